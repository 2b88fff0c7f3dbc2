"""Command-line tools: recipe target checker, Hugging Face export."""
