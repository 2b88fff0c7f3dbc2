"""Data sources feeding the trainers."""
