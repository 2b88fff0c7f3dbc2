"""Parallel runtimes: flat sharded trainer, tensor parallel, Ulysses sequence parallel, peer-memory collectives."""
