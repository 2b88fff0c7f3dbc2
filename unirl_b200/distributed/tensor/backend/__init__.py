"""Tensor-transport backends."""
