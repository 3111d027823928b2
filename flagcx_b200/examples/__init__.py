"""Runnable examples of the PyTorch backend and of the parallel building blocks."""
