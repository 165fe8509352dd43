"""Operators: each has a PyTorch reference (CPU oracle) and an sm_100a kernel path."""
