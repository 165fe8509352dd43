"""Training runtime: loop, checkpoints, metrics."""
