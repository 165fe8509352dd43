"""Process-group plumbing, the flat-buffer training engine and the fused communication paths."""
