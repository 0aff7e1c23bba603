"""bench of gpubridge_b200."""
