"""utils of gpubridge_b200."""
