"""models of gpubridge_b200."""
