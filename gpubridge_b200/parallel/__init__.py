"""parallel of gpubridge_b200."""
