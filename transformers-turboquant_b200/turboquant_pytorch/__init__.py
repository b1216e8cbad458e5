"""Import-name compatibility for `turboquant_pytorch.compressors`."""
