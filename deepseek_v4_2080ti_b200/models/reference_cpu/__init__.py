"""fp32 PyTorch oracles that consume the same checkpoints as the GPU runtimes (run on CPU or GPU)."""
