"""Multi-GPU layer: symmetric heap over NVLink, fused compute+collective kernels, NCCL baselines."""
