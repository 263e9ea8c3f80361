"""Tensor / expert / pipeline parallel plumbing: torch.distributed (NCCL) for bootstrap and baselines,
peer-memory kernels for the hot collectives."""
