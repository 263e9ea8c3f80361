"""B200-native (sm_100a) LLM inference engine with the capabilities of PocketLLM.

Sub-packages:
  ops       ctypes front-ends of the hand-written CUDA kernels + fp32 PyTorch oracles
  models    per-family runtimes (Qwen-style hybrid GDN/GQA, GQA-MoE, MLA-MoE) and CPU oracles
  parallel  tensor / expert / pipeline parallel plumbing over torch.distributed + peer memory
  formats   checkpoint formats: Safetensors FP8/FP4, GGUF k-/i-quants (readers, writers, quantizers)
  runtime   paged KV, scheduler bindings, generation loops, speculative decode
  utils     timing, NVTX ranges, clocks sampling
"""
__version__ = "0.1.0"
