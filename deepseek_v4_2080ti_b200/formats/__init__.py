"""Checkpoint formats: Safetensors FP8 block-128 / FP4 E2M1+UE8M0, GGUF raw blocks."""
