"""Model runtimes: qwen_hybrid (GDN + gated GQA), gqa_moe (MiniMax-shaped), mla_moe (DeepSeek/GLM-shaped)."""
