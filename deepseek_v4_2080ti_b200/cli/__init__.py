"""Command-line tools: ``python -m deepseek_v4_2080ti_b200.cli.<tool>``.

inspect_gguf (spec / validate / capability / placement), generate_gguf (greedy generation from a GGUF checkpoint, one
process per GPU under torchrun), merge_imatrix, make_routed_source_gguf, convert_checkpoint."""
