"""GGUF container and block-quantisation formats (Q8_0, Q2_K, Q4_K, Q5_K, IQ1_M, IQ2_XXS, IQ3_XXS):
reader, writer, quantisers and reference dequantisers.  The reference reads these files
(src/loader/gguf/reader.py:121-204, bundle.py:115-204, tensor_reader.py:258-1009) but has no quantiser;
the quantisers here exist to synthesise checkpoints and are validated by the dequantisers."""
from .constants import BLOCK_BYTES, BLOCK_ELEMS, GGMLType, KERNEL_TYPE_ID  # noqa: F401
from .quant import dequantize, quantize  # noqa: F401
from .reader import GGUFFile, read_bundle  # noqa: F401
from .writer import write_gguf  # noqa: F401
