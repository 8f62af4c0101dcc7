"""GGUF container and block formats (Python face of ``csrc/gguf``).

The model server the reference talks to loads GGUF artifacts and picks the family from
``general.architecture`` (reference: docs/muse/muse-glimmer.md:118-126); Q4_K, Q5_K, Q6_K and
Q8_0 are the formats it names (docs/muse/muse-glimmer.md:112,
apps/pylon/docs/2026-06-09-pylon-qwen35-local-inference-roadmap.md:83-88).
"""
from .formats import (GGML_TYPES, GgmlType, dequantize, quantize, tensor_nbytes, type_block,
                      type_name)
from .file import GGUFFile, GGUFTensor, GGUFWriter

__all__ = ["GGML_TYPES", "GgmlType", "dequantize", "quantize", "tensor_nbytes", "type_block",
           "type_name", "GGUFFile", "GGUFTensor", "GGUFWriter"]
