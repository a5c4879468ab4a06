"""B200-native TurboQuant inference core: CUDA kernels behind the reference's C API.

The package is a thin ctypes layer over libturboquant_b200.so (built in-tree by
`python -m turboquant_mlx_core_b200.build`).  Importing the package does not load the
library; the first call does, and raises if it is missing.
"""
from ._lib import LIB_PATH, TQ_F16, TQ_F32, LibraryMissing, TQError, load  # noqa: F401
from .api import (Codebook, DecodeBuffer, QuantizedWeight, QuantizerConfig, TQKVCache, TurboQuantLinear,  # noqa: F401
                  append_batch, hybrid_attention, apply_inverse_wht_rotation, apply_wht_rotation, codebook_from_centroids, compressed_attention,
                  dequantize_weight, generate_codebook, generate_codebook_from_data, fit_layer_codebooks, adaptive_block_size,
                  layer_index, is_sensitive_layer, qjl_compress, qjl_dot_correction, quantize_weight, forward_group)
from . import checkpoint  # noqa: F401,E402  (TurboQuant safetensors reader / writer)
