"""B200 (sm_100a) kernels for transformer-surgeon's compressed decode hot path.

The package mirrors the reference's interfaces for that path only:
  ops.PackedLinear           LinearCompressed.forward on packed low-rank / quantized factors
  ops.PagedKV + ops.paged_decode_attention   quantized paged KV cache (int8 / fp8 / nvfp4)
  surgeon.pack_model         rebinds LinearCompressed.forward per instance after manager.apply()
  decoder.CompressedDecoder  Qwen2 / Llama decode step built from those kernels
Everything calls libtsb200.so through the C ABI in include/tsb200.h; there is no fallback.
"""
from . import _lib, ops  # noqa: F401
from ._lib import Tsb200Error  # noqa: F401
