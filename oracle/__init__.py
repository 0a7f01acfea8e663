"""CPU oracle for the compressed-decode hot path (TEST INFRASTRUCTURE, not product code).

Only tests, the smoke entry and the CPU-baseline legs of the benchmark may import this
package.  Each function restates, in numpy / CPU torch, the arithmetic of one piece of
the reference (CESOIA/transformer-surgeon) and cites the reference file:line it follows.

Parity status
-------------
* Weight quantization / reconstruction, LinearCompressed.forward, attention(), RoPE,
  RMSNorm, SwiGLU: pinned against outputs of the reference itself (fixtures under
  tests/golden/, produced by tests/golden/make_golden.py importing the reference).
* KV-cache quantization (int8 / FP8-e4m3 / NVFP4) and paging: the reference has no such
  code, so these formats are DEFINED here -> "parity unpinned" for them; only the
  dequantized attention math is pinned (against the reference's attention()).
"""
