"""Torch-facing wrappers over the C ABI (include/tsb200.h).

PyTorch is used for device memory and streams only: every function here takes CUDA
tensors, passes raw pointers plus the current stream to libtsb200.so and returns torch
tensors.  No function has a CPU or eager-PyTorch fallback.
"""
import ctypes as C
import torch

from . import _lib
from ._lib import F32, BF16, KV_INT8, KV_FP8, KV_NVFP4, KV_F32, KV_BF16, LinearDesc, KVDesc, check

from ._lib import Tsb200Error  # noqa: F401  (re-exported)

ATTN_STATUS_OFFSET = 16380      # byte offset of the status word inside an attention workspace (last int of the counter block)
KV_FORMATS = {"int8": KV_INT8, "fp8": KV_FP8, "nvfp4": KV_NVFP4, "fp32": KV_F32, "bf16": KV_BF16}
PAGE = 16


def set_pdl(enabled):
    """Programmatic dependent launch for the decode-step kernels (process-wide); returns the old setting."""
    return bool(_lib.load().tsb200_set_pdl(int(bool(enabled))))


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"unsupported activation dtype {t.dtype} (float32 or bfloat16)")


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _cuda(t, name):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _token_strided(t, name):
    """t [B, T, heads, d] whose (heads, d) block is dense and whose tokens are evenly spaced
    (e.g. a column slice of a fused projection output).  Returns the token stride in elements."""
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    B, T, h, d = t.shape
    if t.numel() == 0:
        return h * d
    if t.stride(3) != 1 or (h > 1 and t.stride(2) != d):     # the stride of a size-1 dimension is arbitrary
        raise ValueError(f"{name}: the (heads, d) block of a token must be dense")
    if T == 1:                       # decode: one token per sequence, spaced by the batch stride
        return t.stride(0) if B > 1 else h * d
    if B > 1 and t.stride(0) != T * t.stride(1):
        raise ValueError(f"{name}: tokens must be evenly strided across the batch")
    return t.stride(1)


# ---------------------------------------------------------------- weights ----------
def precision_code(precision):
    """Reference vocabulary (compression/registry.py): int bits or the string "binary"."""
    if precision == "binary":
        return 0
    p = int(precision)
    if not 2 <= p <= 8:
        raise ValueError(f"precision must be 2..8 or 'binary', got {precision!r}")
    return p


def container_bits(precision, has_zero=False):
    if precision == "binary" or precision == 0:
        return 2 if has_zero else 1
    p = int(precision)
    return 8 if p > 4 else (4 if p > 2 else 2)


def packed_row_bytes(cols, bits):
    return int(_lib.load().tsb200_packed_row_bytes(cols, bits))


def quantize_weight(w, precision, granularity="per_channel", eps=1e-6):
    """vanilla.py:40-49 on the GPU: -> (codes int8 [rows, cols], scales fp32 [rows])."""
    lib = _lib.load()
    w = _cuda(w, "w")
    rows, cols = w.shape
    codes = torch.empty((rows, cols), dtype=torch.int8, device=w.device)
    scales = torch.empty((rows,), dtype=torch.float32, device=w.device)
    ws = torch.empty(16, dtype=torch.uint8, device=w.device)
    check(lib.tsb200_quantize_weight(_p(w), _dt(w), rows, cols, precision_code(precision),
                                     int(granularity == "per_channel"), float(eps), _p(codes), _p(scales),
                                     _p(ws), 16, _stream()), "tsb200_quantize_weight")
    return codes, scales


def pack_codes(codes, bits):
    """-> (packed uint8 [rows, row_bytes], saw_zero: bool (only meaningful for bits == 1))."""
    lib = _lib.load()
    codes = _cuda(codes, "codes")
    rows, cols = codes.shape
    packed = torch.empty((rows, packed_row_bytes(cols, bits)), dtype=torch.uint8, device=codes.device)
    flag = torch.zeros(1, dtype=torch.int32, device=codes.device)
    check(lib.tsb200_pack_codes(_p(codes), rows, cols, bits, _p(packed), _p(flag), _stream()), "tsb200_pack_codes")
    return packed, (bool(flag.item()) if bits == 1 else False)


def unpack_codes(packed, rows, cols, bits):
    lib = _lib.load()
    codes = torch.empty((rows, cols), dtype=torch.int8, device=packed.device)
    check(lib.tsb200_unpack_codes(_p(_cuda(packed, "packed")), rows, cols, bits, _p(codes), _stream()),
          "tsb200_unpack_codes")
    return codes


def dequantize_weight(packed, scales, rows, cols, bits, dtype):
    lib = _lib.load()
    out = torch.empty((rows, cols), dtype=dtype, device=packed.device)
    check(lib.tsb200_dequantize_weight(_p(_cuda(packed, "packed")), _p(_cuda(scales, "scales")), rows, cols, bits,
                                       _dt(out), _p(out), _stream()), "tsb200_dequantize_weight")
    return out


class Factor:
    """One factor of a LinearCompressed layer in kernel form: packed codes + row scales,
    or the dense matrix in the activation dtype."""

    def __init__(self, data, scales, bits, rows, cols):
        self.data, self.scales, self.bits, self.rows, self.cols = data, scales, bits, rows, cols

    @staticmethod
    def dense(w):
        w = _cuda(w, "w")
        bits = 32 if w.dtype == torch.float32 else 16
        _dt(w)
        return Factor(w, None, bits, w.shape[0], w.shape[1])

    @staticmethod
    def from_codes(codes, scales, precision):
        """codes int8 [rows, cols] and scales (any shape with `rows` or 1 elements) as the
        reference's quantize_vanilla returned them."""
        codes = _cuda(codes.to(torch.int8), "codes")
        rows, cols = codes.shape
        s = scales.detach().reshape(-1).to(device=codes.device, dtype=torch.float32)
        if s.numel() == 1:
            s = s.expand(rows)
        s = s.contiguous()
        bits = container_bits(precision)
        packed, zero = pack_codes(codes, bits)
        if bits == 1 and zero:
            bits = 2
            packed, _ = pack_codes(codes, bits)
        return Factor(packed, s, bits, rows, cols)

    @staticmethod
    def quantize(w, precision, granularity="per_channel", eps=1e-6):
        codes, scales = quantize_weight(w, precision, granularity, eps)
        return Factor.from_codes(codes, scales, precision)

    def codes(self):
        return unpack_codes(self.data, self.rows, self.cols, self.bits)

    def state(self, prefix=""):
        """Tensors that rebuild this factor without re-quantizing: the packed container (or dense
        matrix), the row scales and a meta vector [bits, rows, cols]."""
        d = {prefix + "data": self.data, prefix + "meta": torch.tensor([self.bits, self.rows, self.cols], dtype=torch.int64)}
        if self.scales is not None:
            d[prefix + "scales"] = self.scales
        return d

    @staticmethod
    def from_state(sd, prefix="", device="cuda"):
        bits, rows, cols = (int(v) for v in sd[prefix + "meta"].tolist())
        data = sd[prefix + "data"].to(device).contiguous()
        scales = sd.get(prefix + "scales")
        if bits >= 16:
            if tuple(data.shape) != (rows, cols):
                raise ValueError("dense factor: shape does not match its meta record")
            return Factor(data, None, bits, rows, cols)
        if data.dtype != torch.uint8 or tuple(data.shape) != (rows, packed_row_bytes(cols, bits)):
            raise ValueError("packed factor: container shape does not match its meta record")
        if scales is None or scales.numel() != rows:
            raise ValueError("packed factor: one fp32 scale per row is required")
        return Factor(data, scales.to(device=device, dtype=torch.float32).contiguous(), bits, rows, cols)

    def reconstruct(self, dtype):
        if self.bits >= 16:
            return self.data
        return dequantize_weight(self.data, self.scales, self.rows, self.cols, self.bits, dtype)


_workspaces = {}


def workspace(device, nbytes, kind="linear"):
    """Grow-only scratch buffer per (device, kind) (PyTorch owns the memory).  Linear layers and
    attention keep separate buffers: the head of a linear workspace holds a status word and
    split-K counters that must stay zero between calls, attention overwrites its whole buffer."""
    key = (device, kind)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)   # status word / counters start at 0
        _workspaces[key] = buf
    return buf


class PackedLinear:
    """Kernel-side state of one LinearCompressed (blocks/linear_compressed.py:9): U factor,
    optional V factor, bias; __call__ is LinearCompressed.forward."""

    def __init__(self, u, v=None, bias=None, act_dtype=torch.bfloat16):
        self.u, self.v, self.bias, self.act_dtype = u, v, bias, act_dtype
        self.out_features = u.rows
        self.rank = v.rows if v is not None else 0
        self.in_features = v.cols if v is not None else u.cols
        if v is not None and u.cols != v.rows:
            raise ValueError("U is [out, rank] and V is [rank, in]: inner sizes differ")
        if bias is not None:
            self.bias = _cuda(bias.to(act_dtype), "bias")
        self.desc = LinearDesc(self.in_features, self.out_features, self.rank,
                               BF16 if act_dtype == torch.bfloat16 else F32, u.bits, v.bits if v is not None else 0, 0,
                               u.data.data_ptr(), 0 if u.scales is None else u.scales.data_ptr(),
                               0 if v is None else v.data.data_ptr(),
                               0 if v is None or v.scales is None else v.scales.data_ptr(),
                               0 if self.bias is None else self.bias.data_ptr())
        self.force_simt = False

    def workspace_bytes(self, M):
        return int(_lib.load().tsb200_linear_workspace_bytes(C.byref(self.desc), M))

    def state(self, prefix=""):
        """Flat dict of tensors (torch.save / safetensors friendly) that `from_state` turns back into
        the same layer: codes and scales are stored, never re-derived."""
        d = self.u.state(prefix + "u.")
        if self.v is not None:
            d.update(self.v.state(prefix + "v."))
        if self.bias is not None:
            d[prefix + "bias"] = self.bias
        d[prefix + "act_bf16"] = torch.tensor([1 if self.act_dtype == torch.bfloat16 else 0], dtype=torch.int64)
        return d

    @staticmethod
    def from_state(sd, prefix="", device="cuda"):
        act = torch.bfloat16 if int(sd[prefix + "act_bf16"].item()) else torch.float32
        u = Factor.from_state(sd, prefix + "u.", device)
        v = Factor.from_state(sd, prefix + "v.", device) if prefix + "v.meta" in sd else None
        bias = sd.get(prefix + "bias")
        return PackedLinear(u, v, None if bias is None else bias.to(device), act)

    def __call__(self, x, out=None, ws=None):
        lib = _lib.load()
        if x.is_cuda and not x.is_contiguous():
            x = x.contiguous()          # LinearCompressed.forward takes any view (e.g. hidden_states[:, -1:, :])
        x = _cuda(x, "x")
        if x.dtype != self.act_dtype:
            raise TypeError(f"x is {x.dtype}, layer was packed for {self.act_dtype}")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        if out is None:
            out = torch.empty((M, self.out_features), dtype=x.dtype, device=x.device)
        nbytes = self.workspace_bytes(M)
        if ws is None:
            ws = workspace(x.device, nbytes)
        fn = lib.tsb200_linear_simt if self.force_simt else lib.tsb200_linear
        check(fn(C.byref(self.desc), _p(x2), _p(out), M, _p(ws), ws.numel(), _stream()), "tsb200_linear")
        return out.reshape(*lead, self.out_features)

    def argmax_workspace_bytes(self, M):
        return int(_lib.load().tsb200_linear_argmax_workspace_bytes(C.byref(self.desc), M))

    def argmax(self, x, out=None, ws=None):
        """Greedy head: argmax over the layer's outputs per row of x [M, in] -> int64 [M]; equals
        torch.argmax(self(x), -1) (first maximum on ties).  A dense bf16 head reduces inside the GEMM's epilogue
        and never writes the logits."""
        lib = _lib.load()
        x = _cuda(x, "x")
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        if out is None:
            out = torch.empty(M, dtype=torch.int64, device=x.device)
        if ws is None:
            ws = workspace(x.device, self.argmax_workspace_bytes(M), "head")
        check(lib.tsb200_linear_argmax(C.byref(self.desc), _p(x2), _p(out), M, _p(ws), ws.numel(), _stream()), "tsb200_linear_argmax")
        return out

    @staticmethod
    def device_status(ws=None, device=None):
        """Status word of a workspace (synchronises): 0, or the code of a bounded wait that ran out."""
        ws = ws if ws is not None else _workspaces[(device, "linear")]
        return int(ws[:4].view(torch.int32).item())


class GatedMLP:
    """down(silu(gate(x)) * up(x)): MLPGated.forward (blocks/mlp.py:171-185) on three PackedLinear."""

    def __init__(self, gate, up, down):
        self.gate, self.up, self.down = gate, up, down

    def workspace_bytes(self, M):
        return int(_lib.load().tsb200_mlp_gated_workspace_bytes(C.byref(self.gate.desc), C.byref(self.up.desc),
                                                                C.byref(self.down.desc), M))

    def __call__(self, x, out=None, ws=None):
        lib = _lib.load()
        x = _cuda(x, "x")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        if out is None:
            out = torch.empty((M, self.down.out_features), dtype=x.dtype, device=x.device)
        if ws is None:
            ws = workspace(x.device, self.workspace_bytes(M), "mlp")
        check(lib.tsb200_mlp_gated(C.byref(self.gate.desc), C.byref(self.up.desc), C.byref(self.down.desc), _p(x2),
                                   _p(out), M, _p(ws), ws.numel(), _stream()), "tsb200_mlp_gated")
        return out.reshape(*lead, self.down.out_features)


# ---------------------------------------------------------------- KV cache ---------
def kv_record_bytes(fmt, head_dim):
    return int(_lib.load().tsb200_kv_record_bytes(fmt, head_dim))


class PagedKV:
    """Pools + block table + lengths of ONE layer's quantized paged KV cache."""

    def __init__(self, fmt, num_pages, hkv, head_dim, block_table, seq_lens, device, k_scale=None, v_scale=None):
        self.fmt = KV_FORMATS[fmt] if isinstance(fmt, str) else fmt
        self.hkv, self.head_dim, self.num_pages = hkv, head_dim, num_pages
        self.rec = kv_record_bytes(self.fmt, head_dim)
        if self.rec == 0:
            raise ValueError("unsupported KV format / head_dim")
        # zero-initialised once: stale slots must hold finite codes and scales
        self.k_pool = torch.zeros((num_pages, hkv, self.rec), dtype=torch.uint8, device=device)
        self.v_pool = torch.zeros((num_pages, hkv, self.rec), dtype=torch.uint8, device=device)
        self.block_table = block_table     # int32 [B, pages_per_seq] (shared between layers)
        self.seq_lens = seq_lens           # int32 [B]               (shared between layers)
        B = block_table.shape[0]
        # FP8 pages: one scale per (sequence, head), amax / 448 over the prompt, frozen for decode.  Until
        # they are set (set_fp8_scales / fill_fp8_scales / constructor arguments) the placeholders are 1.0,
        # which saturates anything above 448 - generate() refuses to run on placeholders.
        self.fp8_scales_set = self.fmt != KV_FP8 or (k_scale is not None and v_scale is not None)
        if self.fmt == KV_FP8:
            self.k_scale = k_scale if k_scale is not None else torch.ones((B, hkv), dtype=torch.float32, device=device)
            self.v_scale = v_scale if v_scale is not None else torch.ones((B, hkv), dtype=torch.float32, device=device)
        else:
            self.k_scale = self.v_scale = None
        self._desc = None

    def fill_fp8_scales(self, k_scale, v_scale):
        """Set the FP8 scales from known values (floats or tensors broadcastable to [B, hkv])."""
        if self.k_scale is None:
            raise ValueError("only FP8 pages carry per-sequence scales")
        self.k_scale.copy_(torch.as_tensor(k_scale, dtype=torch.float32).expand_as(self.k_scale))
        self.v_scale.copy_(torch.as_tensor(v_scale, dtype=torch.float32).expand_as(self.v_scale))
        self.fp8_scales_set = True

    def desc(self, seq_lens=None):
        # rebuilt on every call: block_table / seq_lens tensors may have been swapped
        seq = self.seq_lens if seq_lens is None else seq_lens
        return KVDesc(self.fmt, self.hkv, self.head_dim, 0, self.num_pages, self.k_pool.data_ptr(),
                      self.v_pool.data_ptr(), self.block_table.data_ptr(), self.block_table.shape[1],
                      seq.data_ptr(), 0 if self.k_scale is None else self.k_scale.data_ptr(),
                      0 if self.v_scale is None else self.v_scale.data_ptr())

    def set_fp8_scales(self, k, v, rope=None, pos0=None):
        """scale = amax/448 over the prompt k, v [B, T, hkv, d] (k after RoPE when given)."""
        lib = _lib.load()
        B, T = k.shape[:2]
        cos, sin = (None, None) if rope is None else rope
        check(lib.tsb200_kv_fp8_scales(_p(_cuda(k, "k")), _p(_cuda(v, "v")), _dt(k), B, T, self.hkv, self.head_dim,
                                       _p(pos0), _p(cos), _p(sin), 0 if cos is None else cos.shape[0],
                                       _p(self.k_scale), _p(self.v_scale), _stream()), "tsb200_kv_fp8_scales")
        self.fp8_scales_set = True

    def rope_append(self, q, k, v, rope, new_lens=None, seq_lens=None):
        """One launch: RoPE on q [B, T, H, d] in place, RoPE on k, quantize-and-append k, v."""
        lib = _lib.load()
        B, T = k.shape[:2]
        cos, sin = rope
        d = self.desc(seq_lens)
        qs, ks, vs = _token_strided(q, "q"), _token_strided(k, "k"), _token_strided(v, "v")
        check(lib.tsb200_rope_append(C.byref(d), _p(q), q.shape[2], qs, _p(k), _p(v), _dt(k), ks, vs, B, T,
                                     _p(new_lens), _p(cos), _p(sin), cos.shape[0], _stream()), "tsb200_rope_append")

    def append(self, k, v, new_lens=None, rope=None, seq_lens=None):
        """k, v [B, T, hkv, d]; token j of sequence b -> position seq_lens[b] + j.
        seq_lens is NOT advanced (it is shared by all layers; advance it once per step).
        `seq_lens` overrides the tensor of write positions for this call."""
        lib = _lib.load()
        B, T = k.shape[:2]
        cos, sin = (None, None) if rope is None else rope
        d = self.desc(seq_lens)
        ks, vs = _token_strided(k, "k"), _token_strided(v, "v")
        check(lib.tsb200_kv_append(C.byref(d), _p(k), _p(v), _dt(k), ks, vs, B, T, _p(new_lens),
                                   _p(cos), _p(sin), 0 if cos is None else cos.shape[0], _stream()),
              "tsb200_kv_append")


def kv_gather(kv, L, dtype=torch.bfloat16, seq_lens=None):
    """Dense dequantized copies k, v [B, L, hkv, d] of the first L cached positions of every
    sequence (zeros beyond seq_lens[b]): what an attention over T > 1 query tokens reads."""
    lib = _lib.load()
    B = kv.block_table.shape[0]
    dev = kv.k_pool.device
    k = torch.empty((B, L, kv.hkv, kv.head_dim), dtype=dtype, device=dev)
    v = torch.empty_like(k)
    d = kv.desc(seq_lens)
    check(lib.tsb200_kv_gather(C.byref(d), _p(k), _p(v), _dt(k), B, L, _stream()), "tsb200_kv_gather")
    return k, v


def prefill_attention(kv, q, L, sm_scale=None, out=None, status=None, seq_lens=None):
    """Causal attention of a prompt chunk: q [B, T, H, d] (heads dense, tokens evenly strided; bf16) over the first
    L >= T positions of the cache `kv` (query i at position L - T + i), reading the dequantized cache
    (blocks/mha.py:9-103 for T > 1).  bf16: head-major gather + tcgen05 kernel.  fp32: every query token becomes a
    one-token "sequence" of the paged decode kernel (block-table rows repeated, lengths L - T + i + 1), which reads
    the pages directly in fp32 math.  Returns out [B, T, H, d]."""
    lib = _lib.load()
    B, T, H, d = q.shape
    if sm_scale is None:
        sm_scale = d ** -0.5
    if out is None:
        out = torch.empty((B, T, H, d), dtype=q.dtype, device=q.device)
    if q.dtype == torch.float32:
        lens = (torch.arange(L - T + 1, L + 1, dtype=torch.int32, device=q.device)).repeat(B)          # [B * T]
        base = kv.seq_lens if seq_lens is None else seq_lens
        lens = torch.minimum(lens, base.repeat_interleave(T))
        view = PagedKV.__new__(PagedKV)
        view.__dict__.update(kv.__dict__)
        view.block_table = kv.block_table.repeat_interleave(T, dim=0).contiguous()
        view.seq_lens = lens
        if kv.k_scale is not None:
            view.k_scale, view.v_scale = kv.k_scale.repeat_interleave(T, dim=0).contiguous(), kv.v_scale.repeat_interleave(T, dim=0).contiguous()
        qq = q.reshape(B * T, H, d) if q.is_contiguous() else q.contiguous().reshape(B * T, H, d)
        paged_decode_attention(view, qq, max(int(L), 1), sm_scale=sm_scale, out=out.view(B * T, H, d))
        return out
    if q.dtype != torch.bfloat16:
        raise TypeError("prefill attention takes bf16 (tcgen05) or fp32 (paged kernel) activations")
    qs = _token_strided(q, "q")
    Lp = (L + 63) // 64 * 64
    kd = torch.empty((B, kv.hkv, L, d), dtype=torch.bfloat16, device=q.device)
    vt = torch.empty((B, kv.hkv, d, Lp), dtype=torch.bfloat16, device=q.device)
    desc = kv.desc(seq_lens)
    check(lib.tsb200_kv_gather_heads(C.byref(desc), _p(kd), _p(vt), B, L, Lp, _stream()), "tsb200_kv_gather_heads")
    check(lib.tsb200_prefill_attn(_p(q), qs, _p(kd), _p(vt), _p(out), B, T, L, Lp, H, kv.hkv, d, float(sm_scale), _p(status),
                                  _stream()), "tsb200_prefill_attn")
    return out


def decode_attn_workspace_bytes(B, H, head_dim, max_seq_len):
    return int(_lib.load().tsb200_paged_decode_attn_workspace_bytes(B, H, head_dim, max_seq_len))


def paged_decode_attention(kv, q, max_seq_len, sm_scale=None, out=None, ws=None, simt=False, seq_lens=None):
    """q [B, H, d] -> out [B, H, d]: softmax(q K^T * sm_scale) V over seq_lens[b] cached tokens
    (blocks/mha.py:9-103 for one query token per sequence)."""
    lib = _lib.load()
    if not q.is_cuda:
        raise ValueError("q must be a CUDA tensor (this library has no CPU path)")
    B, H, d = q.shape
    if q.numel() and (q.stride(2) != 1 or q.stride(1) != d):
        raise ValueError("q: heads/d must be dense")
    qs = q.stride(0) if q.numel() else H * d
    if out is None:
        out = torch.empty((B, H, d), dtype=q.dtype, device=q.device)
    nbytes = decode_attn_workspace_bytes(B, H, d, max_seq_len)
    if ws is None:
        ws = workspace(q.device, nbytes, "attention")
    if sm_scale is None:
        sm_scale = d ** -0.5
    fn = lib.tsb200_paged_decode_attn_simt if simt else lib.tsb200_paged_decode_attn
    desc = kv.desc(seq_lens)
    check(fn(C.byref(desc), _p(q), _p(out), _dt(q), qs, B, H, float(sm_scale), int(max_seq_len), _p(ws), ws.numel(),
             _stream()), "tsb200_paged_decode_attn")
    return out


# ---------------------------------------------------------------- small ops --------
def rope_(x, cos, sin, pos0=None):
    """In-place half-split RoPE on x [B, T, heads, d] (blocks/rope.py:140-173)."""
    lib = _lib.load()
    B, T, h, d = x.shape
    xs = _token_strided(x, "x")
    check(lib.tsb200_rope(_p(x), _dt(x), xs, B, T, h, d, _p(pos0), _p(cos), _p(sin), cos.shape[0], _stream()),
          "tsb200_rope")
    return x


def add_rmsnorm(residual, delta, w, eps=1e-6, variant=0, out=None):
    """residual += delta (in place, delta may be None); returns RMSNorm(residual) * w.
    variant 0 = Hugging Face Qwen2/Llama RMSNorm, 1 = blocks/norm.py:8-23."""
    lib = _lib.load()
    r2 = _cuda(residual, "residual").reshape(-1, residual.shape[-1])
    M, hidden = r2.shape
    if out is None:
        out = torch.empty_like(r2)
    check(lib.tsb200_add_rmsnorm(_p(r2), _p(delta), _p(_cuda(w, "w")), _p(out), _dt(r2), M, hidden, float(eps),
                                 variant, _stream()), "tsb200_add_rmsnorm")
    return out.reshape(residual.shape)


def swiglu(gate, up, out=None):
    """silu(gate) * up (blocks/mlp.py:181-183); gate/up may be column slices of one buffer."""
    lib = _lib.load()
    M, n = gate.shape
    if gate.stride(1) != 1 or up.stride(1) != 1:
        raise ValueError("gate/up must be unit-stride in the last dimension")
    if out is None:
        out = torch.empty((M, n), dtype=gate.dtype, device=gate.device)
    check(lib.tsb200_swiglu(_p(gate), _p(up), _p(out), _dt(gate), M, n, gate.stride(0), up.stride(0), out.stride(0),
                            _stream()), "tsb200_swiglu")
    return out
