"""ctypes binding of libtsb200.so (the C ABI declared in include/tsb200.h).

There is no CPU or PyTorch fallback: if the shared library is missing, or a call returns
a non-zero status, an exception is raised.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtsb200.so")

OK, ERR_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6
F32, BF16 = 0, 1
KV_INT8, KV_FP8, KV_NVFP4, KV_F32, KV_BF16 = 0, 1, 2, 3, 4


class Tsb200Error(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__(what)


class LinearDesc(C.Structure):
    _fields_ = [("in_features", C.c_int64), ("out_features", C.c_int64), ("rank", C.c_int64),
                ("act_dtype", C.c_int32), ("u_bits", C.c_int32), ("v_bits", C.c_int32), ("reserved", C.c_int32),
                ("u", C.c_void_p), ("u_scale", C.c_void_p), ("v", C.c_void_p), ("v_scale", C.c_void_p),
                ("bias", C.c_void_p)]


class KVDesc(C.Structure):
    _fields_ = [("format", C.c_int32), ("hkv", C.c_int32), ("head_dim", C.c_int32), ("reserved", C.c_int32),
                ("num_pages", C.c_int64), ("k_pool", C.c_void_p), ("v_pool", C.c_void_p),
                ("block_table", C.c_void_p), ("bt_stride", C.c_int64), ("seq_lens", C.c_void_p),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p)]


class PeerDesc(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("partial", C.c_void_p * 8), ("flags", C.c_void_p * 8),
                ("epoch", C.c_void_p), ("status", C.c_void_p)]


_i64, _i32, _f32, _vp, _sz = C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t
_LD, _KD, _PD = C.POINTER(LinearDesc), C.POINTER(KVDesc), C.POINTER(PeerDesc)

# name -> (restype, argtypes); mirrors include/tsb200.h one to one.
SIGNATURES = {
    "tsb200_strerror": (C.c_char_p, [_i32]),
    "tsb200_version": (_i32, []),
    "tsb200_last_cuda_error": (_i32, []),
    "tsb200_check_device": (_i32, []),
    "tsb200_set_pdl": (_i32, [_i32]),
    "tsb200_packed_row_bytes": (_sz, [_i64, _i32]),
    "tsb200_quantize_weight": (_i32, [_vp, _i32, _i64, _i64, _i32, _i32, _f32, _vp, _vp, _vp, _sz, _vp]),
    "tsb200_pack_codes": (_i32, [_vp, _i64, _i64, _i32, _vp, _vp, _vp]),
    "tsb200_unpack_codes": (_i32, [_vp, _i64, _i64, _i32, _vp, _vp]),
    "tsb200_dequantize_weight": (_i32, [_vp, _vp, _i64, _i64, _i32, _i32, _vp, _vp]),
    "tsb200_linear_workspace_bytes": (_sz, [_LD, _i64]),
    "tsb200_linear": (_i32, [_LD, _vp, _vp, _i64, _vp, _sz, _vp]),
    "tsb200_linear_simt": (_i32, [_LD, _vp, _vp, _i64, _vp, _sz, _vp]),
    "tsb200_linear_argmax_workspace_bytes": (_sz, [_LD, _i64]),
    "tsb200_linear_argmax": (_i32, [_LD, _vp, _vp, _i64, _vp, _sz, _vp]),
    "tsb200_mlp_gated_workspace_bytes": (_sz, [_LD, _LD, _LD, _i64]),
    "tsb200_mlp_gated": (_i32, [_LD, _LD, _LD, _vp, _vp, _i64, _vp, _sz, _vp]),
    "tsb200_kv_record_bytes": (_sz, [_i32, _i32]),
    "tsb200_kv_fp8_scales": (_i32, [_vp, _vp, _i32, _i64, _i64, _i32, _i32, _vp, _vp, _vp, _i64, _vp, _vp, _vp]),
    "tsb200_kv_append": (_i32, [_KD, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "tsb200_kv_gather": (_i32, [_KD, _vp, _vp, _i32, _i64, _i64, _vp]),
    "tsb200_rope_append": (_i32, [_KD, _vp, _i32, _i64, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "tsb200_kv_gather_heads": (_i32, [_KD, _vp, _vp, _i64, _i64, _i64, _vp]),
    "tsb200_prefill_attn": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _f32, _vp, _vp]),
    "tsb200_paged_decode_attn_workspace_bytes": (_sz, [_i64, _i32, _i32, _i64]),
    "tsb200_paged_decode_attn": (_i32, [_KD, _vp, _vp, _i32, _i64, _i64, _i32, _f32, _i64, _vp, _sz, _vp]),
    "tsb200_paged_decode_attn_simt": (_i32, [_KD, _vp, _vp, _i32, _i64, _i64, _i32, _f32, _i64, _vp, _sz, _vp]),
    "tsb200_paged_decode_attn_static_capacity": (_sz, []),
    "tsb200_paged_decode_attn_static": (_i32, [_KD, _vp, _vp, _i32, _i64, _i64, _i32, _f32, _i64, _vp]),
    "tsb200_rope": (_i32, [_vp, _i32, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _vp, _i64, _vp]),
    "tsb200_peer_flag_bytes": (_sz, []),
    "tsb200_enable_peer_access": (_i32, [_i32]),
    "tsb200_ipc_export": (_i32, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "tsb200_ipc_open": (_i32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "tsb200_ipc_close": (_i32, [_vp]),
    "tsb200_peer_allreduce_add_rmsnorm": (_i32, [_PD, _vp, _vp, _vp, _i32, _i64, _i64, _f32, _vp]),
    "tsb200_add_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, _i64, _f32, _i32, _vp]),
    "tsb200_swiglu": (_i32, [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _vp]),
}

_lib = None


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise Tsb200Error(ERR_DEVICE, f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
                          "(there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(status, what):
    if status != OK:
        lib = load()
        msg = lib.tsb200_strerror(status).decode()
        extra = f" (cudaError {lib.tsb200_last_cuda_error()})" if status == ERR_CUDA else ""
        raise Tsb200Error(status, f"{what}: {msg}{extra}")
