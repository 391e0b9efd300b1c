"""ctypes binding of libmagi_attn.so (the C ABI declared in include/magi_attn.h).

There is no fallback: if the library is missing or fails to load, importing this module raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmagi_attn.so")

MAGI_OK = 0
E_BADARG, E_ALIGN, E_ARCH, E_RANGE, E_NOMEM, E_NCCL, E_TIMEOUT, E_CUDA = -1, -2, -3, -4, -5, -6, -7, -8
DTYPE_BF16, DTYPE_FP8_E4M3, DTYPE_F32 = 0, 1, 2
NORM_LAYERNORM_1P, NORM_RMSNORM_1P, NORM_NONE = 0, 1, 2

EXPORTS = [
    "magi_version", "magi_strerror", "magi_ctx_create", "magi_ctx_destroy", "magi_last_error", "magi_ctx_status",
    "magi_qk_norm_rope_fwd", "magi_head_block_copy", "magi_kv_cache_create", "magi_kv_cache_destroy",
    "magi_kv_cache_append", "magi_kv_cache_evict", "magi_kv_cache_read", "magi_kv_cache_bytes",
    "magi_chunk_attn_fwd", "magi_chunk_attn_fwd_simt", "magi_quantize_e4m3_block128", "magi_chunk_attn_fwd_noalloc",
    "magi_peer_alloc", "magi_peer_open", "magi_peer_close", "magi_peer_free", "magi_selftest_bounded_wait",
    "magi_bias_modulate_add", "magi_div_clamp_to_e4m3", "magi_linear_qk_norm_rope_fwd", "magi_linear_qkv_norm_rope_fwd",
    "magi_ulysses_unique_id", "magi_ulysses_create", "magi_ulysses_destroy", "magi_ulysses_a2a_in", "magi_ulysses_a2a_out",
]


class PrologueParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("norm_mode", C.c_int32),
        ("x", C.c_void_p), ("x_stride_t", C.c_int64), ("x_stride_h", C.c_int64),
        ("T", C.c_int32), ("H", C.c_int32),
        ("gamma", C.c_void_p), ("beta", C.c_void_p), ("eps", C.c_float), ("rot_pairs", C.c_int32),
        ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("out", C.c_void_p), ("out_stride_t", C.c_int64), ("out_stride_h", C.c_int64), ("out_stride_block", C.c_int64),
        ("heads_per_block", C.c_int32), ("out_block_ptrs", C.POINTER(C.c_void_p)),
        ("x_heads_per_block", C.c_int32), ("x_stride_block", C.c_int64),
    ]


class LinearPrologueParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("norm_mode", C.c_int32),
        ("x", C.c_void_p), ("x_stride", C.c_int64), ("w", C.c_void_p), ("w_stride", C.c_int64),
        ("T", C.c_int32), ("H", C.c_int32), ("in_features", C.c_int32), ("eps", C.c_float),
        ("gamma", C.c_void_p), ("beta", C.c_void_p), ("rot_pairs", C.c_int32), ("heads_per_block", C.c_int32),
        ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("out", C.c_void_p), ("out_stride_t", C.c_int64), ("out_stride_h", C.c_int64), ("out_stride_block", C.c_int64),
        ("out_block_ptrs", C.POINTER(C.c_void_p)),
        ("dtype", C.c_int32), ("plain_odd_heads", C.c_int32), ("x_scale", C.c_void_p), ("w_scale", C.c_void_p),
    ]


class KVCacheDesc(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32), ("n_layers", C.c_int32), ("max_chunks", C.c_int32),
        ("chunk_tokens", C.c_int32), ("n_kv_heads", C.c_int32),
    ]


class AttnParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype", C.c_int32),
        ("q", C.c_void_p), ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
        ("k", C.c_void_p), ("k_stride_t", C.c_int64), ("k_stride_h", C.c_int64),
        ("v", C.c_void_p), ("v_stride_t", C.c_int64), ("v_stride_h", C.c_int64),
        ("out", C.c_void_p), ("o_stride_t", C.c_int64), ("o_stride_h", C.c_int64),
        ("lse", C.c_void_p),
        ("total_q", C.c_int32), ("total_k", C.c_int32), ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32),
        ("q_ranges", C.c_void_p), ("k_ranges", C.c_void_p), ("k_range_offsets", C.c_void_p),
        ("n_ranges", C.c_int32), ("n_k_ranges", C.c_int32), ("max_seqlen_q", C.c_int32), ("max_seqlen_k", C.c_int32),
        ("softmax_scale", C.c_float),
        ("cache", C.c_void_p), ("layer", C.c_int32), ("n_prefix_chunks", C.c_int32),
        ("prefix_chunk_ids", C.POINTER(C.c_int32)),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("scale_chunk_tokens", C.c_int32), ("reserved", C.c_int32), ("q_lo", C.c_void_p),
        ("o_peer_ptrs", C.POINTER(C.c_void_p)), ("o_peer_offsets", C.POINTER(C.c_int32)),
        ("n_o_peers", C.c_int32), ("o_head_offset", C.c_int32),
        ("o_heads_per_block", C.c_int32), ("reserved2", C.c_int32), ("o_stride_block", C.c_int64),
    ]


class ModulateParams(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("x_dtype", C.c_int32),
        ("x", C.c_void_p), ("x_stride", C.c_int64),
        ("residual", C.c_void_p), ("residual_stride", C.c_int64),
        ("residual_dtype", C.c_int32), ("gate_dtype", C.c_int32),
        ("gate", C.c_void_p), ("gate_stride", C.c_int64),
        ("condition_map", C.c_void_p), ("map_is_int64", C.c_int32), ("n_gates", C.c_int32),
        ("gamma", C.c_void_p), ("beta", C.c_void_p), ("eps", C.c_float), ("gamma_plus_one", C.c_int32),
        ("out", C.c_void_p), ("out_stride", C.c_int64), ("rows", C.c_int32), ("hidden", C.c_int32),
    ]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python magi-1_b200/build.py` (there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
    sig = {
        "magi_version": (C.c_int, []),
        "magi_strerror": (C.c_char_p, [i32]),
        "magi_ctx_create": (C.c_int, [i32, C.POINTER(vp)]),
        "magi_ctx_destroy": (C.c_int, [vp]),
        "magi_last_error": (C.c_char_p, [vp]),
        "magi_ctx_status": (C.c_int, [vp, vp, C.POINTER(C.c_int)]),
        "magi_selftest_bounded_wait": (C.c_int, [vp, C.c_longlong, vp]),
        "magi_ulysses_unique_id": (C.c_int, [vp, vp]),
        "magi_ulysses_create": (C.c_int, [vp, vp, i32, i32, C.POINTER(C.c_int32), C.POINTER(vp)]),
        "magi_ulysses_destroy": (C.c_int, [vp]),
        "magi_ulysses_a2a_in": (C.c_int, [vp, vp, vp, i64, vp]),
        "magi_ulysses_a2a_out": (C.c_int, [vp, vp, vp, i64, vp]),
        "magi_qk_norm_rope_fwd": (C.c_int, [vp, C.POINTER(PrologueParams), vp]),
        "magi_head_block_copy": (C.c_int, [vp, C.POINTER(PrologueParams), vp]),
        "magi_linear_qk_norm_rope_fwd": (C.c_int, [vp, C.POINTER(LinearPrologueParams), vp]),
        "magi_linear_qkv_norm_rope_fwd": (C.c_int, [vp, C.POINTER(LinearPrologueParams), i32, vp]),
        "magi_kv_cache_create": (C.c_int, [vp, C.POINTER(KVCacheDesc), C.POINTER(vp)]),
        "magi_kv_cache_destroy": (C.c_int, [vp]),
        "magi_kv_cache_append": (C.c_int, [vp, i32, i32, vp, i64, i64, vp, i64, i64, i32, i32, vp]),
        "magi_kv_cache_evict": (C.c_int, [vp, i32]),
        "magi_kv_cache_read": (C.c_int, [vp, i32, i32, vp, vp, i32, i32, vp]),
        "magi_kv_cache_bytes": (C.c_int64, [vp]),
        "magi_chunk_attn_fwd": (C.c_int, [vp, C.POINTER(AttnParams), vp]),
        "magi_chunk_attn_fwd_simt": (C.c_int, [vp, C.POINTER(AttnParams), vp]),
        "magi_quantize_e4m3_block128": (C.c_int, [vp, vp, i64, i64, i32, i32, i32, vp, vp, vp, vp]),
        "magi_chunk_attn_fwd_noalloc": (C.c_int, [C.POINTER(AttnParams), vp, vp, C.c_char_p, i32]),
        "magi_bias_modulate_add": (C.c_int, [vp, C.POINTER(ModulateParams), vp]),
        "magi_div_clamp_to_e4m3": (C.c_int, [vp, vp, i64, i32, i32, vp, i32, vp, i64, vp]),
        "magi_peer_alloc": (C.c_int, [vp, C.c_uint64, C.POINTER(vp), C.c_char_p]),
        "magi_peer_open": (C.c_int, [vp, C.c_char_p, C.POINTER(vp)]),
        "magi_peer_close": (C.c_int, [vp, vp]),
        "magi_peer_free": (C.c_int, [vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class MagiError(RuntimeError):
    def __init__(self, code, detail=""):
        self.code = code
        msg = lib.magi_strerror(code).decode()
        super().__init__(f"libmagi_attn: {msg} ({code}){': ' + detail if detail else ''}")


def check(code, ctx=None):
    if code != MAGI_OK:
        detail = lib.magi_last_error(ctx).decode() if ctx else ""
        raise MagiError(code, detail)
