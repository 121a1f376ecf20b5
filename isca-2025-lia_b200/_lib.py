"""ctypes binding of libliab200.so (C ABI declared in include/lia_b200.h).

The reference's only C-ABI precedent is loaded the same way
(lia/cxl/numa_alloc.py:8-26: ctypes.CDLL + argtypes/restype).  There is NO fallback:
if the shared library is missing or a call fails, this module raises.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_longlong, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libliab200.so")

EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_RESIDUAL, EPI_QKV = 0, 1, 2, 3
ABI_VERSION = 9
TP_MAX_WORLD = 8
P2P_HANDLE_BYTES = 64


class LiaQkvArgs(ctypes.Structure):
    _fields_ = [("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("hq", c_int32), ("S", c_int32), ("pos0", c_int32), ("cache_batch", c_int32),
                ("b0", c_int32), ("q_scale", c_float)]


class LiaTpArgs(ctypes.Structure):
    _fields_ = [("rank", c_int32), ("world", c_int32), ("arena", c_void_p * TP_MAX_WORLD),
                ("ctl_off", ctypes.c_uint64), ("recv_off", ctypes.c_uint64), ("recv_bytes", ctypes.c_uint64),
                ("out_off", ctypes.c_uint64), ("mc_arena", c_void_p)]


class LiaError(RuntimeError):
    pass


_PROTOTYPES = {
    "lia_abi_version": (c_int, []),
    "lia_last_error": (c_char_p, []),
    "lia_device_info": (c_int, [POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "lia_layernorm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "lia_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "lia_gemm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              POINTER(LiaQkvArgs), c_void_p, c_size_t, c_void_p]),
    "lia_attn_prefill_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_void_p]),
    "lia_attn_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lia_attn_decode_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lia_kv_append_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_float, c_void_p]),
    "lia_embed_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_void_p]),
    "lia_embed_masked_bf16": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      c_int, c_int, c_void_p]),
    "lia_argmax_bf16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_residual_add_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "lia_tp_ctl_bytes": (c_size_t, []),
    "lia_tp_recv_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lia_gemm_allreduce_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        POINTER(LiaTpArgs), c_void_p, c_size_t, c_void_p]),
    "lia_tp_error": (c_int, [POINTER(LiaTpArgs)]),
    "lia_p2p_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_void_p]),
    "lia_p2p_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "lia_p2p_close": (c_int, [c_void_p]),
    "lia_p2p_free": (c_int, [c_void_p]),
    "lia_host_arena_alloc": (c_void_p, [c_size_t]),
    "lia_host_arena_free": (c_int, [c_void_p, c_size_t]),
    "lia_streamer_create": (c_void_p, [POINTER(c_void_p), c_int, c_size_t]),
    "lia_streamer_prefetch": (c_int, [c_void_p, c_int, c_void_p, c_size_t]),
    "lia_streamer_wait": (c_int, [c_void_p, c_int, c_void_p]),
    "lia_streamer_release": (c_int, [c_void_p, c_int, c_void_p]),
    "lia_streamer_stats": (c_int, [c_void_p, POINTER(c_double), POINTER(c_double)]),
    "lia_streamer_destroy": (c_int, [c_void_p]),
    "lia_program_create": (c_void_p, [c_int]),
    "lia_program_add_layernorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float]),
    "lia_program_add_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                     POINTER(LiaQkvArgs), POINTER(LiaTpArgs)]),
    "lia_program_add_attn_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int]),
    "lia_program_add_embed": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int]),
    "lia_program_add_argmax": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "lia_program_finalize": (c_int, [c_void_p]),
    "lia_program_run": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "lia_program_error": (c_int, [c_void_p]),
    "lia_program_num_ops": (c_int, [c_void_p]),
    "lia_program_destroy": (c_int, [c_void_p]),
    # models with a 32-bit residual stream, matrix-memory mixers and latent-cache attention
    "lia_embed_rmsnorm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_rms_add_norm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float,
                                 c_void_p]),
    "lia_rms_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_clamped_glu": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p]),
    "lia_linear_small": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                 c_void_p]),
    "lia_linear_plain": (c_int, [c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_int,
                                 c_longlong, c_longlong, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_argmax_f32": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_mlstm_scan": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p]),
    "lia_headnorm_gate": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "lia_latent_prep": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_latent_attn_workspace_floats": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lia_latent_attn": (c_int, [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    # models between layer norms: decay / delta-rule recurrences, sliding-window attention, mixture-of-experts feed-forward
    "lia_embed_rows": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_ln_add_norm": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_float, c_void_p]),
    "lia_ln_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_gated_act": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "lia_router_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_moe_tile_rows": (c_int, []),
    "lia_moe_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lia_moe_gemm": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lia_moe_gather": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_moe_expert_gemms": (c_int, [c_void_p, c_void_p, c_longlong, c_void_p, POINTER(c_int), c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                                     c_void_p]),
    "lia_moe_combine": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_conv_prep": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p]),
    "lia_conv_state_update": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                      c_void_p]),
    "lia_linear_scan": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "lia_kv_store": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int,
                             c_int, c_int, c_float, c_int, c_void_p]),
    "lia_window_attn_pairs_per_warp": (c_int, [c_int]),
    "lia_window_attn_smem_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "lia_window_attn_workspace_floats": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lia_window_attn": (c_int, [c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p]),
    # models that norm and gate a sublayer's output and mix all earlier layers' results: attention with a sink, a distance
    # bias and an output gate behind a convolution / norm / rotation / value blend; polynomial activation; identity experts
    "lia_window_attn_ext": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                    c_float, c_int, c_int, c_int, c_void_p]),
    "lia_qkv_prep": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                             c_float, c_float, c_int, c_void_p, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lia_gated_rms_add": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p,
                                  c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_poly_norm": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_router_topk_ext": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_moe_gemm_ext": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lia_moe_combine_ext": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                    c_int, c_void_p]),
    # pre-norm designs with learned positions: latent queries, pairwise rotation, attention maps over shared values under a
    # chunked mask, the forget-gate recurrence, experts with a clamped gated activation
    "lia_embed_scale_pos": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                    c_void_p]),
    "lia_residual_norm": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_float, c_void_p]),
    "lia_rms_norm_rows": (c_int, [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "lia_sigmoid_mul": (c_int, [c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_softcap_f32": (c_int, [c_void_p, c_longlong, c_float, c_void_p]),
    "lia_moe_gemm_act": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p]),
    "lia_forget_gate_prep": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lia_forget_scan": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "lia_window_attn_masked": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p]),
    "lia_qkv_prep_heads": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                   c_float, c_float, c_int, c_void_p, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "lia_diff_combine": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p]),
    "lia_latent_prep_pairs": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_longlong, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
}

EXPORTS = tuple(_PROTOTYPES)

_lib = None


def load():
    """Load libliab200.so once; raise (never fall back) if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LiaError(
                f"{LIB_PATH} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `make -C isca-2025-lia_b200/csrc` (there is no CPU/PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(lib, name)     # AttributeError if a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        if lib.lia_abi_version() != ABI_VERSION:
            raise LiaError(f"ABI mismatch: library {lib.lia_abi_version()} vs binding {ABI_VERSION}")
        _lib = lib
    return _lib


def last_error():
    msg = load().lia_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc, what):
    if rc != 0:
        raise LiaError(f"{what} failed (code {rc}): {last_error()}")


launch_count = 0   # kernels launched through this binding (bench.py's gpu_launches)
