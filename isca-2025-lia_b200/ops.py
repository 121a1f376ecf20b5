"""Tensor-level wrappers over the C ABI (include/lia_b200.h).

PyTorch is plumbing here: it owns device memory and streams; every op below is one
call into libliab200.so on ``torch.cuda.current_stream()``.  No op has a PyTorch
fallback -- a missing library or a non-CUDA tensor raises.
"""
import ctypes
import os

import torch

from . import _lib
from ._lib import EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_RESIDUAL, EPI_QKV, LiaQkvArgs, check  # noqa: F401

BF16 = torch.bfloat16


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return t.data_ptr() if t is not None else None


def _req(t, name, dtype=BF16):
    if not (t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise _lib.LiaError(f"{name}: need a contiguous CUDA {dtype} tensor, got {t.dtype} on {t.device} "
                            f"contiguous={t.is_contiguous()}")
    return t


def count_launches(n=1):
    _lib.launch_count += n


def layernorm(x, w, b, eps=1e-5, out=None):
    """F.layer_norm over the last dim (decoder.py:107-119)."""
    _req(x, "x"); _req(w, "w"); _req(b, "b")
    h = x.shape[-1]
    rows = x.numel() // h
    if out is None:
        out = torch.empty_like(x)
    check(_lib.load().lia_layernorm_bf16(_p(x), _p(w), _p(b), _p(_req(out, "out")), rows, h, eps, _stream()),
          "lia_layernorm_bf16")
    count_launches()
    return out


class GemmWorkspace:
    """Split-K workspace, zero-initialised once (the kernel leaves its counters zeroed)."""

    def __init__(self, nbytes, device):
        self.buf = torch.zeros(max(int(nbytes), 16384), dtype=torch.uint8, device=device)

    @staticmethod
    def bytes_for(shapes):
        lib = _lib.load()
        return max([lib.lia_gemm_workspace_bytes(m, n, k) for (m, n, k) in shapes] + [16384])


def gemm(a, w, bias, out=None, epilogue=EPI_BIAS, residual=None, qkv=None, workspace=None):
    """out = epilogue(a @ w.T) -- a [M,K], w [N,K] (decoder.py:79-105, attentions.py:376-418)."""
    _req(a, "a"); _req(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise _lib.LiaError(f"gemm: a is [{M},{K}] but w is {tuple(w.shape)}")
    if bias is not None:
        _req(bias, "bias")
    if residual is not None:
        _req(residual, "residual")
    if epilogue != EPI_QKV and out is None:
        out = torch.empty(M, N, dtype=BF16, device=a.device)
    if epilogue != EPI_QKV:
        _req(out, "out")
        if tuple(out.shape) != (M, N):
            raise _lib.LiaError(f"gemm: out is {tuple(out.shape)}, need ({M}, {N})")
    if residual is not None and tuple(residual.shape) != (M, N):
        raise _lib.LiaError(f"gemm: residual is {tuple(residual.shape)}, need ({M}, {N})")
    ws_ptr, ws_bytes = (None, 0)
    if workspace is not None:
        ws_ptr, ws_bytes = workspace.buf.data_ptr(), workspace.buf.numel()
    check(_lib.load().lia_gemm_bf16(_p(a), _p(w), _p(bias), _p(residual), _p(out), M, N, K, epilogue,
                                    ctypes.byref(qkv) if qkv is not None else None, ws_ptr, ws_bytes, _stream()),
          "lia_gemm_bf16")
    count_launches()
    return out


def gemm_allreduce(a, w, bias, residual, out, tp_args, workspace=None):
    """Row-parallel projection fused with its all-reduce and residual add (world > 1):
    out = residual + sum_over_ranks(a_r @ w_r.T + bias_r)  (decoder.py:60-77 + 247/317).
    ``tp_args`` is a LiaTpArgs from tp.PeerArena.args(); for M > 128 ``out`` must be an arena tensor."""
    _req(a, "a"); _req(w, "w"); _req(residual, "residual"); _req(out, "out")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise _lib.LiaError(f"gemm_allreduce: a is [{M},{K}] but w is {tuple(w.shape)}")
    if tuple(out.shape) != (M, N) or tuple(residual.shape) != (M, N):
        raise _lib.LiaError(f"gemm_allreduce: out {tuple(out.shape)} / residual {tuple(residual.shape)}, need ({M}, {N})")
    if bias is not None:
        _req(bias, "bias")
    ws_ptr, ws_bytes = (None, 0)
    if workspace is not None:
        ws_ptr, ws_bytes = workspace.buf.data_ptr(), workspace.buf.numel()
    check(_lib.load().lia_gemm_allreduce_bf16(_p(a), _p(w), _p(bias), _p(residual), _p(out), M, N, K,
                                              ctypes.byref(tp_args), ws_ptr, ws_bytes, _stream()),
          "lia_gemm_allreduce_bf16")
    count_launches()
    return out


def _check_cache_rows(k_cache, v_cache, rows, what):
    """The time dimension of the cache bounds every append and every read (the reference's slice assignment
    A:473-491 raises there)."""
    if k_cache.dim() != 4 or k_cache.shape != v_cache.shape:
        raise _lib.LiaError(f"{what}: k_cache {tuple(k_cache.shape)} / v_cache {tuple(v_cache.shape)} must be equal [Tmax,B,H,d]")
    if rows > k_cache.shape[0]:
        raise _lib.LiaError(f"{what}: {rows} cached positions exceed the cache's {k_cache.shape[0]} rows")


def qkv_args(q_out, k_cache, v_cache, S, pos0, b0, scale):
    """k_cache/v_cache: [Tmax, Bc, H, d] time-major (attentions.py:471-472)."""
    _req(q_out, "q_out"); _req(k_cache, "k_cache"); _req(v_cache, "v_cache")
    hq = k_cache.shape[2] * k_cache.shape[3]
    _check_cache_rows(k_cache, v_cache, pos0 + S, "qkv_args")
    return LiaQkvArgs(q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), hq, S, pos0, k_cache.shape[1], b0,
                      float(scale))


def kv_append(q, k, v, k_cache, v_cache, pos0, b0, scale, q_out=None):
    """q_out = q*scale; append k/v rows [B,S,H,d] to the time-major cache (attentions.py:456-491)."""
    _req(q, "q"); _req(k, "k"); _req(v, "v"); _req(k_cache, "k_cache"); _req(v_cache, "v_cache")
    B, S = q.shape[0], q.shape[1]
    hq = k_cache.shape[2] * k_cache.shape[3]
    _check_cache_rows(k_cache, v_cache, pos0 + S, "kv_append")
    if q_out is None:
        q_out = torch.empty_like(q)
    check(_lib.load().lia_kv_append_bf16(_p(q), _p(k), _p(v), _p(q_out), _p(k_cache), _p(v_cache), B, S, hq, pos0,
                                         k_cache.shape[1], b0, float(scale), _stream()), "lia_kv_append_bf16")
    count_launches()
    return q_out


def attn_prefill(q, k_cache, v_cache, B, S, b0=0, out=None):
    """Causal attention over rows [0,S) of the cache (attentions.py:444-449, 493-536)."""
    _req(q, "q"); _req(k_cache, "k_cache"); _req(v_cache, "v_cache")
    _, Bc, H, d = k_cache.shape
    _check_cache_rows(k_cache, v_cache, S, "attn_prefill")
    if out is None:
        out = torch.empty(B * S, H * d, dtype=BF16, device=q.device)
    check(_lib.load().lia_attn_prefill_bf16(_p(q), _p(k_cache), _p(v_cache), _p(_req(out, "out")), B, H, S, d, Bc, b0,
                                            _stream()), "lia_attn_prefill_bf16")
    count_launches()
    return out


_SM_COUNT = {}


def _sm_count(device):
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SM_COUNT[key]


def attn_decode_launches(B, H, T, splits, has_workspace, sms):
    """Kernels one lia_attn_decode_bf16 call launches: 1, or 2 when it splits the keys (the split kernel and the combine).
    Bookkeeping for ``gpu_launches`` only -- restates the choice made in csrc/attn_decode.cu (pick_splits and the fallbacks
    after it); the kernel never sees this."""
    fewest = (T + 4095) // 4096
    if splits <= 0:
        per_sm = -splits
        if per_sm == 0:
            env = os.environ.get("LIA_ATTN_CTAS_PER_SM", "")
            per_sm = int(env) if env.isdigit() and int(env) > 0 else 2
        want = (per_sm * sms + B * H - 1) // (B * H)
        splits = max(min(want, max(T // 128, 1), 32), fewest)
    if splits > 1 and not has_workspace:
        splits = fewest
    t_chunk = (T + splits - 1) // splits
    return 2 if (T + t_chunk - 1) // t_chunk > 1 else 1


def attn_decode(q, k_cache, v_cache, B, T, b0=0, out=None, splits=0, workspace=None):
    """One query token per sequence over T cached positions, no mask (attentions.py:395-399, 500)."""
    _req(q, "q"); _req(k_cache, "k_cache"); _req(v_cache, "v_cache")
    _, Bc, H, d = k_cache.shape
    _check_cache_rows(k_cache, v_cache, T, "attn_decode")
    if out is None:
        out = torch.empty(B, H * d, dtype=BF16, device=q.device)
    ws_ptr, ws_bytes = (None, 0)
    if workspace is not None:
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    check(_lib.load().lia_attn_decode_bf16(_p(q), _p(k_cache), _p(v_cache), _p(_req(out, "out")), B, H, T, d, Bc, b0,
                                           splits, ws_ptr, ws_bytes, _stream()), "lia_attn_decode_bf16")
    count_launches(attn_decode_launches(B, H, T, splits, workspace is not None, _sm_count(q.device)))
    return out


def attn_decode_workspace(B, H, d, device, max_splits=32):
    n = _lib.load().lia_attn_decode_workspace_bytes(B, H, d, max_splits)
    return torch.empty(n // 4, dtype=torch.float32, device=device)


def embed(ids, embed_tokens, embed_positions, past_len, out=None, attention_mask=None):
    """Token + learned positional embedding (lia/modeling_opt.py:1107-1142, 368-378).  ``attention_mask``
    (int64 [B, >= past_len + S], may be a column-slice view of a wider buffer) selects the positions the
    reference derives from its cumsum; None means all ones."""
    _req(ids, "ids", torch.int64)
    if embed_tokens is None and embed_positions is None:
        raise _lib.LiaError("embed: at most one of embed_tokens / embed_positions may be None")
    if embed_tokens is not None:
        _req(embed_tokens, "embed_tokens")
    if embed_positions is not None:
        _req(embed_positions, "embed_positions")
    B, S = ids.shape
    V = embed_tokens.shape[0] if embed_tokens is not None else 0
    h = (embed_tokens if embed_tokens is not None else embed_positions).shape[1]
    if embed_tokens is not None and embed_positions is not None and embed_positions.shape[1] != h:
        raise _lib.LiaError(f"embed: token rows are {h} wide but position rows {embed_positions.shape[1]}")
    P = embed_positions.shape[0] if embed_positions is not None else 0
    if out is not None and (out.numel() != B * S * h):
        raise _lib.LiaError(f"embed: out has {out.numel()} elements, need {B * S * h}")
    if out is None:
        out = torch.empty(B, S, h, dtype=BF16, device=ids.device)
    mask_ptr, mask_ld = None, 0
    if attention_mask is not None:
        am = attention_mask
        if not (am.is_cuda and am.dtype == torch.int64 and am.dim() == 2 and am.shape[0] == B and am.stride(1) == 1):
            raise _lib.LiaError(f"attention_mask: need a CUDA int64 [B, T] tensor with unit column stride, got {am.dtype} "
                                f"{tuple(am.shape)} strides {am.stride()} on {am.device}")
        if am.shape[1] < past_len + S:
            raise _lib.LiaError(f"attention_mask has {am.shape[1]} columns, need past_len + S = {past_len + S}")
        mask_ptr, mask_ld = am.data_ptr(), am.stride(0) if B > 1 else max(am.stride(0), am.shape[1])
    check(_lib.load().lia_embed_masked_bf16(_p(ids), mask_ptr, mask_ld, _p(embed_tokens), _p(embed_positions),
                                            _p(_req(out, "out")), B, S, h, past_len, V, P, _stream()),
          "lia_embed_masked_bf16")
    count_launches()
    return out


def argmax(logits, suppress_id=-1, out=None):
    """Greedy pick with one suppressed id (generation_utils.py:872-880, greedy_search.py:395)."""
    _req(logits, "logits")
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
    check(_lib.load().lia_argmax_bf16(_p(logits), _p(_req(out, "out", torch.int64)), B, V, suppress_id, _stream()),
          "lia_argmax_bf16")
    count_launches()
    return out


def residual_add(x, residual, out=None):
    """out = residual + x after a tensor-parallel all-reduce (decoder.py:247, 317)."""
    _req(x, "x"); _req(residual, "residual")
    if out is None:
        out = torch.empty_like(x)
    check(_lib.load().lia_residual_add_bf16(_p(x), _p(residual), _p(_req(out, "out")), x.numel(), _stream()),
          "lia_residual_add_bf16")
    count_launches()
    return out


# ------------------------------------------------------------------------------------------------------------------
# Models with a 32-bit residual stream, matrix-memory (mLSTM) mixers and latent-cache attention.  Activations are bf16
# or fp32 tensors; norm weights, gates, recurrent state and the residual stream are fp32.  (The reference has no such
# models: its one family is OPT.)
# ------------------------------------------------------------------------------------------------------------------
F32 = torch.float32


def _f32(t):
    """1 for an fp32 tensor, 0 for bf16; anything else is refused."""
    if t.dtype == F32:
        return 1
    if t.dtype == BF16:
        return 0
    raise _lib.LiaError(f"need a bf16 or fp32 tensor, got {t.dtype}")


def _dev(t, name, dtype=None):
    if not t.is_cuda or (dtype is not None and t.dtype != dtype):
        raise _lib.LiaError(f"{name}: need a CUDA {dtype or ''} tensor, got {t.dtype} on {t.device}")
    return t


def _rowmajor(t, name):
    """A 2-D view whose rows are contiguous (column slices of a wider buffer are fine): returns its row stride."""
    _dev(t, name)
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise _lib.LiaError(f"{name}: need a 2-D tensor with unit column stride, got {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def embed_rmsnorm(ids, table, w, x, eps):
    """x[r] = w * e / sqrt(mean(e^2) + eps) with e = table[ids[r]]: the token embedding followed by the model's norm."""
    _req(ids, "ids", torch.int64); _req(w, "w", F32); _req(x, "x", F32); _dev(table, "table")
    rows, W = x.shape
    check(_lib.load().lia_embed_rmsnorm(_p(ids), _p(table.contiguous()), _f32(table), _p(w), w.numel(), _p(x), rows, W, table.shape[0],
                                        float(eps), _stream()), "lia_embed_rmsnorm")
    count_launches()
    return x


def rms_add_norm(x, y, w_post, w_pre, h, eps):
    """x += w_post * y / rms(y) (when y is given), then h = w_pre * x / rms(x) (when h is given); x is the fp32 residual
    stream, updated in place."""
    _req(x, "x", F32)
    rows, W = x.shape
    for t, n in ((y, "y"), (h, "h")):
        if t is not None and not (t.is_cuda and t.is_contiguous() and tuple(t.shape) == (rows, W)):
            raise _lib.LiaError(f"rms_add_norm: {n} must be a contiguous CUDA [{rows}, {W}] tensor")
    check(_lib.load().lia_rms_add_norm(_p(x), _p(y), _f32(y) if y is not None else 0, _p(w_post), w_post.numel() if w_post is not None else 0,
                                       _p(w_pre), w_pre.numel() if w_pre is not None else 0, _p(h), _f32(h) if h is not None else 0,
                                       rows, W, float(eps), _stream()), "lia_rms_add_norm")
    count_launches()
    return x


def rms_gather(x, rows, w, h, eps):
    """h[r] = w * x[rows[r]] / rms(x[rows[r]]): the final norm of the rows whose logits are wanted."""
    _req(x, "x", F32); _req(rows, "rows", torch.int32); _req(w, "w", F32)
    n, W = h.shape
    if rows.numel() != n or x.shape[1] != W or not h.is_contiguous():
        raise _lib.LiaError("rms_gather: shapes do not agree")
    check(_lib.load().lia_rms_gather(_p(x), _p(rows), _p(w), w.numel(), _p(h), _f32(h), n, W, float(eps), _stream()), "lia_rms_gather")
    count_launches()
    return h


def clamped_glu(gate_up, up_off, F, out, limit, alpha):
    """out = g * sigmoid(alpha g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    ld = _rowmajor(gate_up, "gate_up")
    M = gate_up.shape[0]
    if tuple(out.shape) != (M, F) or not out.is_contiguous() or out.dtype != gate_up.dtype:
        raise _lib.LiaError("clamped_glu: out must be a contiguous [M, F] tensor of the input's dtype")
    check(_lib.load().lia_clamped_glu(_p(gate_up), ld, up_off, _p(out), _f32(out), M, F, float(limit), float(alpha), _stream()),
          "lia_clamped_glu")
    count_launches()
    return out


GATE_NONE, GATE_LOG_INPUT_FORGET, GATE_SIGMOID = 0, 1, 2


def linear_small(a, w, bias, out, mode=GATE_NONE, cap=1.0):
    """out = act(a @ w.T + bias) for a handful of outputs (per-head gates), fp32 out."""
    lda = _rowmajor(a, "a")
    _dev(w, "w"); _req(out, "out", F32)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or tuple(out.shape) != (M, N):
        raise _lib.LiaError(f"linear_small: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _req(bias, "bias", F32)
    check(_lib.load().lia_linear_small(_p(a), _f32(a), lda, _p(w), _f32(w), _p(bias), _p(out), M, N, K, mode, float(cap), _stream()),
          "lia_linear_small")
    count_launches()
    return out


def linear_plain(a, w, out, scale=1.0, batch=1, a_batch_stride=0, w_batch_stride=0, out_batch_stride=0, n=None, k=None):
    """out[b] = scale * a[b] @ w[b].T on the CUDA cores with fp32 products and sums.  ``a`` / ``out`` are row-major 2-D
    views (row stride free); batches are taken at element strides from their first element; ``n``, ``k`` give the
    per-batch problem when the views are wider than one batch."""
    lda, ldc = _rowmajor(a, "a"), _rowmajor(out, "out")
    _dev(w, "w")
    M = a.shape[0]
    K = k if k is not None else a.shape[1]
    N = n if n is not None else out.shape[1]
    ldw = w.stride(-2) if w.dim() >= 2 else K
    if out.shape[0] != M:
        raise _lib.LiaError("linear_plain: a and out differ in rows")
    check(_lib.load().lia_linear_plain(_p(a), _f32(a), lda, a_batch_stride, _p(w), _f32(w), ldw, w_batch_stride, _p(out), _f32(out), ldc,
                                       out_batch_stride, M, N, K, batch, float(scale), _stream()), "lia_linear_plain")
    count_launches()
    return out


def argmax_f32(logits, suppress_id=-1, out=None):
    """Greedy pick over fp32 logits (lowest index on ties)."""
    _req(logits, "logits", F32)
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
    check(_lib.load().lia_argmax_f32(_p(logits), _p(_req(out, "out", torch.int64)), B, V, suppress_id, _stream()), "lia_argmax_f32")
    count_launches()
    return out


def mlstm_scan(q, k, v, gates, state_S, state_n, state_m, segs, H, dim, vdim, q_scale, den_eps, o):
    """Matrix-memory recurrence over every portion of the step (csrc/mlstm.cu).  q, k, v: column slices of one projection
    output (same row stride); gates [rows, 2H] fp32 (log input, log forget); state tensors indexed by slot."""
    ld = _rowmajor(q, "q")
    if _rowmajor(k, "k") != ld or _rowmajor(v, "v") != ld or k.dtype != q.dtype or v.dtype != q.dtype:
        raise _lib.LiaError("mlstm_scan: q, k, v must be slices of one buffer")
    _req(gates, "gates", F32); _req(state_S, "state_S", F32); _req(state_n, "state_n", F32); _req(state_m, "state_m", F32)
    _req(segs, "segs", torch.int32); _req(o, "o", F32)
    M = q.shape[0]
    if tuple(gates.shape) != (M, 2 * H) or tuple(o.shape) != (M, H * vdim) or tuple(state_S.shape[1:]) != (H, vdim, dim):
        raise _lib.LiaError("mlstm_scan: shapes do not agree")
    check(_lib.load().lia_mlstm_scan(_p(q), _p(k), _p(v), _f32(q), ld, _p(gates), _p(state_S), _p(state_n), _p(state_m), _p(segs),
                                     segs.shape[0], H, dim, vdim, float(q_scale), float(den_eps), _p(o), _stream()), "lia_mlstm_scan")
    count_launches()
    return o


def headnorm_gate(o, w, gate, out, H, vdim, eps, gate_silu=False):
    """out = o / rms_per_head(o) * w * sigmoid(gate) (``gate_silu``: * silu(gate); ``gate`` None: the norm alone)."""
    _req(o, "o", F32); _req(w, "w", F32)
    ldg = _rowmajor(gate, "gate") if gate is not None else 0
    M = o.shape[0]
    if not out.is_contiguous() or tuple(out.shape) != (M, H * vdim) or (gate is not None and out.dtype != gate.dtype):
        raise _lib.LiaError("headnorm_gate: out must be a contiguous [M, H*vdim] tensor of the gate's dtype")
    check(_lib.load().lia_headnorm_gate(_p(o), _p(w), _p(gate), ldg, _p(out), _f32(out), M, H, vdim, float(eps), int(gate_silu), _stream()),
          "lia_headnorm_gate")
    count_launches()
    return out


def latent_prep(q, dkv, c_norm_w, inv_freq, meta, cache, qa, H, dim, rot, rot_dims, kv_rank, eps, pairs=False, rot_mag=1.0):
    """Normalised latent + rotated shared key part into ``cache[slot, pos]``; rotated query parts into ``qa[..., kv_rank:]``.
    ``pairs``: channels (2i, 2i+1) turn together by angles from a float64 frequency table, cos and sin times ``rot_mag``;
    otherwise channel i turns with i + rot_dims/2 by fp32 angles."""
    ldq, ldd = _rowmajor(q, "q"), _rowmajor(dkv, "dkv")
    _req(c_norm_w, "c_norm_w", F32); _req(meta, "meta", torch.int32); _req(qa, "qa", F32)
    _req(inv_freq, "inv_freq", torch.float64 if pairs else F32)
    M = q.shape[0]
    if cache.dtype != q.dtype or dkv.dtype != q.dtype or not cache.is_contiguous() or cache.shape[2] != kv_rank + rot or inv_freq.numel() != rot_dims // 2:
        raise _lib.LiaError("latent_prep: cache must be a contiguous [slots, capacity, kv_rank + rot] tensor of the activations' dtype, rot_dims / 2 frequencies")
    if pairs:
        check(_lib.load().lia_latent_prep_pairs(_p(q), ldq, _p(dkv), ldd, _f32(q), _p(c_norm_w), _p(inv_freq), float(rot_mag), _p(meta), _p(cache),
                                                cache.stride(0), _p(qa), M, H, dim, rot, rot_dims, kv_rank, float(eps), _stream()), "lia_latent_prep_pairs")
    else:
        check(_lib.load().lia_latent_prep(_p(q), ldq, _p(dkv), ldd, _f32(q), _p(c_norm_w), _p(inv_freq), _p(meta), _p(cache), cache.stride(0),
                                          _p(qa), M, H, dim, rot, rot_dims, kv_rank, float(eps), _stream()), "lia_latent_prep")
    count_launches()


LATENT_SPLIT_KEYS, LATENT_MAX_SPLITS = 64, 32


def latent_attn_split_class(max_ctx):
    """All that ``latent_attn_splits`` takes from the history's length: two lengths of one class launch alike."""
    return min(max_ctx // LATENT_SPLIT_KEYS, LATENT_MAX_SPLITS)


def latent_attn_splits(M, H, max_ctx, sms):
    """Key ranges per row: 1 when the rows alone fill the GPU (prompts), more when a few rows face a long history."""
    blocks = M * ((H + 7) // 8)
    want = (2 * sms + blocks - 1) // blocks
    return max(1, min(want, latent_attn_split_class(max_ctx)))


def latent_attn(qa, cache, meta, gate, out, H, kv_rank, rot, scale, max_ctx=0):
    """Causal softmax attention of every row over its sequence's cached latent rows (csrc/latent_attn.cu).  ``max_ctx``: an
    upper bound of the rows' history lengths (0: unknown, no split of the keys)."""
    _req(qa, "qa", F32); _req(meta, "meta", torch.int32); _req(out, "out", F32)
    if gate is not None:
        _req(gate, "gate", F32)
    M = qa.shape[0]
    nsplit = latent_attn_splits(M, H, max_ctx, _sm_count(qa.device))
    ws = None
    if nsplit > 1:
        ws = torch.empty(_lib.load().lia_latent_attn_workspace_floats(M, H, kv_rank, nsplit), dtype=F32, device=qa.device)
    check(_lib.load().lia_latent_attn(_p(qa), _p(cache), _f32(cache), cache.stride(0), _p(meta), _p(gate), _p(out), _p(ws), nsplit, M, H,
                                      kv_rank, rot, float(scale), _stream()), "lia_latent_attn")
    count_launches(2 if nsplit > 1 else 1)
    return out


# ------------------------------------------------------------------------------------------------------------------
# Models whose sublayers sit between layer norms on a 32-bit residual stream: decay / delta-rule recurrences, sliding-window
# attention with grouped key/value heads, dense and mixture-of-experts feed-forwards.  (Not in the reference either.)
# ------------------------------------------------------------------------------------------------------------------
ACT_NONE, ACT_RELU, ACT_SILU, ACT_GELU_ERF, ACT_GELU_TANH, ACT_CLAMPED_SWISH = 0, 1, 2, 3, 4, 5
I32 = torch.int32


def embed_rows(ids, table, x, x_copy=None):
    """x[r] = table[ids[r]] in fp32; ``x_copy`` receives the same rows (the copy a looped block adds back before a repeat)."""
    _req(ids, "ids", torch.int64); _req(x, "x", F32); _dev(table, "table")
    rows, W = x.shape
    if x_copy is not None:
        _req(x_copy, "x_copy", F32)
    check(_lib.load().lia_embed_rows(_p(ids), _p(table), _f32(table), _p(x), _p(x_copy), rows, W, table.shape[0], _stream()), "lia_embed_rows")
    count_launches()
    return x


def ln_add_norm(x, y, post, mult, pre, h, eps, extra=None):
    """x += mult * LN(y; post) when y is given, x += extra when given, then h = LN(x; pre) when h is given.  ``post`` and
    ``pre`` are (weight, bias) pairs of fp32 vectors; x is the fp32 residual stream, updated in place."""
    _req(x, "x", F32)
    rows, W = x.shape
    for t, n in ((y, "y"), (h, "h"), (extra, "extra")):
        if t is not None and not (t.is_cuda and t.is_contiguous() and tuple(t.shape) == (rows, W)):
            raise _lib.LiaError(f"ln_add_norm: {n} must be a contiguous CUDA [{rows}, {W}] tensor")
    for pair, n in ((post, "post"), (pre, "pre")):
        if pair is not None and not all(t.dtype == F32 and t.numel() == W and t.is_cuda for t in pair):
            raise _lib.LiaError(f"ln_add_norm: {n} must be a (weight, bias) pair of fp32 [{W}] vectors")
    if extra is not None:
        _req(extra, "extra", F32)
    wp, bp = post if post is not None else (None, None)
    wn, bn = pre if pre is not None else (None, None)
    check(_lib.load().lia_ln_add_norm(_p(x), _p(y), _f32(y) if y is not None else 0, _p(wp), _p(bp), float(mult), _p(extra), _p(wn), _p(bn),
                                      _p(h), _f32(h) if h is not None else 0, rows, W, float(eps), _stream()), "lia_ln_add_norm")
    count_launches()
    return x


def ln_gather(x, rows, norm, h, eps):
    """h[r] = LN(x[rows[r]]; norm): the final norm of the rows whose logits are wanted."""
    _req(x, "x", F32); _req(rows, "rows", I32)
    n, W = h.shape
    w, b = norm
    if rows.numel() != n or x.shape[1] != W or not h.is_contiguous() or w.numel() != W or b.numel() != W:
        raise _lib.LiaError("ln_gather: shapes do not agree")
    check(_lib.load().lia_ln_gather(_p(x), _p(rows), _p(_req(w, "w", F32)), _p(_req(b, "b", F32)), _p(h), _f32(h), n, W, float(eps), _stream()),
          "lia_ln_gather")
    count_launches()
    return h


def gated_act(inp, F, out, act, up_off=-1):
    """out = act(inp[:, :F]) * inp[:, up_off:up_off + F] (``up_off`` < 0: no second factor)."""
    ld = _rowmajor(inp, "inp")
    M = inp.shape[0]
    if tuple(out.shape) != (M, F) or not out.is_contiguous() or out.dtype != inp.dtype:
        raise _lib.LiaError("gated_act: out must be a contiguous [M, F] tensor of the input's dtype")
    check(_lib.load().lia_gated_act(_p(inp), ld, up_off, _p(out), _f32(out), M, F, act, _stream()), "lia_gated_act")
    count_launches()
    return out


def router_topk(logits, top, idx, wt, correction=None, renorm=True):
    """Softmax over the experts, the ``top`` largest scores and their weights: idx int32 [M, top], wt fp32.  ``correction``
    [E] is added to the scores for the choice only; ``renorm`` divides the chosen scores by their sum."""
    _req(logits, "logits", F32); _req(idx, "idx", I32); _req(wt, "wt", F32)
    M, E = logits.shape
    if tuple(idx.shape) != (M, top) or tuple(wt.shape) != (M, top) or (correction is not None and correction.numel() != E):
        raise _lib.LiaError("router_topk: idx and wt must be [M, top], the correction [E]")
    if correction is not None:
        _req(correction, "correction", F32)
    check(_lib.load().lia_router_topk_ext(_p(logits), _p(correction), int(renorm), _p(idx), _p(wt), M, E, top, _stream()), "lia_router_topk")
    count_launches()


def moe_tiles(pairs, E):
    """Row tiles that always hold ``pairs`` (token, choice) pairs grouped by expert."""
    tm = _lib.load().lia_moe_tile_rows()
    return (pairs + min(E, pairs) * (tm - 1)) // tm, tm


def moe_plan(idx, E, perm, tile_expert, pos_of):
    _req(idx, "idx", I32); _req(perm, "perm", I32); _req(tile_expert, "tile_expert", I32); _req(pos_of, "pos_of", I32)
    check(_lib.load().lia_moe_plan(_p(idx), idx.numel(), E, tile_expert.numel(), _p(perm), _p(tile_expert), _p(pos_of), _stream()), "lia_moe_plan")
    count_launches()


def moe_gemm(a, w, out, idx, wt, top, up, act=ACT_NONE, perm=None, tile_expert=None, gated=False, act_params=(0.0, 0.0)):
    """One projection of every expert over its own rows; ``w`` [E, N, K].  up: out[place] = act(a[token] @ w[e].T);
    down: out[pair] = wt[pair] * a[place] @ w[e].T (fp32).  Without a plan (``perm`` None) a pair's place is the pair.
    ``gated`` (up only): ``w`` is [E, 2N, K], N gate rows then N up rows, and out = act(gate) * up.  Pairs whose expert
    index is E or more (experts without weights) are left out.  ``act_params``: (limit, alpha) of ACT_CLAMPED_SWISH, the gated
    activation g' sigmoid(alpha g') (u' + 1) on g' = min(g, limit), u' = clamp(u, -limit, limit)."""
    _dev(a, "a"); _dev(w, "w"); _dev(out, "out")
    E, N, K = w.shape
    if gated:
        N //= 2
    if not (w.is_contiguous() and a.is_contiguous() and out.is_contiguous() and a.shape[1] == K and out.shape[1] == N):
        raise _lib.LiaError(f"moe_gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    check(_lib.load().lia_moe_gemm_act(_p(a), _f32(a), K, _p(w), _f32(w), w.stride(0), _p(out), _f32(out), N, _p(perm), _p(tile_expert),
                                       tile_expert.numel() if tile_expert is not None else 0, _p(idx), _p(wt), idx.numel(), top, N, K, int(up), act,
                                       int(gated), E, float(act_params[0]), float(act_params[1]), _stream()), "lia_moe_gemm")
    count_launches()
    return out


def moe_gather(src, perm, dst, top):
    """dst[place] = src[perm[place] // top], zeros in the plan's padding."""
    _req(perm, "perm", I32)
    if not (src.is_contiguous() and dst.is_contiguous() and src.dtype == dst.dtype and dst.shape[0] == perm.numel() and dst.shape[1] == src.shape[1]):
        raise _lib.LiaError("moe_gather: dst must be a contiguous [places, W] tensor of the source's dtype")
    check(_lib.load().lia_moe_gather(_p(src), _f32(src), _p(perm), _p(dst), perm.numel(), src.shape[1], top, _stream()), "lia_moe_gather")
    count_launches()
    return dst


def moe_expert_gemms(a, w, out, tiles_per_expert, tile_rows, workspace):
    """out[rows of e] = a[rows of e] @ w[e].T on the tensor-core GEMM, expert after expert: expert e owns the next
    ``tiles_per_expert[e] * tile_rows`` rows of ``a`` and ``out`` (bf16; ``tiles_per_expert`` is a host list)."""
    _req(a, "a"); _req(w, "w"); _req(out, "out")
    E, N, K = w.shape
    rows = sum(tiles_per_expert) * tile_rows
    if len(tiles_per_expert) != E or a.shape[1] != K or out.shape[1] != N or a.shape[0] < rows or out.shape[0] < rows:
        raise _lib.LiaError(f"moe_expert_gemms: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, {rows} rows planned")
    counts = (ctypes.c_int * E)(*tiles_per_expert)
    check(_lib.load().lia_moe_expert_gemms(_p(a), _p(w), N * K, _p(out), counts, E, tile_rows, N, K, workspace.buf.data_ptr(), workspace.buf.numel(),
                                           _stream()), "lia_moe_expert_gemms")
    count_launches(sum(1 for n in tiles_per_expert if n))
    return out


def moe_combine(ypair, shared, y, top, pos_of=None, wt=None, identity=None):
    """y[m] = sum over the token's choices (+ the shared expert's output).  Without a plan ``ypair`` holds the weighted
    outputs pair by pair; with ``pos_of`` and ``wt`` it holds the unweighted outputs in the plan's order.  ``identity`` =
    (idx, first identity expert, h, wt): a pair routed to an expert from that index on contributes wt * h[m]."""
    _dev(ypair, "ypair"); _req(y, "y", F32)
    M, W = y.shape
    if shared is not None and not (shared.is_contiguous() and tuple(shared.shape) == (M, W)):
        raise _lib.LiaError("moe_combine: the shared expert's output must be a contiguous [M, W] tensor")
    if not ypair.is_contiguous() or ypair.shape[1] != W or (pos_of is None) != (wt is None):
        raise _lib.LiaError("moe_combine: ypair must be a contiguous [.., W] tensor; pos_of and wt go together")
    idx, n_real, h = None, 0, None
    if identity is not None:
        idx, n_real, h, wt_id = identity
        _req(idx, "idx", I32); _req(wt_id, "wt", F32)
        if not (h.is_contiguous() and tuple(h.shape) == (M, W)) or (shared is not None and shared.dtype != h.dtype):
            raise _lib.LiaError("moe_combine: the experts' input must be a contiguous [M, W] tensor of the shared expert's type")
        wt = wt_id
    act = h if h is not None else shared
    check(_lib.load().lia_moe_combine_ext(_p(ypair), _f32(ypair), _p(pos_of), _p(wt), _p(shared), _f32(act) if act is not None else 1, _p(idx),
                                          n_real, _p(h), _p(y), M, W, top, _stream()), "lia_moe_combine")
    count_launches()
    return y


def conv_prep(y, offs, wconv, conv_state, meta, gates, a_log, dt_bias, qk, v, G, H, dim, vdim, taps, q_scale, unit_eps=1e-6):
    """Short convolution + SiLU of the q | k | v columns of ``y`` (column offsets ``offs``), unit q and k per head, and the
    gates beta | g in place of the raw gate projections in ``gates`` [M, 2H]."""
    ld = _rowmajor(y, "y")
    for t, n in ((wconv, "wconv"), (conv_state, "conv_state"), (gates, "gates"), (a_log, "a_log"), (dt_bias, "dt_bias"), (qk, "qk"), (v, "v")):
        _req(t, n, F32)
    _req(meta, "meta", I32)
    M, C = y.shape[0], 2 * G * dim + H * vdim
    if tuple(wconv.shape) != (C, taps) or tuple(conv_state.shape[1:]) != (max(taps - 1, 1), C) or tuple(gates.shape) != (M, 2 * H) \
            or tuple(qk.shape) != (M, 2 * G * dim) or tuple(v.shape) != (M, H * vdim):
        raise _lib.LiaError("conv_prep: shapes do not agree")
    check(_lib.load().lia_conv_prep(_p(y), _f32(y), ld, offs[0], offs[1], offs[2], _p(wconv), _p(conv_state), _p(meta), _p(gates), _p(a_log),
                                    _p(dt_bias), _p(qk), _p(v), M, G, H, dim, vdim, taps, float(q_scale), float(unit_eps), _stream()), "lia_conv_prep")
    count_launches()


def conv_state_update(y, offs, nqk, nv, conv_state, segs, taps, nk=None):
    """The last ``taps`` - 1 inputs of every portion become its sequence's convolution state (after ``conv_prep`` or
    ``qkv_prep``).  ``nqk`` channels of q and ``nk`` of k (None: as many), ``nv`` of v."""
    ld = _rowmajor(y, "y")
    _req(conv_state, "conv_state", F32); _req(segs, "segs", I32)
    if taps > 1:
        check(_lib.load().lia_conv_state_update(_p(y), _f32(y), ld, offs[0], offs[1], offs[2], nqk, nqk if nk is None else nk, nv, _p(conv_state), _p(segs), segs.shape[0],
                                                taps, _stream()), "lia_conv_state_update")
        count_launches()


def linear_scan(q, k, v, state_S, segs, H, G, dim, vdim, o, decay=None, gates=None, in_silu=False):
    """Matrix-state recurrence over every portion of the step (csrc/linear_scan.cu): with ``decay`` [H] the fixed-decay form,
    with ``gates`` [rows, 2H] = beta | g the gated delta rule.  q, k: column slices with one row stride, G heads."""
    ld = _rowmajor(q, "q")
    if _rowmajor(k, "k") != ld or k.dtype != q.dtype or v.dtype != q.dtype:
        raise _lib.LiaError("linear_scan: q and k must be slices of one buffer, v of the same type")
    ldv = _rowmajor(v, "v")
    _req(state_S, "state_S", F32); _req(segs, "segs", I32); _req(o, "o", F32)
    if (decay is None) == (gates is None):
        raise _lib.LiaError("linear_scan: give either decay or gates")
    M = q.shape[0]
    if tuple(o.shape) != (M, H * vdim) or tuple(state_S.shape[1:]) != (H, vdim, dim) or (gates is not None and tuple(gates.shape) != (M, 2 * H)) \
            or (decay is not None and decay.numel() != H):
        raise _lib.LiaError("linear_scan: shapes do not agree")
    check(_lib.load().lia_linear_scan(_p(q), _p(k), ld, _p(v), ldv, _f32(q), int(in_silu), _p(_req(decay, "decay", F32) if decay is not None else None),
                                      _p(_req(gates, "gates", F32) if gates is not None else None), _p(state_S), _p(segs), segs.shape[0], H, G, dim,
                                      vdim, _p(o), _stream()), "lia_linear_scan")
    count_launches()
    return o


def kv_store(k, v, meta, kcache, vcache, G, dim, vdim, eps, norm_values=True):
    """Keys as they are, values divided by their per-head root mean square, into the caches at every row's (slot, position)."""
    ldk, ldv = _rowmajor(k, "k"), _rowmajor(v, "v")
    _req(meta, "meta", I32)
    if not (kcache.dtype == vcache.dtype == k.dtype == v.dtype and kcache.is_contiguous() and vcache.is_contiguous()
            and kcache.shape[2] == G * dim and vcache.shape[2] == G * vdim):
        raise _lib.LiaError("kv_store: caches must be contiguous [slots, capacity, G * dim | G * vdim] tensors of the activations' dtype")
    check(_lib.load().lia_kv_store(_p(k), ldk, _p(v), ldv, _f32(k), _p(meta), _p(kcache), kcache.stride(0), _p(vcache), vcache.stride(0), k.shape[0],
                                   G, dim, vdim, float(eps), int(norm_values), _stream()), "lia_kv_store")
    count_launches()


WINDOW_SPLIT_KEYS, WINDOW_MAX_SPLITS = 64, 32


def window_attn_split_class(max_ctx, window):
    """All that ``window_attn_plan`` takes from the history's length: two lengths of one class launch alike."""
    return min(min(max_ctx, window) // WINDOW_SPLIT_KEYS, WINDOW_MAX_SPLITS)


def window_attn_plan(M, nseg, H, G, dim, vdim, window, max_ctx, sms):
    """(query heads per block, rows per block, key ranges per row).  Heads: whole groups of H/G query heads while they fit 8
    warps and 96 KB of staged keys and values, else a divisor of one group.  Rows: a step of prompts lets the rows of a block
    share the staged keys; a step of single tokens takes one row per block and, when the rows alone do not fill the GPU,
    splits each row's window over several blocks."""
    lib = _lib.load()
    rep = H // G
    if rep >= 8:
        hb = max(d for d in range(1, 9) if rep % d == 0)
    else:
        ng = min(8 // rep, G)
        while ng > 1 and lib.lia_window_attn_smem_bytes(ng * rep, ng, max(1, 32 // (ng * rep)), dim, vdim) > 96 * 1024:
            ng -= 1
        hb = ng * rep
    qr = 1 if M < 2 * nseg else max(1, 8 * lib.lia_window_attn_pairs_per_warp(vdim) // hb)
    blocks = (M + qr - 1) // qr * ((H + hb - 1) // hb)
    want = max(1, 2 * sms // blocks)          # two blocks fit an SM: as many key ranges as keep all blocks in ONE wave
    nsplit = max(1, min(want, window_attn_split_class(max_ctx, window))) if qr == 1 and max_ctx > 0 else 1
    return hb, qr, nsplit


def window_attn(q, kcache, vcache, meta, temp, out, H, G, dim, vdim, window, scale, softcap, nseg=None, max_ctx=0, slopes=None, sink=None,
                gate=None, gate_per_head=False, chunk=0, v_div=1):
    """Softmax attention of every row over the last ``window`` cached positions of its sequence (csrc/window_attn.cu);
    ``window`` <= 0: over its whole history.  ``nseg``: portions in the step (None: one row each); ``max_ctx``: an upper
    bound of the rows' history lengths (0: unknown, no split of the keys).  ``temp`` [H] multiplies the scores, ``slopes``
    [H] take slope * distance off them, ``sink`` [H] joins the denominator; ``gate`` multiplies the output: fp32 [M, H]
    as it is (``gate_per_head``), else sigmoid of a pre-activation per channel (a column slice of the activations' type).
    ``q`` may be fp32 while the caches are bf16, and so may ``out``.  ``chunk`` > 0: a position sees only the keys of its own
    block of ``chunk`` positions (blocks counted from the sequence's start).  ``v_div``: key head g reads value head g // v_div
    (the value cache holds G // v_div heads: several attention maps over one set of values)."""
    ldq = _rowmajor(q, "q")
    _req(meta, "meta", I32)
    for t, n in ((temp, "temp"), (slopes, "slopes"), (sink, "sink")):
        if t is not None and (_req(t, n, F32).numel() != H):
            raise _lib.LiaError(f"window_attn: {n} must be [H]")
    M = q.shape[0]
    if not (out.is_contiguous() and tuple(out.shape) == (M, H * vdim) and kcache.dtype == vcache.dtype and out.dtype in (F32, kcache.dtype)
            and q.dtype in (F32, kcache.dtype)):
        raise _lib.LiaError("window_attn: out must be a contiguous [M, H * vdim] tensor, out and q of the caches' dtype or fp32")
    if v_div < 1 or G % v_div or chunk < 0:
        raise _lib.LiaError(f"window_attn: {G} key heads do not share value heads in groups of {v_div} (chunk {chunk})")
    gate_mode, ldg = 0, 0
    if gate is not None:
        ldg = _rowmajor(gate, "gate")
        if gate_per_head:
            gate_mode = 1
            if gate.dtype != F32 or tuple(gate.shape) != (M, H) or ldg != H:
                raise _lib.LiaError("window_attn: a per-head gate must be a contiguous fp32 [M, H] tensor")
        else:
            gate_mode = 2
            if gate.dtype != kcache.dtype or tuple(gate.shape) != (M, H * vdim):
                raise _lib.LiaError("window_attn: a per-channel gate must be an [M, H * vdim] slice of the activations' dtype")
    window = int(window) if window > 0 else 1 << 30
    span = min(window, int(chunk)) if chunk > 0 else window               # the most keys a row can see
    hb, qr, nsplit = window_attn_plan(M, nseg if nseg is not None else M, H, G, dim, vdim, span, max_ctx, _sm_count(q.device))
    ws = None
    if nsplit > 1:
        ws = torch.empty(_lib.load().lia_window_attn_workspace_floats(M, H, vdim, nsplit), dtype=F32, device=q.device)
    check(_lib.load().lia_window_attn_masked(_p(q), ldq, _f32(q), _f32(kcache), _p(kcache), kcache.stride(0), _p(vcache), vcache.stride(0), _p(meta),
                                             _p(temp), _p(slopes), _p(sink), _p(gate), gate_mode, ldg, _p(out), _f32(out), _p(ws), M, H, G, int(v_div),
                                             dim, vdim, window, int(chunk), float(scale), float(softcap), hb, qr, nsplit, _stream()), "lia_window_attn")
    count_launches(2 if nsplit > 1 else 1)
    return out


# ------------------------------------------------------------------------------------------------------------------
# Models that norm and gate a sublayer's OUTPUT and hand on a weighted mix of all earlier layers' results; attention inputs
# behind a bias, a short convolution, a norm, a temperature, a rotation and a blend of values.  (Not in the reference either.)
# ------------------------------------------------------------------------------------------------------------------
NORM_NONE, NORM_WHOLE, NORM_PER_HEAD = 0, 1, 2
VMIX_NONE, VMIX_PUBLISH, VMIX_BLEND = 0, 1, 2


def qkv_prep(y, offs, meta, q_out, kcache, vcache, H, G, dim, vdim, eps, bias=None, wconv=None, conv_state=None, taps=1, norm_mode=NORM_NONE,
             qnorm_w=None, knorm_w=None, temp_coef=0.0, temp_every=0, freq=None, rot_dims=0, rot_halves=False, rot_mag=1.0, vmix_mode=VMIX_NONE,
             vmix=0.0, v_first=None, v_heads=None):
    """The q | k | v columns of ``y`` (column offsets ``offs``) become attention inputs (csrc/window_attn.cu, qkv_prep): bias,
    short causal convolution, RMS norm of q and k, query temperature, rotation of channel pairs, value blend; q into ``q_out``
    (fp32), k and v into the caches at every row's (slot, position).  ``v_heads``: value heads if they are not as many as
    the G key heads."""
    ld = _rowmajor(y, "y")
    _req(meta, "meta", I32); _req(q_out, "q_out", F32)
    Gv = G if v_heads is None else int(v_heads)
    M, C = y.shape[0], (H + G) * dim + Gv * vdim
    for t, n, shape in ((bias, "bias", (C,)), (wconv, "wconv", (C, taps)), (v_first, "v_first", (M, Gv * vdim))):
        if t is not None and tuple(_req(t, n, F32).shape) != shape:
            raise _lib.LiaError(f"qkv_prep: {n} must be fp32 {shape}, got {tuple(t.shape)}")
    if taps > 1 and (conv_state is None or tuple(_req(conv_state, "conv_state", F32).shape[1:]) != (taps - 1, C)):
        raise _lib.LiaError("qkv_prep: the convolution's state must be fp32 [slots, taps - 1, channels]")
    nw = {NORM_NONE: (0, 0), NORM_WHOLE: (H * dim, G * dim), NORM_PER_HEAD: (dim, dim)}[norm_mode]
    if norm_mode != NORM_NONE and (_req(qnorm_w, "qnorm_w", F32).numel(), _req(knorm_w, "knorm_w", F32).numel()) != nw:
        raise _lib.LiaError(f"qkv_prep: norm weights must have {nw} numbers")
    if rot_dims and (freq is None or freq.dtype != torch.float64 or not freq.is_cuda or freq.numel() != rot_dims // 2):
        raise _lib.LiaError("qkv_prep: the rotation needs rot_dims / 2 frequencies as a CUDA float64 tensor")
    if not (kcache.dtype == vcache.dtype == y.dtype and kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[2] == G * dim
            and vcache.shape[2] == Gv * vdim and tuple(q_out.shape) == (M, H * dim)):
        raise _lib.LiaError("qkv_prep: caches must be contiguous [slots, capacity, G * dim | G * vdim] tensors of the activations' dtype, q_out [M, H * dim]")
    check(_lib.load().lia_qkv_prep_heads(_p(y), _f32(y), ld, offs[0], offs[1], offs[2], _p(bias), _p(wconv), _p(conv_state) if taps > 1 else None, int(taps) if wconv is not None else 1,
                                   norm_mode, _p(qnorm_w), _p(knorm_w), float(eps), float(temp_coef), int(temp_every), _p(freq), int(rot_dims),
                                   int(rot_halves), float(rot_mag), vmix_mode, float(vmix), _p(v_first), _p(meta), _p(q_out), _p(kcache),
                                   kcache.stride(0), _p(vcache), vcache.stride(0), M, H, G, Gv, dim, vdim, _stream()), "lia_qkv_prep")
    count_launches()


def gated_rms_add(x, y, w, h, eps, gate=None, gate_bias=None, stack=None, n_mix=0, mix=None):
    """x += w * g / rms(g) with g = y * sigmoid(gate + gate_bias) (``gate``: a column slice of the activations' dtype; None: g = y;
    ``y`` None: nothing is added).  With ``stack`` [n, rows, W] fp32: stack[n_mix - 1] = x and x = sum_j mix[j] * stack[j], j < n_mix.
    ``h`` (may be None) receives x in the activations' dtype.  x is the fp32 residual stream, updated in place."""
    _req(x, "x", F32)
    rows, W = x.shape
    for t, n in ((y, "y"), (h, "h")):
        if t is not None and not (t.is_cuda and t.is_contiguous() and tuple(t.shape) == (rows, W)):
            raise _lib.LiaError(f"gated_rms_add: {n} must be a contiguous CUDA [{rows}, {W}] tensor")
    ldr = 0
    if gate is not None:
        ldr = _rowmajor(gate, "gate")
        if h is None or gate.dtype != h.dtype or tuple(gate.shape) != (rows, W):
            raise _lib.LiaError("gated_rms_add: the gate must be a [rows, W] slice of h's dtype")
    for t, n in ((w, "w"), (gate_bias, "gate_bias")):
        if t is not None and _req(t, n, F32).numel() != W:
            raise _lib.LiaError(f"gated_rms_add: {n} must be fp32 [{W}]")
    if stack is not None:
        _req(stack, "stack", F32); _req(mix, "mix", F32)
        if tuple(stack.shape[1:]) != (rows, W) or not 1 <= n_mix <= stack.shape[0] or mix.numel() < n_mix:
            raise _lib.LiaError("gated_rms_add: stack must be [n, rows, W] with n >= n_mix, mix at least n_mix numbers")
    act = h if h is not None else gate
    check(_lib.load().lia_gated_rms_add(_p(x), _p(y), _f32(y) if y is not None else 0, _p(gate), ldr, _p(gate_bias), _p(w), _p(stack),
                                        stack.stride(0) if stack is not None else 0, int(n_mix), _p(mix), _p(h), _f32(act) if act is not None else 1,
                                        rows, W, float(eps), _stream()), "lia_gated_rms_add")
    count_launches()
    return x


def poly_norm(inp, F, coef, out, eps):
    """out = k1 R(z) + k2 R(z*z) + k3 R(z*z*z) + k0 over z = inp[:, :F], R = division by the row's root mean square; coef = (k1, k2, k3, k0) fp32."""
    ld = _rowmajor(inp, "inp")
    M = inp.shape[0]
    if tuple(out.shape) != (M, F) or not out.is_contiguous() or out.dtype != inp.dtype or _req(coef, "coef", F32).numel() != 4:
        raise _lib.LiaError("poly_norm: out must be a contiguous [M, F] tensor of the input's dtype, coef fp32 [4]")
    check(_lib.load().lia_poly_norm(_p(inp), ld, _p(coef), _p(out), _f32(out), M, F, float(eps), _stream()), "lia_poly_norm")
    count_launches()
    return out


# ------------------------------------------------------------------------------------------------------------------
# Pre-norm designs with learned positions and per-channel norm weights: latent queries, several attention maps over shared
# values, the forget-gate recurrence.  (Not in the reference either.)
# ------------------------------------------------------------------------------------------------------------------
def embed_scale_pos(ids, table, pos_table, scale, meta, x, cat=None):
    """x[r] = table[ids[r]] * scale + pos_table[position of row r] in fp32 (``pos_table`` may be None).  ``cat`` [rows, 2 W]
    (activations' dtype) receives the row twice, side by side."""
    _req(ids, "ids", torch.int64); _req(x, "x", F32); _req(meta, "meta", I32); _dev(table, "table")
    rows, W = x.shape
    if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.shape[1] != W or not pos_table.is_contiguous()):
        raise _lib.LiaError("embed_scale_pos: the position table must be a contiguous [positions, W] tensor of the token table's dtype")
    if cat is not None and not (cat.is_cuda and cat.is_contiguous() and tuple(cat.shape) == (rows, 2 * W)):
        raise _lib.LiaError("embed_scale_pos: cat must be a contiguous [rows, 2 W] tensor")
    check(_lib.load().lia_embed_scale_pos(_p(ids), _p(table), _p(pos_table), _f32(table), float(scale), _p(meta), _p(x), _p(cat),
                                          _f32(cat) if cat is not None else 0, rows, W, table.shape[0],
                                          pos_table.shape[0] if pos_table is not None else 0, _stream()), "lia_embed_scale_pos")
    count_launches()
    return x


def residual_norm(x, y, w, h, eps, replace=False, bias=None):
    """x = (0 if ``replace`` else x) + y + bias, then h = w * x / rms(x) (``w`` None: h = x in its dtype).  x is the fp32 residual
    stream, updated in place; ``y`` [rows, W], ``bias`` fp32 [W] and ``h`` (a row-major view: it may be the left half of a wider
    buffer) may each be None."""
    _req(x, "x", F32)
    rows, W = x.shape
    if y is not None and not (y.is_cuda and y.is_contiguous() and tuple(y.shape) == (rows, W)):
        raise _lib.LiaError(f"residual_norm: y must be a contiguous CUDA [{rows}, {W}] tensor")
    ldh = 0
    if h is not None:
        ldh = _rowmajor(h, "h")
        if tuple(h.shape) != (rows, W):
            raise _lib.LiaError(f"residual_norm: h must be [{rows}, {W}]")
    for t, n in ((bias, "bias"), (w, "w")):
        if t is not None and _req(t, n, F32).numel() != W:
            raise _lib.LiaError(f"residual_norm: {n} must be fp32 [{W}]")
    check(_lib.load().lia_residual_norm(_p(x), _p(y), _f32(y) if y is not None else 0, int(replace), _p(bias), _p(w), _p(h),
                                        _f32(h) if h is not None else 0, ldh, rows, W, float(eps), _stream()), "lia_residual_norm")
    count_launches()
    return x


def rms_norm_rows(inp, w, out, eps):
    """out = w * z / rms(z) over the rows z of ``inp`` (a column slice is fine); out contiguous."""
    ld = _rowmajor(inp, "inp")
    M, N = inp.shape
    if not (out.is_cuda and out.is_contiguous() and tuple(out.shape) == (M, N)) or _req(w, "w", F32).numel() != N:
        raise _lib.LiaError("rms_norm_rows: out must be a contiguous [M, N] tensor, w fp32 [N]")
    check(_lib.load().lia_rms_norm_rows(_p(inp), _f32(inp), ld, _p(w), _p(out), _f32(out), M, N, float(eps), _stream()), "lia_rms_norm_rows")
    count_launches()
    return out


def sigmoid_mul(a, gate, out):
    """out = a * sigmoid(gate), element by element; ``a`` fp32 or the activations' dtype, ``gate`` and ``out`` the activations' dtype."""
    lda, ldg = _rowmajor(a, "a"), _rowmajor(gate, "gate")
    M, F = a.shape
    if tuple(gate.shape) != (M, F) or not (out.is_cuda and out.is_contiguous() and tuple(out.shape) == (M, F) and out.dtype == gate.dtype):
        raise _lib.LiaError("sigmoid_mul: gate [M, F], out a contiguous [M, F] tensor of the gate's dtype")
    check(_lib.load().lia_sigmoid_mul(_p(a), _f32(a), lda, _p(gate), _f32(gate), ldg, _p(out), _f32(out), M, F, _stream()), "lia_sigmoid_mul")
    count_launches()
    return out


def softcap(x, cap):
    """x = cap * tanh(x / cap) in place (fp32)."""
    _req(x, "x", F32)
    check(_lib.load().lia_softcap_f32(_p(x), x.numel(), float(cap), _stream()), "lia_softcap_f32")
    count_launches()
    return x


def forget_gate_prep(y, offs, f_bias, low, out, nq, nv):
    """The q | f | v columns of ``y`` (column offsets ``offs``) -> out [M, 2 nq + nv] fp32 = silu(q) | low + (1 - low) sigmoid(f + f_bias) | v."""
    ld = _rowmajor(y, "y")
    M = y.shape[0]
    _req(out, "out", F32)
    if tuple(out.shape) != (M, 2 * nq + nv) or _req(low, "low", F32).numel() != nq or (f_bias is not None and _req(f_bias, "f_bias", F32).numel() != nq):
        raise _lib.LiaError("forget_gate_prep: out must be [M, 2 nq + nv], low and f_bias fp32 [nq]")
    check(_lib.load().lia_forget_gate_prep(_p(y), _f32(y), ld, offs[0], offs[1], offs[2], _p(f_bias), _p(low), _p(out), M, nq, nv, _stream()),
          "lia_forget_gate_prep")
    count_launches()
    return out


def forget_scan(q, f, v, state_S, segs, H, dim, vdim, o):
    """Per head and channel d: S[d] <- f[d] S[d] + (1 - f[d]) v, then o = sum_d q[d] S[d], over every portion of the step (csrc/linear_scan.cu); q, f: fp32 column
    slices of one buffer, v fp32; state_S [slots, H, vdim, dim]."""
    ld = _rowmajor(q, "q")
    if _rowmajor(f, "f") != ld or not (q.dtype == f.dtype == v.dtype == F32):
        raise _lib.LiaError("forget_scan: q and f must be fp32 slices of one buffer, v fp32")
    ldv = _rowmajor(v, "v")
    _req(state_S, "state_S", F32); _req(segs, "segs", I32); _req(o, "o", F32)
    M = q.shape[0]
    if tuple(o.shape) != (M, H * vdim) or tuple(state_S.shape[1:]) != (H, vdim, dim) or q.shape[1] != H * dim or v.shape[1] != H * vdim:
        raise _lib.LiaError("forget_scan: shapes do not agree")
    check(_lib.load().lia_forget_scan(_p(q), _p(f), ld, _p(v), ldv, _p(state_S), _p(segs), segs.shape[0], H, dim, vdim, _p(o), _stream()),
          "lia_forget_scan")
    count_launches()
    return o


def diff_combine(a, out, H, G, vdim, lam, mult, eps):
    """a [M, G, 2, H // G, vdim] fp32 (two attention maps per query head, grouped by key/value head) -> out [M, H * vdim]:
    o = a1 - lam * a2, out = mult * o / rms(o) per head."""
    _req(a, "a", F32)
    M = a.shape[0]
    if a.numel() != M * 2 * H * vdim or not (out.is_cuda and out.is_contiguous() and tuple(out.shape) == (M, H * vdim)):
        raise _lib.LiaError("diff_combine: a must hold [M, 2 H vdim] numbers, out a contiguous [M, H * vdim] tensor")
    check(_lib.load().lia_diff_combine(_p(a), _p(out), _f32(out), M, H, G, vdim, float(lam), float(mult), float(eps), _stream()), "lia_diff_combine")
    count_launches()
    return out
