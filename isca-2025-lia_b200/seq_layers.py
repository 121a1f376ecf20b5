"""Sequence mixers and feed-forwards that run on a 32-bit residual stream, each with its constants as parameters so that
any model design can assemble them: a matrix-memory recurrent mixer (mLSTM), attention over a latent key/value cache with
a partly rotated query/key and an output gate (queries direct or through a latent of their own), linear attention with a fixed
decay per head, linear attention with a forget gate per channel, the gated delta rule behind a short convolution, differential
attention (two softmax maps over shared values, subtracted) under a chunked or sliding mask, sliding-window attention with grouped key/value heads, attention over the whole history with a sink in the
softmax (behind an optional bias, convolution, norm, temperature and rotation of its inputs, with a distance bias, a blend of
values across layers and an output gate), and the feed-forwards -- clamped gated, plain gated with any activation, one with a
polynomial activation between norms, and a routed mixture of experts (plain or gated experts, a shared expert, experts that
hand the token back).  Each object owns its (fused) weights,
registers its per-sequence state with a ``seq_state.SlotState`` and runs one step over a batch of portions
(``StepBatch``) through the kernels of ``ops``.

Projections go through ``Linear``: the tensor-core GEMM of the OPT path (csrc/gemm_sm100.cu) for bf16 activations, the
plain CUDA-core kernel for fp32 activations and for shapes the tensor-core kernel does not take.
"""
import os

import torch

from . import ops

BF16, F32 = torch.bfloat16, torch.float32


def _pad8(n):
    return (n + 7) // 8 * 8


class StepBatch:
    """The token rows of one step: ``segs`` int32 [n, 4] = (slot, first position, first row, rows) per portion and
    ``meta`` int32 [rows, 2] = (slot, position) per row, both on the device."""

    def __init__(self, rows, segs, meta, max_ctx=0):
        self.rows, self.segs, self.meta = rows, segs, meta
        self.max_ctx = max_ctx              # longest history (tokens cached after this step) among the step's sequences
        self.scratch = {}                   # what one layer of this step leaves for later layers (per-token tensors)


class Linear:
    """y = x @ W.T for one or several weight matrices stacked by rows (one launch, outputs side by side; each block's
    first column is a multiple of 8 so that every slice stays 16-byte aligned in bf16)."""

    _gemm_ws = {}

    def __init__(self, weights, dtype, device):
        ws = [w.to(device=device, dtype=dtype) for w in weights]
        self.K = ws[0].shape[1]
        self.offsets, n = [], 0
        for w in ws:
            self.offsets.append(_pad8(n))
            n = self.offsets[-1] + w.shape[0]
        self.sizes = [w.shape[0] for w in ws]
        self.N = n
        self.weight = torch.zeros(n, self.K, dtype=dtype, device=device)
        for o, w in zip(self.offsets, ws):
            self.weight[o:o + w.shape[0]] = w
        self.dtype = dtype
        self.tensor_core = (dtype == BF16 and self.K % 8 == 0 and self.N % 8 == 0 and os.environ.get("LIA_PLAIN_LINEAR", "0") == "0")

    def _workspace(self, M, device):
        key = (device, M <= 128)
        need = ops.GemmWorkspace.bytes_for([(M, self.N, self.K)])
        ws = Linear._gemm_ws.get(key)
        if ws is None or ws.buf.numel() < need:
            ws = Linear._gemm_ws[key] = ops.GemmWorkspace(need, device)
        return ws

    def __call__(self, x, out=None):
        M = x.shape[0]
        if out is None:
            out = torch.empty(M, self.N, dtype=self.dtype, device=x.device)
        if self.tensor_core and x.is_contiguous() and x.data_ptr() % 16 == 0:
            ops.gemm(x, self.weight, None, out=out, workspace=self._workspace(M, x.device))
        else:
            ops.linear_plain(x, self.weight, out)
        return out

    def part(self, y, i):
        return y[:, self.offsets[i]:self.offsets[i] + self.sizes[i]]


class MLSTMMixer:
    """Matrix-memory recurrent mixer.  q = Wq h * dim^-1/2, k = Wk h, v = Wv h; per head a log input gate
    cap*tanh((Wi h + bi)/cap) and a log forget gate logsigmoid(cap*tanh((Wf h + bf)/cap)); the stabilised recurrence of
    csrc/mlstm.cu; each head's output RMS-normed, times a per-channel weight, times sigmoid(Wg h), then Wo."""

    def __init__(self, w, heads, dim, vdim, gate_cap, norm_eps, dtype, device, den_eps=1e-6):
        self.H, self.dim, self.vdim, self.cap, self.eps, self.den_eps = heads, dim, vdim, float(gate_cap), float(norm_eps), den_eps
        self.dtype = dtype
        self.proj = Linear([w["q"], w["k"], w["v"], w["g"]], dtype, device)
        self.w_gates = torch.cat([w["i"], w["f"]], 0).to(device=device, dtype=dtype).contiguous()
        self.b_gates = torch.cat([w["i.b"], w["f.b"]], 0).to(device=device, dtype=F32).contiguous()
        self.norm_w = w["norm"].to(device=device, dtype=F32).contiguous()
        self.out = Linear([w["o"]], dtype, device)
        self.q_scale = float(dim) ** -0.5

    def new_state(self, slots):
        return (slots.add_recurrent((self.H, self.vdim, self.dim)), slots.add_recurrent((self.H, self.dim)),
                slots.add_recurrent((self.H,)))

    def __call__(self, h, batch, state):
        S, n, m = state
        M, H = h.shape[0], self.H
        y = self.proj(h)
        q, k, v, g = (self.proj.part(y, i) for i in range(4))
        gates = torch.empty(M, 2 * H, dtype=F32, device=h.device)
        ops.linear_small(h, self.w_gates, self.b_gates, gates, ops.GATE_LOG_INPUT_FORGET, self.cap)
        o = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        ops.mlstm_scan(q, k, v, gates, S, n, m, batch.segs, H, self.dim, self.vdim, self.q_scale, self.den_eps, o)
        on = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.headnorm_gate(o, self.norm_w, g, on, H, self.vdim, self.eps)
        return self.out(on)


def rotary_inv_freq(dims, base, device):
    """f_i = base^(-2i/dims), i < dims/2, rounded once to fp32."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return (float(base) ** (-2.0 * i / dims)).to(F32).to(device)


class LatentAttentionMixer:
    """Attention over a latent cache: per token one normalised latent (kv_rank) and one rotated key part (rot_dim) shared by
    the heads are cached; head h's unrotated key and value are Wuk_h c and Wuv_h c.  Queries are laid out per head as
    [dim unrotated | rot_dim rotated]; causal softmax with ``scale``; then Wo.  The kernels work in the latent space
    (csrc/latent_attn.cu), so Wuk is applied to the query and Wuv to the attention's output.  Options:
      ``q_rank``      None: q = Wq h ("q"); a number: q = Wuq RMSnorm(Wdq h) with the plain weight "dq.norm" ("dq", "uq");
      ``rot_pairs``   False: rotary "rotate half" over the first ``rot_dims`` channels of the rotated part (fp32 angles);
                      True: channels (2i, 2i+1) turn together, angles from float64 frequencies, ``rot_scaling`` interpolates them
                      (``scaled_rotary_freq``) and sets the amplitude of cos and sin;
      ``gate``        "head": head outputs times sigmoid(Wg h)_h ("g" [H, W]); "channel": the concatenated heads times
                      sigmoid(Wg h) element by element ("g" [H * vdim, W]); None: no gate."""

    def __init__(self, w, heads, dim, rot_dim, vdim, kv_rank, rot_dims, rot_base, scale, norm_eps, dtype, device, q_rank=None, rot_pairs=False,
                 rot_scaling=None, gate="head"):
        if gate not in (None, "head", "channel"):
            raise ValueError(f"unknown output gate {gate!r}")
        if rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
            raise ValueError(f"cannot rotate {rot_dims} of {rot_dim} channels")
        if rot_scaling and not rot_pairs:
            raise ValueError("interpolated frequencies come with the pairwise rotation")
        self.H, self.dim, self.rot, self.vdim, self.rank = heads, dim, rot_dim, vdim, kv_rank
        self.rot_dims, self.scale, self.eps, self.dtype = rot_dims, float(scale), float(norm_eps), dtype
        self.q_rank, self.gate, self.rot_pairs = q_rank, gate, bool(rot_pairs)
        stacked = [w["dq"] if q_rank else w["q"], w["dkv"]] + ([w["g"]] if gate == "channel" else [])
        self.proj = Linear(stacked, dtype, device)
        if q_rank:
            self.q_norm_w = w["dq.norm"].to(device=device, dtype=F32).contiguous()
            self.up_q = Linear([w["uq"]], dtype, device)
        self.w_gate = w["g"].to(device=device, dtype=dtype).contiguous() if gate == "head" else None
        self.c_norm_w = w["dkv.norm"].to(device=device, dtype=F32).contiguous()
        # Wuk [H*dim, rank] -> per head [rank, dim]: the projection that carries a query into the latent space
        self.w_uk_t = w["uk"].to(device=device, dtype=dtype).view(heads, dim, kv_rank).transpose(1, 2).contiguous()
        self.w_uv = w["uv"].to(device=device, dtype=dtype).contiguous()            # [H*vdim, rank]
        self.out = Linear([w["o"]], dtype, device)
        self.rot_mag = 1.0
        if self.rot_pairs:
            f, self.rot_mag = scaled_rotary_freq(rot_dims, rot_base, rot_scaling)
            self.inv_freq = f.to(device).contiguous()                                    # float64
        else:
            self.inv_freq = rotary_inv_freq(rot_dims, rot_base, device)

    def new_state(self, slots):
        return (slots.add_rows(self.rank + self.rot, self.dtype),)

    def __call__(self, h, batch, state):
        (cache,) = state
        M, H, D = h.shape[0], self.H, self.rank + self.rot
        y = self.proj(h)
        q, dkv = self.proj.part(y, 0), self.proj.part(y, 1)
        if self.q_rank:
            cq = torch.empty(M, self.q_rank, dtype=self.dtype, device=h.device)
            ops.rms_norm_rows(q, self.q_norm_w, cq, self.eps)
            q = self.up_q(cq)
        gate = None
        if self.gate == "head":
            gate = torch.empty(M, H, dtype=F32, device=h.device)
            ops.linear_small(h, self.w_gate, None, gate, ops.GATE_SIGMOID)
        qa = torch.empty(M, H * D, dtype=F32, device=h.device)
        ops.latent_prep(q, dkv, self.c_norm_w, self.inv_freq, batch.meta, cache, qa, H, self.dim, self.rot, self.rot_dims, self.rank,
                        self.eps, pairs=self.rot_pairs, rot_mag=self.rot_mag)
        # q~[m, h, :rank] = Wuk_h^T q[m, h, :dim]
        ops.linear_plain(q, self.w_uk_t, qa, batch=H, a_batch_stride=self.dim + self.rot, w_batch_stride=self.rank * self.dim,
                         out_batch_stride=D, n=self.rank, k=self.dim)
        lat = torch.empty(M, H * self.rank, dtype=F32, device=h.device)
        ops.latent_attn(qa, cache, batch.meta, gate, lat, H, self.rank, self.rot, self.scale, batch.max_ctx)
        channel = self.gate == "channel"
        o = torch.empty(M, H * self.vdim, dtype=F32 if channel else self.dtype, device=h.device)
        ops.linear_plain(lat, self.w_uv, o, batch=H, a_batch_stride=self.rank, w_batch_stride=self.vdim * self.rank,
                         out_batch_stride=self.vdim, n=self.vdim, k=self.rank)
        if channel:
            og = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
            o = ops.sigmoid_mul(o, self.proj.part(y, 2), og)
        return self.out(o)


class ClampedGLU:
    """Dense gated feed-forward: g = min(Wgate h, limit), u = clamp(Wup h, -limit, limit),
    y = g * sigmoid(alpha g) * (u + 1), output Wdown y."""

    def __init__(self, w, ff, limit, dtype, device, alpha=1.702):
        self.ff, self.limit, self.alpha, self.dtype = ff, float(limit), float(alpha), dtype
        self.gate_up = Linear([w["gate"], w["up"]], dtype, device)
        self.down = Linear([w["down"]], dtype, device)

    def __call__(self, h):
        gu = self.gate_up(h)
        y = torch.empty(h.shape[0], self.ff, dtype=self.dtype, device=h.device)
        ops.clamped_glu(gu, self.gate_up.offsets[1], self.ff, y, self.limit, self.alpha)
        return self.down(y)


class DecayLinearAttentionMixer:
    """Linear attention with a fixed decay per head ("lightning" attention): q, k, v = act(Wq h), act(Wk h), act(Wv h);
    S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (csrc/linear_scan.cu), act = SiLU; the concatenated heads RMS-normed together with a per-channel weight, times sigmoid(Wg h), then Wo."""

    def __init__(self, w, heads, dim, vdim, decay, norm_eps, dtype, device):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        self.H, self.dim, self.vdim, self.eps, self.dtype = heads, dim, vdim, float(norm_eps), dtype
        self.proj = Linear([w["q"], w["k"], w["v"], w["g"]], dtype, device)
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float64).to(device=device, dtype=F32)
        self.norm_w = w["norm"].to(device=device, dtype=F32).contiguous()
        self.out = Linear([w["o"]], dtype, device)

    def new_state(self, slots):
        return (slots.add_recurrent((self.H, self.vdim, self.dim)),)

    def __call__(self, h, batch, state):
        (S,) = state
        M, H = h.shape[0], self.H
        y = self.proj(h)
        g = self.proj.part(y, 3)
        # SiLU of q | k | v in one pass over their columns (every block of the scan that shares a head would repeat it otherwise)
        F_, offs = self.proj.offsets[3], self.proj.offsets
        act = torch.empty(M, F_, dtype=self.dtype, device=h.device)
        ops.gated_act(y, F_, act, ops.ACT_SILU)
        q, k, v = act[:, offs[0]:offs[0] + H * self.dim], act[:, offs[1]:offs[1] + H * self.dim], act[:, offs[2]:offs[2] + H * self.vdim]
        o = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        ops.linear_scan(q, k, v, S, batch.segs, H, H, self.dim, self.vdim, o, decay=self.decay)
        on = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.headnorm_gate(o, self.norm_w, g, on, 1, H * self.vdim, self.eps)       # one norm over all heads
        return self.out(on)


class DeltaRuleMixer:
    """Gated delta rule.  q, k (kv_heads x dim) and v (heads x vdim) pass a short causal convolution per channel and SiLU; q, k
    become unit vectors per head (q times dim^-1/2); per head beta = sigmoid(Wb h) and g = exp(-exp(A_log) softplus(Wa h + dt_bias));
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; each head's o RMS-normed with a weight shared by the heads, times
    silu(Wg h); then Wo.  Per-sequence state: S and the last taps - 1 inputs of the convolution."""

    def __init__(self, w, heads, kv_heads, dim, vdim, taps, norm_eps, dtype, device, unit_eps=1e-6):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads do not divide into {kv_heads} query/key heads")
        self.H, self.G, self.dim, self.vdim, self.taps = heads, kv_heads, dim, vdim, int(taps)
        self.eps, self.unit_eps, self.dtype = float(norm_eps), float(unit_eps), dtype
        self.proj = Linear([w["q"], w["k"], w["v"], w["g"]], dtype, device)
        self.w_gates = torch.cat([w["b"], w["a"]], 0).to(device=device, dtype=dtype).contiguous()        # -> beta | decay inputs
        self.w_conv = torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0).to(device=device, dtype=F32).contiguous()
        self.a_log = w["A_log"].to(device=device, dtype=F32).contiguous()
        self.dt_bias = w["dt_bias"].to(device=device, dtype=F32).contiguous()
        self.norm_w = w["norm"].to(device=device, dtype=F32).repeat(heads).contiguous()
        self.out = Linear([w["o"]], dtype, device)
        self.channels = 2 * kv_heads * dim + heads * vdim

    def new_state(self, slots):
        return (slots.add_recurrent((self.H, self.vdim, self.dim)), slots.add_recurrent((max(self.taps - 1, 1), self.channels)))

    def __call__(self, h, batch, state):
        S, conv = state
        M, H, G = h.shape[0], self.H, self.G
        y = self.proj(h)
        gates = torch.empty(M, 2 * H, dtype=F32, device=h.device)
        ops.linear_small(h, self.w_gates, None, gates, ops.GATE_NONE)
        qk = torch.empty(M, 2 * G * self.dim, dtype=F32, device=h.device)
        v = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        offs = self.proj.offsets[:3]
        ops.conv_prep(y, offs, self.w_conv, conv, batch.meta, gates, self.a_log, self.dt_bias, qk, v, G, H, self.dim, self.vdim, self.taps,
                      float(self.dim) ** -0.5, self.unit_eps)
        ops.conv_state_update(y, offs, G * self.dim, H * self.vdim, conv, batch.segs, self.taps)
        o = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        ops.linear_scan(qk[:, :G * self.dim], qk[:, G * self.dim:], v, S, batch.segs, H, G, self.dim, self.vdim, o, gates=gates)
        on = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.headnorm_gate(o, self.norm_w, self.proj.part(y, 3), on, H, self.vdim, self.eps, gate_silu=True)
        return self.out(on)


class WindowAttentionMixer:
    """Softmax attention over the last ``window`` positions, ``kv_heads`` key/value heads shared by groups of query heads, no
    positional rotation.  Values are divided by their per-head root mean square before they are cached; a score is
    (q . k) * scale * temp_h, then softcap * tanh(score / softcap) (csrc/window_attn.cu); output Wo on the concatenated heads."""

    def __init__(self, w, heads, kv_heads, dim, vdim, window, scale, softcap, norm_eps, dtype, device, norm_values=True):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads do not divide into {kv_heads} key/value heads")
        self.H, self.G, self.dim, self.vdim, self.window = heads, kv_heads, dim, vdim, int(window)
        self.scale, self.softcap, self.eps, self.dtype, self.norm_values = float(scale), float(softcap), float(norm_eps), dtype, norm_values
        self.proj = Linear([w["q"], w["k"], w["v"]], dtype, device)
        temp = w.get("temp")
        self.temp = (temp if temp is not None else torch.ones(heads)).to(device=device, dtype=F32).contiguous()
        self.out = Linear([w["o"]], dtype, device)

    def new_state(self, slots):
        return (slots.add_rows(self.G * self.dim, self.dtype), slots.add_rows(self.G * self.vdim, self.dtype))

    def __call__(self, h, batch, state):
        kc, vc = state
        M = h.shape[0]
        y = self.proj(h)
        q, k, v = (self.proj.part(y, i) for i in range(3))
        ops.kv_store(k, v, batch.meta, kc, vc, self.G, self.dim, self.vdim, self.eps, self.norm_values)
        o = torch.empty(M, self.H * self.vdim, dtype=self.dtype, device=h.device)
        ops.window_attn(q, kc, vc, batch.meta, self.temp, o, self.H, self.G, self.dim, self.vdim, self.window, self.scale, self.softcap,
                        nseg=batch.segs.shape[0], max_ctx=batch.max_ctx)
        return self.out(o)


class ForgetGateLinearAttentionMixer:
    """Keyless linear attention whose per-channel forget gate f doubles as the write strength 1 - f (HGRN2's recurrence): q = silu(Wq h), v = Wv h,
    f = low + (1 - low) * sigmoid(Wf h + bf) per head and channel with the learned lower bound ``low``; per head
    row d of the state follows S[d] <- f[d] S[d] + (1 - f[d]) v and the output is o = sum_d q[d] S[d] (no key, no further scale; csrc/linear_scan.cu); each head's o RMS-normed
    over vdim with a plain weight shared by the heads; then Wo.  Gates, state and sums are fp32."""

    def __init__(self, w, heads, dim, vdim, norm_eps, dtype, device):
        self.H, self.dim, self.vdim, self.eps, self.dtype = heads, dim, vdim, float(norm_eps), dtype
        self.proj = Linear([w["q"], w["f"], w["v"]], dtype, device)
        self.f_bias = w["f.b"].to(device=device, dtype=F32).contiguous()
        self.low = w["lower"].to(device=device, dtype=F32).contiguous()
        self.norm_w = w["norm"].to(device=device, dtype=F32).repeat(heads).contiguous()
        self.out = Linear([w["o"]], dtype, device)

    def new_state(self, slots):
        return (slots.add_recurrent((self.H, self.vdim, self.dim)),)

    def __call__(self, h, batch, state):
        (S,) = state
        M, nq, nv = h.shape[0], self.H * self.dim, self.H * self.vdim
        y = self.proj(h)
        qfv = torch.empty(M, 2 * nq + nv, dtype=F32, device=h.device)
        ops.forget_gate_prep(y, self.proj.offsets, self.f_bias, self.low, qfv, nq, nv)
        o = torch.empty(M, nv, dtype=F32, device=h.device)
        ops.forget_scan(qfv[:, :nq], qfv[:, nq:2 * nq], qfv[:, 2 * nq:], S, batch.segs, self.H, self.dim, self.vdim, o)
        on = torch.empty(M, nv, dtype=self.dtype, device=h.device)
        ops.headnorm_gate(o, self.norm_w, None, on, self.H, self.vdim, self.eps)
        return self.out(on)


def wavelength_scaled_rotary_freq(dims, base, scaling=None):
    """Rotation frequencies f_i = base^(-2i/dims), i < dims/2, as float64.  With ``scaling`` {factor, low, high, original}
    (the rule Llama 3.1 uses): a pair whose wavelength 2 pi / f is shorter than original / high keeps f, one longer than
    original / low gets f / factor, and between the two the blend weight t = (original / wavelength - low) / (high - low)
    gives f * (t + (1 - t) / factor)."""
    import math
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    wave = 2.0 * math.pi / f
    t = (original / wave - low) / (high - low)
    mid = f * (t + (1.0 - t) / factor)
    return torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, mid))


class DifferentialAttentionMixer:
    """Differential attention with grouped key/value heads: every query head carries two softmax attention maps (q and k have
    2 * dim channels per head, [map 1 | map 2]) over the SAME values; with a1, a2 the maps' outputs,
    o = a1 - lam * a2, then o / rms(o) per head (no weight) times (1 - diff), then Wo;
    lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff is a single scalar per layer.  q and k turn in channel pairs (2i, 2i+1) over the
    first ``rot["dims"]`` channels of every map (``rot["scaling"]``: the wavelength rule).  Mask: causal, and ``chunk`` > 0 keeps
    only the keys of the query's own block of ``chunk`` positions, ``window`` > 0 only the last ``window`` positions.
    The key cache holds 2 G heads ([g][map]), the value cache G; the query projection's rows are regrouped at load time as
    [g][map][head of the group] so that the attention kernel's plain grouping (csrc/window_attn.cu) pairs every map with its key
    head, and value head = key head // 2.  Scores, weights, sums, the difference and the norm are fp32."""

    def __init__(self, w, heads, kv_heads, dim, vdim, scale, diff, norm_eps, dtype, device, rot=None, chunk=0, window=0):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads do not divide into {kv_heads} key/value heads")
        self.H, self.G, self.dim, self.vdim = heads, kv_heads, dim, vdim
        self.scale, self.diff, self.eps, self.dtype = float(scale), float(diff), float(norm_eps), dtype
        self.chunk, self.window = int(chunk or 0), int(window or 0)
        rep = heads // kv_heads
        wq = w["q"].view(kv_heads, rep, 2, dim, -1).permute(0, 2, 1, 3, 4).reshape(heads * 2 * dim, -1)      # [g][r][map] -> [g][map][r]
        self.proj = Linear([wq, w["k"], w["v"]], dtype, device)
        d64 = torch.float64
        self.lam = float(torch.exp((w["lq1"].to(d64) * w["lk1"].to(d64)).sum()) - torch.exp((w["lq2"].to(d64) * w["lk2"].to(d64)).sum())) + self.diff
        self.rot_dims, self.freq = 0, None
        if rot:
            self.rot_dims = int(rot["dims"])
            if self.rot_dims % 2 or not 0 < self.rot_dims <= dim:
                raise ValueError(f"cannot rotate {self.rot_dims} of {dim} channels")
            self.freq = wavelength_scaled_rotary_freq(self.rot_dims, rot["base"], rot.get("scaling")).to(device).contiguous()
        self.out = Linear([w["o"]], dtype, device)

    @property
    def span(self):
        """The most keys a query can see (0: the whole history)."""
        lim = [n for n in (self.chunk, self.window) if n > 0]
        return min(lim) if lim else 0

    def new_state(self, slots):
        return (slots.add_rows(2 * self.G * self.dim, self.dtype), slots.add_rows(self.G * self.vdim, self.dtype))

    def __call__(self, h, batch, state):
        kc, vc = state
        M, H2, G2 = h.shape[0], 2 * self.H, 2 * self.G
        y = self.proj(h)
        q = torch.empty(M, H2 * self.dim, dtype=F32, device=h.device)
        ops.qkv_prep(y, self.proj.offsets, batch.meta, q, kc, vc, H2, G2, self.dim, self.vdim, self.eps, freq=self.freq, rot_dims=self.rot_dims,
                     v_heads=self.G)
        a = torch.empty(M, H2 * self.vdim, dtype=F32, device=h.device)
        ops.window_attn(q, kc, vc, batch.meta, None, a, H2, G2, self.dim, self.vdim, self.window, self.scale, 0.0, nseg=batch.segs.shape[0],
                        max_ctx=batch.max_ctx, chunk=self.chunk, v_div=2)
        o = torch.empty(M, self.H * self.vdim, dtype=self.dtype, device=h.device)
        ops.diff_combine(a, o, self.H, self.G, self.vdim, self.lam, 1.0 - self.diff, self.eps)
        return self.out(o)


def scaled_rotary_freq(dims, base, scaling=None):
    """Rotation frequencies f_i = base^(-2i/dims), i < dims/2, as float64, and the factor on cos and sin.  With ``scaling``
    {factor, original, fast, slow} (the "YaRN" interpolation): pairs that turn more than ``fast`` times within ``original``
    positions keep f_i, those that turn fewer than ``slow`` times get f_i / factor, the ones between are blended linearly in
    the pair index, and the rotation's amplitude becomes 1 + 0.1 ln(factor)."""
    import math
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_at(turns):                     # the (real-valued) pair index whose frequency makes `turns` turns in `original` positions
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(pair_at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_at(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class SinkAttentionMixer:
    """Causal softmax attention over the whole history with grouped key/value heads and one learned sink per head in the
    softmax's denominator (a term without key or value).  Everything else is an option, so that designs which differ in them
    share the mixer:
      ``biases``   q, k, v projections with biases ("q.b", ...);
      ``taps``     a short causal convolution along the sequence on every channel of q, k, v right after the projection ("q.conv"
                   [channels, taps], ...; None: no convolution); the last taps - 1 projected rows are per-sequence state;
      ``norm``     "whole": one RMS norm over all of q and one over all of k ("q.norm" [H*dim], "k.norm" [G*dim]);
                   "head": per head with a weight [dim] shared by the heads;
      ``q_temp``   (coef, every): q times 1 + coef * ln(floor((pos + 1) / every) + 1);
      ``rot``      {"dims", "base", "scaling"}: the first ``dims`` channels of every q and k head turn in pairs (2i, 2i+1);
      ``slopes``   [H]: every position between query and key costs head h slopes[h] of the score;
      ``v_mix``    "publish": this layer's values are left in the step's scratch for later layers; "blend": v becomes
                   (1 - vmix) v + vmix v_published before it is cached;
      ``gate``     "head": head h's output times sigmoid(Wg h)_h; "channel": the concatenated heads times sigmoid(Wg h);
      ``ride_along`` further weight matrices that read the same input: they join the stacked projection and their outputs
                   (column slices) are appended to ``extras`` by ``__call__``.
    Norms, temperature, angles, scores, weights and sums are fp32; q stays fp32 up to the scores; the caches hold the
    model's dtype (csrc/window_attn.cu)."""

    def __init__(self, w, heads, kv_heads, dim, vdim, scale, norm_eps, dtype, device, norm=None, biases=False, taps=None, q_temp=None, rot=None,
                 slopes=None, v_mix=None, gate=None, ride_along=()):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads do not divide into {kv_heads} key/value heads")
        if norm not in (None, "whole", "head") or gate not in (None, "head", "channel") or v_mix not in (None, "publish", "blend"):
            raise ValueError(f"unknown option: norm={norm!r} gate={gate!r} v_mix={v_mix!r}")
        self.H, self.G, self.dim, self.vdim, self.taps = heads, kv_heads, dim, vdim, int(taps or 1)
        self.scale, self.eps, self.dtype = float(scale), float(norm_eps), dtype
        nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
        self.channels = nq + nk + nv
        stacked = [w["q"], w["k"], w["v"]] + ([w["g"]] if gate == "channel" else []) + list(ride_along)
        self.n_ride, self.gate = len(ride_along), gate
        self.proj = Linear(stacked, dtype, device)
        f32 = dict(device=device, dtype=F32)
        self.bias = torch.cat([w["q.b"], w["k.b"], w["v.b"]]).to(**f32).contiguous() if biases else None
        self.w_conv = torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0).to(**f32).contiguous() if taps else None
        self.norm_mode = {None: ops.NORM_NONE, "whole": ops.NORM_WHOLE, "head": ops.NORM_PER_HEAD}[norm]
        self.q_norm = w["q.norm"].to(**f32).contiguous() if norm else None
        self.k_norm = w["k.norm"].to(**f32).contiguous() if norm else None
        self.temp_coef, self.temp_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
        self.rot_dims, self.freq, self.rot_mag = 0, None, 1.0
        if rot:
            self.rot_dims = int(rot["dims"])
            if self.rot_dims % 2 or not 0 < self.rot_dims <= dim:
                raise ValueError(f"cannot rotate {self.rot_dims} of {dim} channels")
            f, self.rot_mag = scaled_rotary_freq(self.rot_dims, rot["base"], rot.get("scaling"))
            self.freq = f.to(device).contiguous()
        self.slopes = torch.tensor([float(x) for x in slopes], dtype=torch.float64).to(**f32) if slopes is not None else None
        self.sink = w["sink"].to(**f32).contiguous()
        self.vmix_mode = {None: ops.VMIX_NONE, "publish": ops.VMIX_PUBLISH, "blend": ops.VMIX_BLEND}[v_mix]
        self.vmix = float(w["vmix"]) if v_mix == "blend" else 0.0
        self.w_gate = w["g"].to(device=device, dtype=dtype).contiguous() if gate == "head" else None
        self.out = Linear([w["o"]], dtype, device)

    def new_state(self, slots):
        st = (slots.add_rows(self.G * self.dim, self.dtype), slots.add_rows(self.G * self.vdim, self.dtype))
        if self.taps > 1:
            st += (slots.add_recurrent((self.taps - 1, self.channels)),)
        return st

    def __call__(self, h, batch, state, extras=None):
        kc, vc = state[0], state[1]
        conv = state[2] if self.taps > 1 else None
        M, H, G = h.shape[0], self.H, self.G
        y = self.proj(h)
        first_ride = 3 + (self.gate == "channel")
        if extras is not None:
            extras.extend(self.proj.part(y, first_ride + i) for i in range(self.n_ride))
        gate = None
        if self.gate == "head":
            gate = torch.empty(M, H, dtype=F32, device=h.device)
            ops.linear_small(h, self.w_gate, None, gate, ops.GATE_SIGMOID)
        elif self.gate == "channel":
            gate = self.proj.part(y, 3)
        v_first = None
        if self.vmix_mode == ops.VMIX_PUBLISH:
            v_first = batch.scratch["v_first"] = torch.empty(M, G * self.vdim, dtype=F32, device=h.device)
        elif self.vmix_mode == ops.VMIX_BLEND:
            v_first = batch.scratch["v_first"]
            if v_first.shape[1] != G * self.vdim:
                raise ValueError(f"values of {G * self.vdim} numbers cannot be blended with published values of {v_first.shape[1]}")
        q = torch.empty(M, H * self.dim, dtype=F32, device=h.device)
        offs = self.proj.offsets[:3]
        ops.qkv_prep(y, offs, batch.meta, q, kc, vc, H, G, self.dim, self.vdim, self.eps, bias=self.bias, wconv=self.w_conv, conv_state=conv,
                     taps=self.taps, norm_mode=self.norm_mode, qnorm_w=self.q_norm, knorm_w=self.k_norm, temp_coef=self.temp_coef,
                     temp_every=self.temp_every, freq=self.freq, rot_dims=self.rot_dims, rot_mag=self.rot_mag, vmix_mode=self.vmix_mode,
                     vmix=self.vmix, v_first=v_first)
        if self.taps > 1:
            ops.conv_state_update(y, offs, H * self.dim, G * self.vdim, conv, batch.segs, self.taps, nk=G * self.dim)
        o = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.window_attn(q, kc, vc, batch.meta, None, o, H, G, self.dim, self.vdim, 0, self.scale, 0.0, nseg=batch.segs.shape[0],
                        max_ctx=batch.max_ctx, slopes=self.slopes, sink=self.sink, gate=gate, gate_per_head=self.gate == "head")
        return self.out(o)


class PolyNormMLP:
    """Wdown act(Wup h) with the polynomial activation between norms: act(z) = k1 R(z) + k2 R(z*z) + k3 R(z*z*z) + k0, products taken
    element by element, R = division of a token's ff numbers by their root mean square (fp32).  ``ride_along``: further weight
    matrices that read the same input and join the up projection (outputs appended to ``extras``)."""

    def __init__(self, w, ff, norm_eps, dtype, device, ride_along=()):
        self.ff, self.eps, self.dtype, self.n_ride = ff, float(norm_eps), dtype, len(ride_along)
        self.up = Linear([w["up"]] + list(ride_along), dtype, device)
        self.coef = w["act"].to(device=device, dtype=F32).contiguous()
        self.down = Linear([w["down"]], dtype, device)

    def __call__(self, h, extras=None):
        u = self.up(h)
        if extras is not None:
            extras.extend(self.up.part(u, 1 + i) for i in range(self.n_ride))
        y = torch.empty(h.shape[0], self.ff, dtype=self.dtype, device=h.device)
        ops.poly_norm(u, self.ff, self.coef, y, self.eps)
        return self.down(y)


class GatedMLP:
    """Dense gated feed-forward: Wdown (act(Wgate h) * (Wup h))."""

    def __init__(self, w, ff, act, dtype, device):
        self.ff, self.act, self.dtype = ff, act, dtype
        self.gate_up = Linear([w["gate"], w["up"]], dtype, device)
        self.down = Linear([w["down"]], dtype, device)

    def __call__(self, h):
        gu = self.gate_up(h)
        y = torch.empty(h.shape[0], self.ff, dtype=self.dtype, device=h.device)
        ops.gated_act(gu, self.ff, y, self.act, up_off=self.gate_up.offsets[1])
        return self.down(y)


class PlainMLP:
    """Wdown act(Wup h)."""

    def __init__(self, w, ff, act, dtype, device):
        self.ff, self.act, self.dtype = ff, act, dtype
        self.up = Linear([w["up"]], dtype, device)
        self.down = Linear([w["down"]], dtype, device)

    def __call__(self, h):
        u = self.up(h)
        y = torch.empty(h.shape[0], self.ff, dtype=self.dtype, device=h.device)
        ops.gated_act(u, self.ff, y, self.act)
        return self.down(y)


class MoEFeedForward:
    """Routed mixture of experts: router logits in fp32, softmax over all experts, the ``top`` largest scores (``correction``,
    one number per router output, is added for the choice only) as weights, renormalised (divided by their sum + 1e-20) if
    ``renorm``; every expert is Wdown act(Wup h), or Wdown (act(Wgate h) * Wup h) when ``experts_w`` carry a "gate"; the last
    ``identity`` router outputs are experts without weights that hand the token back; ``act`` = ops.ACT_CLAMPED_SWISH with
    ``act_params`` = (limit, alpha) makes a gated expert Wdown (g' sigmoid(alpha g') (u' + 1)), g' = min(Wgate h, limit), u' = clamp(Wup h, +-limit);
    with ``renorm`` the weights equal a softmax restricted to the selected experts' logits; a shared expert (optional) runs for
    every token and is added.  ``experts_w``: list of {"up", "down"[, "gate"]} per expert.  The (token, choice) pairs are
    grouped by expert on the device (no host round trip) and each projection runs as one grouped launch; a handful of pairs
    (decoding) take the form with one warp per output instead.  The result is fp32."""

    FEW_PAIRS = 48            # up to here: one warp per output, no plan
    TENSOR_CORE_PAIRS = 512   # from here (bf16, sizes that are multiples of 8): every expert's rows through the tensor-core GEMM

    def __init__(self, router_w, experts_w, top, ff, act, shared, dtype, device, correction=None, renorm=True, identity=0, act_params=(0.0, 0.0)):
        self.E, self.top, self.ff, self.act, self.dtype = len(experts_w), int(top), ff, act, dtype
        self.act_params = (float(act_params[0]), float(act_params[1]))      # ACT_CLAMPED_SWISH (gated experts): (limit, alpha)
        self.identity, self.renorm = int(identity), bool(renorm)
        self.R = self.E + self.identity                          # router outputs
        if not 1 <= self.top <= self.R or self.E < 1 or router_w.shape[0] != self.R:
            raise ValueError(f"top = {top} of {self.E} experts + {self.identity} identity experts, router of {router_w.shape[0]} outputs")
        self.router = router_w.to(device=device, dtype=dtype).contiguous()
        self.correction = correction.to(device=device, dtype=F32).contiguous() if correction is not None else None
        self.gated = "gate" in experts_w[0]
        # [E, ff, W], or [E, 2 ff, W] with every expert's gate rows before its up rows
        self.w_up = torch.stack([torch.cat([e["gate"], e["up"]], 0) if self.gated else e["up"] for e in experts_w]).to(device=device, dtype=dtype).contiguous()
        self.w_down = torch.stack([e["down"] for e in experts_w]).to(device=device, dtype=dtype).contiguous()     # [E, W, ff]
        self.shared = shared
        W = self.w_up.shape[2]
        self.tensor_core = dtype == BF16 and W % 8 == 0 and ff % 8 == 0 and os.environ.get("LIA_PLAIN_LINEAR", "0") == "0"

    def _workspace(self, rows, N, K, device):
        """One split-K workspace large enough for every row count among the experts' launches."""
        key = (device, "experts")
        need = ops.GemmWorkspace.bytes_for([(m, N, K) for m in set(rows)])
        ws = Linear._gemm_ws.get(key)
        if ws is None or ws.buf.numel() < need:
            ws = Linear._gemm_ws[key] = ops.GemmWorkspace(need, device)
        return ws

    def _experts_tensor_core(self, h, idx, wt, y):
        """Prompts: the pairs grouped by expert (tiles of 64 rows), the rows gathered into that order, then one tensor-core
        GEMM per expert and projection on its contiguous rows (launched back to back from the library).  The tile table comes to the host once per call (the only
        round trip; decode steps never take this path, so they stay capturable)."""
        M, W = h.shape
        E, R, top, ff, dev = self.E, self.R, self.top, self.ff, h.device
        pairs = M * top
        n_tiles, tm = ops.moe_tiles(pairs, R)
        perm = torch.empty(n_tiles * tm, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(n_tiles, dtype=torch.int32, device=dev)
        pos_of = torch.empty(pairs, dtype=torch.int32, device=dev)
        ops.moe_plan(idx, R, perm, tile_expert, pos_of)
        xs = torch.empty(n_tiles * tm, W, dtype=self.dtype, device=dev)
        ops.moe_gather(h, perm, xs, top)
        counts = torch.bincount(tile_expert.cpu().long() + 1, minlength=R + 1)[1:E + 1].tolist()     # tiles per expert that has weights (they come first)
        used, rows = max(sum(counts), 1) * tm, [n * tm for n in counts if n]
        n_up = self.w_up.shape[1]
        up = torch.empty(used, n_up, dtype=self.dtype, device=dev)
        mid = torch.empty(used, ff, dtype=self.dtype, device=dev)
        ys = torch.empty(used, W, dtype=self.dtype, device=dev)
        if rows:
            ops.moe_expert_gemms(xs, self.w_up, up, counts, tm, self._workspace(rows, n_up, W, dev))
            if self.act == ops.ACT_CLAMPED_SWISH:
                ops.clamped_glu(up, ff, ff, mid, *self.act_params)
            else:
                ops.gated_act(up, ff, mid, self.act, up_off=ff if self.gated else -1)
            ops.moe_expert_gemms(mid, self.w_down, ys, counts, tm, self._workspace(rows, W, ff, dev))
        ops.moe_combine(ys, self.shared(h) if self.shared is not None else None, y, top, pos_of=pos_of, wt=wt,
                        identity=(idx, E, h, wt) if self.identity else None)
        return y

    def __call__(self, h, router_input=None):
        """``router_input``: the same rows before they were rounded to the activations' dtype (the fp32 residual stream), for
        router logits that do not see that rounding; None: the router reads ``h``."""
        M, W, dev = h.shape[0], h.shape[1], h.device
        R, top = self.R, self.top
        logits = torch.empty(M, R, dtype=F32, device=dev)
        ops.linear_small(h if router_input is None else router_input, self.router, None, logits, ops.GATE_NONE)
        idx = torch.empty(M, top, dtype=torch.int32, device=dev)
        wt = torch.empty(M, top, dtype=F32, device=dev)
        ops.router_topk(logits, top, idx, wt, correction=self.correction, renorm=self.renorm)
        identity = (idx, self.E, h, wt) if self.identity else None
        pairs = M * top
        y = torch.empty(M, W, dtype=F32, device=dev)
        if self.tensor_core and pairs >= self.TENSOR_CORE_PAIRS and h.is_contiguous() and not torch.cuda.is_current_stream_capturing():
            return self._experts_tensor_core(h, idx, wt, y)
        ypair = torch.empty(pairs, W, dtype=F32, device=dev)
        if pairs <= self.FEW_PAIRS:
            mid = torch.empty(pairs, self.ff, dtype=self.dtype, device=dev)
            ops.moe_gemm(h, self.w_up, mid, idx, wt, top, True, self.act, gated=self.gated, act_params=self.act_params)
            ops.moe_gemm(mid, self.w_down, ypair, idx, wt, top, False)
        else:
            n_tiles, tm = ops.moe_tiles(pairs, R)
            perm = torch.empty(n_tiles * tm, dtype=torch.int32, device=dev)
            tile_expert = torch.empty(n_tiles, dtype=torch.int32, device=dev)
            pos_of = torch.empty(pairs, dtype=torch.int32, device=dev)
            ops.moe_plan(idx, R, perm, tile_expert, pos_of)
            mid = torch.empty(n_tiles * tm, self.ff, dtype=self.dtype, device=dev)
            ops.moe_gemm(h, self.w_up, mid, idx, wt, top, True, self.act, perm, tile_expert, gated=self.gated, act_params=self.act_params)
            ops.moe_gemm(mid, self.w_down, ypair, idx, wt, top, False, ops.ACT_NONE, perm, tile_expert)
        ops.moe_combine(ypair, self.shared(h) if self.shared is not None else None, y, top, identity=identity)
        return y
