"""GPU checks of the Bizetar path against the plain float64 oracle (tests/bizetar_oracle.py): every new kernel and both mixers
alone, then the model through the step engine -- whole prompts, token-by-token decoding, portions down to two tokens (shorter
than the convolution's state), unequal requests in one step, slots that are freed and reused, a key far back among hundreds,
keys at the edges of the attention kernel's own tiles (32 cached positions per stage, 64 per key range), the sink, the
positions where the query temperature steps, the first tokens, long decoding, greedy generation through generate(), the trace
runner and the command line."""
import copy
import json
import math
import os

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import ops, registry
from lia_b200.checkpoint import write_safetensors
from lia_b200.engine import Engine
from lia_b200.modeling_bizetar import BizetarConfig, BizetarForCausalLM, distance_slopes
from lia_b200.seq_layers import MoEFeedForward, PolyNormMLP, SinkAttentionMixer, StepBatch, scaled_rotary_freq
from lia_b200.seq_state import SlotState

import bizetar_oracle as O
from bizetar_cases import CASES, attention, attention_2, config, dense, moe

pytestmark = pytest.mark.gpu
BF16, F32, F64 = torch.bfloat16, torch.float32, torch.float64
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def bf(t):
    """bf16-representable fp32 numbers."""
    return t.to(BF16).float()


def make_batch(portions):
    """portions: (slot, first position, tokens) in row order."""
    segs, meta, row = [], [], 0
    for slot, p0, n in portions:
        segs.append((slot, p0, row, n))
        meta += [(slot, p0 + i) for i in range(n)]
        row += n
    return StepBatch(row, i32(segs), i32(meta), max(p0 + n for _, p0, n in portions))


CUTS = {"whole": [60], "token by token": [1] * 60, "twos": [2] * 30, "ragged": [31, 1, 1, 2, 22, 3], "stage edges": [32, 1, 27]}


# ------------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("W", [44, 256, 1000])
def test_gated_residual_norm_and_layer_mix(W):
    g = gen(0)
    rows, n_stack = 9, 5
    x0 = torch.randn(rows, W, generator=g)
    y = torch.randn(rows, W, generator=g) * 3.0
    r = torch.randn(rows, W + 8, generator=g) * 2.0                   # the gate is a column slice of a wider buffer
    rb, w = torch.randn(W, generator=g), torch.randn(W, generator=g)
    mix = torch.randn(n_stack, generator=g)
    earlier = torch.randn(n_stack, rows, W, generator=g)
    for dt, tol in ((F32, 2e-6), (BF16, 5e-3)):
        yy, rr = y.to(dt), r.to(dt)
        gated = yy.double() * torch.sigmoid(rr.double()[:, 8:] + rb.double())
        # the gated, normed add alone
        x = x0.clone().to(DEV)
        h = torch.empty(rows, W, dtype=dt, device=DEV)
        ops.gated_rms_add(x, yy.to(DEV), w.to(DEV), h, 1e-5, gate=rr.to(DEV)[:, 8:], gate_bias=rb.to(DEV))
        want = x0.double() + O.rms_norm(gated, w.double(), 1e-5)
        assert rel(x, want) < 2e-6 and rel(h, want) < tol             # the residual sum is fp32 whatever the activations are
        # the same, then the result joins the stack and a mix of entries 0 .. 3 goes on
        x = x0.clone().to(DEV)
        stack = earlier.clone().to(DEV)
        ops.gated_rms_add(x, yy.to(DEV), w.to(DEV), h, 1e-5, gate=rr.to(DEV)[:, 8:], gate_bias=rb.to(DEV), stack=stack, n_mix=4, mix=mix.to(DEV))
        assert rel(stack[3], want) < 2e-6 and torch.equal(stack[4].cpu(), earlier[4]) and torch.equal(stack[:3].cpu(), earlier[:3])
        mixed = sum(mix[j].double() * earlier[j].double() for j in range(3)) + mix[3].double() * want
        assert rel(x, mixed) < 4e-6 and rel(h, mixed) < tol
        # no gate: the plain norm of the sublayer's output
        x = x0.clone().to(DEV)
        ops.gated_rms_add(x, yy.to(DEV), w.to(DEV), None, 1e-5)
        assert rel(x, x0.double() + O.rms_norm(yy.double(), w.double(), 1e-5)) < 2e-6
    # nothing added: the row joins the stack as entry 0 with weight 1 (the embedding's way in) and comes out in the activations' type
    x = x0.clone().to(DEV)
    stack = torch.zeros(2, rows, W, device=DEV)
    h = torch.empty(rows, W, dtype=BF16, device=DEV)
    ops.gated_rms_add(x, None, None, h, 1e-5, stack=stack, n_mix=1, mix=torch.ones(1, device=DEV))
    assert torch.equal(x.cpu(), x0) and torch.equal(stack[0].cpu(), x0) and torch.equal(h.cpu(), x0.to(BF16))


@pytest.mark.parametrize("F", [30, 256, 1100])
def test_polynomial_activation_between_norms(F):
    g = gen(1)
    z = torch.randn(7, F + 16, generator=g) * 2.0
    coef = torch.tensor([0.9, -0.4, 0.3, 0.2])
    for dt, tol in ((F32, 3e-6), (BF16, 6e-3)):
        zz = z.to(dt)
        out = torch.empty(7, F, dtype=dt, device=DEV)
        ops.poly_norm(zz.to(DEV), F, coef.to(DEV), out, 1e-5)
        assert rel(out, O.poly_norm(zz.double()[:, :F], coef, 1e-5)) < tol
    w = {"up": bf(torch.randn(F, 44, generator=g) * 44 ** -0.5), "down": bf(torch.randn(44, F, generator=g) * F ** -0.5), "act": coef}
    h = bf(torch.randn(70, 44, generator=g))
    ride = bf(torch.randn(44, 44, generator=g))
    extras = []
    got = PolyNormMLP(w, F, 1e-5, F32, DEV, ride_along=[ride])(h.to(DEV), extras)
    assert rel(got, O.dense_ff(h.double(), {k: v.double() for k, v in w.items()}, "", 1e-5)) < 1e-5
    assert rel(extras[0], h.double() @ ride.double().T) < 1e-5


def test_router_chooses_with_the_correction_and_weighs_without():
    g = gen(2)
    M, E, top = 50, 11, 3
    z = torch.randn(M, E, generator=g)
    corr = torch.randn(E, generator=g) * 0.3 - 0.5                     # choice scores below zero as well
    idx = torch.empty(M, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(M, top, dtype=F32, device=DEV)
    ops.router_topk(z.to(DEV), top, idx, wt, correction=corr.to(DEV), renorm=False)
    s = torch.softmax(z.double(), -1)
    want_idx = (s + corr.double()).topk(top, -1).indices
    assert torch.equal(idx.cpu().long(), want_idx)
    assert rel(wt, torch.gather(s, -1, want_idx)) < 1e-6
    assert not torch.equal(want_idx, s.topk(top, -1).indices)          # the correction did change some choices
    ops.router_topk(z.to(DEV), top, idx, wt)                           # the earlier form: plain scores, renormalised
    assert torch.equal(idx.cpu().long(), s.topk(top, -1).indices) and rel(wt.sum(-1), torch.ones(M)) < 1e-6


@pytest.mark.parametrize("M,dtype", [(5, F32), (5, BF16), (90, F32), (300, BF16), (300, F32)])
def test_gated_experts_with_identity_experts_in_every_form(M, dtype):
    """Few pairs (one warp per output), the grouped launch, and (bf16, many pairs) the tensor-core form; expert 1 gets no token
    and the identity experts take many of them (a strong correction in their favour)."""
    g = gen(3)
    W, ff, E, ident, top = 64, 24, 5, 2, 3
    cfg = {"router": {"experts": E, "identity": ident, "top": top}, "expert": {"ff": ff}}
    w = {"router": bf(torch.randn(E + ident, W, generator=g) * 3 * W ** -0.5), "correction": torch.tensor([0.0, -5.0, 0.0, 0.0, 0.0, 0.3, 0.1])}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = bf(torch.randn(ff, W, generator=g) * W ** -0.5), bf(torch.randn(ff, W, generator=g) * W ** -0.5)
        w[f"e{e}.down"] = bf(torch.randn(W, ff, generator=g) * ff ** -0.5)
    h = bf(torch.randn(M, W, generator=g))
    want = O.moe(h.double(), {k: v.double() for k, v in w.items()}, "", cfg)
    experts = [{k: w[f"e{e}.{k}"] for k in ("gate", "up", "down")} for e in range(E)]
    m = MoEFeedForward(w["router"], experts, top, ff, ops.ACT_SILU, None, dtype, DEV, correction=w["correction"], renorm=False, identity=ident)
    old = MoEFeedForward.TENSOR_CORE_PAIRS
    MoEFeedForward.TENSOR_CORE_PAIRS = 512
    try:
        got = m(h.to(device=DEV, dtype=dtype))
    finally:
        MoEFeedForward.TENSOR_CORE_PAIRS = old
    idx, _ = O.route(h.double(), w["router"].double(), w["correction"].double(), top)
    assert int((idx >= E).sum()) > M // 2 and int((idx == 1).sum()) == 0
    assert rel(got, want) < (1e-5 if dtype == F32 else 2e-2)


def _attn_inputs(H, G, dim, vdim, n, seed):
    g = gen(seed)
    q = torch.randn(n, H * dim, generator=g)
    k = bf(torch.randn(n, G * dim, generator=g))
    v = bf(torch.randn(n, G * vdim, generator=g))
    return q, k, v


@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 16, 24), (9, 3, 72, 40), (1, 1, 12, 10), (8, 1, 96, 136)])
def test_attention_kernel_with_sink_slopes_and_gates(H, G, dim, vdim):
    """Prompt rows and single rows (keys split over blocks) at histories that end at the kernel's tile edges; fp32 queries on
    bf16 caches; per-head and per-channel gates."""
    n = 200
    q, k, v = _attn_inputs(H, G, dim, vdim, n, 4)
    sink = torch.randn(H, generator=gen(5))
    slopes = torch.tensor(distance_slopes(H))
    gate_h = torch.rand(n, H, generator=gen(6))
    gate_c = torch.randn(n, H * vdim + 8, generator=gen(7))
    pos = torch.arange(n)
    plain = O.sink_attention(q.double().view(n, H, dim), k.double().view(n, G, dim), v.double().view(n, G, vdim), pos, 0.3, sink.double(), slopes.double())
    for cache_dt, tol in ((F32, 2e-5), (BF16, 8e-3)):
        kc = torch.zeros(2, n, G * dim, dtype=cache_dt, device=DEV)
        vc = torch.zeros(2, n, G * vdim, dtype=cache_dt, device=DEV)
        kc[1], vc[1] = k.to(DEV), v.to(DEV)
        meta = i32([(1, p) for p in range(n)])
        out = torch.empty(n, H * vdim, dtype=cache_dt, device=DEV)
        # the whole prompt in one step, one gate per head
        ops.window_attn(q.to(DEV), kc, vc, meta, None, out, H, G, dim, vdim, 0, 0.3, 0.0, nseg=1, max_ctx=n, slopes=slopes.to(DEV), sink=sink.to(DEV),
                        gate=gate_h.to(DEV), gate_per_head=True)
        assert rel(out, (plain * gate_h.double()[:, :, None]).reshape(n, -1)) < tol
        # single rows at the tile edges, keys split over blocks, a gate per channel read from a wider buffer
        gc = gate_c.to(cache_dt)
        want = plain.reshape(n, -1) * torch.sigmoid(gc.double()[:, 8:])
        for p in (0, 1, 31, 32, 33, 63, 64, 65, 127, 128, 199):
            o1 = torch.empty(1, H * vdim, dtype=cache_dt, device=DEV)
            ops.window_attn(q[p:p + 1].to(DEV), kc, vc, i32([(1, p)]), None, o1, H, G, dim, vdim, 0, 0.3, 0.0, max_ctx=p + 1, slopes=slopes.to(DEV),
                            sink=sink.to(DEV), gate=gc.to(DEV)[p:p + 1, 8:])
            assert rel(o1, want[p:p + 1]) < tol, p


def test_attention_sink_and_distance_bias_show():
    """Weights made so that a fault shows: with zero queries the scores are the distance bias alone, so the weights are
    exp(-slope (i - j)) against exp(sink); a huge sink empties the output; a far key among hundreds that matches the query
    takes all the weight although 300 keys lie between."""
    H, G, dim, vdim, n = 2, 1, 8, 8, 400
    g = gen(8)
    k = bf(torch.randn(n, dim, generator=g))
    v = bf(torch.randn(n, vdim, generator=g))
    kc, vc = k.to(DEV).view(1, n, dim).contiguous(), v.to(DEV).view(1, n, vdim).contiguous()
    slopes = torch.tensor([0.5, 0.01])
    sink = torch.tensor([0.7, 4.0])
    p = n - 1
    out = torch.empty(1, H * vdim, dtype=F32, device=DEV)
    zero_q = torch.zeros(1, H * dim, device=DEV)
    ops.window_attn(zero_q, kc, vc, i32([(0, p)]), None, out, H, G, dim, vdim, 0, 1.0, 0.0, max_ctx=n, slopes=slopes.to(DEV), sink=sink.to(DEV))
    dist = (p - torch.arange(n)).double()
    for h in range(H):
        wts = torch.exp(-slopes[h].double() * dist)
        want = (wts[:, None] * v.double()).sum(0) / (wts.sum() + math.exp(float(sink[h])))
        assert rel(out[0, h * vdim:(h + 1) * vdim], want) < 1e-5
        without_sink = (wts[:, None] * v.double()).sum(0) / wts.sum()
        assert rel(want, without_sink) > 0.05                        # a kernel that left the sink out would be far off
    ops.window_attn(zero_q, kc, vc, i32([(0, p)]), None, out, H, G, dim, vdim, 0, 1.0, 0.0, max_ctx=n, sink=torch.tensor([40.0, 40.0], device=DEV))
    assert float(out.abs().max()) < 1e-12
    far = 57
    k2 = k.clone()
    k2[:, 0] = 0.0
    k2[far, 0] = 1.0                                                   # channel 0 marks the far key alone
    q = torch.zeros(1, H * dim)
    q[0, 0] = 30.0                                                     # head 0: score 30 at the far key, 0 at every other
    ops.window_attn(q.to(DEV), k2.to(DEV).view(1, n, dim).contiguous(), vc, i32([(0, p)]), None, out, H, G, dim, vdim, 0, 1.0, 0.0, max_ctx=n, sink=sink.to(DEV))
    assert rel(out[0, :vdim], v[far]) < 1e-6


def _prep_reference(y, pos_first, w, m, kind, eps, past, v_first):
    """q, k, v as the oracle's mixers make them, for rows that continue a sequence whose earlier projected rows are ``past``."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = y["q"].shape[0]
    pos = torch.arange(pos_first, pos_first + T)
    if kind == "attention":
        q = O.rms_norm(y["q"], w["q.norm"], eps) * (1.0 + m["q_temp"]["coef"] * torch.log(torch.floor((pos.double() + 1) / m["q_temp"]["every"]) + 1.0))[:, None]
        k = O.rms_norm(y["k"], w["k.norm"], eps)
        v = y["v"]
    else:
        u = {n: y[n] + w[n + ".b"] for n in "qkv"}
        u = {n: O.causal_conv(u[n], w[n + ".conv"], past[n] + w[n + ".b"] if past[n].shape[0] else past[n]) for n in "qkv"}       # one tap: a factor per channel
        q = O.rms_norm(u["q"].view(T, H, d), w["q.norm"], eps)
        k = O.rms_norm(u["k"].view(T, G, d), w["k.norm"], eps)
        if m.get("rot"):
            cos, sin = O.yarn_tables(pos, m["rot"])
            q, k = O.rotate_pairs(q, cos, sin, m["rot"]["dims"]), O.rotate_pairs(k, cos, sin, m["rot"]["dims"])
        q, k, v = q.reshape(T, -1), k.reshape(T, -1), u["v"]
    if v_first is not None:
        v = (1 - 0.3) * v + 0.3 * v_first
    return q, k, v


@pytest.mark.parametrize("kind,H,G,dim,vdim,taps,rot_dims", [("attention", 6, 2, 24, 16, 1, 0), ("attention_2", 4, 2, 16, 24, 4, 16),
                                                              ("attention_2", 3, 1, 10, 7, 1, 6), ("attention_2", 3, 3, 12, 34, 5, 0),
                                                              ("attention_2", 2, 1, 136, 120, 3, 136)])
def test_attention_inputs_kernel(kind, H, G, dim, vdim, taps, rot_dims):
    """Bias, convolution across a portion's start (state) and across the sequence's start (zeros), both norms, the temperature
    at the positions where it steps, the rotation far into a sequence, the value blend; two sequences side by side."""
    g = gen(9)
    nq, nk, nv = H * dim, G * dim, G * vdim
    C = nq + nk + nv
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "q_temp": {"coef": 0.8, "every": 5}}
    if taps > 1:
        m["conv"] = taps
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": 300.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}
    w = {"q.norm": torch.randn(nq if kind == "attention" else dim, generator=g).double(), "k.norm": torch.randn(nk if kind == "attention" else dim, generator=g).double()}
    for n, c in (("q", nq), ("k", nk), ("v", nv)):
        w[n + ".b"] = torch.randn(c, generator=g).double()
        w[n + ".conv"] = torch.randn(c, max(taps, 1), generator=g).double()
    # sequence A: 3 rows at positions 0..2 (the convolution reaches before the start); sequence B: 4 rows from position 1021 on
    ya = {n: torch.randn(3, c, generator=g).double() for n, c in (("q", nq), ("k", nk), ("v", nv))}
    yb = {n: torch.randn(4, c, generator=g).double() for n, c in (("q", nq), ("k", nk), ("v", nv))}
    past_b = {n: torch.randn(max(taps - 1, 0) + 2, c, generator=g).double() for n, c in (("q", nq), ("k", nk), ("v", nv))}
    empty = {n: torch.zeros(0, c, dtype=F64) for n, c in (("q", nq), ("k", nk), ("v", nv))}
    vf = torch.randn(7, nv, generator=g).double()
    ra = _prep_reference(ya, 0, w, m, kind, 1e-5, empty, vf[:3])
    rb = _prep_reference(yb, 1021, w, m, kind, 1e-5, past_b, vf[3:])
    # the projection's output with q | k | v at column offsets 8, 8 + nq + 8, ...
    offs = [8, 8 + nq + 8, 8 + nq + 8 + nk + 8]
    y = torch.zeros(7, offs[2] + nv + 8, dtype=F64)
    for n, o, c in (("q", offs[0], nq), ("k", offs[1], nk), ("v", offs[2], nv)):
        y[:3, o:o + c], y[3:, o:o + c] = ya[n], yb[n]
    kc = torch.zeros(3, 1100, nk, device=DEV)
    vc = torch.zeros(3, 1100, nv, device=DEV)
    conv_state = None
    if taps > 1:
        conv_state = torch.zeros(3, taps - 1, C, device=DEV)
        conv_state[2] = torch.cat([past_b[n][-(taps - 1):] for n in "qkv"], 1).float()       # sequence B lives in slot 2
    q_out = torch.empty(7, nq, device=DEV)
    batch = make_batch([(0, 0, 3), (2, 1021, 4)])
    f, mag = scaled_rotary_freq(rot_dims, 300.0, m["rot"]["scaling"]) if rot_dims else (None, 1.0)
    ops.qkv_prep(y.float().to(DEV), offs, batch.meta, q_out, kc, vc, H, G, dim, vdim, 1e-5,
                 bias=torch.cat([w[n + ".b"] for n in "qkv"]).float().to(DEV) if kind == "attention_2" else None,
                 wconv=torch.cat([w[n + ".conv"] for n in "qkv"], 0).float().to(DEV) if kind == "attention_2" else None, conv_state=conv_state, taps=taps,
                 norm_mode=ops.NORM_WHOLE if kind == "attention" else ops.NORM_PER_HEAD, qnorm_w=w["q.norm"].float().to(DEV), knorm_w=w["k.norm"].float().to(DEV),
                 temp_coef=0.8 if kind == "attention" else 0.0, temp_every=5 if kind == "attention" else 0, freq=f.to(DEV) if rot_dims else None,
                 rot_dims=rot_dims, rot_mag=mag, vmix_mode=ops.VMIX_BLEND, vmix=0.3, v_first=vf.float().to(DEV))
    assert rel(q_out[:3], ra[0]) < 5e-6 and rel(q_out[3:], rb[0]) < 5e-6
    assert rel(kc[0, :3], ra[1]) < 5e-6 and rel(kc[2, 1021:1025], rb[1]) < 5e-6
    assert rel(vc[0, :3], ra[2]) < 5e-6 and rel(vc[2, 1021:1025], rb[2]) < 5e-6
    assert float(kc[1].abs().max()) == 0 and float(kc[0, 3:].abs().max()) == 0 and float(kc[2, :1021].abs().max()) == 0      # nothing else was touched
    if taps > 1:                # the state moves on: the last taps - 1 projected rows (without bias) of each sequence
        ops.conv_state_update(y.float().to(DEV), offs, nq, nv, conv_state, batch.segs, taps, nk=nk)
        full_a = torch.cat([torch.zeros(taps - 1, C, dtype=F64), torch.cat([ya[n] for n in "qkv"], 1)])
        full_b = torch.cat([torch.cat([past_b[n] for n in "qkv"], 1), torch.cat([yb[n] for n in "qkv"], 1)])
        assert rel(conv_state[0], full_a[-(taps - 1):]) < 1e-6 and rel(conv_state[2], full_b[-(taps - 1):]) < 1e-6


def test_published_values_are_the_unblended_ones():
    g = gen(10)
    y = torch.randn(5, 3 * 16, generator=g)
    kc, vc = torch.zeros(1, 8, 16, device=DEV), torch.zeros(1, 8, 16, device=DEV)
    q_out, vf = torch.empty(5, 16, device=DEV), torch.zeros(5, 16, device=DEV)
    ops.qkv_prep(y.to(DEV), [0, 16, 32], i32([(0, p) for p in range(5)]), q_out, kc, vc, 2, 2, 8, 8, 1e-5, vmix_mode=ops.VMIX_PUBLISH, vmix=0.9, v_first=vf)
    assert torch.equal(vf.cpu(), y[:, 32:]) and torch.equal(vc[0, :5].cpu(), y[:, 32:]) and torch.equal(q_out.cpu(), y[:, :16])


def test_rotation_frequencies():
    f, mag = scaled_rotary_freq(16, 1000.0, None)
    assert mag == 1.0 and rel(f, 1000.0 ** (-torch.arange(8).double() / 8)) < 1e-15
    rot = {"dims": 34, "base": 50.0, "scaling": {"factor": 16.0, "original": 32, "fast": 1000.0, "slow": 500.0}}
    f, mag = scaled_rotary_freq(34, 50.0, rot["scaling"])
    cos, sin = O.yarn_tables(torch.tensor([1]), rot)
    assert rel(torch.cos(f) * mag, cos[0]) < 1e-14 and rel(torch.sin(f) * mag, sin[0]) < 1e-14
    plain = 50.0 ** (-torch.arange(17).double() / 17)
    assert f[0] == 1.0 and rel(f[1:], plain[1:] / 16.0) < 1e-14 and abs(mag - (0.1 * math.log(16.0) + 1)) < 1e-15     # every pair but the first is interpolated


# ------------------------------------------------------------------------------------------------ mixers alone
def _mixer_weights(shapes, seed):
    g = gen(seed)
    out = {}
    for k, shp in shapes.items():
        if k.endswith(".conv"):
            out[k] = bf(torch.randn(shp, generator=g) * 0.5)
        elif len(shp) == 2:
            out[k] = bf(torch.randn(shp, generator=g) * shp[1] ** -0.5)
        elif len(shp) == 0:
            out[k] = bf(torch.tensor(0.4))
        else:
            out[k] = bf(torch.randn(shp, generator=g) * 0.5 + (1.0 if k.endswith("norm") else 0.0))
    return out


def run_mixer(mixer, h, cuts, v_first=None, slot=1, n_slots=3):
    slots = SlotState(n_slots, h.shape[0], DEV)
    state = mixer.new_state(slots)
    outs, at = [], 0
    for c in cuts:
        batch = make_batch([(slot, at, c)])
        if v_first is not None:
            batch.scratch["v_first"] = v_first[at:at + c].float().to(DEV).contiguous()
        outs.append(mixer(h[at:at + c].to(device=DEV, dtype=mixer.dtype).contiguous(), batch, state).float().cpu())
        at += c
    assert at == h.shape[0]
    return torch.cat(outs)


@pytest.mark.parametrize("H,G,dim,vdim,W", [(6, 2, 24, 16, 64), (1, 1, 12, 10, 44), (9, 3, 72, 40, 96)])
def test_attention_mixer_alone(H, G, dim, vdim, W):
    w = _mixer_weights({"q": (H * dim, W), "k": (G * dim, W), "v": (G * vdim, W), "q.norm": (H * dim,), "k.norm": (G * dim,), "vmix": (), "sink": (H,),
                        "g": (H, W), "o": (W, H * vdim)}, 11)
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 * 3, "q_temp": {"coef": 0.5, "every": 7}, "v_mix": True}
    h = bf(torch.randn(60, W, generator=gen(12)))
    vf = torch.randn(60, G * vdim, generator=gen(13)).double()
    want = O.attention_mixer(h.double(), torch.arange(60), {k: v.double() for k, v in w.items()}, "", m, 1e-5, {}, {"v_first": vf}, 1)
    mx = SinkAttentionMixer(w, H, G, dim, vdim, m["scale"], 1e-5, F32, DEV, norm="whole", q_temp=(0.5, 7), slopes=distance_slopes(H), gate="head", v_mix="blend")
    for label, cuts in CUTS.items():
        assert rel(run_mixer(mx, h, cuts, vf), want) < 5e-5, label


@pytest.mark.parametrize("H,G,dim,vdim,taps,rot_dims,W", [(4, 2, 16, 24, 4, 16, 64), (3, 1, 10, 7, 1, 6, 44), (3, 3, 12, 34, 5, 0, 44), (2, 1, 136, 120, 3, 136, 96)])
def test_attention_2_mixer_alone(H, G, dim, vdim, taps, rot_dims, W):
    shapes = {"q": (H * dim, W), "k": (G * dim, W), "v": (G * vdim, W), "q.b": (H * dim,), "k.b": (G * dim,), "v.b": (G * vdim,), "q.norm": (dim,),
              "k.norm": (dim,), "sink": (H,), "g": (H * vdim, W), "o": (W, H * vdim)}
    if taps > 1:
        shapes.update({"q.conv": (H * dim, taps), "k.conv": (G * dim, taps), "v.conv": (G * vdim, taps)})
    w = _mixer_weights(shapes, 14)
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 * 3}
    if taps > 1:
        m["conv"] = taps
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    h = bf(torch.randn(60, W, generator=gen(15)))
    shared = {}
    want = O.attention_2_mixer(h.double(), torch.arange(60), {k: v.double() for k, v in w.items()}, "", m, 1e-5, {}, shared, 0)
    ride = bf(torch.randn(W, W, generator=gen(16)) * W ** -0.5)
    mx = SinkAttentionMixer(w, H, G, dim, vdim, m["scale"], 1e-5, F32, DEV, norm="head", biases=True, taps=taps if taps > 1 else None, rot=m.get("rot"), gate="channel",
                            ride_along=[ride])
    for label, cuts in CUTS.items():             # "twos" and "token by token" are shorter than the convolution's state
        assert rel(run_mixer(mx, h, cuts), want) < 5e-5, label
    extras = []
    mx(h.to(DEV), make_batch([(0, 0, 60)]), mx.new_state(SlotState(1, 60, DEV)), extras)
    assert rel(extras[0], h.double() @ ride.double().T) < 1e-5


def test_two_sequences_in_one_batch_keep_their_own_state():
    """Portions of two sequences side by side in one step: the convolution must not read across the border, and each
    sequence attends to its own cache."""
    H, G, dim, vdim, taps, W = 4, 2, 16, 24, 4, 64
    w = _mixer_weights({"q": (H * dim, W), "k": (G * dim, W), "v": (G * vdim, W), "q.b": (H * dim,), "k.b": (G * dim,), "v.b": (G * vdim,), "q.norm": (dim,),
                        "k.norm": (dim,), "sink": (H,), "g": (H * vdim, W), "o": (W, H * vdim), "q.conv": (H * dim, taps), "k.conv": (G * dim, taps),
                        "v.conv": (G * vdim, taps)}, 17)
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": 0.4, "conv": taps, "rot": {"dims": 8, "base": 100.0}}
    ha, hb = bf(torch.randn(20, W, generator=gen(18))), bf(torch.randn(9, W, generator=gen(19)))
    wd = {k: v.double() for k, v in w.items()}
    want_a = O.attention_2_mixer(ha.double(), torch.arange(20), wd, "", m, 1e-5, {}, {}, 0)
    want_b = O.attention_2_mixer(hb.double(), torch.arange(9), wd, "", m, 1e-5, {}, {}, 0)
    mx = SinkAttentionMixer(w, H, G, dim, vdim, 0.4, 1e-5, F32, DEV, norm="head", biases=True, taps=taps, rot=m["rot"], gate="channel")
    state = mx.new_state(SlotState(3, 32, DEV))
    got_a, got_b = [], []
    ia = ib = 0
    for na, nb in [(12, 1), (1, 2), (7, 6)]:                          # tokens of a, of b per step; b sits in the rows right after a
        rows = torch.cat([ha[ia:ia + na], hb[ib:ib + nb]]).to(DEV)
        out = mx(rows, make_batch([(2, ia, na), (0, ib, nb)]), state).cpu()
        got_a.append(out[:na]); got_b.append(out[na:])
        ia += na; ib += nb
    assert rel(torch.cat(got_a), want_a) < 5e-5 and rel(torch.cat(got_b), want_b) < 5e-5


# ------------------------------------------------------------------------------------------------ the model
def build(name, dtype, seed=11, std_scale=1.0):
    cfg = CASES[name] if isinstance(name, str) else name
    w = O.random_weights(cfg, seed, std_scale)
    m = BizetarForCausalLM(BizetarConfig.from_dict(copy.deepcopy(cfg)), DEV, dtype).load_weights(lambda n: w[n])
    return cfg, w, m


def oracle_logits(cfg, w, toks, trace=None):
    with torch.no_grad():
        return O.forward(toks, w, cfg, O.new_state(cfg), trace)


def toks_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=gen(seed)).tolist()


def err(got, want, reduce="max"):
    """The measure a serving check would use: rms over the vocabulary of the centred difference, relative to the logits' rms."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    e = d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    return float(e.max() if reduce == "max" else e.mean())


@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompt_fp32_and_every_layer(name):
    cfg, w, m = build(name, F32)
    toks = toks_for(cfg, 45, 1)
    trace_o, trace_m = [], []
    want = oracle_logits(cfg, w, toks, trace_o)
    got = Engine(m, 64, 2).step([{"id": 0, "tokens": toks, "want": list(range(45))}], trace=trace_m)
    assert len(trace_m) == len(trace_o) == len(cfg["layers"])
    for r, (a, b) in enumerate(zip(trace_m, trace_o)):
        assert rel(a, b) < 2e-4, f"what layer {r} hands on"
    assert err(got, want) < 2e-4


@pytest.mark.parametrize("name", sorted(CASES))
def test_bf16_model_stays_within_rounding(name):
    cfg, w, m = build(name, BF16)
    toks = toks_for(cfg, 70, 2)
    got = Engine(m, 80, 1).step([{"id": 0, "tokens": toks, "want": list(range(70))}])
    # bf16 rounding of the projections through a few narrow layers: a few percent of the logits' rms, where a wrong slice,
    # state or constant shows as an error of order 1.  (A routed layer may send a token to another expert when two scores are
    # within rounding of each other; the mean shows that this is rare.)
    assert err(got, oracle_logits(cfg, w, toks), "mean") < 0.08


@pytest.mark.parametrize("name,dtype", [("even", F32), ("odd", F32), ("wide", F32), ("even", BF16)])
def test_portions_and_decoding_equal_the_whole_prompt(name, dtype):
    cfg, w, m = build(name, dtype)
    n = 75
    toks = toks_for(cfg, n, 3)
    eng = Engine(m, 100, 2)
    whole = eng.step([{"id": "w", "tokens": toks, "want": list(range(n))}], end=["w"])
    schedules = {"token by token": [1] * n, "twos": [2] * 37 + [1], "ragged": [31, 1, 1, 2, 30, 3, 7], "stage edges": [32, 32, 8, 1, 1, 1],
                 "prompt then decode": [n - 33] + [1] * 33}
    for label, cuts in schedules.items():
        assert sum(cuts) == n
        outs, at = [], 0
        for c in cuts:
            outs.append(eng.step([{"id": label, "tokens": toks[at:at + c], "want": list(range(c))}]))
            at += c
        eng.step([], end=[label])
        if dtype == F32:
            assert err(torch.cat(outs), whole.double().cpu()) < 1e-4, label
        else:       # bf16: GEMM tiles differ with the row count, so portions differ by rounding
            assert err(torch.cat(outs), whole.double().cpu(), "mean") < 0.08, label
    if dtype == F32:
        assert err(whole, oracle_logits(cfg, w, toks)) < 2e-4


def test_unequal_requests_in_one_step_equal_each_alone():
    cfg, w, m = build("even", F32)
    eng = Engine(m, 64, 4)
    prompts = {"a": toks_for(cfg, 40, 4), "b": toks_for(cfg, 3, 5), "c": toks_for(cfg, 17, 6)}
    alone = {k: eng.step([{"id": k, "tokens": t, "want": list(range(len(t)))}], end=[k]) for k, t in prompts.items()}
    got = {k: [] for k in prompts}
    plan = [{"a": 25, "b": 3, "c": 1}, {"a": 1, "c": 10}, {"a": 14, "c": 6}]
    at = {k: 0 for k in prompts}
    for step in plan:
        entries = [{"id": k, "tokens": prompts[k][at[k]:at[k] + n], "want": list(range(n))} for k, n in step.items()]
        out = eng.step(entries)
        o = 0
        for k, n in step.items():
            got[k].append(out[o:o + n])
            o += n
            at[k] += n
    for k in prompts:
        assert at[k] == len(prompts[k])
        assert err(torch.cat(got[k]), alone[k].double().cpu()) < 1e-4, k
        assert err(alone[k], oracle_logits(cfg, w, prompts[k])) < 2e-4


def test_freed_slots_are_reused_clean_and_passes_cut_long_entries():
    cfg, w, m = build("odd", F32)
    eng = Engine(m, 48, 2, max_rows=16)                              # a 40-token entry runs as passes of 16, 16 and 8 rows
    t1, t2, t3 = toks_for(cfg, 40, 7), toks_for(cfg, 33, 8), toks_for(cfg, 9, 9)
    a = eng.step([{"id": 1, "tokens": t1, "want": [0, 15, 16, 39]}], end=[1])
    assert err(a, oracle_logits(cfg, w, t1)[[0, 15, 16, 39]]) < 2e-4
    b = eng.step([{"id": 2, "tokens": t2, "want": [32]}, {"id": 3, "tokens": t3, "want": [8]}], end=[2])       # slot 0 again
    assert err(b[:1], oracle_logits(cfg, w, t2)[[32]]) < 2e-4 and err(b[1:], oracle_logits(cfg, w, t3)[[8]]) < 2e-4
    c = eng.step([{"id": 4, "tokens": t1[:5], "want": [4]}], end=[3, 4])                                    # and once more
    assert err(c, oracle_logits(cfg, w, t1[:5])[[4]]) < 2e-4
    assert eng.slots.live_tokens == 0


@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_a_far_token_still_moves_the_logits_through_the_model(kind):
    """One attention layer with sharp scores: among the tokens about 350 positions back, the one whose replacement moves the
    last position's logits most (found with the oracle) is replaced; the model follows the oracle with and without the
    replacement -- in a whole prompt, when the tail is decoded token by token, and in portions."""
    layer = attention(2, 1, 16, 16, scale=2.0, q_temp=(0.3, 64)) if kind == "attention" else attention_2(2, 1, 16, 16, conv=2, rot_dims=4, scale=2.0)
    cfg = config([layer], vocab=50, width=32)
    _, w, m = build(cfg, F32, seed=12)
    n = 400
    toks = toks_for(cfg, n, 10)
    base = oracle_logits(cfg, w, toks)[-1:]
    best = (0.0, None, None)
    for far in range(n - 366, n - 346):
        variant = list(toks)
        variant[far] = (variant[far] + 7) % cfg["vocab"]
        moved = oracle_logits(cfg, w, variant)[-1:]
        best = max(best, (err(moved, base), variant, moved), key=lambda t: t[0])
    effect, variant, moved = best
    assert effect > 5e-4
    eng = Engine(m, n, 1)
    for seq, want in ((toks, base), (variant, moved)):
        assert err(eng.step([{"id": 0, "tokens": seq, "want": [n - 1]}], end=[0]), want) < 1e-4
        eng.step([{"id": 1, "tokens": seq[:n - 40], "want": []}])
        for t in seq[n - 40:-1]:
            eng.step([{"id": 1, "tokens": [t], "want": []}])
        assert err(eng.step([{"id": 1, "tokens": seq[-1:], "want": [0]}], end=[1]), want) < 1e-4
        at = 0
        for c in [100, 2, 61, 130, 3, 104]:
            out = eng.step([{"id": 2, "tokens": seq[at:at + c], "want": [c - 1]}])
            at += c
        eng.step([], end=[2])
        assert at == n and err(out, want) < 1e-4


def test_long_decoding_keeps_the_state_exact():
    """260 decoded tokens: the history passes the attention's stage and key-range edges and the query temperature steps
    several times (every 7 positions in one layer, every position in another)."""
    cfg, w, m = build("even", F32)
    n = 264
    toks = toks_for(cfg, n, 13)
    eng = Engine(m, n, 1)
    eng.step([{"id": 0, "tokens": toks[:4], "want": []}])
    outs = [eng.step([{"id": 0, "tokens": [t], "want": [0]}]) for t in toks[4:]]
    assert err(torch.cat(outs), oracle_logits(cfg, w, toks)[4:]) < 2e-4


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_graphed_decode_passes_equal_eager_ones_bit_for_bit(dtype):
    cfg, w, m = build("even", dtype)
    a, b, c = toks_for(cfg, 129, 40), toks_for(cfg, 60, 41), toks_for(cfg, 30, 42)

    def play(graphs):
        eng = Engine(m, 130, 2, graphs=graphs)
        outs = [eng.step([{"id": "a", "tokens": a[:50], "want": [49]}, {"id": "b", "tokens": b[:3], "want": [2]}])]
        for i in range(50):
            want = [] if i % 7 == 3 else [0]
            o = eng.step([{"id": "a", "tokens": [a[50 + i]], "want": want}, {"id": "b", "tokens": [b[3 + i]], "want": want}])
            assert (o is None) == (not want)
            if o is not None:
                outs.append(o)
        eng.step([], end=["b"])
        outs.append(eng.step([{"id": "c", "tokens": c[:1], "want": [0]}]))           # b's slot again; alone in its pass
        for i in range(1, 30):
            outs.append(eng.step([{"id": "c", "tokens": [c[i]], "want": [0]}, {"id": "a", "tokens": [a[99 + i]], "want": [0]}]))
        return torch.cat(outs), eng

    eager, _ = play(False)
    graphed, eng = play(True)
    assert sum(g.graph is not None for g in eng._step_graphs.values()) >= 2           # several shapes were captured and replayed
    assert torch.equal(eager, graphed)
    if dtype == F32:
        la, lc = oracle_logits(cfg, w, a), oracle_logits(cfg, w, c)
        assert err(graphed[-2:-1], lc[29:30]) < 2e-4 and err(graphed[-1:], la[128:129]) < 2e-4


def test_first_tokens_and_single_token_prompts():
    cfg, w, m = build("wide", F32)
    eng = Engine(m, 8, 3)
    for seed in (20, 21, 22):
        t = toks_for(cfg, 1, seed)
        assert err(eng.step([{"id": seed, "tokens": t, "want": [0]}]), oracle_logits(cfg, w, t)) < 2e-4
    t = toks_for(cfg, 5, 23)
    eng.step([], end=[20, 21, 22])
    got = torch.cat([eng.step([{"id": "s", "tokens": [x], "want": [0]}]) for x in t])
    assert err(got, oracle_logits(cfg, w, t)) < 2e-4


def test_layers_without_options_and_equal_sizes():
    """What a configuration may leave out or make equal: no temperature, no convolution, no rotation, no value mixing, no
    feed-forward, one head, heads as wide as the model, a router that takes every output."""
    cfg = config([attention(1, 1, 32, 32, q_temp=None), attention_2(2, 2, 16, 16, conv=None, rot_dims=None, mlp=moe(2, 3, 8, identity=1)),
                  attention_2(4, 1, 8, 8, conv=1, rot_dims=2, scaling=None, v_mix=True, mlp=dense(32))], vocab=32, width=32)
    _, w, m = build(cfg, F32, seed=5)
    toks = toks_for(cfg, 40, 24)
    eng = Engine(m, 40, 1)
    got = torch.cat([eng.step([{"id": 0, "tokens": toks[:17], "want": list(range(17))}]), eng.step([{"id": 0, "tokens": toks[17:], "want": list(range(23))}])])
    assert err(got, oracle_logits(cfg, w, toks)) < 2e-4


def _write_checkpoint(tmp_path, cfg, seed):
    w = O.random_weights(cfg, seed)
    d = tmp_path / "ckpt"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: v.to(BF16) for k, v in w.items()})
    return str(d), w


def test_greedy_generation_through_generate_and_from_pretrained(tmp_path):
    cfg = CASES["even"]
    ckpt, w = _write_checkpoint(tmp_path, cfg, 14)
    m = registry.load_model(ckpt, device=DEV, dtype=F32)
    assert isinstance(m, BizetarForCausalLM)
    prompts = torch.tensor([toks_for(cfg, 12, 30), toks_for(cfg, 12, 31)])
    new = 10
    out = m.generate(prompts, max_new_tokens=new)
    out_chunked = m.generate(prompts, max_new_tokens=new, chunk=5)
    assert out.shape == (2, 12 + new) and torch.equal(out[:, :12], prompts)
    for b in range(2):      # teacher-forced against the oracle: every greedy pick is its argmax wherever the top-2 margin is not a near-tie
        lg = oracle_logits(cfg, w, out[b].tolist())
        for t in range(new):
            top = lg[11 + t].topk(2)
            if float(top.values[0] - top.values[1]) > 1e-3:
                assert int(out[b, 12 + t]) == int(top.indices[0]), (b, t)
                assert int(out_chunked[b, 12 + t]) == int(out[b, 12 + t])


def test_trace_runner_and_command_line_as_a_user_calls_them(tmp_path):
    """The two programs a user runs, as child processes on a small checkpoint: the trace runner in both dtypes against the
    oracle, and run.py's generation summary."""
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CASES["even"]
    ckpt, w = _write_checkpoint(tmp_path, cfg, 15)
    a, b = toks_for(cfg, 41, 50), toks_for(cfg, 6, 51)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},              # nothing wanted: no file
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:40], "want": [7]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[40:41], "want": [0]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]}]               # a's slot, handed out again
    la, lb = oracle_logits(cfg, w, a), oracle_logits(cfg, w, b)
    want = {0: la[[0, 29]], 2: la[[39]], 3: la[[40]], 4: lb[[5]]}
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 0.2)):
        out = tmp_path / ("out_" + dtype)
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", ckpt, "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == ["done %d" % s["step"] for s in steps]
        assert sorted(os.listdir(out)) == ["%d.f32" % k for k in sorted(want)]
        for k, ref in want.items():
            got = torch.from_numpy(np.fromfile(out / ("%d.f32" % k), dtype="<f4").reshape(-1, cfg["vocab"]).copy())
            assert got.shape == ref.shape and err(got, ref) < tol, (dtype, k)
    p = subprocess.run([sys.executable, os.path.join(root, "run.py"), "-m", ckpt, "--dtype", "float32", "--input-tokens", "9", "--max-new-tokens", "5",
                        "--batch-size", "2", "--num-iter", "2", "--num-warmup", "1"], text=True, capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "Inference latency:" in p.stdout and "Throughput:" in p.stdout and "[5, 5]" in p.stdout
