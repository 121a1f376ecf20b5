"""GPU checks of the Zatusun path against the plain float64 oracle (tests/zatusun_oracle.py): every new kernel and all three
mixers alone, then the model through the step engine -- whole prompts, token-by-token decoding, portions down to two tokens,
unequal requests in one step, slots that are freed and reused, a key far back among hundreds, keys just inside and just outside
a chunk (in prompts and in decoding), keys at the edges of the attention kernels' own tiles (32 cached positions per stage, 64 per
key range), the first tokens, long decoding, sizes that are equal or 1, greedy generation through generate(), the trace runner and
the command line."""
import copy
import json
import os

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import ops, registry
from lia_b200.checkpoint import write_safetensors
from lia_b200.engine import Engine
from lia_b200.modeling_zatusun import ZatusunConfig, ZatusunForCausalLM
from lia_b200.seq_layers import (DifferentialAttentionMixer, ForgetGateLinearAttentionMixer, LatentAttentionMixer, MoEFeedForward, StepBatch)
from lia_b200.seq_state import SlotState

import zatusun_oracle as O
from zatusun_cases import CASES, config, differential, hgrn2, latent, moe

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
def test_embedding_with_scale_and_learned_positions(W):
    g = gen(0)
    table, pos = bf(torch.randn(50, W, generator=g)), bf(torch.randn(40, W, generator=g))
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int64)
    batch = make_batch([(2, 37, 3), (0, 0, 2)])
    want = table[ids].double() * 2.75 + pos[[37, 38, 39, 0, 1]].double()
    for dt in (F32, BF16):
        x = torch.empty(5, W, device=DEV)
        cat = torch.empty(5, 2 * W, dtype=dt, device=DEV)
        ops.embed_scale_pos(ids.to(DEV), table.to(DEV, dt), pos.to(DEV, dt), 2.75, batch.meta, x, cat)
        assert rel(x, want) < 2e-7                                    # the stream is fp32 whatever the tables are
        assert torch.equal(cat[:, :W], cat[:, W:]) and torch.equal(cat[:, :W].cpu(), x.cpu().to(dt))
    x2 = torch.empty(5, W, device=DEV)
    ops.embed_scale_pos(ids.to(DEV), table.to(DEV), None, 0.5, batch.meta, x2)
    assert rel(x2, table[ids].double() * 0.5) < 2e-7


@pytest.mark.parametrize("W", [44, 256, 1000])
def test_residual_update_with_the_next_norm(W):
    g = gen(1)
    rows = 9
    x0, y = torch.randn(rows, W, generator=g) * 4.0, torch.randn(rows, W, generator=g)
    bias, w = torch.randn(W, generator=g), 1.0 + 0.3 * torch.randn(W, generator=g)
    for dt, tol in ((F32, 2e-6), (BF16, 5e-3)):
        yy = y.to(dt)
        x = x0.clone().to(DEV)
        h = torch.empty(rows, W, dtype=dt, device=DEV)
        ops.residual_norm(x, yy.to(DEV), w.to(DEV), h, 1e-5)
        s = x0.double() + yy.double()
        assert rel(x, s) < 2e-7 and rel(h, O.rms_norm(s, w.double(), 1e-5)) < tol
        # the stream is replaced by y + bias; the row goes out unnormed into the left half of a wider buffer
        x = x0.clone().to(DEV)
        wide = torch.full((rows, 2 * W), 7.0, dtype=dt, device=DEV)
        ops.residual_norm(x, yy.to(DEV), None, wide[:, :W], 1e-5, replace=True, bias=bias.to(DEV))
        s = yy.double() + bias.double()
        assert rel(x, s) < 2e-7 and torch.equal(wide[:, :W].cpu(), x.cpu().to(dt)) and bool((wide[:, W:] == 7.0).all())
        # the norm alone: the stream stays as it is
        x = x0.clone().to(DEV)
        ops.residual_norm(x, None, w.to(DEV), h, 1e-5)
        assert torch.equal(x.cpu(), x0) and rel(h, O.rms_norm(x0.double(), w.double(), 1e-5)) < tol
        # the last update of a model: nothing reads a norm
        ops.residual_norm(x, yy.to(DEV), None, None, 1e-5)
        assert rel(x, x0.double() + yy.double()) < 2e-7


def test_row_norm_gate_product_and_soft_cap():
    g = gen(2)
    z = torch.randn(70, 50, generator=g) * 3.0
    w = torch.randn(37, generator=g)
    gate = torch.randn(70, 48, generator=g) * 2.0
    for dt, tol in ((F32, 2e-6), (BF16, 5e-3)):
        zz = z.to(dt)
        out = torch.empty(70, 37, dtype=dt, device=DEV)
        ops.rms_norm_rows(zz.to(DEV)[:, 5:42], w.to(DEV), out, 1e-6)              # a column slice of a wider buffer
        assert rel(out, O.rms_norm(zz.double()[:, 5:42], w.double(), 1e-6)) < tol
        gg = gate.to(dt)
        prod = torch.empty(70, 37, dtype=dt, device=DEV)
        ops.sigmoid_mul(z.to(DEV)[:, 5:42], gg.to(DEV)[:, 11:], prod)             # fp32 values, gate in the activations' type
        assert rel(prod, z.double()[:, 5:42] * torch.sigmoid(gg.double()[:, 11:])) < tol
    x = (torch.randn(33, 61, generator=g) * 30.0).to(DEV)
    want = 12.5 * torch.tanh(x.double().cpu() / 12.5)
    assert rel(ops.softcap(x, 12.5), want) < 1e-6 and float(x.abs().max()) <= 12.5


@pytest.mark.parametrize("M,dtype,E,top", [(5, F32, 6, 2), (5, BF16, 6, 2), (90, F32, 5, 3), (300, BF16, 6, 2), (300, F32, 4, 4), (7, F32, 1, 1)])
def test_clamped_gated_experts_in_every_form(M, dtype, E, top):
    """Few pairs (one warp per output), the grouped launch, and (bf16, many pairs) the tensor-core form; expert 1 gets no token;
    the limit is low enough to clamp both factors often; the weights are a softmax restricted to the selected experts' logits."""
    g = gen(3)
    W, ff, limit = 64, 24, 0.6
    router = bf(torch.randn(E, W, generator=g) * 4.0 * W ** -0.5)
    if E > top:
        router[1] = 0.0
        router[1, 0] = -30.0                                           # h[:, 0] > 0 below: expert 1 never wins
    experts = [{"gate": bf(torch.randn(ff, W, generator=g) * 2.0 * W ** -0.5), "up": bf(torch.randn(ff, W, generator=g) * 2.0 * W ** -0.5),
                "down": bf(torch.randn(W, ff, generator=g) * ff ** -0.5)} for _ in range(E)]
    h = bf(torch.randn(M, W, generator=g))
    h[:, 0] = h[:, 0].abs() + 0.5
    w = {"router": router.double()}
    for e, ex in enumerate(experts):
        w.update({f"e{e}.{k}": v.double() for k, v in ex.items()})
    want = O.moe(h.double(), w, "", {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}})
    ff_ = MoEFeedForward(router, experts, top, ff, ops.ACT_CLAMPED_SWISH, None, dtype, DEV, renorm=True, act_params=(limit, 1.702))
    got = ff_(h.to(DEV, dtype))
    assert got.dtype == F32 and rel(got, want) < (2e-5 if dtype == F32 else 2e-2)
    g_raw = h.double() @ experts[0]["gate"].double().T
    assert bool((g_raw > limit).any()) and bool(((h.double() @ experts[0]["up"].double().T).abs() > limit).any())       # the clamps were at work


@pytest.mark.parametrize("H,dim,vdim", [(1, 12, 10), (2, 24, 16), (2, 72, 136), (3, 128, 40)])
def test_forget_gate_recurrence_kernel(H, dim, vdim):
    g = gen(4)
    n = 70
    q, v = torch.randn(n, H * dim, generator=g), torch.randn(n, H * vdim, generator=g)
    f = torch.rand(n, H * dim, generator=g)
    f.view(n, H, dim)[:, :, 0] = 1.0                                   # a channel that never forgets (and so never writes)
    f.view(n, H, dim)[:, :, 1] = 0.0                                   # one that keeps only the current token
    S0 = torch.randn(H, dim, vdim, generator=g)
    S, want = S0.double().clone(), torch.zeros(n, H, vdim, dtype=F64)
    for t in range(n):
        ft = f[t].double().view(H, dim, 1)
        S = ft * S + (1.0 - ft) * v[t].double().view(H, 1, vdim)
        want[t] = torch.einsum("hdv,hd->hv", S, q[t].double().view(H, dim))
    qfv = torch.cat([q, f, v], 1).to(DEV)
    nq = H * dim
    for cuts in ([n], [1] * n, [33, 2, 35]):
        state = torch.zeros(3, H, vdim, dim, device=DEV)
        state[1] = S0.transpose(1, 2).to(DEV)
        o = torch.empty(n, H * vdim, device=DEV)
        at = 0
        for c in cuts:
            rows = qfv[at:at + c]
            ops.forget_scan(rows[:, :nq], rows[:, nq:2 * nq], rows[:, 2 * nq:], state, i32([(1, at, 0, c)]), H, dim, vdim, o[at:at + c])
            at += c
        assert rel(o, want.view(n, -1)) < 2e-5, cuts
        assert rel(state[1].transpose(1, 2), S) < 2e-5 and not state[0].any() and not state[2].any()
        assert torch.equal(state[1, :, :, 0].cpu(), S0[:, 0, :])        # the channel that never forgets holds its row bit for bit


def test_forget_gates_from_the_projection():
    g = gen(5)
    M, nq, nv = 40, 36, 20
    y = torch.randn(M, 8 + nq + 4 + nq + nv, generator=g) * 2.0
    fb, low = torch.randn(nq, generator=g), torch.rand(nq, generator=g)
    offs = (8, 8 + nq + 4, 8 + nq + 4 + nq)
    for dt, tol in ((F32, 2e-6), (BF16, 2e-6)):                       # bf16 inputs, but everything the gate computes is fp32
        yy = y.to(dt)
        out = torch.empty(M, 2 * nq + nv, device=DEV)
        ops.forget_gate_prep(yy.to(DEV), offs, fb.to(DEV), low.to(DEV), out, nq, nv)
        yd = yy.double()
        want = torch.cat([O.silu(yd[:, 8:8 + nq]), low.double() + (1 - low.double()) * torch.sigmoid(yd[:, offs[1]:offs[1] + nq] + fb.double()), yd[:, offs[2]:]], 1)
        assert rel(out, want) < tol
        fgate = out[:, nq:2 * nq].cpu()
        assert bool((fgate >= low).all()) and bool((fgate <= 1.0).all())


def _maps_reference(q, k, v, pos0, H2, G2, dim, vdim, scale, chunk):
    """q [T, H2*dim] for positions pos0 .., k [N, G2*dim], v [N, (G2/2)*vdim]: every query head over its key head and the value
    head that pairs of key heads share, under the chunked mask."""
    T, N = q.shape[0], k.shape[0]
    mask = O.visible(pos0, T, chunk)[:, :N]
    out = torch.zeros(T, H2, vdim, dtype=F64)
    rep = H2 // G2
    for h in range(H2):
        kh = h // rep
        s = q.view(T, H2, dim)[:, h].double() @ k.view(N, G2, dim)[:, kh].double().T * scale
        out[:, h] = O.masked_softmax(s, mask) @ v.view(N, G2 // 2, vdim)[:, kh // 2].double()
    return out.view(T, -1)


@pytest.mark.parametrize("H2,G2,dim,vdim,chunk", [(8, 4, 16, 8, 11), (6, 6, 10, 34, 5), (12, 4, 40, 72, 40), (2, 2, 6, 3, 64), (4, 2, 24, 136, 33)])
def test_attention_kernel_with_chunks_and_shared_value_heads(H2, G2, dim, vdim, chunk):
    g = gen(6)
    n = 150
    for dt, tol in ((F32, 2e-5), (BF16, 2e-5)):                       # bf16 caches hold the same numbers: the output is fp32 either way
        k, v = bf(torch.randn(n, G2 * dim, generator=g)), bf(torch.randn(n, (G2 // 2) * vdim, generator=g))
        q = torch.randn(n, H2 * dim, generator=g)
        kc = torch.zeros(2, n, G2 * dim, dtype=dt, device=DEV)
        vc = torch.zeros(2, n, (G2 // 2) * vdim, dtype=dt, device=DEV)
        kc[1], vc[1] = k.to(DEV, dt), v.to(DEV, dt)
        want = _maps_reference(q, k, v, 0, H2, G2, dim, vdim, 0.3, chunk)
        # a prompt, then portions, then single rows whose keys are split over several blocks
        for cuts in ([n], [64, 2, 31, 53], [1] * n):
            out = torch.empty(n, H2 * vdim, device=DEV)
            at = 0
            for c in cuts:
                b = make_batch([(1, at, c)])
                ops.window_attn(q[at:at + c].to(DEV), kc, vc, b.meta, None, out[at:at + c], H2, G2, dim, vdim, 0, 0.3, 0.0, nseg=1, max_ctx=at + c,
                                chunk=chunk, v_div=2)
                at += c
            assert rel(out, want) < tol, (dt, cuts[:3])


def test_a_key_just_inside_the_chunk_takes_all_the_weight_and_just_outside_none():
    """One key is made to score far above the others for every query.  Queries of its own chunk that come after it return its
    value; the first query of the next chunk does not see it at all -- in a prompt and row by row."""
    g = gen(7)
    H2, G2, dim, vdim, chunk, n = 4, 2, 16, 8, 37, 140
    star = 70                                                         # chunk [37, 74): positions 70 .. 73 see it, 74 is the next chunk's first
    k, v = bf(torch.randn(n, G2 * dim, generator=g) * 0.1), bf(torch.randn(n, vdim, generator=g))
    q = torch.randn(n, H2 * dim, generator=g) * 0.1
    k.view(n, G2, dim)[star, :, 0] = 8.0
    q.view(n, H2, dim)[:, :, 0] = 8.0
    kc, vc = k.to(DEV).unsqueeze(0).contiguous(), v.to(DEV).unsqueeze(0).contiguous()
    want = _maps_reference(q, k, v, 0, H2, G2, dim, vdim, 1.0, chunk)
    for cuts in ([n], [1] * n, [72, 2, 66]):
        out = torch.empty(n, H2 * vdim, device=DEV)
        at = 0
        for c in cuts:
            b = make_batch([(0, at, c)])
            ops.window_attn(q[at:at + c].to(DEV), kc, vc, b.meta, None, out[at:at + c], H2, G2, dim, vdim, 0, 1.0, 0.0, nseg=1, max_ctx=at + c, chunk=chunk, v_div=2)
            at += c
        assert rel(out, want) < 2e-5
        o = out.view(n, H2, vdim).cpu()
        for p in (70, 71, 73):
            assert rel(o[p, 0], v[star]) < 1e-6                        # all the weight on the marked key
        assert rel(o[74, 0], v[74]) < 1e-6                             # the next chunk's first position sees only itself
        assert rel(o[69, 0], v[star]) > 0.1 and rel(o[75, 0], v[star]) > 0.1


def test_difference_of_two_maps_and_its_norm():
    g = gen(8)
    M, H, G, vdim = 21, 6, 2, 34
    a = torch.randn(M, G, 2, H // G, vdim, generator=g)
    lam, diff = 0.73, 0.35
    want = O.rms_div(a[:, :, 0].double() - lam * a[:, :, 1].double(), 1e-5).reshape(M, H * vdim) * (1 - diff)
    for dt, tol in ((F32, 2e-6), (BF16, 5e-3)):
        out = torch.empty(M, H * vdim, dtype=dt, device=DEV)
        ops.diff_combine(a.to(DEV).view(M, -1), out, H, G, vdim, lam, 1 - diff, 1e-5)
        assert rel(out, want) < tol


# ------------------------------------------------------------------------------------------------ mixers alone
def _weights(shapes, seed, scale=1.0):
    g = gen(seed)
    w = {}
    for k, shp in shapes.items():
        if k == "lower":
            t = 0.95 * torch.rand(shp, generator=g)
        elif len(shp) == 2:
            t = torch.randn(shp, generator=g) * scale * shp[1] ** -0.5
        elif k.endswith("norm"):
            t = 1.0 + 0.2 * torch.randn(shp, generator=g)
        else:
            t = 0.4 * torch.randn(shp, generator=g)
        w[k] = bf(t)
    return w


def run_mixer(mixer, h, cuts, slot=1, n_slots=3):
    state = mixer.new_state(SlotState(n_slots, h.shape[0], DEV))
    outs, at = [], 0
    for c in cuts:
        outs.append(mixer(h[at:at + c].to(DEV), make_batch([(slot, at, c)]), state).float().cpu())
        at += c
    return torch.cat(outs)


@pytest.mark.parametrize("H,dim,rot,vdim,rank,qr,W", [(4, 16, 8, 24, 32, 24, 64), (3, 10, 6, 7, 20, 9, 44), (9, 24, 16, 40, 264, 48, 96)])
def test_latent_attention_mixer_alone(H, dim, rot, vdim, rank, qr, W):
    w = _weights({"dq": (qr, W), "dq.norm": (qr,), "uq": (H * (dim + rot), qr), "dkv": (rank + rot, W), "dkv.norm": (rank,), "uk": (H * dim, rank),
                  "uv": (H * vdim, rank), "g": (H * vdim, W), "o": (W, H * vdim)}, 20, scale=2.0)
    m = latent(H, dim, rot, vdim, rank, qr, base=100.0, scaling=(4.0, 16, 4.0, 1.0))["mixer"]
    h = bf(torch.randn(60, W, generator=gen(21)))
    want = O.latent_attention(h.double(), torch.arange(60), {k: v.double() for k, v in w.items()}, "", m, 1e-5, {})
    mx = LatentAttentionMixer(w, H, dim, rot, vdim, rank, rot, 100.0, m["scale"], 1e-5, F32, DEV, q_rank=qr, rot_pairs=True, rot_scaling=m["rot"]["scaling"],
                              gate="channel")
    for label, cuts in CUTS.items():
        assert rel(run_mixer(mx, h, cuts), want) < 5e-5, label


@pytest.mark.parametrize("H,G,dim,vdim,chunk,rot_dims,W", [(4, 2, 16, 8, 11, 8, 64), (3, 3, 10, 34, 5, 6, 44), (6, 2, 40, 72, 40, 40, 96), (1, 1, 6, 3, 64, 6, 44)])
def test_differential_attention_mixer_alone(H, G, dim, vdim, chunk, rot_dims, W):
    w = _weights({"q": (2 * H * dim, W), "k": (2 * G * dim, W), "v": (G * vdim, W), "lq1": (dim,), "lk1": (dim,), "lq2": (dim,), "lk2": (dim,),
                  "o": (W, H * vdim)}, 22, scale=2.0)
    m = differential(H, G, dim, vdim, chunk, rot_dims=rot_dims, base=100.0, scaling=(8.0, 1.0, 4.0, 16))["mixer"]
    h = bf(torch.randn(60, W, generator=gen(23)))
    want = O.differential_attention(h.double(), torch.arange(60), {k: v.double() for k, v in w.items()}, "", m, 1e-5, {})
    mx = DifferentialAttentionMixer(w, H, G, dim, vdim, m["scale"], m["diff"], 1e-5, F32, DEV, rot=m["rot"], chunk=chunk)
    assert abs(mx.lam - O.differential_lambda({k: v.double() for k, v in w.items()}, "", m["diff"])) < 1e-12
    for label, cuts in CUTS.items():
        assert rel(run_mixer(mx, h, cuts), want) < 5e-5, label


@pytest.mark.parametrize("H,dim,vdim,W", [(2, 24, 16, 64), (1, 12, 10, 44), (2, 72, 136, 96)])
def test_forget_gate_mixer_alone(H, dim, vdim, W):
    w = _weights({"q": (H * dim, W), "f": (H * dim, W), "f.b": (H * dim,), "lower": (H * dim,), "v": (H * vdim, W), "norm": (vdim,), "o": (W, H * vdim)}, 24, scale=2.0)
    h = bf(torch.randn(60, W, generator=gen(25)))
    want = O.hgrn2(h.double(), {k: v.double() for k, v in w.items()}, "", {"heads": H, "dim": dim, "vdim": vdim}, 1e-5, {})
    mx = ForgetGateLinearAttentionMixer(w, H, dim, vdim, 1e-5, F32, DEV)
    for label, cuts in CUTS.items():
        assert rel(run_mixer(mx, h, cuts), want) < 5e-5, label


def test_two_sequences_in_one_batch_keep_their_own_state():
    """Portions of two sequences side by side in one step, for each mixer: each attends to its own cache from its own positions
    (chunks are counted from each sequence's start) and carries its own recurrent state."""
    W = 64
    wl = _weights({"dq": (24, W), "dq.norm": (24,), "uq": (4 * 24, 24), "dkv": (40, W), "dkv.norm": (32,), "uk": (64, 32), "uv": (96, 32), "g": (96, W), "o": (W, 96)}, 26)
    ml = latent(4, 16, 8, 24, 32, 24)["mixer"]
    wa = _weights({"q": (128, W), "k": (64, W), "v": (16, W), "lq1": (16,), "lk1": (16,), "lq2": (16,), "lk2": (16,), "o": (W, 32)}, 27)
    ma = differential(4, 2, 16, 8, 7, rot_dims=8)["mixer"]
    wh = _weights({"q": (48, W), "f": (48, W), "f.b": (48,), "lower": (48,), "v": (32, W), "norm": (16,), "o": (W, 32)}, 28)
    mh = {"heads": 2, "dim": 24, "vdim": 16}
    mixers = [(LatentAttentionMixer(wl, 4, 16, 8, 24, 32, 8, ml["rot"]["base"], ml["scale"], 1e-5, F32, DEV, q_rank=24, rot_pairs=True, rot_scaling=ml["rot"]["scaling"],
                                    gate="channel"), lambda h, n: O.latent_attention(h, torch.arange(n), {k: v.double() for k, v in wl.items()}, "", ml, 1e-5, {})),
              (DifferentialAttentionMixer(wa, 4, 2, 16, 8, ma["scale"], ma["diff"], 1e-5, F32, DEV, rot=ma["rot"], chunk=7),
               lambda h, n: O.differential_attention(h, torch.arange(n), {k: v.double() for k, v in wa.items()}, "", ma, 1e-5, {})),
              (ForgetGateLinearAttentionMixer(wh, 2, 24, 16, 1e-5, F32, DEV), lambda h, n: O.hgrn2(h, {k: v.double() for k, v in wh.items()}, "", mh, 1e-5, {}))]
    ha, hb = bf(torch.randn(20, W, generator=gen(29))), bf(torch.randn(9, W, generator=gen(30)))
    for mx, oracle in mixers:
        want_a, want_b = oracle(ha.double(), 20), oracle(hb.double(), 9)
        state = mx.new_state(SlotState(3, 32, DEV))
        got_a, got_b = [], []
        ia = ib = 0
        for na, nb in [(12, 1), (1, 2), (7, 6)]:                      # tokens of a, of b per step; b sits in the rows right after a
            rows = torch.cat([ha[ia:ia + na], hb[ib:ib + nb]]).to(DEV)
            out = mx(rows, make_batch([(2, ia, na), (0, ib, nb)]), state).cpu()
            got_a.append(out[:na]); got_b.append(out[na:])
            ia += na; ib += nb
        assert rel(torch.cat(got_a), want_a) < 5e-5 and rel(torch.cat(got_b), want_b) < 5e-5, type(mx).__name__


# ------------------------------------------------------------------------------------------------ the model
def build(name, dtype, seed=11, std_scale=1.0):
    cfg = CASES[name] if isinstance(name, str) else name
    w = O.random_weights(cfg, seed, std_scale)
    m = ZatusunForCausalLM(ZatusunConfig.from_dict(copy.deepcopy(cfg)), DEV, dtype).load_weights(lambda n: w[n])
    return cfg, w, m


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
    want = O.logits_of(cfg, w, toks, trace_o)
    got = Engine(m, 64, 2).step([{"id": 0, "tokens": toks, "want": list(range(45))}], trace=trace_m)
    assert len(trace_m) == len(trace_o) == len(O.layer_runs(cfg))
    for r, (a, b) in enumerate(zip(trace_m, trace_o)):
        assert rel(a, b) < 2e-4, f"what layer run {r} hands on"
    assert err(got, want) < 2e-4


@pytest.mark.parametrize("name", sorted(CASES))
def test_bf16_model_stays_within_rounding(name):
    cfg, w, m = build(name, BF16)
    toks = toks_for(cfg, 70, 2)
    got = Engine(m, 80, 1).step([{"id": 0, "tokens": toks, "want": list(range(70))}])
    assert err(got, O.logits_of(cfg, w, toks), "mean") < 0.06


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
        assert err(whole, O.logits_of(cfg, w, toks)) < 2e-4


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
        assert err(alone[k], O.logits_of(cfg, w, prompts[k])) < 2e-4


def test_freed_slots_are_reused_clean_and_passes_cut_long_entries():
    cfg, w, m = build("odd", F32)
    eng = Engine(m, 48, 2, max_rows=16)                              # a 40-token entry runs as passes of 16, 16 and 8 rows
    t1, t2, t3 = toks_for(cfg, 40, 7), toks_for(cfg, 33, 8), toks_for(cfg, 9, 9)
    a = eng.step([{"id": 1, "tokens": t1, "want": [0, 15, 16, 39]}], end=[1])
    assert err(a, O.logits_of(cfg, w, t1)[[0, 15, 16, 39]]) < 2e-4
    b = eng.step([{"id": 2, "tokens": t2, "want": [32]}, {"id": 3, "tokens": t3, "want": [8]}], end=[2])       # slot 0 again: its recurrent state starts at zero
    assert err(b[:1], O.logits_of(cfg, w, t2)[[32]]) < 2e-4 and err(b[1:], O.logits_of(cfg, w, t3)[[8]]) < 2e-4
    c = eng.step([{"id": 4, "tokens": t1[:5], "want": [4]}], end=[3, 4])                                    # and once more
    assert err(c, O.logits_of(cfg, w, t1[:5])[[4]]) < 2e-4
    assert eng.slots.live_tokens == 0


def _replay(eng, seq, rid, cuts):
    at = 0
    for c in cuts:
        out = eng.step([{"id": rid, "tokens": seq[at:at + c], "want": [c - 1]}])
        at += c
    eng.step([], end=[rid])
    assert at == len(seq)
    return out


def test_a_token_just_outside_the_chunk_changes_nothing_and_just_inside_does():
    """A model of one differential-attention layer: the last position's logits depend on the tokens of its own chunk alone.
    Replacing the chunk's first token moves them as the oracle says; replacing the token right before the chunk leaves them
    exactly as they were -- in a whole prompt, with the tail decoded token by token, and in portions cut inside the chunk."""
    chunk, n = 50, 230                                                # the last position, 229, lies in chunk [200, 250)
    cfg = config([differential(2, 1, 16, 16, chunk=chunk, rot_dims=8, scale=0.4)], vocab=50, width=32)
    _, w, m = build(cfg, F32, seed=12)
    toks = toks_for(cfg, n, 10)
    inside, outside = list(toks), list(toks)
    inside[200] = (inside[200] + 7) % cfg["vocab"]
    outside[199] = (outside[199] + 7) % cfg["vocab"]
    base, moved = O.logits_of(cfg, w, toks)[-1:], O.logits_of(cfg, w, inside)[-1:]
    assert err(moved, base) > 1e-3 and err(O.logits_of(cfg, w, outside)[-1:], base) < 1e-12
    eng = Engine(m, n, 1)
    for cuts in ([n], [n - 40] + [1] * 40, [100, 2, 99, 1, 3, 25], [199, 1, 30], [200, 30], [201, 29]):
        got = {k: _replay(eng, seq, k, cuts) for k, seq in (("base", toks), ("inside", inside), ("outside", outside))}
        assert err(got["base"], base) < 1e-4 and err(got["inside"], moved) < 1e-4, cuts
        assert torch.equal(got["outside"], got["base"]), cuts


@pytest.mark.parametrize("kind", ["latent_attention", "hgrn2"])
def test_a_far_token_still_moves_the_logits_through_the_model(kind):
    """One layer with a long memory (sharp attention scores; forget gates bounded close to one): among the tokens about 350
    positions back, the one whose replacement moves the last position's logits most (found with the oracle) is replaced; the
    model follows the oracle with and without the replacement -- in a whole prompt, when the tail is decoded token by token,
    and in portions."""
    layer = latent(2, 16, 8, 16, 24, 16, scale=1.0) if kind == "latent_attention" else hgrn2(2, 16, 16)
    cfg = config([layer], vocab=50, width=32)
    _, w, m = build(cfg, F32, seed=12, std_scale=2.0 if kind == "latent_attention" else 1.0)
    if kind == "hgrn2":
        w["l0.mix.lower"] = bf(0.98 + 0.02 * torch.rand(32, generator=gen(13)))
        m.load_weights(lambda n: w[n])
    n = 400
    toks = toks_for(cfg, n, 10)
    base = O.logits_of(cfg, w, toks)[-1:]
    best = (0.0, None, None)
    for far in range(n - 366, n - 346):
        variant = list(toks)
        variant[far] = (variant[far] + 7) % cfg["vocab"]
        moved = O.logits_of(cfg, w, variant)[-1:]
        best = max(best, (err(moved, base), variant, moved), key=lambda t: t[0])
    effect, variant, moved = best
    assert effect > 5e-4
    eng = Engine(m, n, 1)
    for seq, want in ((toks, base), (variant, moved)):
        for cuts in ([n], [n - 40] + [1] * 40, [100, 2, 61, 130, 3, 104]):
            assert err(_replay(eng, seq, 0, cuts), want) < 1e-4, cuts


def test_long_decoding_keeps_the_state_exact():
    """260 decoded tokens: the history passes the attention kernels' stage and key-range edges and many chunk borders, and the
    recurrent state is carried 260 times."""
    cfg, w, m = build("even", F32)
    n = 264
    toks = toks_for(cfg, n, 13)
    eng = Engine(m, n, 1)
    eng.step([{"id": 0, "tokens": toks[:4], "want": []}])
    outs = [eng.step([{"id": 0, "tokens": [t], "want": [0]}]) for t in toks[4:]]
    assert err(torch.cat(outs), O.logits_of(cfg, w, toks)[4:]) < 2e-4


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
        la, lc = O.logits_of(cfg, w, a), O.logits_of(cfg, w, c)
        assert err(graphed[-2:-1], lc[29:30]) < 2e-4 and err(graphed[-1:], la[128:129]) < 2e-4


def test_first_tokens_and_single_token_prompts():
    cfg, w, m = build("wide", F32)
    eng = Engine(m, 8, 3)
    for seed in (20, 21, 22):
        t = toks_for(cfg, 1, seed)
        assert err(eng.step([{"id": seed, "tokens": t, "want": [0]}]), O.logits_of(cfg, w, t)) < 2e-4
    t = toks_for(cfg, 5, 23)
    eng.step([], end=[20, 21, 22])
    got = torch.cat([eng.step([{"id": "s", "tokens": [x], "want": [0]}]) for x in t])
    assert err(got, O.logits_of(cfg, w, t)) < 2e-4


def test_sizes_that_are_equal_or_one():
    """What a configuration may make equal or 1: one head, heads as wide as the model, a latent as wide as the model, a chunk of
    one position (every token sees itself alone), a chunk longer than the sequence, one expert, a router that takes every
    expert, a loop of one pass, no soft cap, an embedding scale of 1."""
    cfg = config([differential(1, 1, 32, 32, chunk=1, scaling=None, diff=0.0), latent(1, 32, 32, 32, 32, 32, scaling=None, mlp=moe(1, 1, 32)),
                  hgrn2(1, 32, 32, mlp=moe(3, 3, 8)), differential(2, 2, 16, 16, chunk=500, rot_dims=2)], vocab=32, width=32, loop=(1, 2, 1), scale=1.0,
                 softcap=0.0)
    _, w, m = build(cfg, F32, seed=5)
    toks = toks_for(cfg, 40, 24)
    eng = Engine(m, 40, 1)
    got = torch.cat([eng.step([{"id": 0, "tokens": toks[:17], "want": list(range(17))}]), eng.step([{"id": 0, "tokens": toks[17:], "want": list(range(23))}])])
    assert err(got, O.logits_of(cfg, w, toks)) < 2e-4


def test_a_sequence_cannot_outgrow_the_position_table():
    cfg = config([hgrn2(1, 8, 8)], vocab=20, width=16, max_positions=12)
    _, w, m = build(cfg, F32)
    eng = Engine(m, 64, 1)
    toks = toks_for(cfg, 12, 1)
    assert err(eng.step([{"id": 0, "tokens": toks, "want": [11]}]), O.logits_of(cfg, w, toks)[-1:]) < 2e-4       # the last row of the table is used
    with pytest.raises(Exception):
        eng.step([{"id": 0, "tokens": [1], "want": [0]}])


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
    assert isinstance(m, ZatusunForCausalLM)
    prompts = torch.tensor([toks_for(cfg, 12, 30), toks_for(cfg, 12, 31)])
    new = 10
    out = m.generate(prompts, max_new_tokens=new)
    out_chunked = m.generate(prompts, max_new_tokens=new, chunk=5)
    assert out.shape == (2, 12 + new) and torch.equal(out[:, :12], prompts)
    for b in range(2):      # teacher-forced against the oracle: every greedy pick is its argmax wherever the top-2 margin is not a near-tie
        lg = O.logits_of(cfg, w, out[b].tolist())
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
    la, lb = O.logits_of(cfg, w, a), O.logits_of(cfg, w, b)
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
