"""`bench.py --compare-davasun`: prefill and decode throughput of Davasun at layer sizes of a real model (random weights)
beside OPT -- the closest existing model -- at equal width and depth, with every kernel's time against its roofline.
`bench.py --compare-bebulorn`: the same for Bebulorn beside Davasun, the closest existing model (step-served, recurrent and
attention mixers on a 32-bit residual stream).
`bench.py --compare-bizetar`: the same for Bizetar beside Bebulorn, the closest existing model (softmax attention with grouped
key/value heads on the same attention kernel, dense and mixture-of-experts feed-forwards, step-served).
`bench.py --compare-zatusun`: the same for Zatusun beside Bebulorn, the closest existing model (a matrix-state recurrence, masked
softmax attention and routed experts on the same kernels, a looped block, step-served).

Each operation of ``ops`` is wrapped for the duration of an instrumented pass: CUDA events around the call, and the
operation's algorithmic FLOPs and bytes from its arguments.  roofline time = max(FLOPs / peak, bytes / HBM bandwidth)
with the measured cuBLAS bf16 peak for tensor-core GEMMs, the nominal fp32 FMA rate of the CUDA cores (SMs x 128 lanes x
2 x max SM clock) for the kernels whose arithmetic must be fp32, and the measured copy bandwidth.  The throughput numbers
come from separate, uninstrumented passes (>= 3 warm-ups; weights + state exceed L2).
"""
import time

import torch

from . import ops

BF16 = torch.bfloat16


def _nbytes(*ts):
    return sum(t.numel() * t.element_size() for t in ts if t is not None)


def _cost(name, a, kw):
    """(flops, bytes, kind) of one call; kind: 'tc' tensor-core GEMM, 'f32' CUDA-core fp32 arithmetic, 'mem' memory-bound."""
    if name == "gemm":
        x, w = a[0], a[1]
        M, K, N = x.shape[0], x.shape[1], w.shape[0]
        return 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N), "tc"
    if name == "linear_plain":
        x, w, out = a[0], a[1], a[2]
        b = kw.get("batch", 1)
        K = kw.get("k") or x.shape[1]
        N = kw.get("n") or out.shape[1]
        M = x.shape[0]
        return 2.0 * b * M * N * K, M * b * K * x.element_size() + _nbytes(w) + M * b * N * out.element_size(), "f32"
    if name == "linear_small":
        x, w, out = a[0], a[1], a[3]
        return 2.0 * x.shape[0] * w.shape[0] * w.shape[1], _nbytes(x, w, out), "mem"
    if name == "mlstm_scan":
        q, S, segs, H, dim, vdim, o = a[0], a[4], a[7], a[8], a[9], a[10], a[13]
        M = q.shape[0]
        state = 2.0 * segs.shape[0] * H * dim * vdim * 4
        return 4.0 * M * H * dim * vdim, state + M * H * (2 * dim + vdim) * q.element_size() + _nbytes(o), "f32"
    if name == "latent_attn":
        qa, cache, meta, out, H, rank, rot = a[0], a[1], a[2], a[4], a[5], a[6], a[7]
        keys = float(kw.get("_keys", 0))                                           # sum over rows of visible keys
        return 2.0 * keys * H * (2 * rank + rot), _nbytes(qa, out) + kw.get("_ctx", 0) * (rank + rot) * cache.element_size(), "f32"
    if name == "linear_scan":
        q, S, segs, H, G, dim, vdim, o = a[0], a[3], a[4], a[5], a[6], a[7], a[8], a[9]
        M = q.shape[0]
        state = 2.0 * segs.shape[0] * H * dim * vdim * 4
        per_token = 8.0 if kw.get("gates") is not None else 4.0                    # delta: two dot products and two updates per cell
        return per_token * M * H * dim * vdim, state + M * (2 * G * dim + H * vdim) * q.element_size() + _nbytes(o), "f32"
    if name == "forget_scan":
        q, S, segs, H, dim, vdim, o = a[0], a[3], a[4], a[5], a[6], a[7], a[8]
        M = q.shape[0]
        return 4.0 * M * H * dim * vdim, 2.0 * segs.shape[0] * H * dim * vdim * 4 + M * H * (2 * dim + vdim) * 4 + _nbytes(o), "f32"
    if name == "window_attn":
        q, kc, out, H, G, dim, vdim = a[0], a[1], a[5], a[6], a[7], a[8], a[9]
        keys = float(kw.get("_wkeys", 0))                                          # sum over rows of keys inside the window
        return 2.0 * keys * H * (dim + vdim), _nbytes(q, out) + kw.get("_wctx", 0) * G * (dim + vdim) * kc.element_size(), "f32"
    if name == "qkv_prep":
        y, q_out, kc, vc = a[0], a[3], a[4], a[5]
        M = y.shape[0]
        C = q_out.shape[1] + kc.shape[2] + vc.shape[2]
        return 0.0, M * (C * y.element_size() + q_out.shape[1] * 4 + (kc.shape[2] + vc.shape[2]) * kc.element_size()), "mem"
    if name == "gated_rms_add":
        x, y, h = a[0], a[1], a[3]
        n_mix = kw.get("n_mix", 0) if kw.get("stack") is not None else 0
        gate = kw.get("gate")
        return 0.0, _nbytes(x) * (2 + n_mix) + _nbytes(y, h) + (x.shape[0] * x.shape[1] * gate.element_size() if gate is not None else 0), "mem"
    if name == "poly_norm":
        inp, F, out = a[0], a[1], a[3]
        return 0.0, 2.0 * inp.shape[0] * F * inp.element_size() + _nbytes(out), "mem"
    if name == "moe_gemm":
        x, w, out, idx = a[0], a[1], a[2], a[3]
        pairs, N, K = idx.numel(), w.shape[1], w.shape[2]
        touched = min(w.shape[0], pairs)
        kind = "tc" if x.dtype == BF16 and pairs > 64 else "mem"
        return 2.0 * pairs * N * K, pairs * (K * x.element_size() + N * out.element_size()) + touched * N * K * w.element_size(), kind
    if name == "moe_expert_gemms":
        x, w, counts, tm = a[0], a[1], a[3], a[4]
        rows, N, K = sum(counts) * tm, w.shape[1], w.shape[2]
        return 2.0 * rows * N * K, 2.0 * (rows * K + sum(1 for n in counts if n) * N * K + rows * N), "tc"
    if name == "attn_prefill":
        q, kc, B, S = a[0], a[1], a[3], a[4]
        H, d = kc.shape[2], kc.shape[3]
        return 2.0 * B * H * S * S * d, 4.0 * B * S * H * d * 2, "tc"            # causal: half of 4 B H S^2 d
    if name == "attn_decode":
        q, kc, B, T = a[0], a[1], a[3], a[4]
        H, d = kc.shape[2], kc.shape[3]
        return 4.0 * B * H * T * d, 4.0 * B * T * H * d, "mem"
    ts = [t for t in list(a) + list(kw.values()) if isinstance(t, torch.Tensor) and t.is_cuda]
    return 0.0, float(_nbytes(*ts)), "mem"


class Instrument:
    NAMES = ("gemm", "linear_plain", "linear_small", "mlstm_scan", "headnorm_gate", "latent_prep", "latent_attn", "clamped_glu",
             "rms_add_norm", "embed_rmsnorm", "rms_gather", "layernorm", "attn_prefill", "attn_decode", "embed", "argmax", "argmax_f32",
             "linear_scan", "conv_prep", "conv_state_update", "kv_store", "window_attn", "ln_add_norm", "embed_rows", "ln_gather", "gated_act",
             "router_topk", "moe_plan", "moe_gemm", "moe_gather", "moe_expert_gemms", "moe_combine", "qkv_prep", "gated_rms_add", "poly_norm",
             "embed_scale_pos", "residual_norm", "rms_norm_rows", "sigmoid_mul", "softcap", "forget_gate_prep", "forget_scan", "diff_combine")

    def __init__(self):
        self.records, self.saved, self.extra = [], {}, {}

    def __enter__(self):
        for n in self.NAMES:
            fn = getattr(ops, n)
            self.saved[n] = fn

            def wrapped(*a, _n=n, _fn=fn, **kw):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = _fn(*a, **kw)
                e1.record()
                self.records.append((_n, e0, e1, _cost(_n, a, dict(kw, **self.extra))))
                return r
            setattr(ops, n, wrapped)
        return self

    def __exit__(self, *exc):
        for n, fn in self.saved.items():
            setattr(ops, n, fn)

    def table(self, pk):
        torch.cuda.synchronize()
        agg = {}
        for n, e0, e1, (fl, by, kind) in self.records:
            peak = pk["bf16_burst"] * 1e12 if kind == "tc" else pk["fp32_nominal_tflops"] * 1e12
            ideal = max(fl / peak if kind != "mem" else 0.0, by / (pk["hbm_gbs"] * 1e9))
            r = agg.setdefault(n, {"calls": 0, "ms": 0.0, "roofline_ms": 0.0, "gflop": 0.0, "mb": 0.0, "bound": kind})
            r["calls"] += 1
            r["ms"] += e0.elapsed_time(e1)
            r["roofline_ms"] += ideal * 1e3
            r["gflop"] += fl / 1e9
            r["mb"] += by / 1e6
        for r in agg.values():
            r["of_roofline"] = round(r["roofline_ms"] / r["ms"], 4) if r["ms"] > 0 else None
            for k in ("ms", "roofline_ms", "gflop", "mb"):
                r[k] = round(r[k], 4)
        return agg


def davasun_config(width, n_layers):
    """Layer sizes of a ~1-3 B model: mLSTM heads of 256 x 512, latent attention with 128 + 64 query/key channels and a
    512-wide latent, a 2.75 x feed-forward on the attention layers; one attention layer in every four."""
    H = max(1, width // 512)
    ml = {"type": "mlstm", "mixer": {"heads": H, "dim": 256, "vdim": 512, "gate_cap": 15.0}, "mlp": None}
    la = {"type": "latent_attention",
          "mixer": {"heads": width // 128, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "rot": {"base": 10000.0, "dims": 64},
                    "scale": 192 ** -0.5},
          "mlp": {"kind": "dense", "ff": width * 11 // 4, "limit": 7.0}}
    layers = [la if i % 4 == 1 else ml for i in range(n_layers)]
    return {"architecture": "Davasun", "vocab": 32000, "width": width, "layers": layers, "loop": {"start": 0, "stop": 0, "times": 1},
            "norm": {"eps": 1e-6}, "logit_scale": 1.0}


def bebulorn_config(width, n_layers):
    """Layer sizes of a ~1-3 B model: heads of 128 x 128 throughout; delta layers with half as many query/key heads as value
    heads and a 4-tap convolution; attention with 8 key/value heads and a window of 1024; feed-forwards alternate between a
    dense 2.75 x one and 16 experts of 0.6875 x (2 chosen) plus a shared expert of the same size.  Order: delta, lightning,
    lightning, attention."""
    H = width // 128
    dense = {"kind": "dense", "ff": width * 11 // 4}
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": width * 11 // 16}, "shared": {"ff": width * 11 // 16}}
    li = lambda mlp: {"type": "lightning", "mlp": mlp,  # noqa: E731
                      "mixer": {"heads": H, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** -(1 + 7 * i / max(H - 1, 1)) for i in range(H)]}}
    de = {"type": "delta", "mixer": {"heads": H, "kv_heads": max(1, H // 2), "dim": 128, "vdim": 128, "conv": 4}, "mlp": dense}
    at = {"type": "attention", "mlp": moe,
          "mixer": {"heads": H, "kv_heads": min(8, H), "dim": 128, "vdim": 128, "mask": {"size": 1024}, "scale": 128 ** -0.5, "softcap": 50.0}}
    pattern = [de, li(moe), li(dense), at]
    return {"architecture": "Bebulorn", "vocab": 32000, "width": width, "layers": [pattern[i % 4] for i in range(n_layers)],
            "loop": {"start": 0, "stop": 0, "times": 1}, "norm": {"eps": 1e-6}, "residual_mult": 0.5}


def bizetar_config(width, n_layers):
    """Layer sizes of a ~1-3 B model: heads of 128 x 128 on 8 key/value heads throughout; three layers in four rotate half of
    every head behind a 4-tap convolution, the fourth norms the whole projection and takes a distance bias; every layer mixes
    values; feed-forwards alternate between a dense 2.75 x one and 16 gated experts of 0.6875 x (2 chosen) with 2 identity experts."""
    H = width // 128
    G = min(8, H)
    dense = {"kind": "dense", "ff": width * 11 // 4}
    moe = {"kind": "moe", "router": {"experts": 16, "identity": 2, "top": 2}, "expert": {"ff": width * 11 // 16}}
    base = {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "v_mix": True}
    rot = {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}
    a2 = lambda mlp: {"type": "attention_2", "mixer": dict(base, conv=4, rot=rot), "mlp": mlp}  # noqa: E731
    a1 = {"type": "attention", "mixer": dict(base, q_temp={"coef": 0.1, "every": 256}), "mlp": moe}
    pattern = [a2(dense), a1, a2(moe), a2(dense)]
    return {"architecture": "Bizetar", "vocab": 32000, "width": width, "layers": [pattern[i % 4] for i in range(n_layers)], "norm": {"eps": 1e-6}}


def zatusun_config(width, n_runs):
    """Layer sizes of a ~1-3 B model in ``n_runs`` layer runs: latent attention with heads of 128 + 64 query/key channels, a 512-wide
    latent and queries through a latent of half the width; the forget-gate recurrence with heads of 128 x 128; differential
    attention with two maps of 128 channels and values of 256 per head on 4 key/value heads, in chunks of 1024; every layer with
    16 clamped gated experts of 0.6875 x (2 chosen).  Order: latent, recurrence (these two form the loop, run twice), then
    latent, differential, recurrence, ... for the rest."""
    H = width // 128
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": width * 11 // 16, "limit": 7.0}}
    la = {"type": "latent_attention", "mlp": moe,
          "mixer": {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": width // 2, "scale": 192 ** -0.5,
                    "rot": {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}}
    hg = {"type": "hgrn2", "mlp": moe, "mixer": {"heads": H, "dim": 128, "vdim": 128}}
    Hd = max(1, width // 256)
    di = {"type": "attention", "mlp": moe,
          "mixer": {"heads": Hd, "kv_heads": min(4, Hd), "dim": 128, "vdim": 256, "diff": 0.5, "mask": {"size": 1024}, "scale": 128 ** -0.5,
                    "rot": {"dims": 128, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 1024}}}}
    rest = [la, di, hg]
    layers = [la, hg] + [rest[i % 3] for i in range(max(n_runs - 4, 0))]
    return {"architecture": "Zatusun", "vocab": 32000, "width": width, "max_positions": 8192, "layers": layers, "loop": {"start": 0, "stop": 2, "times": 2},
            "norm": {"eps": 1e-6}, "embedding": {"scale": float(width) ** 0.5}, "logit_softcap": 30.0}


def _window_keys(layers, n_new, ctx_before):
    """Sum over the new rows of the keys inside the first attention layer's window (the whole history where a layer names
    none), and the cached rows those windows span."""
    first = next((l for l in layers if l["type"].startswith("attention")), None)
    win = first["mixer"].get("mask", {}).get("size", 1 << 30) if first else 0
    if not win:
        return 0, 0
    if "diff" in first["mixer"]:              # a chunked mask: a row sees the keys of its own block of `win` positions
        return sum((ctx_before + i) % win + 1 for i in range(n_new)), min(ctx_before + n_new, win + n_new - 1)
    keys = sum(min(win, ctx_before + i + 1) for i in range(n_new))
    return keys, min(ctx_before + n_new, win + n_new - 1)


def step_model(m, cfg, pk, g, prompt, decode_ctx, decode_batches, new):
    """Prefill and decode numbers of a model served by the step engine, with the per-kernel table of one instrumented pass."""
    from .engine import Engine
    toks = torch.randint(0, cfg.vocab, (prompt,), generator=g).tolist()
    eng = Engine(m, max_tokens=decode_ctx + new + 8, max_requests=max(decode_batches), max_rows=prompt)

    def prefill():
        eng.step([{"id": "p", "tokens": toks, "want": [prompt - 1]}], end=["p"])
    ms = _timed(prefill)
    d = {"prefill_ms": round(ms, 3), "prefill_tokens_per_s": round(prompt / ms * 1e3, 1)}
    with Instrument() as ins:
        wk, wc = _window_keys(cfg.layers, prompt, 0)
        ins.extra = {"_keys": prompt * (prompt + 1) / 2, "_ctx": prompt, "_wkeys": wk, "_wctx": wc}
        prefill()
    d["prefill_kernels"] = ins.table(pk)
    for B in decode_batches:
        ids = list(range(B))
        ctx = torch.randint(0, cfg.vocab, (decode_ctx,), generator=g).tolist()
        for i in ids:
            eng.step([{"id": i, "tokens": ctx, "want": []}])
        step = lambda: eng.step([{"id": i, "tokens": [7], "want": [0]} for i in ids])  # noqa: E731
        ms = _timed(step, warmup=3, iters=new - 4)
        d[f"decode_b{B}_ms_per_step"] = round(ms, 3)
        d[f"decode_b{B}_tokens_per_s"] = round(B / ms * 1e3, 1)
        eng.graphs = False                    # the timed steps above replay a CUDA graph; the per-kernel pass launches eagerly
        ms = _timed(step, warmup=1, iters=2)
        d[f"decode_b{B}_ms_per_step_eager"] = round(ms, 3)
        with Instrument() as ins:
            wk, wc = _window_keys(cfg.layers, 1, decode_ctx + new)
            ins.extra = {"_keys": B * (decode_ctx + new), "_ctx": B * (decode_ctx + new), "_wkeys": B * wk, "_wctx": B * wc}
            step()
        eng.graphs = True
        d[f"decode_b{B}_kernels"] = ins.table(pk)
        eng.step([], end=ids)
    return d


def run_bebulorn(pk, widths=(2048, 4096), n_layers=8, prompt=2048, decode_ctx=2048, decode_batches=(1, 16), new=16):
    """Bebulorn beside Davasun at equal width and depth."""
    from .modeling_bebulorn import BebulornConfig, BebulornForCausalLM
    from .modeling_davasun import DavasunConfig, DavasunForCausalLM
    dev = torch.device("cuda", 0)
    props = torch.cuda.get_device_properties(dev)
    pk = dict(pk, fp32_nominal_tflops=props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12)
    out = {"peaks": pk, "sizes": []}
    g = torch.Generator().manual_seed(0)
    for width in widths:
        rec = {"width": width, "layers": n_layers, "prompt": prompt, "decode_context": decode_ctx}
        for name, make in (("bebulorn", lambda: BebulornForCausalLM(BebulornConfig.from_dict(bebulorn_config(width, n_layers)), dev, BF16)),
                           ("davasun", lambda: DavasunForCausalLM(DavasunConfig.from_dict(davasun_config(width, n_layers)), dev, BF16))):
            m = make().init_weights(seed=1)
            rec[name] = step_model(m, m.config, pk, g, prompt, decode_ctx, decode_batches, new)
            del m
            torch.cuda.empty_cache()
        out["sizes"].append(rec)
    return out


def run_zatusun(pk, widths=(2048, 4096), n_layers=8, prompt=2048, decode_ctx=2048, decode_batches=(1, 16), new=16):
    """Zatusun beside Bebulorn at equal width and number of layer runs."""
    from .modeling_bebulorn import BebulornConfig, BebulornForCausalLM
    from .modeling_zatusun import ZatusunConfig, ZatusunForCausalLM
    dev = torch.device("cuda", 0)
    props = torch.cuda.get_device_properties(dev)
    pk = dict(pk, fp32_nominal_tflops=props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12)
    out = {"peaks": pk, "sizes": []}
    g = torch.Generator().manual_seed(0)
    for width in widths:
        rec = {"width": width, "layers": n_layers, "prompt": prompt, "decode_context": decode_ctx}
        for name, make in (("zatusun", lambda: ZatusunForCausalLM(ZatusunConfig.from_dict(zatusun_config(width, n_layers)), dev, BF16)),
                           ("bebulorn", lambda: BebulornForCausalLM(BebulornConfig.from_dict(bebulorn_config(width, n_layers)), dev, BF16))):
            m = make().init_weights(seed=1)
            rec[name] = step_model(m, m.config, pk, g, prompt, decode_ctx, decode_batches, new)
            del m
            torch.cuda.empty_cache()
        out["sizes"].append(rec)
    return out


def run_bizetar(pk, widths=(2048, 4096), n_layers=8, prompt=2048, decode_ctx=2048, decode_batches=(1, 16), new=16):
    """Bizetar beside Bebulorn at equal width and depth."""
    from .modeling_bebulorn import BebulornConfig, BebulornForCausalLM
    from .modeling_bizetar import BizetarConfig, BizetarForCausalLM
    dev = torch.device("cuda", 0)
    props = torch.cuda.get_device_properties(dev)
    pk = dict(pk, fp32_nominal_tflops=props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12)
    out = {"peaks": pk, "sizes": []}
    g = torch.Generator().manual_seed(0)
    for width in widths:
        rec = {"width": width, "layers": n_layers, "prompt": prompt, "decode_context": decode_ctx}
        for name, make in (("bizetar", lambda: BizetarForCausalLM(BizetarConfig.from_dict(bizetar_config(width, n_layers)), dev, BF16)),
                           ("bebulorn", lambda: BebulornForCausalLM(BebulornConfig.from_dict(bebulorn_config(width, n_layers)), dev, BF16))):
            m = make().init_weights(seed=1)
            rec[name] = step_model(m, m.config, pk, g, prompt, decode_ctx, decode_batches, new)
            del m
            torch.cuda.empty_cache()
        out["sizes"].append(rec)
    return out


def _timed(fn, warmup=3, iters=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run(pk, widths=(2048, 4096), n_layers=8, prompt=2048, decode_ctx=2048, decode_batches=(1, 16), new=16):
    from .modeling_davasun import DavasunConfig, DavasunForCausalLM
    from .modeling_opt import OPTConfig, OPTForCausalLM
    dev = torch.device("cuda", 0)
    props = torch.cuda.get_device_properties(dev)
    pk = dict(pk, fp32_nominal_tflops=props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12)
    out = {"peaks": pk, "sizes": []}
    g = torch.Generator().manual_seed(0)
    for width in widths:
        rec = {"width": width, "layers": n_layers, "prompt": prompt, "decode_context": decode_ctx}
        # ---------------- Davasun
        cfg = DavasunConfig.from_dict(davasun_config(width, n_layers))
        m = DavasunForCausalLM(cfg, dev, BF16).init_weights(seed=1)
        d = step_model(m, cfg, pk, g, prompt, decode_ctx, decode_batches, new)
        rec["davasun"] = d
        del eng, m
        torch.cuda.empty_cache()
        # ---------------- OPT at equal width and depth (head_dim 128, 4x feed-forward)
        ocfg = OPTConfig(hidden_size=width, num_hidden_layers=n_layers, num_attention_heads=width // 128, ffn_dim=4 * width,
                         vocab_size=32000, max_position_embeddings=prompt + decode_ctx + new + 8, name=f"opt-w{width}")
        om = OPTForCausalLM(ocfg, dev).init_weights(seed=1)
        o = {}
        ids1 = torch.randint(3, 32000, (1, prompt), generator=g).to(dev)
        gen = lambda x, n: om.generate(x, max_new_tokens=n, min_new_tokens=n, prefill_policy=0, decoding_policy=0)  # noqa: E731
        _timed(lambda: gen(ids1, 1), warmup=3, iters=1)
        ms = om.last_timing["prefill_s"] * 1e3
        o["prefill_ms"] = round(ms, 3)
        o["prefill_tokens_per_s"] = round(prompt / ms * 1e3, 1)
        om.use_cuda_graphs = False
        with Instrument() as ins:
            gen(ids1, 1)
        o["prefill_kernels"] = ins.table(pk)
        for B in decode_batches:
            idsb = torch.randint(3, 32000, (B, decode_ctx), generator=g).to(dev)
            om.use_cuda_graphs = True
            _timed(lambda: gen(idsb, new), warmup=3, iters=1)
            dec = om.last_timing["decode_s"]
            ms = sum(dec) / len(dec) * 1e3
            o[f"decode_b{B}_ms_per_step"] = round(ms, 3)
            o[f"decode_b{B}_tokens_per_s"] = round(B / ms * 1e3, 1)
            om.use_cuda_graphs = False
            before = None
            with Instrument() as ins:
                gen(idsb, 2)
            # keep the records of the decode step only (after the prefill's): the last layer loop + head
            per_step = len(ins.records) - next(i for i, r in enumerate(ins.records) if r[0] == "attn_decode") + 2
            ins.records = ins.records[-per_step:]
            o[f"decode_b{B}_kernels"] = ins.table(pk)
        rec["opt"] = o
        del om
        torch.cuda.empty_cache()
        out["sizes"].append(rec)
    return out
