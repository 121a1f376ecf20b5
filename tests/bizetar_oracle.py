"""Plain, slow restatement of the Bizetar design, one function per mechanism, in float64 PyTorch on the CPU.  It shares no
code with the product: attention builds the full score matrix over the whole history with an explicit mask and an explicit
sink term, the convolution is a Python loop over taps on a zero-padded history, experts are visited token by token, and
state is a dict per layer that holds the history itself (convolution inputs, keys, values).

Weights: dict name -> tensor ('l<i>.mix.q', ...), config: the dict of config.json.
"""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ norms and activations
def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_div(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def poly_norm(z, coef, eps):
    """k1 R(z) + k2 R(z*z) + k3 R(z*z*z) + k0 with R = division by the row's root mean square; coef = (k1, k2, k3, k0)."""
    a, b, c, e = (float(t) for t in coef)
    return a * rms_div(z, eps) + b * rms_div(z * z, eps) + c * rms_div(z * z * z, eps) + e


# ------------------------------------------------------------------------------------------------ feed-forwards
def dense_ff(h, w, p, eps):
    return poly_norm(h @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def gated_expert(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def route(h, w_router, correction, top):
    """Chosen outputs [T, top] of the router and their weights: softmax over all outputs, the choice made on the scores plus
    the correction, the weights being the plain scores of the chosen (not renormalised)."""
    s = torch.softmax(h @ w_router.T, -1)
    _, idx = torch.topk(s + correction, top, dim=-1)
    return idx, torch.gather(s, -1, idx)


def moe(h, w, p, cfg):
    r = cfg["router"]
    real = r["experts"]
    idx, wt = route(h, w[p + "router"], w[p + "correction"], r["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            if e >= real:                        # an identity expert hands the token back
                out[t] += wt[t, j] * h[t]
            else:
                out[t] += wt[t, j] * gated_expert(h[t], w[p + f"e{e}.gate"], w[p + f"e{e}.up"], w[p + f"e{e}.down"])
    return out


# ------------------------------------------------------------------------------------------------ pieces of the mixers
def causal_conv(u, w_conv, past):
    """u [T, C] new inputs, past [P, C] all earlier inputs of the sequence, w_conv [C, taps]: the last column of w_conv weighs
    the current input, the one before it the previous input, and so on; inputs at negative positions count as 0."""
    taps = w_conv.shape[1]
    full = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=F64), past, u], 0)
    P = past.shape[0]
    y = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            y[t] += w_conv[:, j] * full[(taps - 1) + P + t - taps + 1 + j]
    return y


def yarn_tables(pos, rot):
    """cos, sin [T, dims/2] of the rotation at positions ``pos``."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc is not None:
        def where(t):
            return dims * math.log(sc["original"] / (2 * math.pi * t)) / (2 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / sc["factor"] * ramp + f * (1 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    ang = pos.to(F64)[:, None] * f[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate_pairs(x, cos, sin, dims):
    """x [T, heads, dim]: channels (2i, 2i+1) of the first ``dims`` channels turn by the angle of pair i."""
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def sink_attention(q, k, v, pos, scale, sink, slopes=None):
    """q [T, H, d] at positions pos [T]; k [N, G, d], v [N, G, e]: the whole history, key j at position j.  Softmax over the
    visible keys plus one sink term exp(sink_h) that has no value; optionally every position of distance costs head h slopes[h] of the score."""
    T, H, _ = q.shape
    N, G = k.shape[0], k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    j = torch.arange(N)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        dist = (pos[:, None] - j[None, :]).to(F64)
        if slopes is not None:
            s = s - slopes[h] * dist
        s = s.masked_fill(dist < 0, float("-inf"))
        full = torch.cat([s, sink[h].expand(T, 1)], 1)
        p = torch.softmax(full, -1)[:, :N]
        out[:, h] = p @ v[:, g]
    return out


def mix_values(v, layer_index, w, p, shared):
    """Value mixing: the first layer that mixes publishes its values; every later one blends them into its own."""
    if "v_first" not in shared:
        shared["v_first"] = v
        return v
    lam = float(w[p + "vmix"])
    return (1.0 - lam) * v + lam * shared["v_first"]


# ------------------------------------------------------------------------------------------------ mixers
def attention_mixer(h, pos, w, p, m, eps, state, shared, layer_index):
    """The mixer with a norm over the whole query / key projection, a query temperature, a distance bias and one gate per head."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps)
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps)
    v = h @ w[p + "v"].T
    qt = m.get("q_temp")
    if qt is not None:
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((pos.to(F64) + 1) / qt["every"]) + 1.0))[:, None]
    if m.get("v_mix"):
        v = mix_values(v, layer_index, w, p, shared)
    state["k"] = torch.cat([state["k"], k.view(T, G, d)], 0) if "k" in state else k.view(T, G, d)
    state["v"] = torch.cat([state["v"], v.view(T, G, e)], 0) if "v" in state else v.view(T, G, e)
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)], dtype=F64)
    o = sink_attention(q.view(T, H, d), state["k"], state["v"], pos, m["scale"], w[p + "sink"], slopes)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * e) @ w[p + "o"].T


def attention_2_mixer(h, pos, w, p, m, eps, state, shared, layer_index):
    """The mixer with biased projections behind a short convolution, a norm per head, rotated queries and keys and a gate per channel."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for n in ("q", "k", "v"):
        u = h @ w[p + n].T + w[p + n + ".b"]
        if m.get("conv"):
            past = state.get("u" + n, torch.zeros(0, u.shape[1], dtype=F64))
            proj[n] = causal_conv(u, w[p + n + ".conv"], past)
            state["u" + n] = torch.cat([past, u], 0)
        else:
            proj[n] = u
    q = rms_norm(proj["q"].view(T, H, d), w[p + "q.norm"], eps)
    k = rms_norm(proj["k"].view(T, G, d), w[p + "k.norm"], eps)
    v = proj["v"]
    rot = m.get("rot")
    if rot is not None:
        cos, sin = yarn_tables(pos, rot)
        q, k = rotate_pairs(q, cos, sin, rot["dims"]), rotate_pairs(k, cos, sin, rot["dims"])
    if m.get("v_mix"):
        v = mix_values(v, layer_index, w, p, shared)
    state["k"] = torch.cat([state["k"], k], 0) if "k" in state else k
    state["v"] = torch.cat([state["v"], v.view(T, G, e)], 0) if "v" in state else v.view(T, G, e)
    o = sink_attention(q, state["k"], state["v"], pos, m["scale"], w[p + "sink"])
    o = o.reshape(T, H * e) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


MIXERS = {"attention": attention_mixer, "attention_2": attention_2_mixer}


# ------------------------------------------------------------------------------------------------ the model
def new_state(config):
    return {"pos": 0, "layers": [dict() for _ in config["layers"]]}


def forward(tokens, w, config, state, trace=None):
    """Feeds ``tokens`` (the next tokens of one sequence) and returns logits [T, vocab] in float64.  ``state`` carries the
    sequence from call to call; ``trace`` (a list) receives what each layer hands on."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    pos = torch.arange(state["pos"], state["pos"] + T)
    state["pos"] += T
    x = rms_norm(w["embed"][torch.tensor(tokens)], w["embed.norm"], eps)
    results = [x]                        # X_0 and every layer's own result
    shared = {}                          # what layers of one forward pass hand to later layers (the first mixed values)
    for i, l in enumerate(config["layers"]):
        p = f"l{i}."
        y = MIXERS[l["type"]](x, pos, w, p + "mix.", l["mixer"], eps, state["layers"][i], shared, i)
        y = y * torch.sigmoid(x @ w[p + "rg1"].T + w[p + "rg1.b"])
        x = x + rms_norm(y, w[p + "norm1"], eps)
        mlp = l.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, p + "mlp.", eps) if mlp["kind"] == "dense" else moe(x, w, p + "mlp.", mlp)
            y = y * torch.sigmoid(x @ w[p + "rg2"].T + w[p + "rg2.b"])
            x = x + rms_norm(y, w[p + "norm2"], eps)
        results.append(x)
        x = sum(float(w[p + "dwa"][j]) * results[j] for j in range(i + 2))
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


# ------------------------------------------------------------------------------------------------ checkpoints for the tests
def tensor_shapes(config):
    W, V = config["width"], config["vocab"]
    out = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,), "head": (V, W)}
    for i, l in enumerate(config["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, d = m["heads"], m["dim"]
        G, e = m.get("kv_heads", H), m.get("vdim", d)
        out[p + "norm1"], out[p + "rg1"], out[p + "rg1.b"], out[p + "dwa"] = (W,), (W, W), (W,), (i + 2,)
        out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = (H * d, W), (G * d, W), (G * e, W)
        out[p + "mix.sink"], out[p + "mix.o"] = (H,), (W, H * e)
        if m.get("v_mix"):
            out[p + "mix.vmix"] = ()
        if l["type"] == "attention":
            out[p + "mix.q.norm"], out[p + "mix.k.norm"], out[p + "mix.g"] = (H * d,), (G * d,), (H, W)
        else:
            out[p + "mix.q.norm"], out[p + "mix.k.norm"], out[p + "mix.g"] = (d,), (d,), (H * e, W)
            for n, c in (("q", H * d), ("k", G * d), ("v", G * e)):
                out[p + f"mix.{n}.b"] = (c,)
                if m.get("conv"):
                    out[p + f"mix.{n}.conv"] = (c, m["conv"])
        mlp = l.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"], out[p + "rg2"], out[p + "rg2.b"] = (W,), (W, W), (W,)
        if mlp["kind"] == "dense":
            out[p + "mlp.up"], out[p + "mlp.down"], out[p + "mlp.act"] = (mlp["ff"], W), (W, mlp["ff"]), (4,)
        else:
            f, r = mlp["expert"]["ff"], mlp["router"]
            for x in range(r["experts"]):
                out[p + f"mlp.e{x}.gate"], out[p + f"mlp.e{x}.up"], out[p + f"mlp.e{x}.down"] = (f, W), (f, W), (W, f)
            n_out = r["experts"] + r.get("identity", 0)
            out[p + "mlp.router"], out[p + "mlp.correction"] = (n_out, W), (n_out,)
    return out


def random_weights(config, seed, std_scale=1.0):
    """bf16-representable random weights: projections N(0, 1/in), norm weights near 1, biases and sinks near 0, routers wide
    enough that two scores are rarely within rounding of each other, layer mixes that sum to about 1."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shp in tensor_shapes(config).items():
        if name.endswith(".conv"):
            t = torch.randn(shp, generator=g) * 0.5
        elif name.endswith(".dwa"):
            t = torch.full(shp, 1.0 / shp[0]) + 0.2 * torch.randn(shp, generator=g)
        elif name.endswith(".vmix"):
            t = 0.2 + 0.5 * torch.rand(shp, generator=g)
        elif name.endswith(".act"):
            t = torch.tensor([1.0, 0.5, 0.25, 0.1]) + 0.2 * torch.randn(shp, generator=g)
        elif name.endswith(".correction"):
            t = 0.05 * torch.randn(shp, generator=g)
        elif name.endswith(".router"):
            t = torch.randn(shp, generator=g) * 2.0 * shp[1] ** -0.5
        elif len(shp) == 2:
            t = torch.randn(shp, generator=g) * std_scale * shp[1] ** -0.5
        elif name.endswith(".b") or name.endswith(".sink"):
            t = 0.5 * torch.randn(shp, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shp, generator=g)
        out[name] = t.to(torch.bfloat16).float()
    return out
