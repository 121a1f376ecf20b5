"""Plain, slow restatement of the Zatusun design, one function per mechanism, in float64 PyTorch on the CPU.  It shares no
code with the product: both attentions build the full score matrix over the whole history with an explicit mask (the latent
attention expands every cached latent into per-head keys and values first), the recurrence is a Python loop over tokens,
experts are visited token by token, and state is a dict per layer run that holds the history itself (latents, keys, values)
or the recurrent matrix.

Weights: dict name -> tensor ('l<i>.mix.q', ...), config: the dict of config.json.
"""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ norms and activations
def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    """Plain weight."""
    return rms_div(x, eps) * w


def rms_norm_around_zero(x, w, eps):
    """The weight is stored as its distance from one."""
    return rms_div(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------------ rotation
def plain_freq(dims, base):
    return torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def yarn_freq(dims, base, s):
    """Frequencies and the amplitude on cos and sin: pairs below ``first`` keep their frequency, pairs above ``last`` are slowed by
    ``factor``, the ones between blend linearly."""
    f = plain_freq(dims, base)
    if not s:
        return f, 1.0

    def pair_of(turns):
        return dims * math.log(s["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    first = max(math.floor(pair_of(s["fast"])), 0)
    last = min(math.ceil(pair_of(s["slow"])), dims - 1)
    span = max(last - first, 0.001)
    out = f.clone()
    for i in range(dims // 2):
        slowed = min(max((i - first) / span, 0.0), 1.0)           # 0: the pair keeps its frequency, 1: it is slowed by the whole factor
        out[i] = f[i] * ((1.0 - slowed) + slowed / s["factor"])
    return out, 0.1 * math.log(s["factor"]) + 1.0


def llama3_freq(dims, base, s):
    """Frequencies by wavelength: short waves stay, long waves are slowed by ``factor``, the ones between blend."""
    f = plain_freq(dims, base)
    if not s:
        return f, 1.0
    out = f.clone()
    for i in range(dims // 2):
        wave = 2.0 * math.pi / float(f[i])
        if wave < s["original"] / s["high"]:
            continue
        if wave > s["original"] / s["low"]:
            out[i] = f[i] / s["factor"]
        else:
            t = (s["original"] / wave - s["low"]) / (s["high"] - s["low"])
            out[i] = (1.0 - t) * f[i] / s["factor"] + t * f[i]
    return out, 1.0


def rotate_pairs(x, pos, freq, amp):
    """x [T, n, d]: channels (2i, 2i+1), i < len(freq), of every vector turn by pos * freq[i]; the rest pass."""
    out = x.clone()
    for i in range(freq.numel()):
        a = pos.to(F64) * freq[i]
        c, s = (torch.cos(a) * amp)[:, None], (torch.sin(a) * amp)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ feed-forward
def clamped_expert(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def route(h, w_router, top):
    """The ``top`` largest logits and the softmax over just those."""
    z = h @ w_router.T
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def moe(h, w, p, cfg):
    idx, wt = route(h, w[p + "router"], cfg["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * clamped_expert(h[t], w[p + f"e{e}.gate"], w[p + f"e{e}.up"], w[p + f"e{e}.down"], cfg["expert"]["limit"])
    return out


# ------------------------------------------------------------------------------------------------ mixers
def visible(P, T, chunk=0):
    """mask [T, P + T]: new token t (position P + t) sees position j if j <= P + t and, with a chunked mask, both lie in the
    same block of ``chunk`` positions counted from the sequence's start."""
    i = (P + torch.arange(T))[:, None]
    j = torch.arange(P + T)[None, :]
    m = j <= i
    if chunk:
        m = m & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    return m


def masked_softmax(s, mask):
    return torch.softmax(s.masked_fill(~mask, float("-inf")), -1)


def latent_attention(h, pos, w, p, m, eps, state):
    """state: {"c": [P, kv_rank], "kr": [P, rot_dim]} of the earlier tokens (rotated key part as cached)."""
    T, H, d, r, vd, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    freq, amp = yarn_freq(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    kr = rotate_pairs(dkv[:, None, rank:], pos, freq, amp)[:, 0]
    q_rot = rotate_pairs(q[..., d:], pos, freq, amp)
    c_all = torch.cat([state.get("c", c[:0]), c], 0)
    kr_all = torch.cat([state.get("kr", kr[:0]), kr], 0)
    state["c"], state["kr"] = c_all, kr_all
    P = c_all.shape[0] - T
    k = (c_all @ w[p + "uk"].T).view(-1, H, d)               # every cached latent expanded into per-head keys and values
    v = (c_all @ w[p + "uv"].T).view(-1, H, vd)
    mask = visible(P, T)
    out = torch.zeros(T, H, vd, dtype=F64)
    for hq in range(H):
        s = (q[:, hq, :d] @ k[:, hq].T + q_rot[:, hq] @ kr_all.T) * m["scale"]
        out[:, hq] = masked_softmax(s, mask) @ v[:, hq]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * vd) * gate) @ w[p + "o"].T


def differential_lambda(w, p, diff):
    return math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff


def differential_attention(h, pos, w, p, m, eps, state):
    """state: {"k": [P, G, 2, dim] rotated, "v": [P, G, vdim]} of the earlier tokens."""
    T, H, G, d, vd = h.shape[0], m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    rot = m.get("rot")
    q, k = (h @ w[p + "q"].T).view(T, H * 2, d), (h @ w[p + "k"].T).view(T, G * 2, d)
    if rot:
        freq, amp = llama3_freq(rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate_pairs(q, pos, freq, amp), rotate_pairs(k, pos, freq, amp)
    q, k = q.view(T, H, 2, d), k.view(T, G, 2, d)
    v = (h @ w[p + "v"].T).view(T, G, vd)
    k_all = torch.cat([state.get("k", k[:0]), k], 0)
    v_all = torch.cat([state.get("v", v[:0]), v], 0)
    state["k"], state["v"] = k_all, v_all
    P = k_all.shape[0] - T
    lam = differential_lambda(w, p, m["diff"])
    mask = visible(P, T, (m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, vd, dtype=F64)
    for hq in range(H):
        g = hq // (H // G)
        maps = [masked_softmax(q[:, hq, a] @ k_all[:, g, a].T * m["scale"], mask) @ v_all[:, g] for a in range(2)]
        out[:, hq] = rms_div(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    return out.reshape(T, H * vd) @ w[p + "o"].T


def hgrn2(h, w, p, m, eps, state):
    """state: {"S": [H, dim, vdim]}; rows of S belong to the query's channels."""
    T, H, d, vd = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, vd)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[p + "f"].T + w[p + "f.b"])).view(T, H, d)
    S = state.get("S", torch.zeros(H, d, vd, dtype=F64))
    out = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    state["S"] = S
    return rms_norm(out, w[p + "norm"], eps).reshape(T, H * vd) @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------ the model
def layer_runs(cfg):
    """(layer, pass number or None) per run: the looped block ``times`` times in a row; the pass number marks a pass's first layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


class Oracle:
    """Feeds portions of one sequence; keeps the sequence's state between calls."""

    def __init__(self, cfg, weights):
        self.cfg = cfg
        self.w = {k: v.to(F64) for k, v in weights.items()}
        self.runs = layer_runs(cfg)
        self.state = [dict() for _ in self.runs]
        self.n = 0

    def forward(self, tokens, trace=None):
        """logits [T, vocab] of the next ``tokens``; ``trace`` receives the stream after every layer run."""
        cfg, w, eps = self.cfg, self.w, cfg_eps(self.cfg)
        T = len(tokens)
        pos = torch.arange(self.n, self.n + T)
        self.n += T
        x0 = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"] + w["pos"][pos]
        x = x0
        for r, (li, t) in enumerate(self.runs):
            if t is not None:
                x = torch.cat([x, x0], -1) @ w["loop.in"].T + w["loop.step"][t]
            l, p = cfg["layers"][li], f"l{li}."
            h = rms_norm_around_zero(x, w[p + "norm1"], eps)
            if l["type"] == "latent_attention":
                y = latent_attention(h, pos, w, p + "mix.", l["mixer"], eps, self.state[r])
            elif l["type"] == "attention":
                y = differential_attention(h, pos, w, p + "mix.", l["mixer"], eps, self.state[r])
            elif l["type"] == "hgrn2":
                y = hgrn2(h, w, p + "mix.", l["mixer"], eps, self.state[r])
            else:
                raise ValueError(l["type"])
            x = x + y
            if l.get("mlp") is not None:
                x = x + moe(rms_norm_around_zero(x, w[p + "norm2"], eps), w, p + "mlp.", l["mlp"])
            if trace is not None:
                trace.append(x.clone())
        z = rms_norm_around_zero(x, w["final.norm"], eps) @ w["head"].T
        cap = cfg.get("logit_softcap")
        return cap * torch.tanh(z / cap) if cap else z


def cfg_eps(cfg):
    return cfg["norm"]["eps"]


# ------------------------------------------------------------------------------------------------ weights for the tests
def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "pos": (cfg["max_positions"], W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("loop"):
        out["loop.in"], out["loop.step"] = (W, 2 * W), (cfg["loop"]["times"], W)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        out[p + "norm1"] = (W,)
        H, d, v = m["heads"], m["dim"], m["vdim"]
        if l["type"] == "latent_attention":
            r, c, qr = m["rot_dim"], m["kv_rank"], m["q_rank"]
            for k, shp in (("dq", (qr, W)), ("dq.norm", (qr,)), ("uq", (H * (d + r), qr)), ("dkv", (c + r, W)), ("dkv.norm", (c,)), ("uk", (H * d, c)),
                           ("uv", (H * v, c)), ("g", (H * v, W)), ("o", (W, H * v))):
                out[p + "mix." + k] = shp
        elif l["type"] == "attention":
            G = m.get("kv_heads", H)
            for k, shp in (("q", (2 * H * d, W)), ("k", (2 * G * d, W)), ("v", (G * v, W)), ("lq1", (d,)), ("lk1", (d,)), ("lq2", (d,)), ("lk2", (d,)),
                           ("o", (W, H * v))):
                out[p + "mix." + k] = shp
        else:
            for k, shp in (("q", (H * d, W)), ("f", (H * d, W)), ("f.b", (H * d,)), ("lower", (H * d,)), ("v", (H * v, W)), ("norm", (v,)), ("o", (W, H * v))):
                out[p + "mix." + k] = shp
        if l.get("mlp") is not None:
            out[p + "norm2"] = (W,)
            f, E = l["mlp"]["expert"]["ff"], l["mlp"]["router"]["experts"]
            for e in range(E):
                out[p + f"mlp.e{e}.gate"], out[p + f"mlp.e{e}.up"], out[p + f"mlp.e{e}.down"] = (f, W), (f, W), (W, f)
            out[p + "mlp.router"] = (E, W)
    return out


def random_weights(cfg, seed, std_scale=1.0):
    """bf16-representable fp32 tensors: projections N(0, std_scale / sqrt(inputs)), norm weights around their neutral value, gate
    bounds in (0, 0.95), routers sharp enough that choices are no close calls."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shp in tensor_shapes(cfg).items():
        if name == "embed":
            t = torch.randn(shp, generator=g)
        elif name == "pos":
            t = 0.5 * torch.randn(shp, generator=g)
        elif name.endswith(".lower"):
            t = 0.95 * torch.rand(shp, generator=g)
        elif name.endswith("router"):
            t = 3.0 * torch.randn(shp, generator=g) * shp[1] ** -0.5
        elif name == "loop.in":
            t = torch.randn(shp, generator=g) * (2.0 / shp[1]) ** 0.5
        elif len(shp) == 2 and name != "loop.step":
            t = torch.randn(shp, generator=g) * std_scale * shp[1] ** -0.5
        elif name.endswith((".dq.norm", ".dkv.norm", "mix.norm")):
            t = 1.0 + 0.2 * torch.randn(shp, generator=g)
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            t = 0.4 * torch.randn(shp, generator=g)
        else:                                           # norm weights that are offsets from one, the gate's bias, the passes' step vectors
            t = 0.3 * torch.randn(shp, generator=g)
        out[name] = t.to(torch.bfloat16).float()
    return out


def logits_of(cfg, weights, tokens, trace=None):
    with torch.no_grad():
        return Oracle(cfg, weights).forward(tokens, trace)
