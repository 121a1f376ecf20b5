"""Bizetar: a decoder-only language model whose sublayers read the 32-bit residual stream itself and are normed, and gated,
on their OUTPUT, and whose layers hand on a learned mix of every earlier layer's result instead of the last one.

    X_0 = RMS(embed[token]; embed.norm);  x = X_0
    per layer i:   a   = mixer(x) * sigmoid(rg1 x + rg1.b);      x' = x + RMS(a; norm1)
                   b   = ff(x') * sigmoid(rg2 x' + rg2.b);       X_(i+1) = x' + RMS(b; norm2)        (no ff: X_(i+1) = x')
                   x   = sum_(j <= i+1) dwa_i[j] X_j
    logits = head RMS(x; final.norm)

Two mixers, both causal softmax attention over the whole history with grouped key/value heads and a sink per head in the
softmax's denominator (``seq_layers.SinkAttentionMixer`` with different options):
  ``attention``    one RMS norm over the whole query projection and one over the whole key projection, a query temperature
                   that grows with the logarithm of the position, no rotation but a per-head distance bias
                   (head n of H, counted from 1, takes 2^(-8n/H) off a score per position between query and key), and one
                   output gate per head;
  ``attention_2``  projections with biases behind a short causal convolution, a norm per head, rotated channel pairs with
                   interpolated frequencies, and one output gate per channel.
Layers that say ``v_mix`` blend their values with those of the first such layer (same token) before caching them.
Feed-forwards: dense with a polynomial activation between norms (``PolyNormMLP``), or a routed mixture of gated SiLU experts
whose router adds a correction for the choice only, does not renormalise the chosen scores and ends in ``identity`` experts
that hand the token back (``MoEFeedForward``).

``config.json`` gives every size and constant (``BizetarConfig``); tensor names are ``embed``, ``embed.norm``, ``l<i>.norm1|norm2``,
``l<i>.rg1|rg2`` (+ ``.b``), ``l<i>.dwa``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.  Per-sequence state lives in
a ``seq_state.SlotState``; serving goes through ``engine.Engine`` (the model only implements ``new_state`` and ``forward_rows``).

dtype bfloat16: projections and caches in bf16 with fp32 accumulation; positions, angles, norms, routers, attention scores and
weights, the polynomial activation's norms and the residual stream in fp32.  dtype float32: everything in true fp32.
"""
import json
import os
from dataclasses import dataclass, field

import torch

from . import _lib, ops
from .seq_layers import Linear, MoEFeedForward, PolyNormMLP, SinkAttentionMixer
from .seq_state import SlotState

BF16, F32 = torch.bfloat16, torch.float32
MIXERS = ("attention", "attention_2")
MLP_KINDS = ("dense", "moe")


@dataclass
class BizetarConfig:
    vocab: int = 0
    width: int = 0
    layers: list = field(default_factory=list)          # dicts: type, mixer {...}, mlp {...} | None
    norm_eps: float = 1e-6
    name: str = "bizetar"
    architectures: list = field(default_factory=lambda: ["Bizetar"])
    eos_token_id: int = -1

    @classmethod
    def from_dict(cls, c, name="bizetar"):
        layers = c["layers"]
        for i, l in enumerate(layers):
            if l.get("type") not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {l.get('type')!r} (known: {MIXERS})")
            mlp = l.get("mlp")
            if mlp is not None:
                mlp.setdefault("kind", "moe" if "router" in mlp else "dense")
                if mlp["kind"] not in MLP_KINDS:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r} (known: {MLP_KINDS})")
                if mlp["kind"] == "moe":
                    r = mlp["router"]
                    r.setdefault("identity", 0)
                    if not 1 <= r["top"] <= r["experts"] + r["identity"] or r["experts"] < 1:
                        raise ValueError(f"layer {i}: router takes {r['top']} of {r['experts']} + {r['identity']} experts")
            m = l["mixer"]
            m.setdefault("vdim", m["dim"])
            m.setdefault("kv_heads", m["heads"])
            if m["heads"] % m["kv_heads"]:
                raise ValueError(f"layer {i}: {m['heads']} heads do not divide into {m['kv_heads']} groups")
            rot = m.get("rot")
            if rot is not None and (rot["dims"] % 2 or not 0 < rot["dims"] <= m["dim"]):
                raise ValueError(f"layer {i}: cannot rotate {rot['dims']} of {m['dim']} channels")
        widths = {l["mixer"]["kv_heads"] * l["mixer"]["vdim"] for l in layers if l["mixer"].get("v_mix")}
        if len(widths) > 1:
            raise ValueError(f"layers that mix values must agree on kv_heads * vdim, got {sorted(widths)}")
        return cls(vocab=int(c["vocab"]), width=int(c["width"]), layers=layers, norm_eps=float(c["norm"]["eps"]), name=name)

    def to_dict(self):
        return {"architecture": "Bizetar", "vocab": self.vocab, "width": self.width, "layers": self.layers, "norm": {"eps": self.norm_eps}}

    def first_mixing_layer(self):
        """Index of the first layer that says ``v_mix`` (its values are the ones later layers blend in), or None."""
        return next((i for i, l in enumerate(self.layers) if l["mixer"].get("v_mix")), None)

    def tensor_shapes(self):
        """name -> shape of every tensor of a checkpoint of this configuration."""
        W, V = self.width, self.vocab
        out = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,), "head": (V, W)}
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "norm1": (W,), p + "rg1": (W, W), p + "rg1.b": (W,), p + "dwa": (i + 2,),
                        p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * v, W), p + "mix.sink": (H,), p + "mix.o": (W, H * v)})
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
            if l["type"] == "attention":
                out.update({p + "mix.q.norm": (H * d,), p + "mix.k.norm": (G * d,), p + "mix.g": (H, W)})
            else:
                out.update({p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.g": (H * v, W),
                            p + "mix.q.b": (H * d,), p + "mix.k.b": (G * d,), p + "mix.v.b": (G * v,)})
                taps = m.get("conv")
                if taps:
                    out.update({p + "mix.q.conv": (H * d, taps), p + "mix.k.conv": (G * d, taps), p + "mix.v.conv": (G * v, taps)})
            mlp = l.get("mlp")
            if mlp is None:
                continue
            out.update({p + "norm2": (W,), p + "rg2": (W, W), p + "rg2.b": (W,)})
            if mlp["kind"] == "dense":
                f = mlp["ff"]
                out.update({p + "mlp.up": (f, W), p + "mlp.down": (W, f), p + "mlp.act": (4,)})
            else:
                f, r = mlp["expert"]["ff"], mlp["router"]
                for e in range(r["experts"]):
                    out.update({p + f"mlp.e{e}.gate": (f, W), p + f"mlp.e{e}.up": (f, W), p + f"mlp.e{e}.down": (W, f)})
                out[p + "mlp.router"] = (r["experts"] + r["identity"], W)
                out[p + "mlp.correction"] = (r["experts"] + r["identity"],)
        return out


def distance_slopes(heads):
    """What each head takes off a score per position of distance: head n of H, counted from 1, takes 2^(-8n/H)."""
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


class _Prefixed:
    """``w[name]`` -> the checkpoint's tensor ``prefix + name``, read when it is asked for."""

    def __init__(self, fetch, prefix):
        self.fetch, self.prefix = fetch, prefix

    def __getitem__(self, name):
        return self.fetch(self.prefix + name)


class _Layer:
    def __init__(self, mixer, mlp, norm1, norm2, rg1_b, rg2, rg2_b, dwa):
        self.mixer, self.mlp, self.norm1, self.norm2 = mixer, mlp, norm1, norm2
        self.rg1_b, self.rg2, self.rg2_b, self.dwa = rg1_b, rg2, rg2_b, dwa     # rg2: its own projection when the feed-forward cannot carry it


class BizetarForCausalLM:
    step_serving = True          # served through engine.Engine (requests, slots, portions)

    def __init__(self, config, device="cuda", dtype=BF16):
        _lib.load()
        if dtype not in (BF16, F32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.config, self.device, self.dtype = config, torch.device(device), dtype
        self.layers = []
        self.embed = self.embed_norm = self.head = self.final_norm = None

    # ---- weights
    def load_weights(self, get):
        """``get(name)`` -> CPU tensor (checkpoint dtype).  Projection weights take the model's dtype; norm weights, biases and
        the small per-head vectors stay fp32.  The residual gate of a sublayer rides on that sublayer's first projection."""
        cfg, dev, dt = self.config, self.device, self.dtype
        shapes = cfg.tensor_shapes()

        def fetch(name):
            t = get(name)
            if tuple(t.shape) != tuple(shapes[name]):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration needs {tuple(shapes[name])}")
            return t.float()

        def vec(name):
            return fetch(name).to(dev).contiguous()

        self.embed = fetch("embed").to(device=dev, dtype=dt).contiguous()
        self.embed_norm = vec("embed.norm")
        self.head = Linear([fetch("head")], dt, dev)
        self.final_norm = vec("final.norm")
        first_mix = cfg.first_mixing_layer()
        self.layers = []
        for i, l in enumerate(cfg.layers):
            p, m = f"l{i}.", l["mixer"]
            w = _Prefixed(fetch, p + "mix.")              # the mixer asks for the tensors its options need, and no others
            v_mix = None if not m.get("v_mix") else ("publish" if i == first_mix else "blend")
            common = dict(norm_eps=cfg.norm_eps, dtype=dt, device=dev, v_mix=v_mix, ride_along=[fetch(p + "rg1")])
            if l["type"] == "attention":
                qt = m.get("q_temp")
                mixer = SinkAttentionMixer(w, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], norm="whole",
                                           q_temp=(qt["coef"], qt["every"]) if qt else None, slopes=distance_slopes(m["heads"]), gate="head", **common)
            else:
                mixer = SinkAttentionMixer(w, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], norm="head", biases=True,
                                           taps=m.get("conv"), rot=m.get("rot"), gate="channel", **common)
            mlp = norm2 = rg2 = rg2_b = None
            spec = l.get("mlp")
            if spec is not None:
                q = p + "mlp."
                norm2, rg2_b = vec(p + "norm2"), vec(p + "rg2.b")
                if spec["kind"] == "dense":
                    mlp = PolyNormMLP({k: fetch(q + k) for k in ("up", "down", "act")}, spec["ff"], cfg.norm_eps, dt, dev, ride_along=[fetch(p + "rg2")])
                else:
                    r = spec["router"]
                    experts = [{k: fetch(q + f"e{e}." + k) for k in ("gate", "up", "down")} for e in range(r["experts"])]
                    mlp = MoEFeedForward(fetch(q + "router"), experts, r["top"], spec["expert"]["ff"], ops.ACT_SILU, None, dt, dev,
                                         correction=fetch(q + "correction"), renorm=False, identity=r["identity"])
                    rg2 = Linear([fetch(p + "rg2")], dt, dev)
            self.layers.append(_Layer(mixer, mlp, vec(p + "norm1"), norm2, vec(p + "rg1.b"), rg2, rg2_b, vec(p + "dwa")))
        return self

    def init_weights(self, seed=0, std=None):
        """Random weights (bf16-representable) for tests and benchmarks: N(0, K^-1/2) projections, norm weights near 1, biases,
        sinks and corrections near 0, mixing weights that sum to about 1."""
        g = torch.Generator().manual_seed(seed)
        shapes = self.config.tensor_shapes()

        def make(name):
            shp = shapes[name]
            if name.endswith(".conv"):
                t = torch.randn(shp, generator=g) * 0.5
            elif name.endswith(".dwa"):
                t = torch.full(shp, 1.0 / shp[0]) + 0.1 * torch.randn(shp, generator=g)
            elif name.endswith(".vmix"):
                t = torch.rand(shp, generator=g) * 0.5 + 0.2
            elif name.endswith(".act"):
                t = torch.tensor([1.0, 0.5, 0.25, 0.0]) + 0.1 * torch.randn(shp, generator=g)
            elif name.endswith(".correction"):
                t = 0.02 * torch.randn(shp, generator=g)
            elif len(shp) == 2:
                t = torch.randn(shp, generator=g) * (std if std is not None else shp[1] ** -0.5)
            elif name.endswith((".b", ".sink")):
                t = 0.5 * torch.randn(shp, generator=g)
            else:
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            return t.to(BF16)

        cache = {}
        return self.load_weights(lambda n: cache.setdefault(n, make(n)))

    @classmethod
    def from_pretrained(cls, path, device="cuda", dtype=BF16, **unused):
        from .checkpoint import SafetensorsFile
        cfg = BizetarConfig.from_dict(json.load(open(os.path.join(path, "config.json"))),
                                      name=os.path.basename(os.path.abspath(path)) or "bizetar")
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        try:
            return cls(cfg, device, dtype).load_weights(f.get)
        finally:
            f.close()

    def eval(self):
        return self

    # ---- serving interface (engine.Engine)
    def new_state(self, n_slots, capacity):
        slots = SlotState(n_slots, capacity, self.device)
        slots.run_state = [layer.mixer.new_state(slots) for layer in self.layers]
        return slots

    def forward_rows(self, ids, batch, want, slots, trace=None):
        """One step: ``ids`` int64 [rows] on the device, ``batch`` a StepBatch, ``want`` int32 row indices (device) whose
        logits are returned as fp32 [len(want), vocab] (None when empty).  ``trace``: a list that receives a copy of what
        every layer hands on."""
        cfg, dev, dt = self.config, self.device, self.dtype
        M, W, eps, L = batch.rows, cfg.width, cfg.norm_eps, len(self.layers)
        stack = torch.empty(L + 1, M, W, dtype=F32, device=dev)           # X_0 and every layer's own result
        x = torch.empty(M, W, dtype=F32, device=dev)
        h = torch.empty(M, W, dtype=dt, device=dev)
        ops.embed_rmsnorm(ids, self.embed, self.embed_norm, x, eps)
        ops.gated_rms_add(x, None, None, h, eps, stack=stack, n_mix=1, mix=self._one(dev))     # X_0 = x joins the stack, h = x in the model's dtype
        for i, layer in enumerate(self.layers):
            extras = []
            y = layer.mixer(h, batch, slots.run_state[i], extras)
            last = dict(stack=stack, n_mix=i + 2, mix=layer.dwa)         # the layer's result joins the stack and the mix goes on
            if layer.mlp is None:
                ops.gated_rms_add(x, y, layer.norm1, h, eps, gate=extras[0], gate_bias=layer.rg1_b, **last)
            else:
                ops.gated_rms_add(x, y, layer.norm1, h, eps, gate=extras[0], gate_bias=layer.rg1_b)
                extras = []
                if layer.rg2 is not None:
                    extras.append(layer.rg2(h))
                    y = layer.mlp(h, router_input=x)             # the router reads the fp32 stream itself
                else:
                    y = layer.mlp(h, extras)
                ops.gated_rms_add(x, y, layer.norm2, h, eps, gate=extras[0], gate_bias=layer.rg2_b, **last)
            if trace is not None:
                trace.append(x.clone())
        if want is None or want.numel() == 0:
            return None
        n = want.numel()
        hn = torch.empty(n, W, dtype=dt, device=dev)
        ops.rms_gather(x, want, self.final_norm, hn, eps)
        logits = torch.empty(n, cfg.vocab, dtype=F32, device=dev)
        ops.linear_plain(hn, self.head.weight, logits)
        return logits

    def _one(self, dev):
        if getattr(self, "_one_t", None) is None:
            self._one_t = torch.ones(1, dtype=F32, device=dev)
        return self._one_t

    def graph_class(self, max_ctx):
        """What a decode pass's launches depend on besides the contents of the static buffers: the number of key ranges the
        attention splits the longest history into."""
        return ops.window_attn_split_class(max_ctx, 1 << 30)

    def generate(self, input_ids, max_new_tokens=32, chunk=None, **unused):
        """Greedy generation of a batch of prompts through the step engine; returns ids [B, S + new] on the input's device."""
        from .engine import Engine
        prompts = [[int(t) for t in row] for row in input_ids.tolist()]
        eng = Engine(self, max_tokens=len(prompts[0]) + max_new_tokens, max_requests=len(prompts))
        out = eng.generate(prompts, max_new_tokens, chunk=chunk)
        return torch.tensor(out, dtype=torch.int64, device=input_ids.device)
