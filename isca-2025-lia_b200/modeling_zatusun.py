"""Zatusun: a pre-norm decoder-only language model with learned positions that mixes three kinds of sequence mixer -- attention
over a latent key/value cache with latent queries, a pairwise rotation with interpolated ("YaRN") frequencies and a per-channel
output gate; differential attention (two softmax maps over shared values) with grouped heads under a chunked mask; and the
forget-gate linear recurrence of HGRN2 -- each followed by a routed mixture of clamped gated experts, on a 32-bit residual stream,
with a block of layers that is run several times over (same weights, separate state per pass) behind an input projection that
sees the stream and the embedding side by side.

    x0 = embed[token] * scale + pos[position];  x = x0
    per layer run:  (first layer of a pass t:  x = Win [x ; x0] + step[t])
                    x += mixer(N1(x));   if the layer has a feed-forward:  x += ff(N2(x))
    logits = cap * tanh(head(Nf(x)) / cap)                 N(x) = x / rms(x) * (1 + w)

``config.json`` gives every size and constant (``ZatusunConfig``); tensor names are ``embed``, ``pos``, ``loop.in``, ``loop.step``,
``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.  The mixers and the feed-forward are the general ones
of ``seq_layers``; per-sequence state lives in a ``seq_state.SlotState``; serving goes through ``engine.Engine`` (the model only
implements ``new_state`` and ``forward_rows``).

dtype bfloat16: projections and their activations in bf16 with fp32 accumulation; positions and angles, norms, routers, gates of
the recurrence and its state, attention scores, weights and sums, and the residual stream in fp32.  dtype float32: everything in
true fp32.
"""
import json
import os
from dataclasses import dataclass, field

import torch

from . import _lib, ops
from .seq_layers import (DifferentialAttentionMixer, ForgetGateLinearAttentionMixer, LatentAttentionMixer, Linear, MoEFeedForward)
from .seq_state import SlotState

BF16, F32 = torch.bfloat16, torch.float32
MIXERS = ("latent_attention", "attention", "hgrn2")
EXPERT_ALPHA = 1.702            # the experts' gate is g * sigmoid(1.702 g): fixed by the design


@dataclass
class ZatusunConfig:
    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    layers: list = field(default_factory=list)          # dicts: type, mixer {...}, mlp {...} | None
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0                                 # 0: no looped block (no input projection either)
    norm_eps: float = 1e-6
    embed_scale: float = 1.0
    logit_softcap: float = 0.0                          # 0: none
    name: str = "zatusun"
    architectures: list = field(default_factory=lambda: ["Zatusun"])
    eos_token_id: int = -1

    @classmethod
    def from_dict(cls, c, name="zatusun"):
        layers = c["layers"]
        for i, l in enumerate(layers):
            if l.get("type") not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {l.get('type')!r} (known: {MIXERS})")
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            m = l["mixer"]
            if l["type"] == "attention":
                m.setdefault("kv_heads", m["heads"])
                if m["heads"] % m["kv_heads"]:
                    raise ValueError(f"layer {i}: {m['heads']} heads do not divide into {m['kv_heads']} groups")
            if l["type"] == "latent_attention" and m["rot"]["dims"] > m["rot_dim"]:
                raise ValueError(f"layer {i}: rot.dims {m['rot']['dims']} exceeds rot_dim {m['rot_dim']}")
        loop = c.get("loop")
        start = stop = times = 0
        if loop:
            start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ValueError(f"bad loop {loop} for {len(layers)} layers")
            if start == stop:                           # a block without layers: no pass ever begins
                start = stop = times = 0
        return cls(vocab=int(c["vocab"]), width=int(c["width"]), max_positions=int(c["max_positions"]), layers=layers, loop_start=start,
                   loop_stop=stop, loop_times=times, norm_eps=float(c["norm"]["eps"]), embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)),
                   logit_softcap=float(c.get("logit_softcap") or 0.0), name=name)

    def to_dict(self):
        d = {"architecture": "Zatusun", "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions, "layers": self.layers,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embed_scale}}
        if self.loop_times:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d

    def layer_runs(self):
        """(layer index, pass number or None) of every run, in order: the layers before the loop once, the looped block ``times``
        times in a row, the rest once.  The pass number marks the first layer of every pass (the first pass too): the input
        projection and that pass's step vector come right before it."""
        if not self.loop_times:
            return [(i, None) for i in range(len(self.layers))]
        runs = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            runs += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, None) for i in range(self.loop_stop, len(self.layers))]

    def tensor_shapes(self):
        """name -> shape of every tensor of a checkpoint of this configuration."""
        W, V = self.width, self.vocab
        out = {"embed": (V, W), "pos": (self.max_positions, W), "final.norm": (W,), "head": (V, W)}
        if self.loop_times:
            out.update({"loop.in": (W, 2 * W), "loop.step": (self.loop_times, W)})
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            out[p + "norm1"] = (W,)
            H, d, v = m["heads"], m["dim"], m["vdim"]
            if l["type"] == "latent_attention":
                r, c, qr = m["rot_dim"], m["kv_rank"], m["q_rank"]
                out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + r), qr), p + "mix.dkv": (c + r, W),
                            p + "mix.dkv.norm": (c,), p + "mix.uk": (H * d, c), p + "mix.uv": (H * v, c), p + "mix.g": (H * v, W),
                            p + "mix.o": (W, H * v)})
            elif l["type"] == "attention":
                G = m["kv_heads"]
                out.update({p + "mix.q": (H * 2 * d, W), p + "mix.k": (G * 2 * d, W), p + "mix.v": (G * v, W), p + "mix.lq1": (d,),
                            p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,), p + "mix.o": (W, H * v)})
            else:
                out.update({p + "mix.q": (H * d, W), p + "mix.f": (H * d, W), p + "mix.f.b": (H * d,), p + "mix.lower": (H * d,),
                            p + "mix.v": (H * v, W), p + "mix.norm": (v,), p + "mix.o": (W, H * v)})
            mlp = l.get("mlp")
            if mlp is None:
                continue
            out[p + "norm2"] = (W,)
            f = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out.update({p + f"mlp.e{e}.gate": (f, W), p + f"mlp.e{e}.up": (f, W), p + f"mlp.e{e}.down": (W, f)})
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
        return out


class _Layer:
    def __init__(self, mixer, mlp, norm1, norm2):
        self.mixer, self.mlp, self.norm1, self.norm2 = mixer, mlp, norm1, norm2      # norm weights as 1 + w, fp32


class ZatusunForCausalLM:
    step_serving = True          # served through engine.Engine (requests, slots, portions)

    def __init__(self, config, device="cuda", dtype=BF16):
        _lib.load()
        if dtype not in (BF16, F32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.config, self.device, self.dtype = config, torch.device(device), dtype
        self.layers = []
        self.runs = config.layer_runs()
        self.embed = self.pos = self.head = self.final_norm = self.loop_in = self.loop_step = None

    # ---- weights
    def load_weights(self, get):
        """``get(name)`` -> CPU tensor (checkpoint dtype).  Projection weights and the two embedding tables take the model's dtype;
        norm weights (the checkpoint holds w, the model keeps 1 + w), biases, gate bounds and step vectors stay fp32."""
        cfg, dev, dt = self.config, self.device, self.dtype
        shapes = cfg.tensor_shapes()

        def fetch(name):
            t = get(name)
            if tuple(t.shape) != tuple(shapes[name]):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration needs {tuple(shapes[name])}")
            return t.float()

        def norm(name):
            return (1.0 + fetch(name)).to(dev).contiguous()

        self.embed = fetch("embed").to(device=dev, dtype=dt).contiguous()
        self.pos = fetch("pos").to(device=dev, dtype=dt).contiguous()
        self.head = Linear([fetch("head")], dt, dev)
        self.final_norm = norm("final.norm")
        if cfg.loop_times:
            self.loop_in = Linear([fetch("loop.in")], dt, dev)
            self.loop_step = fetch("loop.step").to(dev).contiguous()
        self.layers = []
        for i, l in enumerate(cfg.layers):
            p, m = f"l{i}.", l["mixer"]
            w = {k[len(p) + 4:]: fetch(k) for k in shapes if k.startswith(p + "mix.")}
            if l["type"] == "latent_attention":
                rot = m["rot"]
                mixer = LatentAttentionMixer(w, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], rot["dims"], rot["base"], m["scale"],
                                             cfg.norm_eps, dt, dev, q_rank=m["q_rank"], rot_pairs=True, rot_scaling=rot.get("scaling"), gate="channel")
            elif l["type"] == "attention":
                mixer = DifferentialAttentionMixer(w, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m["diff"], cfg.norm_eps, dt, dev,
                                                   rot=m.get("rot"), chunk=(m.get("mask") or {}).get("size", 0))
            else:
                mixer = ForgetGateLinearAttentionMixer(w, m["heads"], m["dim"], m["vdim"], cfg.norm_eps, dt, dev)
            mlp, n2 = None, None
            spec = l.get("mlp")
            if spec is not None:
                q = p + "mlp."
                experts = [{k: fetch(q + f"e{e}." + k) for k in ("gate", "up", "down")} for e in range(spec["router"]["experts"])]
                mlp = MoEFeedForward(fetch(q + "router"), experts, spec["router"]["top"], spec["expert"]["ff"], ops.ACT_CLAMPED_SWISH, None, dt, dev,
                                     renorm=True, act_params=(spec["expert"]["limit"], EXPERT_ALPHA))
                n2 = norm(p + "norm2")
            self.layers.append(_Layer(mixer, mlp, norm(p + "norm1"), n2))
        return self

    def init_weights(self, seed=0, std=None):
        """Random weights (bf16-representable) for tests and benchmarks: N(0, K^-1/2) projections, norm weights near their
        neutral value (0 for the norms whose weight is an offset from one, 1 for the plain ones), small biases and vectors, lower bounds in (0, 1)."""
        g = torch.Generator().manual_seed(seed)
        shapes = self.config.tensor_shapes()

        def make(name):
            shp = shapes[name]
            if name in ("embed", "pos"):
                t = torch.randn(shp, generator=g) * (0.5 if name == "pos" else 1.0)
            elif name.endswith(".lower"):
                t = torch.rand(shp, generator=g) * 0.9
            elif len(shp) == 2 and name != "loop.step":
                t = torch.randn(shp, generator=g) * (std if std is not None else shp[1] ** -0.5)
            elif name.endswith((".dq.norm", ".dkv.norm", "mix.norm")):
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
                t = 0.3 * torch.randn(shp, generator=g)
            else:                                    # norms around zero, biases, step vectors
                t = 0.1 * torch.randn(shp, generator=g)
            return t.to(BF16)

        cache = {}
        return self.load_weights(lambda n: cache.setdefault(n, make(n)))

    @classmethod
    def from_pretrained(cls, path, device="cuda", dtype=BF16, **unused):
        from .checkpoint import SafetensorsFile
        c = json.load(open(os.path.join(path, "config.json")))
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        if "max_positions" not in c and "pos" in f.header:         # the table's own height says how far positions go
            c["max_positions"] = int(f.header["pos"]["shape"][0])
        cfg = ZatusunConfig.from_dict(c, name=os.path.basename(os.path.abspath(path)) or "zatusun")
        try:
            return cls(cfg, device, dtype).load_weights(f.get)
        finally:
            f.close()

    def eval(self):
        return self

    # ---- serving interface (engine.Engine)
    def new_state(self, n_slots, capacity):
        """A sequence cannot grow past the position table."""
        slots = SlotState(n_slots, min(int(capacity), self.config.max_positions), self.device)
        slots.run_state = [self.layers[i].mixer.new_state(slots) for i, _ in self.runs]      # one state per layer RUN
        return slots

    def forward_rows(self, ids, batch, want, slots, trace=None):
        """One step: ``ids`` int64 [rows] on the device, ``batch`` a StepBatch, ``want`` int32 row indices (device) whose
        logits are returned as fp32 [len(want), vocab] (None when empty).  ``trace``: a list that receives a copy of the
        residual stream after every layer run."""
        cfg, dev, dt = self.config, self.device, self.dtype
        M, W, eps = batch.rows, cfg.width, cfg.norm_eps
        x = torch.empty(M, W, dtype=F32, device=dev)
        h = torch.empty(M, W, dtype=dt, device=dev)
        # [x ; x0] in the projections' dtype, the input of a pass's projection: the right half stays the embedding, the left
        # half is written by the residual update that precedes a pass
        cat = torch.empty(M, 2 * W, dtype=dt, device=dev) if cfg.loop_times else None
        ops.embed_scale_pos(ids, self.embed, self.pos, cfg.embed_scale, batch.meta, x, cat)
        if self.runs and self.runs[0][1] is None:
            ops.residual_norm(x, None, self.layers[self.runs[0][0]].norm1, h, eps)
        for r, (li, t) in enumerate(self.runs):
            layer = self.layers[li]
            if t is not None:                            # a pass begins: x = Win [x ; x0] + step[t], then this layer's first norm
                ops.residual_norm(x, self.loop_in(cat), layer.norm1, h, eps, replace=True, bias=self.loop_step[t])
            y = layer.mixer(h, batch, slots.run_state[r])
            if layer.mlp is not None:
                ops.residual_norm(x, y, layer.norm2, h, eps)
                y = layer.mlp(h)
            # the last residual update of the run also makes what the next run reads: its first norm, or (before a pass) the
            # stream itself in the projections' dtype
            if r + 1 == len(self.runs):
                ops.residual_norm(x, y, None, None, eps)
            elif self.runs[r + 1][1] is not None:
                ops.residual_norm(x, y, None, cat[:, :W], eps)
            else:
                ops.residual_norm(x, y, self.layers[self.runs[r + 1][0]].norm1, h, eps)
            if trace is not None:
                trace.append(x.clone())
        if want is None or want.numel() == 0:
            return None
        n = want.numel()
        hn = torch.empty(n, W, dtype=dt, device=dev)
        ops.rms_gather(x, want, self.final_norm, hn, eps)
        logits = torch.empty(n, cfg.vocab, dtype=F32, device=dev)
        ops.linear_plain(hn, self.head.weight, logits)
        if cfg.logit_softcap > 0:
            ops.softcap(logits, cfg.logit_softcap)
        return logits

    def graph_class(self, max_ctx):
        """What a decode pass's launches depend on besides the contents of the static buffers: the number of key ranges each
        kind of attention splits the longest history into."""
        key = set()
        for l in self.layers:
            if isinstance(l.mixer, LatentAttentionMixer):
                key.add(("latent", ops.latent_attn_split_class(max_ctx)))
            elif isinstance(l.mixer, DifferentialAttentionMixer):
                key.add(("maps", ops.window_attn_split_class(max_ctx, l.mixer.span or (1 << 30))))
        return tuple(sorted(key))

    def generate(self, input_ids, max_new_tokens=32, chunk=None, **unused):
        """Greedy generation of a batch of prompts through the step engine; returns ids [B, S + new] on the input's device."""
        from .engine import Engine
        prompts = [[int(t) for t in row] for row in input_ids.tolist()]
        eng = Engine(self, max_tokens=len(prompts[0]) + max_new_tokens, max_requests=len(prompts))
        out = eng.generate(prompts, max_new_tokens, chunk=chunk)
        return torch.tensor(out, dtype=torch.int64, device=input_ids.device)
