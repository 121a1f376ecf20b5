"""CPU-side checks of the Bizetar integration: configuration, tensor table, registry, the rotation's frequency table, and the
oracle's own consistency (a prompt fed whole, in portions and token by token gives the same logits; the sink, the distance bias,
the router's correction and the identity experts behave as stated)."""
import copy
import json
import math

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import registry
from lia_b200.modeling_bizetar import BizetarConfig, distance_slopes
from lia_b200.seq_layers import scaled_rotary_freq

import bizetar_oracle as O
from bizetar_cases import CASES, attention, attention_2, config, dense, moe


def cfg_of(c):
    return BizetarConfig.from_dict(copy.deepcopy(c))


def test_shapes_and_the_first_mixing_layer():
    for name in CASES:
        c = cfg_of(CASES[name])
        assert c.tensor_shapes() == O.tensor_shapes(CASES[name])
        assert cfg_of(c.to_dict()).tensor_shapes() == c.tensor_shapes()
    assert cfg_of(CASES["even"]).first_mixing_layer() == 1 and cfg_of(CASES["odd"]).first_mixing_layer() is None
    assert cfg_of(CASES["wide"]).first_mixing_layer() == 0
    s = cfg_of(CASES["even"]).tensor_shapes()
    assert s["l0.mix.q"] == (64, 64) and s["l0.mix.v.conv"] == (48, 4) and s["l0.mix.q.norm"] == (16,) and s["l0.mix.g"] == (96, 64)
    assert s["l1.mix.q.norm"] == (144,) and s["l1.mix.k.norm"] == (48,) and s["l1.mix.g"] == (6, 64) and s["l1.mix.vmix"] == ()
    assert "l0.mix.vmix" not in s and "l1.mix.q.b" not in s and "l1.mix.q.conv" not in s
    assert s["l1.mlp.router"] == (8, 64) and s["l1.mlp.correction"] == (8,) and s["l1.mlp.e5.gate"] == (24, 64) and "l1.mlp.e6.up" not in s
    assert s["l0.mlp.act"] == (4,) and s["l3.dwa"] == (5,) and "l4.norm2" not in s and "l4.rg2" not in s and s["l4.rg1.b"] == (64,)


def test_config_rejects_unknown_parts_and_fills_defaults():
    with pytest.raises(ValueError):
        cfg_of(config([{"type": "mlstm", "mixer": {}, "mlp": None}], 10, 8))
    with pytest.raises(ValueError):
        cfg_of(config([attention(1, 1, 4, 4, mlp={"kind": "glu", "ff": 8})], 10, 8))
    with pytest.raises(ValueError):
        cfg_of(config([attention(3, 2, 4, 4)], 10, 8))
    with pytest.raises(ValueError):
        cfg_of(config([attention_2(2, 1, 8, 4, rot_dims=10)], 10, 8))
    with pytest.raises(ValueError):
        cfg_of(config([attention(2, 1, 8, 4, mlp=moe(2, 4, 8, identity=1))], 10, 8))
    with pytest.raises(ValueError):        # layers that mix values must have values of one size
        cfg_of(config([attention(2, 1, 8, 4, v_mix=True), attention(2, 2, 8, 4, v_mix=True)], 10, 8))
    a = attention(4, 4, 8, 8)
    del a["mixer"]["kv_heads"], a["mixer"]["vdim"]
    a["mlp"] = {"router": {"experts": 2, "top": 1}, "expert": {"ff": 4}}
    c = cfg_of(config([a], 10, 8))
    s = c.tensor_shapes()
    assert s["l0.mix.k"] == (32, 8) and s["l0.mix.v"] == (32, 8) and s["l0.mlp.router"] == (2, 8) and c.layers[0]["mlp"]["kind"] == "moe"


def test_registry_picks_the_class_from_config_json(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(CASES["odd"]))
    assert registry.architecture_of(str(d)) == "bizetar"
    assert registry.model_class(str(d)).__name__ == "BizetarForCausalLM"
    assert registry.model_class(str(d)).step_serving


def test_frequency_table_and_slopes():
    assert distance_slopes(4) == [0.25, 0.0625, 0.015625, 0.00390625]
    f, mag = scaled_rotary_freq(8, 10000.0)
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=torch.float64))
    rot = {"dims": 16, "base": 1000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}
    f, mag = scaled_rotary_freq(16, 1000.0, rot["scaling"])
    plain = 1000.0 ** (-torch.arange(8).double() / 8)
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert f[0] == plain[0] and abs(float(f[-1]) - float(plain[-1]) / 4.0) < 1e-18         # the fastest pair as it is, the slowest divided
    assert all(plain[i] / 4.0 <= f[i] <= plain[i] for i in range(8)) and any(plain[i] / 4.0 < f[i] < plain[i] for i in range(8))
    cos, sin = O.yarn_tables(torch.tensor([3]), rot)
    assert torch.allclose(torch.cos(3 * f) * mag, cos[0], atol=1e-14) and torch.allclose(torch.sin(3 * f) * mag, sin[0], atol=1e-14)


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_portions_equal_the_whole_prompt(name):
    cfg = CASES[name]
    w = O.random_weights(cfg, 3)
    toks = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = O.forward(toks, w, cfg, O.new_state(cfg))
    for cuts in ([1] * 23, [2] * 11 + [1], [7, 1, 2, 13]):
        st, outs, at = O.new_state(cfg), [], 0
        for c in cuts:
            outs.append(O.forward(toks[at:at + c], w, cfg, st))
            at += c
        assert float((torch.cat(outs) - whole).abs().max()) < 1e-9


def test_oracle_sink_and_distance_bias():
    g = torch.Generator().manual_seed(0)
    k, v = torch.randn(9, 1, 4, generator=g).double(), torch.randn(9, 1, 4, generator=g).double()
    q = torch.zeros(1, 2, 4).double()
    pos = torch.tensor([8])
    sink = torch.tensor([0.5, -30.0]).double()
    out = O.sink_attention(q, k, v, pos, 1.0, sink)
    assert torch.allclose(out[0, 0], v[:, 0].sum(0) / (9 + math.exp(0.5)))                 # zero scores: every key weighs 1, the sink e^0.5
    assert torch.allclose(out[0, 1], v[:, 0].mean(0))                                      # a sink far below the scores does not count
    out = O.sink_attention(q, k, v, pos, 1.0, torch.tensor([-30.0, -30.0]).double(), torch.tensor([100.0, 0.0]).double())
    assert torch.allclose(out[0, 0], v[8, 0]) and torch.allclose(out[0, 1], v[:, 0].mean(0))    # a steep slope leaves the key at distance 0
    out = O.sink_attention(q, k[:4], v[:4], torch.tensor([3]), 1.0, sink)                   # causal: keys after the query do not exist yet
    assert torch.allclose(out[0, 1], v[:4, 0].mean(0))


def test_oracle_router_and_identity_experts():
    g = torch.Generator().manual_seed(2)
    h, wr = torch.randn(40, 8, generator=g).double(), torch.randn(5, 8, generator=g).double()
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 10.0]).double()
    idx, wt = O.route(h, wr, corr, 2)
    s = torch.softmax(h @ wr.T, -1)
    assert bool((idx[:, 0] == 4).all())                                                    # the correction decides the choice ...
    assert torch.allclose(wt[:, 0], s[:, 4]) and float(wt.sum(-1).max()) < 1.0             # ... but not the weight, and nothing is renormalised
    cfg = {"router": {"experts": 1, "identity": 4, "top": 2}, "expert": {"ff": 3}}
    w = {"router": wr, "correction": torch.tensor([-10.0, 0.0, 0.0, 0.0, 0.0]).double(), "e0.gate": torch.randn(3, 8, generator=g).double(),
         "e0.up": torch.randn(3, 8, generator=g).double(), "e0.down": torch.randn(8, 3, generator=g).double()}
    idx, wt = O.route(h, wr, w["correction"], 2)
    assert bool((idx >= 1).all())
    assert torch.allclose(O.moe(h, w, "", cfg), wt.sum(-1, keepdim=True) * h)              # identity experts only: the token, weighted


class _RowEcho:
    """Stands in for a model: the logits of a wanted row are its token id in every column."""

    class config:
        vocab = 50

    device = torch.device("cpu")

    def new_state(self, n, cap):
        from lia_b200.seq_state import SlotState
        return SlotState(n, cap, "cpu")

    def forward_rows(self, ids, batch, want, slots, trace=None):
        return None if want is None else ids[want.long()].float()[:, None].expand(-1, 50).contiguous()

    def graph_class(self, max_ctx):
        return 0


def test_engine_returns_wanted_places_in_the_order_asked_for():
    """Places that are not ascending, a place asked for twice, an entry that is cut into several passes, two entries."""
    from lia_b200.engine import Engine
    e = Engine(_RowEcho(), max_tokens=64, max_requests=2, max_rows=4)
    out = e.step([{"id": "x", "tokens": [10, 11, 12, 13, 14, 15, 16], "want": [6, 0, 3, 3, 5]}, {"id": "y", "tokens": [20, 21, 22], "want": [2, 1]}])
    assert out[:, 0].tolist() == [16, 10, 13, 13, 15, 22, 21]
    out = e.step([{"id": "x", "tokens": [30, 31], "want": [0, 1]}, {"id": "y", "tokens": [40], "want": []}])
    assert out[:, 0].tolist() == [30, 31]
