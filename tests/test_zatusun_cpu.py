"""CPU checks of the Zatusun path: configuration, run order, tensor shapes, registry, the frequency tables, and the oracle's own
consistency (portions against a whole prompt, its chunked mask, its router, the forget gate's limits)."""
import copy
import json
import math

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import registry
from lia_b200.modeling_zatusun import ZatusunConfig
from lia_b200.seq_layers import scaled_rotary_freq, wavelength_scaled_rotary_freq

import zatusun_oracle as O
from zatusun_cases import CASES, config, differential, hgrn2, latent, moe

F64 = torch.float64


def toks_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("name", sorted(CASES))
def test_configuration_shapes_and_run_order(name):
    cfg = CASES[name]
    c = ZatusunConfig.from_dict(copy.deepcopy(cfg))
    assert {k: tuple(v) for k, v in c.tensor_shapes().items()} == O.tensor_shapes(cfg)
    assert c.layer_runs() == O.layer_runs(cfg)
    back = ZatusunConfig.from_dict(copy.deepcopy(c.to_dict()))
    assert back.layer_runs() == c.layer_runs() and back.tensor_shapes() == c.tensor_shapes()
    assert back.embed_scale == cfg["embedding"]["scale"] and back.logit_softcap == cfg["logit_softcap"]


def test_run_order_marks_the_first_layer_of_every_pass():
    cfg = config([hgrn2(1, 4, 4)] * 5, 10, 8, loop=(1, 4, 3))
    runs = ZatusunConfig.from_dict(copy.deepcopy(cfg)).layer_runs()
    assert runs == [(0, None), (1, 0), (2, None), (3, None), (1, 1), (2, None), (3, None), (1, 2), (2, None), (3, None), (4, None)]
    one = ZatusunConfig.from_dict(copy.deepcopy(config([hgrn2(1, 4, 4)] * 2, 10, 8, loop=(0, 1, 1))))
    assert one.layer_runs() == [(0, 0), (1, None)] and "loop.in" in one.tensor_shapes()         # one pass still goes through the projection
    empty = ZatusunConfig.from_dict(copy.deepcopy(config([hgrn2(1, 4, 4)] * 2, 10, 8, loop=(1, 1, 3))))
    assert empty.layer_runs() == [(0, None), (1, None)]                                           # a block without layers: no pass begins
    none = ZatusunConfig.from_dict(copy.deepcopy(config([hgrn2(1, 4, 4)] * 2, 10, 8)))
    assert none.layer_runs() == [(0, None), (1, None)] and "loop.in" not in none.tensor_shapes()


def test_configuration_refuses_what_it_does_not_know():
    bad = copy.deepcopy(CASES["odd"])
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError):
        ZatusunConfig.from_dict(bad)
    bad = copy.deepcopy(CASES["even"])
    bad["layers"][2]["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        ZatusunConfig.from_dict(bad)
    bad = copy.deepcopy(CASES["even"])
    bad["loop"] = {"start": 3, "stop": 2, "times": 2}
    with pytest.raises(ValueError):
        ZatusunConfig.from_dict(bad)
    bad = copy.deepcopy(CASES["even"])
    bad["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(ValueError):
        ZatusunConfig.from_dict(bad)


def test_registry_knows_the_design(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CASES["odd"]))
    assert registry.architecture_of(str(tmp_path)) == "zatusun"
    assert registry.model_class(str(tmp_path)).__name__ == "ZatusunForCausalLM"


def test_frequency_tables_agree_with_the_plain_ones():
    for dims, base, s in ((8, 500.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}), (40, 1e4, {"factor": 16.0, "low": 0.5, "high": 64.0, "original": 1000}),
                          (6, 100.0, None)):
        want, _ = O.llama3_freq(dims, base, s)
        assert torch.allclose(wavelength_scaled_rotary_freq(dims, base, s), want, rtol=1e-14, atol=0)
    s = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}
    f, plain = wavelength_scaled_rotary_freq(8, 500.0, s), O.plain_freq(8, 500.0)
    assert f[0] == plain[0] and f[-1] == plain[-1] / 8.0 and any(0 < float(1 - a / b) < 1 - 1 / 8.0 for a, b in zip(f, plain))     # all three regimes occur
    for dims, base, s in ((16, 1000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}), (6, 50.0, {"factor": 16.0, "original": 32, "fast": 1000.0, "slow": 500.0})):
        want, amp = O.yarn_freq(dims, base, s)
        got, mag = scaled_rotary_freq(dims, base, s)
        assert torch.allclose(got, want, rtol=1e-14, atol=0) and mag == amp == 0.1 * math.log(s["factor"]) + 1.0


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_portions_equal_the_whole_prompt(name):
    cfg = CASES[name]
    w = O.random_weights(cfg, 3)
    toks = toks_for(cfg, 31, 1)
    whole = O.logits_of(cfg, w, toks)
    o = O.Oracle(cfg, w)
    with torch.no_grad():
        parts = torch.cat([o.forward(toks[a:b]) for a, b in ((0, 7), (7, 8), (8, 10), (10, 27), (27, 31))])
    assert float((parts - whole).abs().max()) < 1e-9
    assert float(whole.abs().max()) <= cfg["logit_softcap"]


def test_oracle_chunked_mask_and_router_and_forget_gate():
    m = O.visible(3, 4, chunk=5)                                      # positions 3 .. 6 over keys 0 .. 6
    assert m.tolist() == [[True, True, True, True, False, False, False], [True, True, True, True, True, False, False],
                          [False, False, False, False, False, True, False], [False, False, False, False, False, True, True]]
    h = torch.randn(9, 12, dtype=F64, generator=torch.Generator().manual_seed(0))
    wr = torch.randn(5, 12, dtype=F64, generator=torch.Generator().manual_seed(1))
    idx, wt = O.route(h, wr, 2)
    z = h @ wr.T
    assert torch.equal(idx[:, 0], z.argmax(-1)) and torch.allclose(wt.sum(-1), torch.ones(9, dtype=F64))
    assert torch.allclose(wt[:, 0] / wt[:, 1], torch.exp(z.gather(1, idx[:, :1]) - z.gather(1, idx[:, 1:]))[:, 0])
    # a forget gate held at 1 keeps the state, at its lower bound 0 with a closed sigmoid it writes v whole
    w = {"q": torch.eye(4, dtype=F64), "v": torch.eye(4, dtype=F64), "f": torch.zeros(4, 4, dtype=F64), "f.b": torch.full((4,), -50.0, dtype=F64),
         "lower": torch.zeros(4, dtype=F64), "norm": torch.ones(4, dtype=F64), "o": torch.eye(4, dtype=F64)}
    st = {}
    O.hgrn2(torch.ones(3, 4, dtype=F64), w, "", {"heads": 1, "dim": 4, "vdim": 4}, 1e-6, st)
    assert torch.allclose(st["S"][0], torch.ones(4, 4, dtype=F64))
    w["lower"] = torch.ones(4, dtype=F64)
    O.hgrn2(7 * torch.ones(2, 4, dtype=F64), w, "", {"heads": 1, "dim": 4, "vdim": 4}, 1e-6, st)
    assert torch.allclose(st["S"][0], torch.ones(4, 4, dtype=F64))
