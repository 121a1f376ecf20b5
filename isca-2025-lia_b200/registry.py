"""Model registry: ``config.json`` -> model class.  A checkpoint directory names its design either the Hugging Face way
(``architectures: [...]`` / ``model_type``) or with one ``architecture`` string; ``load_model`` picks the class and calls
its ``from_pretrained`` (run_generation.py:159-167 resolves OPT the same way, through its model-type table)."""
import json
import os

MODEL_CLASSES = {}


def register(name, loader):
    """``loader()`` -> class with ``from_pretrained(path, device=, **kw)``; resolved lazily."""
    MODEL_CLASSES[name.lower()] = loader


def _opt():
    from .modeling_opt import OPTForCausalLM
    return OPTForCausalLM


def _davasun():
    from .modeling_davasun import DavasunForCausalLM
    return DavasunForCausalLM


def _bebulorn():
    from .modeling_bebulorn import BebulornForCausalLM
    return BebulornForCausalLM


def _bizetar():
    from .modeling_bizetar import BizetarForCausalLM
    return BizetarForCausalLM


def _zatusun():
    from .modeling_zatusun import ZatusunForCausalLM
    return ZatusunForCausalLM


register("OPTForCausalLM", _opt)
register("opt", _opt)
register("Davasun", _davasun)
register("DavasunForCausalLM", _davasun)
register("Bebulorn", _bebulorn)
register("BebulornForCausalLM", _bebulorn)
register("Bizetar", _bizetar)
register("BizetarForCausalLM", _bizetar)
register("Zatusun", _zatusun)
register("ZatusunForCausalLM", _zatusun)


def architecture_of(path):
    cj = os.path.join(path, "config.json")
    if not os.path.exists(cj):
        if os.path.exists(os.path.join(path, "lia_slabs.json")):
            return "opt"
        raise FileNotFoundError(f"{path}: config.json not found")
    c = json.load(open(cj))
    names = [c.get("architecture")] + list(c.get("architectures") or []) + [c.get("model_type")]
    for n in names:
        if n and n.lower() in MODEL_CLASSES:
            return n.lower()
    raise KeyError(f"{path}: no registered model for {[n for n in names if n]} (known: {sorted(MODEL_CLASSES)})")


def model_class(path):
    return MODEL_CLASSES[architecture_of(path)]()


def load_model(path, device="cuda", **kw):
    return model_class(path).from_pretrained(path, device=device, **kw)
