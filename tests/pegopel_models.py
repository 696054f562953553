"""Small Pegopel configurations with random weights for the tests, and their plain float64 logits.

``P1``: three residual streams, a loop that runs two layers twice, both mixers, two key/value heads for four and six
query heads, a value size unlike the key size, convolutions of three and two taps, bias tables of ten and eight rows, a
rotation over half of a head with stretched low frequencies and one over a whole head without, kept first tokens,
capped and uncapped scores, a layer without a feed-forward, windows that are no multiple of anything.  ``P2``: one
plain residual stream and no loop, one query head per key/value head, a single head, a window of a whole page, no kept
tokens, five taps.  ``P3``: a single stream written as ``streams: 1``, a loop over every layer, a window of one key.
"""
import copy
import json
import os

import torch

import plain_pegopel


def _scaling(factor, original, fast=32.0, slow=1.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _conv(heads, kv_heads, dim, vdim, taps, size, scale, bias_rows, bias_max):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps, "mask": {"size": size},
            "scale": scale, "bias_rows": bias_rows, "bias_max": bias_max}


def _rotary(heads, kv_heads, dim, size, scale, keep_first=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": size}, "scale": scale}
    if keep_first is not None:
        m["mask"]["keep_first"] = keep_first
    if rot is not None:
        m["rot"] = rot
    if softcap is not None:
        m["softcap"] = softcap
    return m


def _ff(n):
    return {"kind": "dense", "ff": n} if n else None


P1 = {"architecture": "Pegopel", "vocab": 307, "width": 96, "max_positions": 400, "streams": 3, "norm": {"eps": 1e-5},
      "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
    {"type": "attention", "mixer": _conv(4, 2, 16, 24, 3, 23, 0.3, 10, 50), "mlp": _ff(136)},
    {"type": "attention_2", "mixer": _rotary(6, 2, 16, 37, 0.25, keep_first=5, softcap=5.0,
                                             rot={"dims": 8, "base": 1e4, "scaling": _scaling(4.0, 64, fast=8.0)}),
     "mlp": None},
    {"type": "attention", "mixer": _conv(2, 1, 24, 40, 2, 9, 0.2, 8, 30), "mlp": _ff(72)},
    {"type": "attention_2", "mixer": _rotary(2, 2, 24, 12, 0.2, keep_first=12, rot={"dims": 24, "base": 500.0}),
     "mlp": _ff(64)},
]}
P2 = {"architecture": "Pegopel", "vocab": 257, "width": 64, "max_positions": 512, "norm": {"eps": 1e-6}, "layers": [
    {"type": "attention_2", "mixer": _rotary(3, 3, 8, 64, 0.35, rot={"dims": 8, "base": 100.0, "scaling": _scaling(1.5, 16, 4.0, 0.5)},
                                             softcap=2.0), "mlp": _ff(100)},
    {"type": "attention", "mixer": _conv(1, 1, 32, 8, 5, 16, 0.18, 6, 12.5), "mlp": None},
    {"type": "attention_2", "mixer": _rotary(4, 1, 12, 17, 0.3, keep_first=1), "mlp": _ff(48)},
]}
P3 = {"architecture": "Pegopel", "vocab": 131, "width": 40, "max_positions": 300, "streams": 1, "norm": {"eps": 1e-5},
      "loop": {"start": 0, "stop": 2, "times": 3}, "layers": [
    {"type": "attention", "mixer": _conv(5, 5, 8, 8, 1, 1, 0.5, 2, 7), "mlp": _ff(24)},
    {"type": "attention_2", "mixer": _rotary(2, 1, 20, 3, 0.2, keep_first=2, softcap=50.0,
                                             rot={"dims": 4, "base": 10.0, "scaling": _scaling(8.0, 32)}), "mlp": _ff(56)},
]}
CONFIGS = {"P1": P1, "P2": P2, "P3": P3}
SIGMA = {"P1": 0.12, "P2": 0.15, "P3": 0.2}


def single_layer(kind, mlp=None, streams=2, **changes):
    """A model of ONE layer of the given mixer (a mechanism alone); ``changes`` replace keys of the mixer."""
    mixer = {"attention": _conv(6, 2, 12, 20, 4, 11, 0.4, 12, 40),
             "attention_2": _rotary(6, 3, 12, 13, 0.4, keep_first=3, softcap=4.0,
                                    rot={"dims": 6, "base": 50.0, "scaling": _scaling(2.0, 24, 6.0, 0.5)})}[kind]
    mixer = copy.deepcopy(mixer)
    for k, v in changes.items():
        if v is None:
            mixer.pop(k, None)
        else:
            mixer[k] = v
    raw = {"architecture": "Pegopel", "vocab": 120, "width": 48, "max_positions": 256, "norm": {"eps": 1e-5},
           "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}
    if streams:
        raw["streams"] = streams
    return raw


def write_model(folder, raw, seed, sigma, dtype=torch.bfloat16):
    """A model folder with random weights.  The connections between the residual streams are drawn around the plain
    residual sum (reads that sum to about one, a mixing matrix around the identity, writes around one), so that every
    layer's output stays in the logits.  The rows of the bias tables are NOT in the written config.json: the engine
    has to take them from the tensors' shapes."""
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    from pih_b200.weights import random_tensors
    from pih_b200.weights.safetensors_io import write_safetensors
    folder = str(folder)
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(expected_tensors(config_from_dict(copy.deepcopy(raw)).model_spec()), seed, sigma, dtype)
    S = raw.get("streams", 0)
    for name, t in tensors.items():
        if ".hc" in name:
            noise = t.float() * 0.5
            if name.endswith(".mix"):
                t = torch.eye(S) + noise
            elif name.endswith(".in"):
                t = 1.0 / S + noise
            else:
                t = 1.0 + noise
            tensors[name] = t.to(dtype)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    out = copy.deepcopy(raw)
    for layer in out["layers"]:
        layer["mixer"].pop("bias_rows", None)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    return folder


def load_plain(model_dir):
    from pih_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with SafetensorsFile(os.path.join(model_dir, "model.safetensors")) as sf:
        w = {n: sf.read_tensor(n).to(torch.float64) for n in sf.names()}
    return cfg, w


_LOGITS = {}


def plain_logits(model_dir, requests):
    """{rid: float64 logits [len, vocab]} of the plain implementation, cached per (folder, request)."""
    cfg, w = None, None
    out = {}
    for rid, toks in requests.items():
        key = (model_dir, tuple(toks))
        if key not in _LOGITS:
            if cfg is None:
                cfg, w = load_plain(model_dir)
            _LOGITS[key] = plain_pegopel.forward(cfg, w, toks)
        out[rid] = _LOGITS[key]
    return out


def random_config(seed):
    """A configuration drawn at random: sizes (odd ones and ones that no fast kernel takes among them), the order of
    layers, a loop or none, the number of streams, windows around and below a page, every constant."""
    import random
    rnd = random.Random(seed)
    width = rnd.choice([40, 56, 64, 72, 96, 136])
    layers = []
    for i in range(rnd.randint(2, 5)):
        kv_heads = rnd.choice([1, 2, 3])
        heads = kv_heads * rnd.choice([1, 2, 4])
        dim = rnd.choice([4, 8, 12, 16, 24, 32, 40, 64])
        size = rnd.choice([1, 2, 7, 15, 16, 17, 31, 33, 64, 100])
        if rnd.random() < 0.5:
            rows = rnd.choice([2, 4, 6, 16, 32])
            mixer = _conv(heads, kv_heads, dim, rnd.choice([8, 12, 16, 24, 40, 64, 72, 136]), rnd.choice([1, 2, 3, 4, 7]), size,
                          rnd.uniform(0.1, 0.6), rows, rows // 2 + rnd.choice([0.5, 3, 20, 200]))
            kind = "attention"
        else:
            rot = None
            if rnd.random() < 0.8:
                rot = {"dims": rnd.choice([d for d in (2, 4, 8, 12, 16, 24, 32, 40, 64) if d <= dim]), "base": rnd.choice([10.0, 1e4, 1e6])}
                if rnd.random() < 0.7:
                    rot["scaling"] = _scaling(rnd.choice([1.0, 2.0, 8.0, 40.0]), rnd.choice([8, 64, 4096]),
                                              rnd.choice([4.0, 32.0]), rnd.choice([0.25, 1.0]))
            mixer = _rotary(heads, kv_heads, dim, size, rnd.uniform(0.1, 0.6), keep_first=rnd.choice([None, 0, 1, 4, 16, 21]),
                            rot=rot, softcap=rnd.choice([None, 1.0, 7.5, 30.0]))
            kind = "attention_2"
        layers.append({"type": kind, "mixer": mixer, "mlp": _ff(rnd.choice([0, 24, 50, 64, 130]))})
    raw = {"architecture": "Pegopel", "vocab": rnd.choice([97, 256, 300]), "width": width, "max_positions": 160,
           "norm": {"eps": rnd.choice([1e-5, 1e-6])}, "layers": layers}
    streams = rnd.choice([0, 1, 2, 3, 4])
    if streams:
        raw["streams"] = streams
    if rnd.random() < 0.6:
        a = rnd.randint(0, len(layers) - 1)
        raw["loop"] = {"start": a, "stop": rnd.randint(a, len(layers)), "times": rnd.randint(1, 3)}
    return raw
