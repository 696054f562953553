"""Small Sagelorn configurations with random weights for the tests, and their plain float64 logits.

Two configurations that differ from each other in every size.  ``S1``: grouped key/value heads, a rotation over part
of a head with stretched slow pairs, a layer that reads another's keys and values through a WIDER window than the
owner's own, latent attention whose values are narrower than its keys and whose window is smaller than a page, a
retention layer with a decay of exactly one, experts of which two are chosen, a layer without a feed-forward.  ``S2``:
one query head per key/value head and a rotation over the whole head without stretching, two readers of one cache (one
with a narrower window, one with a wider one), a latent attention with a stretched rotation, three chosen experts
without a shared one, a retention layer in front, bigram multipliers above the number of buckets, a logit scale above one.
"""
import copy
import json
import os

import torch

import plain_sagelorn


def _rot(dims, base=10000.0, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling:
        out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


def _att(heads, kv_heads, dim, vdim, rot, scale, window, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, rot, scale, window):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot,
            "scale": scale, "mask": {"size": window}}


def _ret(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def _moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def _dense(ff):
    return {"kind": "dense", "ff": ff}


_A1 = dict(heads=4, kv_heads=2, dim=16, vdim=24, rot=_rot(8, 1000.0, (8.0, 1.0, 4.0, 64)), scale=0.3)
S1 = {"architecture": "Sagelorn", "vocab": 311, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.3,
      "embedding": {"bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 5}},
      "layers": [
          {"type": "attention", "mixer": _att(window=20, **_A1), "mlp": _dense(136)},
          {"type": "latent_attention", "mixer": _lat(3, 16, 8, 12, 40, 24, _rot(8, 500.0), 0.25, 11), "mlp": _moe(6, 2, 40, shared=56)},
          {"type": "attention", "mixer": _att(window=37, kv_from=0, **_A1), "mlp": None},
          {"type": "retention", "mixer": _ret(3, 16, 24, [1.0, 0.97, 0.995]), "mlp": _moe(6, 2, 40, shared=56)},
          {"type": "attention", "mixer": _att(2, 1, 24, 40, _rot(24, 1e6), 0.2, 50), "mlp": _dense(72)},
      ]}
_A2 = dict(heads=3, kv_heads=3, dim=8, vdim=12, rot=_rot(8, 100.0), scale=0.5)
S2 = {"architecture": "Sagelorn", "vocab": 257, "width": 64, "norm": {"eps": 1e-6}, "logit_scale": 1.7,
      "embedding": {"bigram": {"buckets": 17, "mul_prev": 40, "mul_cur": 23}},
      "layers": [
          {"type": "retention", "mixer": _ret(5, 8, 40, [0.5, 0.9, 0.999, 0.75, 1.0]), "mlp": _moe(5, 3, 24)},
          {"type": "attention", "mixer": _att(window=24, **_A2), "mlp": _moe(4, 1, 48, shared=16)},
          {"type": "attention", "mixer": _att(window=9, kv_from=1, **_A2), "mlp": None},
          {"type": "latent_attention", "mixer": _lat(2, 24, 4, 40, 28, 36, _rot(4, 10.0, (4.0, 2.0, 8.0, 32)), 0.2, 70),
           "mlp": _dense(100)},
          {"type": "attention", "mixer": _att(window=64, kv_from=1, **_A2), "mlp": _dense(48)},
      ]}
# Sizes that no 16-byte path and no tensor-core instance takes: an odd vocabulary, a width and sizes that are multiples
# of two only, three query heads a key/value head, a window of three keys, all experts but one chosen.
_A3 = dict(heads=3, kv_heads=1, dim=10, vdim=6, rot=_rot(6, 20.0, (3.0, 1.0, 2.0, 10)), scale=0.4)
S3 = {"architecture": "Sagelorn", "vocab": 77, "width": 50, "norm": {"eps": 1e-5}, "logit_scale": 2.5,
      "embedding": {"bigram": {"buckets": 2, "mul_prev": 1, "mul_cur": 1}},
      "layers": [
          {"type": "latent_attention", "mixer": _lat(3, 6, 2, 10, 14, 10, _rot(2, 9.0), 0.3, 3), "mlp": _moe(3, 2, 18, shared=6)},
          {"type": "attention", "mixer": _att(window=5, **_A3), "mlp": _dense(30)},
          {"type": "retention", "mixer": _ret(1, 6, 10, [0.9]), "mlp": None},
          {"type": "attention", "mixer": _att(window=40, kv_from=1, **_A3), "mlp": _moe(2, 1, 10)},
      ]}
CONFIGS = {"S1": S1, "S2": S2}
SIGMA = {"S1": 0.12, "S2": 0.15}


def all_chosen(raw):
    """The configuration with every expert chosen: in bfloat16 the rounding of a router's input flips choices between
    experts whose scores are close, and a flip changes that position outright, so a model with random weights cannot be
    held to a rounding bound.  With every expert chosen the weights still come from the router; the choice itself is
    tested with decided scores."""
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if layer.get("mlp") and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def single_layer(kind, mlp=None, bigram=True, **changes):
    """A model of ONE layer of the given mixer (a mechanism alone), sizes unlike S1's and S2's."""
    mixer = {"retention": _ret(2, 12, 20, [0.93, 0.999]),
             "attention": _att(6, 2, 12, 20, _rot(4, 50.0, (2.0, 1.0, 3.0, 16)), 0.4, 13),
             "latent_attention": _lat(2, 12, 6, 20, 18, 14, _rot(6, 30.0), 0.3, 15)}[kind]
    mixer = copy.deepcopy(mixer)
    mixer.update(changes)
    raw = {"architecture": "Sagelorn", "vocab": 120, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 0.8,
           "layers": [{"type": kind, "mixer": mixer, "mlp": mlp}]}
    if bigram:
        raw["embedding"] = {"bigram": {"buckets": 29, "mul_prev": 3, "mul_cur": 11}}
    return raw


def write_model(folder, raw, seed, sigma):
    from pih_b200.config import config_from_dict
    from pih_b200.weights import write_random_model
    return write_random_model(str(folder), config_from_dict(raw), seed=seed, sigma=sigma)


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
            _LOGITS[key] = plain_sagelorn.model_layers(cfg, w, toks)[1]
        out[rid] = _LOGITS[key]
    return out


def random_config(seed):
    """A configuration drawn at random: sizes (also odd ones and ones that no fast kernel takes), the order of layers,
    which layers read whose keys and values and through which window, every constant."""
    import random
    rnd = random.Random(seed)
    width = rnd.choice([40, 56, 64, 72, 96, 136])
    layers, owners = [], {}
    for i in range(rnd.randint(3, 7)):
        kind = rnd.choice(["attention", "attention", "latent_attention", "retention"])
        if kind == "retention":
            heads = rnd.choice([1, 2, 3, 4])
            mixer = _ret(heads, rnd.choice([4, 8, 12, 16, 20, 32, 64]), rnd.choice([8, 12, 20, 32, 40, 64, 96]),
                         [rnd.choice([1.0, 1.0 - 2.0 ** -rnd.randint(1, 10), rnd.uniform(0.3, 0.999)]) for _ in range(heads)])
        elif kind == "latent_attention":
            rot_dim = rnd.choice([2, 4, 8, 16])
            scaling = rnd.choice([None, (rnd.choice([2.0, 8.0]), 1.0, rnd.choice([2.0, 4.0]), rnd.choice([16, 256]))])
            mixer = _lat(rnd.choice([1, 2, 4, 5]), rnd.choice([4, 8, 16, 24, 32]), rot_dim, rnd.choice([8, 12, 16, 32, 40]),
                         rnd.choice([12, 16, 24, 48, 56, 62]), rnd.choice([8, 20, 32]),
                         _rot(rot_dim, rnd.choice([10.0, 1e4, 2e5]), scaling), rnd.uniform(0.1, 0.5), rnd.choice([1, 2, 7, 16, 33, 200]))
        else:
            if owners and rnd.random() < 0.4:
                j = rnd.choice(list(owners))
                mixer = dict(copy.deepcopy(owners[j]), kv_from=j, heads=owners[j]["kv_heads"] * rnd.choice([1, 2, 3]),
                             scale=rnd.uniform(0.1, 0.6), mask={"size": rnd.choice([1, 3, 8, 17, 40, 300])})
            else:
                kv_heads = rnd.choice([1, 2, 3])
                dim = rnd.choice([4, 8, 12, 16, 24, 32, 40, 64])
                scaling = rnd.choice([None, (rnd.choice([2.0, 3.0, 32.0]), 1.0, rnd.choice([2.0, 4.0]), rnd.choice([8, 64, 512]))])
                mixer = _att(kv_heads * rnd.choice([1, 2, 4]), kv_heads, dim, rnd.choice([8, 12, 16, 24, 40, 64, 72, 128, 136]),
                             _rot(rnd.choice([d for d in (2, 4, 8, 12, 16, 24, 32, 40, 64) if d <= dim]),
                                  rnd.choice([10.0, 1e4, 2e5]), scaling),
                             rnd.uniform(0.1, 0.6), rnd.choice([1, 2, 5, 16, 31, 64, 300]))
                owners[i] = {k: mixer[k] for k in ("kv_heads", "dim", "vdim", "rot")}
        layer = {"type": kind, "mixer": mixer}
        ff = rnd.choice(["dense", "moe", "moe", None])
        if ff == "dense":
            layer["mlp"] = _dense(rnd.choice([24, 50, 64, 130]))
        elif ff == "moe":
            experts = rnd.randint(1, 9)
            layer["mlp"] = _moe(experts, rnd.randint(1, experts), rnd.choice([8, 24, 36, 64]), shared=rnd.choice([None, 16, 40]))
        else:
            layer["mlp"] = None
        layers.append(layer)
    raw = {"architecture": "Sagelorn", "vocab": rnd.choice([97, 256, 300]), "width": width,
           "norm": {"eps": rnd.choice([1e-5, 1e-6])}, "logit_scale": rnd.choice([1.0, 0.25, 0.7, 3.0]), "layers": layers}
    if rnd.random() < 0.8:
        raw["embedding"] = {"bigram": {"buckets": rnd.choice([1, 7, 64, 509]), "mul_prev": rnd.choice([0, 1, 131, 100003]),
                                       "mul_cur": rnd.choice([1, 5, 4099])}}
    return raw
