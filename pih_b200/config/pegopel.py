"""Typed configuration of the Pegopel design, read from its config.json keys.

A Pegopel model is a list of pre-norm layers over several residual streams (hyper-connections), a learned vector per
place added to the embedding, and an output head that is the embedding table.  Each layer has one of two attention
mixers over a sliding window with a sink in the softmax denominator: ``"attention"`` (short convolutions behind the
projections, a learned bias by distance, a learned sink) or ``"attention_2"`` (the values are the keys as projected,
rotation with stretched low frequencies in neighbouring pairs, capped scores, kept first tokens, a sink of score zero,
a gate a head), and a gated feed-forward with the tanh form of GELU, or none.  config.json holds::

    {"architecture": "Pegopel", "vocab": V, "width": W, "max_positions": P, "streams": S, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention" | "attention_2", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

``loop``: layers a .. b-1 run n times in a row with the same weights, each pass with a cache and state of its own; the
schedule names those layers n times.  Without ``streams`` the layers are plain pre-norm layers.  The residual streams
are summed in 32-bit.  Tensor names: ``embed``, ``pos``, ``final.norm``, and ``l<i>.`` + ``norm1`` / ``norm2`` /
``mix.*`` / ``mlp.*`` / ``hc1.*`` / ``hc2.*`` (see the name tables of the part specs).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import register_architecture
from .specs import (BlockSpec, HyperSpec, ModelSpec, NormSpec, ScaledRopeSpec, ScheduleEntry, SwiGLUSpec,
                    WindowAttentionSpec)
from .tuganex import _int, _number, _object


@register_architecture("Pegopel")
@dataclass(frozen=True)
class PegopelConfig:
    vocab: int
    width: int
    max_positions: int
    streams: int                      # 0: one stream, plain residual sums
    norm_eps: float
    loop: Optional[Tuple[int, int, int]]      # (start, stop, times)
    layers: Tuple[dict, ...]          # as in config.json, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "PegopelConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ValueError("config.json: 'norm' must be an object with 'eps'")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        loop = None
        if raw.get("loop") is not None:
            lp = _object(raw, "loop", "config")
            loop = (_int(lp, "start", "loop", 0), _int(lp, "stop", "loop", 0), _int(lp, "times", "loop", 1))
            if not loop[0] <= loop[1] <= len(layers):
                raise ValueError(f"config.json: loop must satisfy start <= stop <= {len(layers)} layers, got {loop[:2]}")
        streams = _int(raw, "streams", "config") if raw.get("streams") is not None else 0
        if streams > 8:
            raise ValueError(f"config.json: streams must be at most 8, got {streams}")
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  max_positions=_int(raw, "max_positions", "config"), streams=streams,
                  norm_eps=_number(norm, "eps", "norm"), loop=loop, layers=tuple(copy.deepcopy(layers)))
        cfg.model_spec()                      # every layer's keys and sizes are checked by building its spec
        return cfg

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
               "layers": copy.deepcopy(list(self.layers))}
        if self.streams:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def layer_order(self):
        """The layers in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    # -- layers -----------------------------------------------------------------
    def _rotation(self, m: dict, where: str, head_dim: int):
        rot = m.get("rot")
        if rot is None:
            return None
        rot = _object(m, "rot", where)
        rw = where + ".rot"
        dims = _int(rot, "dims", rw, minimum=2)
        if dims % 2 or dims > head_dim:
            raise ValueError(f"config.json: {rw}.dims must be even and at most dim ({head_dim}), got {dims}")
        extra = {}
        if rot.get("scaling") is not None:
            sc = _object(rot, "scaling", rw)
            sw = rw + ".scaling"
            extra = dict(factor=_number(sc, "factor", sw), original=_number(sc, "original", sw),
                         fast=_number(sc, "fast", sw), slow=_number(sc, "slow", sw))
        return ScaledRopeSpec(head_dim=head_dim, rotary_dim=dims, theta=_number(rot, "base", rw),
                              max_positions=self.max_positions, interleaved=True, **extra)

    def _mixer_spec(self, i: int):
        layer = self.layers[i]
        if not isinstance(layer, dict):
            raise ValueError(f"config.json: layers[{i}] must be an object")
        where = f"layers[{i}].mixer"
        kind, m = layer.get("type"), layer.get("mixer")
        if kind not in ("attention", "attention_2"):
            raise ValueError(f"config.json: layers[{i}].type must be 'attention' or 'attention_2', got {kind!r}")
        if not isinstance(m, dict):
            raise ValueError(f"config.json: {where} must be an object")
        heads, kv_heads, dim = _int(m, "heads", where), _int(m, "kv_heads", where), _int(m, "dim", where)
        vdim = _int(m, "vdim", where) if m.get("vdim") is not None else dim     # (not given: as wide as the keys)
        if heads % kv_heads:
            raise ValueError(f"config.json: {where}.heads must be a multiple of kv_heads")
        mask = _object(m, "mask", where)
        common = dict(hidden=self.width, heads=heads, kv_heads=kv_heads, key_dim=dim, value_dim=vdim,
                      scale=_number(m, "scale", where), window=_int(mask, "size", where + ".mask"),
                      norm_eps=self.norm_eps)
        if kind == "attention":
            return WindowAttentionSpec(conv_taps=_int(m, "conv", where) if m.get("conv") is not None else 0,
                                       bias_rows=self._bias_rows(i),
                                       bias_far=_number(m, "bias_max", where), sink="learned", **common)
        if vdim != dim:
            raise ValueError(f"config.json: {where}.vdim must equal dim: the values are the keys as projected")
        keep = _int(mask, "keep_first", where + ".mask", 0) if mask.get("keep_first") is not None else 0
        cap = _number(m, "softcap", where) if m.get("softcap") is not None else None
        return WindowAttentionSpec(keep_first=keep, values_from_keys=True, position=self._rotation(m, where, dim),
                                   softcap=cap, sink="zero", head_gate=True, **common)

    def _bias_rows(self, i: int) -> int:
        """Rows of layer i's bias table: ``bias_rows`` of its mixer where the configuration says it, else what the
        weight file's tensor has (``with_shapes``), else 16."""
        m = self.layers[i]["mixer"]
        if m.get("bias_rows") is not None:
            return _int(m, "bias_rows", f"layers[{i}].mixer", 2)
        return 16

    def with_shapes(self, shapes) -> "PegopelConfig":
        """The configuration with the sizes that only the tensors' shapes give: the rows of each bias table
        (``l<i>.mix.rel``: [rows, heads])."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            shape = shapes.get(f"l{i}.mix.rel")
            if layer.get("type") == "attention" and shape is not None and len(shape) == 2:
                layer["mixer"]["bias_rows"] = int(shape[0])
        return PegopelConfig(self.vocab, self.width, self.max_positions, self.streams, self.norm_eps, self.loop,
                             tuple(layers))

    def _ffn_spec(self, i: int):
        f = self.layers[i].get("mlp")
        if f is None:
            return None
        where = f"layers[{i}].mlp"
        if not isinstance(f, dict):
            raise ValueError(f"config.json: {where} must be null or an object")
        if f.get("kind") != "dense":
            raise ValueError(f"config.json: {where}.kind must be 'dense', got {f.get('kind')!r}")
        return SwiGLUSpec(hidden=self.width, intermediate=_int(f, "ff", where), activation="gelu_tanh",
                          names={"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})

    # -- the model as parts --------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        norm = NormSpec(width=self.width, eps=self.norm_eps, weight_name="")
        hyper = HyperSpec(streams=self.streams) if self.streams else None
        blocks = []
        for i in range(len(self.layers)):
            mixer = self._mixer_spec(i)
            ffn = self._ffn_spec(i)
            blocks.append(BlockSpec(prefix=f"l{i}.", mixer=mixer, ffn=ffn, norm_in=norm,
                                    norm_post=norm if ffn is not None else None,
                                    arrangement="hyper" if hyper is not None else "prenorm",
                                    names={"norm_in": "norm1", "norm_post": "norm2"}, hyper=hyper))
        schedule = tuple(ScheduleEntry(i) for i in self.layer_order())
        spec = ModelSpec(vocab=self.vocab, hidden=self.width, blocks=tuple(blocks), schedule=schedule,
                         final_norm=norm, tie_embeddings=True, embed_name="embed", final_norm_prefix="final.norm",
                         head_name="head", max_positions=self.max_positions, stream_dtype="float32",
                         position_name="pos", streams=self.streams)
        spec.validate()
        return spec
