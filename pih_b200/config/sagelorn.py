"""Typed configuration of the Sagelorn design, read from its config.json keys.

A Sagelorn model embeds a token as the sum of its row of the token table and a row of a bigram table chosen by a
hash of (previous token, token), runs a list of layers whose norms sit on the sub-layers' OUTPUTS —
``x += norm1(mixer(x))``, then ``x += norm2(ff(x))``, the norm weights stored around zero (``1 + w`` multiplies) —
and multiplies the logits by one number.  A layer's mixer is one of

* ``"attention"``: softmax attention over a sliding window with a learned sink a head in the denominator, grouped
  key/value heads, an RMS norm of q and of k over the whole projection, a rotation in halves whose low frequencies
  may be stretched by wavelength bands; with ``"kv_from": j`` the layer has no key/value tensors and reads layer j's
  cache with its own queries, window and sink;
* ``"latent_attention"``: attention over a cached latent with queries through a latent of their own, a rotated key
  part shared by the heads (neighbouring pairs), a sliding window, and a sigmoid gate a column of the output;
* ``"retention"``: linear attention with a fixed decay a head and a matrix state per sequence;

and its feed-forward is dense (gated, SiLU), a mixture of experts (sigmoid scores, the chosen experts read the row
times its score, two-matrix experts around the squared ReLU, a shared expert of the same form) or absent.
config.json holds::

    {"architecture": "Sagelorn", "vocab": V, "width": W, "norm": {"eps": e}, "logit_scale": s,
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": ..., "mixer": {...}, "mlp": {...} | null}, ...]}

The residual stream is summed in 32-bit.  Tensor names: ``embed``, ``bigram``, ``head``, ``final.norm``, and
``l<i>.`` + ``norm1`` / ``norm2`` / ``mix.*`` / ``mlp.*`` (see the name tables of the part specs).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import register_architecture
from .specs import (BigramSpec, BlockSpec, ComputedRopeSpec, LatentAttentionSpec, ModelSpec, NormSpec, PlainMLPSpec,
                    RetentionSpec, ScheduleEntry, ScoredMoESpec, SwiGLUSpec, WindowAttentionSpec)
from .tuganex import _int, _number, _object

# The rotations' angles are computed from the position, so the design has no longest context of its own; this bounds
# the engine's default.
DEFAULT_MAX_CONTEXT = 1 << 20

_MIXERS = ("attention", "latent_attention", "retention")


@register_architecture("Sagelorn")
@dataclass(frozen=True)
class SagelornConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    bigram: Optional[Tuple[int, int, int]]    # (buckets, mul_prev, mul_cur)
    layers: Tuple[dict, ...]          # as in config.json, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "SagelornConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ValueError("config.json: 'norm' must be an object with 'eps'")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        bigram = None
        emb = raw.get("embedding")
        if emb is not None:
            if not isinstance(emb, dict):
                raise ValueError("config.json: 'embedding' must be an object")
            if emb.get("bigram") is not None:
                b = _object(emb, "bigram", "embedding")
                bigram = (_int(b, "buckets", "embedding.bigram"), _int(b, "mul_prev", "embedding.bigram", 0),
                          _int(b, "mul_cur", "embedding.bigram", 0))
        scale = _number(raw, "logit_scale", "config") if raw.get("logit_scale") is not None else 1.0
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  norm_eps=_number(norm, "eps", "norm"), logit_scale=scale, bigram=bigram,
                  layers=tuple(copy.deepcopy(layers)))
        cfg.model_spec()                      # every layer's keys and sizes are checked by building its spec
        return cfg

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
               "layers": copy.deepcopy(list(self.layers))}
        if self.bigram is not None:
            out["embedding"] = {"bigram": {"buckets": self.bigram[0], "mul_prev": self.bigram[1],
                                           "mul_cur": self.bigram[2]}}
        return out

    # -- layers -----------------------------------------------------------------
    def _mixer(self, i: int) -> dict:
        layer = self.layers[i]
        if not isinstance(layer, dict):
            raise ValueError(f"config.json: layers[{i}] must be an object")
        if layer.get("type") not in _MIXERS:
            raise ValueError(f"config.json: layers[{i}].type must be one of {list(_MIXERS)}, got {layer.get('type')!r}")
        m = layer.get("mixer")
        if not isinstance(m, dict):
            raise ValueError(f"config.json: layers[{i}].mixer must be an object")
        return m

    def _rotation(self, m: dict, where: str, head_dim: int, interleaved: bool):
        if m.get("rot") is None:
            return None
        rot = _object(m, "rot", where)
        rw = where + ".rot"
        dims = _int(rot, "dims", rw, minimum=2)
        if dims % 2 or dims > head_dim:
            raise ValueError(f"config.json: {rw}.dims must be even and at most {head_dim}, got {dims}")
        stretch = None
        if rot.get("scaling") is not None:
            sc = _object(rot, "scaling", rw)
            sw = rw + ".scaling"
            stretch = (_number(sc, "factor", sw), _number(sc, "low", sw), _number(sc, "high", sw),
                       _number(sc, "original", sw))
            if stretch[1] == stretch[2]:
                raise ValueError(f"config.json: {sw}.low and .high must differ")
        return ComputedRopeSpec(head_dim=head_dim, rotary_dim=dims, theta=_number(rot, "base", rw),
                                interleaved=interleaved, stretch=stretch)

    def _kv_source(self, i: int):
        """The layer whose cache attention layer ``i`` reads (None: its own)."""
        m = self._mixer(i)
        j = m.get("kv_from")
        if self.layers[i]["type"] != "attention" or j is None:
            return None
        where = f"layers[{i}].mixer.kv_from"
        if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < i:
            raise ValueError(f"config.json: {where} must name an earlier layer, got {j!r}")
        other = self.layers[j]
        if not isinstance(other, dict) or other.get("type") != "attention" or not isinstance(other.get("mixer"), dict) \
                or other["mixer"].get("kv_from") is not None:
            raise ValueError(f"config.json: {where} must name an attention layer with keys and values of its own")
        for key in ("kv_heads", "dim", "vdim", "rot"):
            if other["mixer"].get(key) != m.get(key):
                raise ValueError(f"config.json: {where}: layer {j}'s {key} differs from this layer's")
        return j

    def _window(self, m: dict, where: str) -> int:
        """The mask's size; 0 (every earlier key) where the mixer names no mask."""
        if m.get("mask") is None:
            return 0
        return _int(_object(m, "mask", where), "size", where + ".mask")

    def _cache_reach(self, i: int) -> int:
        """How many keys back layer i's cache has to reach: the widest window of the layer and of those that read its
        cache (0: every key)."""
        windows = [self._window(self._mixer(i), f"layers[{i}].mixer")]
        for k in range(i + 1, len(self.layers)):
            if self._kv_source(k) == i:
                windows.append(self._window(self._mixer(k), f"layers[{k}].mixer"))
        return 0 if 0 in windows else max(windows)

    def _mixer_spec(self, i: int):
        m = self._mixer(i)
        kind = self.layers[i]["type"]
        where = f"layers[{i}].mixer"
        if kind == "retention":
            heads, dim = _int(m, "heads", where), _int(m, "dim", where)
            decays = m.get("decay")
            if not isinstance(decays, list) or len(decays) != heads or not all(
                    isinstance(d, (int, float)) and not isinstance(d, bool) and 0.0 < d <= 1.0 for d in decays):
                raise ValueError(f"config.json: {where}.decay must list one number in (0, 1] a head")
            return RetentionSpec(hidden=self.width, heads=heads, key_dim=dim, value_dim=_int(m, "vdim", where),
                                 decays=tuple(float(d) for d in decays), key_scale=dim ** -0.5, norm_eps=self.norm_eps,
                                 position=None)
        if kind == "latent_attention":
            rot_dim = _int(m, "rot_dim", where, 0) if m.get("rot_dim") is not None else 0
            position = self._rotation(m, where, rot_dim, interleaved=True) if rot_dim else None
            if position is not None and position.rotary_dim != rot_dim:
                raise ValueError(f"config.json: {where}.rot.dims must equal rot_dim ({rot_dim})")
            if rot_dim and position is None:
                raise ValueError(f"config.json: {where}.rot_dim needs {where}.rot")
            return LatentAttentionSpec(hidden=self.width, heads=_int(m, "heads", where), key_dim=_int(m, "dim", where),
                                       value_dim=_int(m, "vdim", where), latent_rank=_int(m, "kv_rank", where),
                                       scale=_number(m, "scale", where), norm_eps=self.norm_eps, sink=False, gated=True,
                                       gate_per="column", rotary_dim=rot_dim, position=position,
                                       query_rank=_int(m, "q_rank", where), window=self._window(m, where) or None)
        heads, kv_heads, dim = _int(m, "heads", where), _int(m, "kv_heads", where), _int(m, "dim", where)
        if heads % kv_heads:
            raise ValueError(f"config.json: {where}.heads must be a multiple of kv_heads")
        own = self._kv_source(i) is None
        reach = self._cache_reach(i) if own else 0
        return WindowAttentionSpec(hidden=self.width, heads=heads, kv_heads=kv_heads, key_dim=dim,
                                   value_dim=_int(m, "vdim", where), scale=_number(m, "scale", where),
                                   window=self._window(m, where), norm_eps=self.norm_eps,
                                   position=self._rotation(m, where, dim, interleaved=False), sink="learned",
                                   own_kv=own, cache_window=reach if own else None)

    def _expert(self, f: dict, key: str, where: str, prefix: str) -> PlainMLPSpec:
        return PlainMLPSpec(hidden=self.width, intermediate=_int(_object(f, key, where), "ff", f"{where}.{key}"),
                            names={"up": prefix + "up", "down": prefix + "down"})

    def _ffn_spec(self, i: int):
        f = self.layers[i].get("mlp")
        if f is None:
            return None
        where = f"layers[{i}].mlp"
        if not isinstance(f, dict):
            raise ValueError(f"config.json: {where} must be null or an object")
        if f.get("kind") == "dense":
            return SwiGLUSpec(hidden=self.width, intermediate=_int(f, "ff", where),
                              names={"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})
        if f.get("kind") != "moe":
            raise ValueError(f"config.json: {where}.kind must be 'dense' or 'moe', got {f.get('kind')!r}")
        router = _object(f, "router", where)
        experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
        if top > experts:
            raise ValueError(f"config.json: {where}.router.top exceeds the number of experts")
        shared = self._expert(f, "shared", where, "mlp.shared.") if f.get("shared") is not None else None
        return ScoredMoESpec(hidden=self.width, experts=experts, identity=0, top=top,
                             intermediate=self._expert(f, "expert", where, "").intermediate, shared=shared,
                             activation="relu2", scoring="sigmoid", correction=False, gated=False, weigh="input",
                             shared_gate=False)

    # -- the model as parts --------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        norm = NormSpec(width=self.width, eps=self.norm_eps, weight_name="", offset=1.0)
        blocks, schedule = [], []
        for i in range(len(self.layers)):
            mixer = self._mixer_spec(i)
            ffn = self._ffn_spec(i)
            blocks.append(BlockSpec(prefix=f"l{i}.", mixer=mixer, ffn=ffn, norm_in=norm,
                                    norm_post=norm if ffn is not None else None, arrangement="outnorm",
                                    names={"norm_in": "norm1", "norm_post": "norm2"}))
            schedule.append(ScheduleEntry(i, reads_cache_of=self._kv_source(i)))
        bigram = BigramSpec(*self.bigram) if self.bigram is not None else None
        spec = ModelSpec(vocab=self.vocab, hidden=self.width, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, tie_embeddings=False, embed_name="embed", final_norm_prefix="final.norm",
                         head_name="head", max_positions=DEFAULT_MAX_CONTEXT, stream_dtype="float32",
                         logit_scale=self.logit_scale, bigram=bigram)
        spec.validate()
        return spec
