"""Part specifications: what a model is made of, as plain data.

An architecture's typed configuration (``pih_b200.config.qwen3``) is turned
into a ``ModelSpec``: a list of ``BlockSpec`` (one per distinct layer, each
naming its mixer, feed-forward, norms and position encoding with every size
and constant as a field) and a ``schedule`` — the order in which layers run.
The parts in ``pih_b200.parts`` are built from these specs alone; none of
them knows which architecture it belongs to.

``kind`` strings are keys of the part registries in
``pih_b200.parts.registry``; a new kind of part brings its own spec class
(any dataclass with a ``kind`` field) and registers a builder for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Sequence


def _names(**kw):
    return field(default_factory=lambda: dict(kw))


@dataclass(frozen=True)
class NormSpec:
    width: int
    eps: float
    kind: str = "rmsnorm"
    weight_name: str = "weight"       # behind the norm's prefix ("": the prefix itself names the tensor)
    offset: float = 0.0               # the weight that multiplies is ``offset`` + the stored one (1.0: stored around zero)


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary encoding over the first ``rotary_dim`` columns of a head."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    scale: float                      # applied to q.k after the dot product
    qk_norm_eps: Optional[float]      # None: no per-head q/k norm
    window: Optional[int]             # None: all keys; W: the last W keys
    position: Optional[RopeSpec]
    kind: str = "attention"
    # tensor names below the block's prefix, by role
    names: Mapping[str, str] = _names(q="self_attn.q_proj.weight", k="self_attn.k_proj.weight",
                                      v="self_attn.v_proj.weight", o="self_attn.o_proj.weight",
                                      q_norm="self_attn.q_norm.weight", k_norm="self_attn.k_norm.weight")

    @property
    def q_size(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.kv_heads * self.head_dim


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden: int
    intermediate: int
    activation: str = "silu"
    kind: str = "swiglu"
    names: Mapping[str, str] = _names(gate="mlp.gate_proj.weight", up="mlp.up_proj.weight",
                                      down="mlp.down_proj.weight")


@dataclass(frozen=True)
class ScalarNormSpec:
    """RMS norm whose weight is ONE number for all coordinates (a tensor without axes)."""
    width: int
    eps: float
    kind: str = "scalar_rmsnorm"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Gated delta rule: a matrix state ``S [key_dim, value_dim]`` per head that decays, is corrected towards the
    new value along the new key, and is read with the query.  q and k have ``kv_heads`` heads shared by groups of
    value heads; q, k and v pass a short causal convolution and SiLU; q and k are made unit vectors."""
    hidden: int
    heads: int
    kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float                   # of the per-head RMS norm of the read-out
    unit_eps: float = 1e-6            # inside the root of the unit norm of q and k
    kind: str = "gated_delta"
    names: Mapping[str, str] = _names(q="mix.q", k="mix.k", v="mix.v", q_conv="mix.q.conv", k_conv="mix.k.conv",
                                      v_conv="mix.v.conv", beta="mix.b", decay="mix.a", decay_log="mix.A_log",
                                      decay_bias="mix.dt_bias", out_norm="mix.norm", gate="mix.g", o="mix.o")

    @property
    def qk_size(self) -> int:
        return self.kv_heads * self.key_dim

    @property
    def v_size(self) -> int:
        return self.heads * self.value_dim


@dataclass(frozen=True)
class RGLRUSpec:
    """Recurrent block with a real-gated linear recurrent unit: a GELU branch and a branch of convolution and a
    diagonal recurrence whose decay ``a = exp(-decay_scale * r * softplus(lam))`` and input gate come from
    block-diagonal projections (``blocks`` square blocks) of the convolution's output."""
    hidden: int
    width: int
    blocks: int
    conv_taps: int
    decay_scale: float = 8.0
    kind: str = "rglru"
    names: Mapping[str, str] = _names(y="mix.y", y_bias="mix.y.b", x="mix.x", x_bias="mix.x.b", conv="mix.conv",
                                      conv_bias="mix.conv.b", r="mix.ra", r_bias="mix.ra.b", i="mix.ri",
                                      i_bias="mix.ri.b", lam="mix.lam", o="mix.o")


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are up-projections of one cached latent vector per token
    (``latent_rank`` numbers, RMS-normed); the softmax denominator may hold a learned per-head sink, and a sigmoid
    gate may multiply the output: one number a head (``gate_per`` "head") or one a column of the concatenated heads
    ("column").  Options, each a mechanism of its own:

    * ``rotary_dim`` > 0 with ``position``: beside the ``key_dim`` numbers that come from the latent, every head's
      query has ``rotary_dim`` rotated numbers (a head's query is laid out ``[key_dim | rotary_dim]``), and the down
      projection has ``rotary_dim`` more rows: one rotated key part a token, not normed, shared by all heads and
      cached behind the latent; the score is the sum of both dot products;
    * ``query_rank``: the queries come through a latent of their own, ``q = W_uq rmsnorm(W_dq x)``;
    * ``window``: a row sees the last ``window`` keys, its own included."""
    hidden: int
    heads: int
    key_dim: int
    value_dim: int
    latent_rank: int
    scale: float
    norm_eps: float
    sink: bool = True
    gated: bool = True
    gate_per: str = "head"
    rotary_dim: int = 0
    position: Optional[object] = None
    query_rank: Optional[int] = None
    window: Optional[int] = None
    kind: str = "latent_attention"
    names: Mapping[str, str] = _names(q="mix.q", down="mix.dkv", down_norm="mix.dkv.norm", up_k="mix.uk",
                                      up_v="mix.uv", sink="mix.sink", gate="mix.g", o="mix.o", q_down="mix.dq",
                                      q_down_norm="mix.dq.norm", q_up="mix.uq")

    @property
    def query_dim(self) -> int:
        return self.key_dim + self.rotary_dim

    @property
    def cached_width(self) -> int:
        return self.latent_rank + self.rotary_dim


@dataclass(frozen=True)
class MoESpec:
    """Mixture of gated feed-forward experts: the ``top`` largest router logits choose, the softmax over the
    chosen logits weighs.  ``names["expert"]`` is formatted with the expert's index."""
    hidden: int
    experts: int
    top: int
    intermediate: int
    activation: str = "silu"
    kind: str = "moe"
    names: Mapping[str, str] = _names(router="mlp.router", expert="mlp.e{}.", gate="gate", up="up", down="down")


@dataclass(frozen=True)
class ComputedRopeSpec:
    """Rotary encoding whose angles the kernels compute from the position (32-bit ``position * f_i`` with
    ``f_i = theta^(-2i/rotary_dim)``): no table, so no longest context has to be known.  The pairs are the halves
    ``(i, i + rotary_dim / 2)`` or, with ``interleaved``, the neighbours ``(2i, 2i + 1)``.  ``stretch`` = (factor, low,
    high, original) slows the slow pairs down: with ``turns_i = original f_i / (2 pi)`` (how often pair i goes round
    within ``original`` positions) and ``t_i = clamp((turns_i - low) / (high - low), 0, 1)``, the frequency becomes
    ``f_i (t_i + (1 - t_i) / factor)`` — untouched from ``high`` turns on, divided by ``factor`` up to ``low`` turns."""
    head_dim: int
    rotary_dim: int
    theta: float
    interleaved: bool = False
    stretch: Optional[Sequence[float]] = None
    kind: str = "rope_computed"


@dataclass(frozen=True)
class RetentionSpec:
    """Retention: linear attention with one fixed decay a head and neither softmax nor denominator.  Per head a
    matrix state ``S [key_dim, value_dim]``: ``S <- decay * S + k v^T``, read-out ``S^T q``.  q and k are rotated
    (``position``), k is scaled by ``key_scale`` after the rotation; the read-out of a head is divided by its root
    mean square (``norm_eps``, no weight) and multiplied by ``silu`` of a gate projection."""
    hidden: int
    heads: int
    key_dim: int
    value_dim: int
    decays: Sequence[float]           # one a head, in (0, 1]
    key_scale: float
    norm_eps: float
    position: Optional[object]
    kind: str = "retention"
    names: Mapping[str, str] = _names(q="mix.q", k="mix.k", v="mix.v", gate="mix.g", o="mix.o")

    @property
    def qk_size(self) -> int:
        return self.heads * self.key_dim

    @property
    def v_size(self) -> int:
        return self.heads * self.value_dim


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Differential attention: every head has two maps, each a causal softmax attention of its own (queries and keys
    of ``key_dim``, laid out head by head as [map 1 | map 2]) over the SAME values (``value_dim``); the head's output
    is ``a1 - lambda * a2`` with one ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init`` a layer, divided by
    its root mean square over ``value_dim`` (``norm_eps``, no weight) and multiplied by ``out_scale``.  q and k pass a
    per-map RMS norm (``qk_norm_eps``; None: no norm) and the rotation ``position``.  ``kv_heads`` key/value heads
    serve groups of query heads.  ``own_kv`` False: the mixer has no key/value tensors and reads another entry's
    cache."""
    hidden: int
    heads: int
    kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    lambda_init: float
    out_scale: float
    norm_eps: float
    qk_norm_eps: Optional[float]
    position: Optional[object]
    window: Optional[int] = None
    own_kv: bool = True
    kind: str = "diff_attention"
    names: Mapping[str, str] = _names(q="mix.q", k="mix.k", v="mix.v", o="mix.o", q_norm="mix.q.norm",
                                      k_norm="mix.k.norm", lq1="mix.lq1", lk1="mix.lk1", lq2="mix.lq2", lk2="mix.lk2")

    @property
    def q_size(self) -> int:
        return self.heads * 2 * self.key_dim

    @property
    def k_size(self) -> int:
        return self.kv_heads * 2 * self.key_dim

    @property
    def v_size(self) -> int:
        return self.kv_heads * self.value_dim


@dataclass(frozen=True)
class BiasedMLPSpec:
    """Two-matrix feed-forward with biases: ``W_down act(W_up x + b_up) + b_down``.  ``activation`` "xielu": for
    z > 0 ``softplus(p) z^2 + z / 2``, else ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` with the two learned
    numbers (p, q) of the tensor ``act``."""
    hidden: int
    intermediate: int
    activation: str = "xielu"
    kind: str = "biased_mlp"
    names: Mapping[str, str] = _names(up="mlp.up", up_bias="mlp.up.b", down="mlp.down", down_bias="mlp.down.b",
                                      act="mlp.act")


@dataclass(frozen=True)
class PlainMLPSpec:
    """Two-matrix feed-forward without biases or gate: ``W_down act(W_up x)``; ``activation`` "relu2": the square of
    ``max(z, 0)``."""
    hidden: int
    intermediate: int
    activation: str = "relu2"
    kind: str = "plain_mlp"
    names: Mapping[str, str] = _names(up="mlp.up", down="mlp.down")


@dataclass(frozen=True)
class ScoredMoESpec:
    """Mixture of gated feed-forward experts whose router scores every output with a softmax over ALL of them:
    ``experts`` real experts and behind them ``identity`` experts without tensors whose output is the input itself.
    The choice goes by ``score + correction`` (a learned vector), restricted to the ``groups_keep`` best of
    ``groups`` equal groups of neighbouring outputs (a group's score: its largest choice score); the ``top`` chosen
    outputs weigh with their scores, as they are (``renormalize`` False) or divided by their sum.  ``shared``: a
    gated feed-forward that runs for every row and is added, multiplied by ``sigmoid`` of a one-row projection
    (``shared_gate`` False: added as it is; its spec may be any feed-forward's).

    ``scoring`` "sigmoid": every output's score is the sigmoid of its own logit.  ``correction`` False: there is no
    correction tensor.  ``gated`` False: an expert is ``W_down act(W_up x)`` (no gate matrix; ``activation`` "relu2":
    the square of ``max(z, 0)``).  ``weigh`` "input": the weight multiplies what the expert READS, not what it gives:
    the output is the sum of ``expert(weight * x)``."""
    hidden: int
    experts: int
    identity: int
    top: int
    intermediate: int
    groups: int = 1
    groups_keep: int = 1
    renormalize: bool = False
    shared: Optional[object] = None
    activation: str = "silu"
    scoring: str = "softmax"
    correction: bool = True
    gated: bool = True
    weigh: str = "output"
    shared_gate: bool = True
    kind: str = "scored_moe"
    names: Mapping[str, str] = _names(router="mlp.router", correction="mlp.correction", expert="mlp.e{}.", gate="gate",
                                      up="up", down="down", shared_gate="mlp.shared.sg")

    @property
    def outputs(self) -> int:
        return self.experts + self.identity


@dataclass(frozen=True)
class ScaledRopeSpec:
    """Rotation of the first ``rotary_dim`` columns of a head by a table of cosines and sines per position, the pairs
    being neighbours ``(2i, 2i + 1)`` (``interleaved``) or halves ``(i, i + rotary_dim / 2)``.  With ``factor`` the low
    frequencies are stretched (YaRN): with ``turn(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta)``,
    ``lo = max(floor(turn(fast)), 0)``, ``hi = min(ceil(turn(slow)), rotary_dim - 1)`` and ``ramp_i = clamp((i - lo) /
    max(hi - lo, ramp_floor), 0, 1)`` the frequency of pair i is ``f_i / factor * ramp_i + f_i (1 - ramp_i)``, and
    cosine and sine are multiplied by ``gain_slope ln(factor) + 1``."""
    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    interleaved: bool = True
    factor: Optional[float] = None       # None: the plain frequencies theta^(-2i / rotary_dim)
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0
    gain_slope: float = 0.1
    ramp_floor: float = 0.001
    kind: str = "rope_scaled"


@dataclass(frozen=True)
class WindowAttentionSpec:
    """Softmax attention over a sliding window of ``window`` keys (the row's own included) and the first ``keep_first``
    keys of the sequence, with a term ``exp(sink)`` in the denominator that has no key and no value (``sink``
    "learned": one number a head; "zero": a score of 0, which adds 1; "none").  Options, each a mechanism of its own:

    * ``conv_taps`` > 0: q, k and v pass a short causal convolution per channel right behind their projections (no
      bias, no activation); a sequence's last ``conv_taps - 1`` projected rows are its state;
    * ``norm_eps`` not None: q and k are RMS-normed over their WHOLE projection (all heads at once), a weight a column;
    * ``values_from_keys``: there is no value projection, the values are the keys as projected (before norm and rotation);
    * ``position``: a rotation of q and k;
    * ``bias_rows`` > 0: a learned bias ``rel[bucket(distance), head]`` is added to the scaled score, with
      ``bucket(n) = n`` below ``bias_rows // 2`` and beyond it ``min(bias_rows - 1, half + floor(ln(n / half) /
      ln(bias_far / half) * (bias_rows - half)))``;
    * ``softcap``: the scaled score becomes ``softcap * tanh(score / softcap)``;
    * ``head_gate``: head h's output is multiplied by ``sigmoid`` of a one-row projection of the mixer's input."""
    hidden: int
    heads: int
    kv_heads: int
    key_dim: int
    value_dim: int
    scale: float
    window: int
    keep_first: int = 0
    conv_taps: int = 0
    norm_eps: Optional[float] = None
    values_from_keys: bool = False
    position: Optional[object] = None
    bias_rows: int = 0
    bias_far: float = 0.0
    softcap: Optional[float] = None
    sink: str = "learned"
    head_gate: bool = False
    # False: the mixer has no key/value tensors (projections, their convolutions and norms) and reads another entry's
    # cache, with queries, window, sink and everything else of its own
    own_kv: bool = True
    # how many keys back the cache has to reach (another entry that reads this cache may look further back than
    # ``window``); None: ``window``
    cache_window: Optional[int] = None
    kind: str = "window_attention"
    names: Mapping[str, str] = _names(q="mix.q", k="mix.k", v="mix.v", o="mix.o", q_norm="mix.q.norm", k_norm="mix.k.norm",
                                      q_conv="mix.q.conv", k_conv="mix.k.conv", v_conv="mix.v.conv", bias="mix.rel",
                                      sink="mix.sink", gate="mix.g")

    @property
    def q_size(self) -> int:
        return self.heads * self.key_dim

    @property
    def k_size(self) -> int:
        return self.kv_heads * self.key_dim

    @property
    def v_size(self) -> int:
        return self.kv_heads * self.value_dim


@dataclass(frozen=True)
class HyperSpec:
    """Hyper-connections: ``streams`` copies of the residual stream.  A sub-layer reads ``sum_s in[s] x_s`` and its
    output y is written back as ``x_t <- sum_s mix[s, t] x_s + out[t] y`` for all t at once.  ``names``: the tensors'
    prefixes for the mixer's and the feed-forward's connections."""
    streams: int
    names: Mapping[str, str] = _names(mixer="hc1.", ffn="hc2.")


@dataclass(frozen=True)
class BlockSpec:
    """One layer: ``h += mixer(norm_in(h)); h += ffn(norm_post(h))`` for
    ``arrangement == "prenorm"``; ``h += norm_in(mixer(h)); h += norm_post(ffn(h))``
    for ``arrangement == "outnorm"`` (the norms sit on the sub-layers' outputs,
    the sub-layers read the stream itself); ``arrangement == "hyper"``: the pre-norm
    layer over several streams (``hyper``); ``ffn`` and ``norm_post`` None: the layer has
    no feed-forward.  ``prefix`` is the layer's tensor-name prefix in the
    weight files."""
    prefix: str
    mixer: object
    ffn: Optional[object]
    norm_in: object
    norm_post: Optional[object]
    arrangement: str = "prenorm"
    names: Mapping[str, str] = _names(norm_in="input_layernorm.",
                                      norm_post="post_attention_layernorm.")
    hyper: Optional[HyperSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """Run layer ``layer``.  ``reads_cache_of`` names an earlier entry of the
    schedule (by its index in the list) whose cache this entry's mixer reads
    instead of keeping one of its own."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class BigramSpec:
    """A second embedding by the pair (previous token, token): row ``(previous * mul_prev + token * mul_cur) mod
    buckets`` of the table ``name`` ``[buckets + 1, hidden]`` is added to the token's embedding; a sequence's first
    token takes the table's last row.  The previous token is per-request state."""
    buckets: int
    mul_prev: int
    mul_cur: int
    name: str = "bigram"


@dataclass(frozen=True)
class ModelSpec:
    vocab: int
    hidden: int
    blocks: Sequence[BlockSpec]
    schedule: Sequence[ScheduleEntry]
    final_norm: object
    tie_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    max_positions: int = 0
    eos_token_ids: Sequence[int] = field(default_factory=tuple)
    # "float32": the residual stream is kept and summed in 32-bit whatever the compute dtype (norms read it and
    # give the compute dtype); None: the stream has the compute dtype
    stream_dtype: Optional[str] = None
    # a learned vector per place, added to the embedding (a table [max_positions, hidden]); None: no such table
    position_name: Optional[str] = None
    # > 0: the model keeps this many copies of the residual stream (blocks of the "hyper" arrangement); its output is
    # the final norm of their sum
    streams: int = 0
    # the logits are the head's product times this number
    logit_scale: float = 1.0
    bigram: Optional[BigramSpec] = None

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            if e.reads_cache_of is not None:
                if not 0 <= e.reads_cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, "
                                     "which must be an earlier entry")
                if self.schedule[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, "
                                     "which keeps none of its own")
