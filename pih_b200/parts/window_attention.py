"""Softmax attention over a sliding window with a sink in the denominator, as a mixer.

A row at position p sees the keys j <= p with ``p - j < window`` or ``j < keep_first`` (kept first keys keep their
true positions).  With ``q [heads, key_dim]``, ``k [kv_heads, key_dim]``, ``v [kv_heads, value_dim]`` and query head h
reading key/value head ``h // (heads // kv_heads)``::

    s_j = scale q . k_j;   softcap: s_j <- c tanh(s_j / c);   bias: s_j <- s_j + rel[bucket(p - j), h]
    w_j = exp(s_j) / (sum over the seen keys of exp(s_i) + exp(sink_h))         (sink "zero": + 1; "none": no such term)
    o   = sum_j w_j v_j;   head_gate: o <- o sigmoid(g_h),  g = W_g x

What the spec switches on, each on its own (``WindowAttentionSpec``): short causal convolutions behind the q, k and v
projections (the last ``taps - 1`` projected rows of a request are its state, in a state slot beside the pages); an
RMS norm of q and of k over the WHOLE projection; values that are the keys as projected; a rotation of q and k; the
bias by distance (the learned table ``[bias_rows, heads]`` is spread out once into one number a distance inside the
window, so the kernels index it by the distance itself); capped scores; the gate a head.

The cache holds ONE vector per token, ``[k: kv_heads x key_dim | v: kv_heads x value_dim]`` after norm and rotation
(``PagedVectorNeed`` with the window and the kept first tokens: the pages between them go back to the pool).  Scores,
softmax, sink and gate are 32-bit whatever the compute dtype.

A mixer built with ``own_kv`` False has no key/value tensors: its schedule entry reads another entry's cache, with
queries, window, sink and output projection of its own.  The entry that keeps the cache holds it as far back as
``cache_window`` says (the widest window of those that read it).  The rotation comes from a table of cosines and
sines per position or, from a position part that computes its angles, from frequencies: ``position * f_i`` in 32-bit
inside the kernel.
"""
from __future__ import annotations

import math

import torch

from .registry import PagedStateNeed, PagedVectorNeed, Runtime, StateNeed, TensorInfo, part_class, register_mixer
from ._bind import bind_matrix


def distance_bucket(n: int, rows: int, far: float) -> int:
    """The row of a bias table of ``rows`` rows for the distance ``n >= 0``: one row a distance below ``rows // 2``,
    the other rows spread logarithmically from there up to the distance ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def bias_by_distance(table: torch.Tensor, far: float, distances: int) -> torch.Tensor:
    """fp32 ``[heads, distances]`` from the learned ``[rows, heads]``: column n is the bias at distance n."""
    rows = table.shape[0]
    index = torch.tensor([distance_bucket(n, rows, far) for n in range(distances)], dtype=torch.long)
    return table.to(torch.float32)[index].t().contiguous()


@register_mixer("window_attention")
class WindowAttention:
    pad_safe = True            # rows of no request carry the padding slot: nothing is written for them, and what is
                               # computed for them is never read

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        own = getattr(spec, "own_kv", True)
        out = {n["q"]: TensorInfo((spec.q_size, spec.hidden)), n["o"]: TensorInfo((spec.hidden, spec.heads * spec.value_dim))}
        if own:
            out[n["k"]] = TensorInfo((spec.k_size, spec.hidden))
        if own and not spec.values_from_keys:
            out[n["v"]] = TensorInfo((spec.v_size, spec.hidden))
        if spec.norm_eps is not None:
            out[n["q_norm"]] = TensorInfo((spec.q_size,), "one_plus_normal")
            if own:
                out[n["k_norm"]] = TensorInfo((spec.k_size,), "one_plus_normal")
        if spec.conv_taps > 0:
            out[n["q_conv"]] = TensorInfo((spec.q_size, spec.conv_taps), "conv")
            if own:
                out[n["k_conv"]] = TensorInfo((spec.k_size, spec.conv_taps), "conv")
            if own and not spec.values_from_keys:
                out[n["v_conv"]] = TensorInfo((spec.v_size, spec.conv_taps), "conv")
        if spec.bias_rows > 0:
            out[n["bias"]] = TensorInfo((spec.bias_rows, spec.heads), "unit_normal")
        if spec.sink == "learned":
            out[n["sink"]] = TensorInfo((spec.heads,), "unit_normal")
        if spec.head_gate:
            out[n["gate"]] = TensorInfo((spec.heads, spec.hidden))
        return out

    def __init__(self, spec, weights, rt: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"heads ({spec.heads}) must be a multiple of kv_heads ({spec.kv_heads})")
        if spec.window < 0 or spec.keep_first < 0:
            raise ValueError("window and keep_first must not be negative")
        if spec.values_from_keys and spec.value_dim != spec.key_dim:
            raise ValueError("values that are the keys need value_dim == key_dim")
        if spec.sink not in ("learned", "zero", "none"):
            raise ValueError(f"sink must be 'learned', 'zero' or 'none', got {spec.sink!r}")
        if spec.bias_rows > 0 and (spec.bias_rows < 2 or spec.bias_far <= spec.bias_rows // 2):
            raise ValueError("a bias by distance needs at least 2 rows and a far distance beyond half of them")
        self.spec, self.rt = spec, rt
        self.own_kv = own = getattr(spec, "own_kv", True)
        n = spec.names
        f32 = dict(device=rt.device, dtype=torch.float32)
        # one product for everything that reads the block's input: [q | k | v | gate]
        parts = [weights[n["q"]]] + ([weights[n["k"]]] if own else [])
        if own and not spec.values_from_keys:
            parts.append(weights[n["v"]])
        self.channels = sum(p.shape[0] for p in parts)
        if spec.head_gate:
            parts.append(weights[n["gate"]])
        self.w_in = bind_matrix(torch.cat(parts, dim=0), rt)
        self.w_o = bind_matrix(weights[n["o"]], rt)
        self.w_conv = None
        if spec.conv_taps > 0:
            conv = [weights[n["q_conv"]]] + ([weights[n["k_conv"]]] if own else []) + (
                [weights[n["v_conv"]]] if own and not spec.values_from_keys else [])
            self.w_conv = bind_matrix(torch.cat(conv, dim=0), rt)
        self.q_norm = self.k_norm = None
        if spec.norm_eps is not None:
            self.q_norm = weights[n["q_norm"]].to(**f32).contiguous()
            self.k_norm = weights[n["k_norm"]].to(**f32).contiguous() if own else None
        self.bias = None
        if spec.bias_rows > 0:
            # beyond ``bias_far`` every distance has the last row; inside a window no distance reaches the window's size
            reach = int(math.ceil(spec.bias_far)) + 1
            distances = min(spec.window, reach) if spec.window > 0 else reach
            self.bias = bias_by_distance(weights[n["bias"]], spec.bias_far, distances).to(rt.device)
        self.sink = None
        if spec.sink == "learned":
            self.sink = weights[n["sink"]].to(**f32).contiguous()
        elif spec.sink == "zero":
            self.sink = torch.zeros(spec.heads, **f32)
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, rt)
            if self.position.rotation_table() is None and not hasattr(self.position, "frequencies"):
                raise TypeError("window attention rotates by a table of cosines and sines per position or by frequencies")

    def _state_numbers(self) -> int:
        return max(self.spec.conv_taps - 1, 0) * self.channels

    def cache_need(self):
        s = self.spec
        reach = getattr(s, "cache_window", None)
        reach = s.window if reach is None else reach            # (0: every key stays)
        paged = PagedVectorNeed(s.k_size + s.v_size, reach or None, s.keep_first if reach else 0) if self.own_kv else None
        if self._state_numbers() == 0:
            return paged
        if paged is None:
            return StateNeed((self._state_numbers(),), torch.float32)
        return PagedStateNeed(paged, StateNeed((self._state_numbers(),), torch.float32))

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        if cache.writable != self.own_kv:
            raise ValueError("window attention: the schedule entry's cache does not fit the mixer "
                             "(a mixer without keys and values reads another entry's cache, and only such a mixer)")
        proj = ops.linear(x, self.w_in)                      # [T, q | k | v | gate]
        gate = proj[:, self.channels:] if s.head_gate else None
        src = proj
        if self.w_conv is not None:
            state = cache.state if self._state_numbers() else proj.new_zeros((1, 1), dtype=torch.float32)
            src = ops.causal_conv(proj[:, :self.channels], self.w_conv, step=step, state=state, state_offset=0)
        table = self.position.rotation_table() if self.position is not None else None
        rotation = {}
        if self.position is not None and table is None:
            rotation = dict(frequencies=self.position.frequencies())
        if not self.own_kv:
            rotation["write_kv"] = False
        geometry = dict(heads=s.heads, kv_heads=s.kv_heads, key_dim=s.key_dim, value_dim=s.value_dim)
        q = ops.window_qk_prepare(src, q_norm=self.q_norm, k_norm=self.k_norm, eps=s.norm_eps or 0.0, rope_table=table,
                                  rotary_dim=self.position.rotary_dim if self.position is not None else 0,
                                  interleaved=getattr(self.position, "interleaved", False), positions=step.positions,
                                  slot_mapping=cache.slot_mapping, cache=cache.kv, values_from_keys=s.values_from_keys,
                                  **geometry, **rotation)
        attn = ops.window_attention(q, cache=cache.kv, block_table=cache.block_table, step=step, scale=s.scale,
                                    window=s.window, keep_first=s.keep_first, softcap=s.softcap or 0.0, bias=self.bias,
                                    sink=self.sink, gate=gate, **geometry)
        return ops.linear(attn, self.w_o)
