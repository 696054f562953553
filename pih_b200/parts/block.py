"""The arrangement of parts in a layer.

``prenorm``: ``h += mixer(norm_in(h)); h += ffn(norm_post(h))``
(plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:19-39).  The block
passes on the residual stream ``h`` together with ``delta``, the last
sub-layer's output that is not yet added, so that the add fuses with the
next norm wherever that norm lives (the next block's, or the model's final
norm).  ``delta`` is None when the last sub-layer has added its output itself
(for few rows the output projections add the residual in their epilogue).
A layer whose spec has no feed-forward is ``h += mixer(norm_in(h))`` alone.
"""
from __future__ import annotations

import torch

from .registry import Runtime, TensorInfo, part_class, register_block


def _sub(weights, names, prefix=""):
    return {rel: weights[prefix + rel] for rel in names}


@register_block("prenorm")
class PreNormBlock:
    @classmethod
    def expected_tensors(cls, spec):
        out = {}
        n = spec.names
        for rel, info in part_class("norm", spec.norm_in.kind).expected_tensors(spec.norm_in).items():
            out[n["norm_in"] + rel] = info
        out.update(part_class("mixer", spec.mixer.kind).expected_tensors(spec.mixer))
        if spec.ffn is not None:                   # a layer may have no feed-forward (and then no second norm)
            for rel, info in part_class("norm", spec.norm_post.kind).expected_tensors(spec.norm_post).items():
                out[n["norm_post"] + rel] = info
            out.update(part_class("ffn", spec.ffn.kind).expected_tensors(spec.ffn))
        return out

    def __init__(self, spec, weights, rt: Runtime):
        self.spec = spec
        self.rt = rt
        n = spec.names
        norm_in_cls = part_class("norm", spec.norm_in.kind)
        mixer_cls = part_class("mixer", spec.mixer.kind)
        self.norm_in = norm_in_cls(
            spec.norm_in, _sub(weights, norm_in_cls.expected_tensors(spec.norm_in), n["norm_in"]), rt)
        self.mixer = mixer_cls(spec.mixer, _sub(weights, mixer_cls.expected_tensors(spec.mixer)), rt)
        self.norm_post = self.ffn = None
        if spec.ffn is not None:
            norm_post_cls = part_class("norm", spec.norm_post.kind)
            ffn_cls = part_class("ffn", spec.ffn.kind)
            self.norm_post = norm_post_cls(
                spec.norm_post, _sub(weights, norm_post_cls.expected_tensors(spec.norm_post), n["norm_post"]), rt)
            self.ffn = ffn_cls(spec.ffn, _sub(weights, ffn_cls.expected_tensors(spec.ffn)), rt)
        self._native_ok = None             # decided at the first step

    def forward(self, h, delta, step, cache):
        # kernels that can issue a whole block of these parts from one native call get it (the same kernels in the
        # same order as below; what they do not take comes back as None)
        if self._native_ok is None:
            native = getattr(self.rt.ops, "native_block", None)
            self._native_ok = native is not None and self.rt.ops._native_supports(self)
        if self._native_ok:
            done = self.rt.ops.native_block(self, h, delta, step, cache)
            if done is not None:
                return done
        # a part that can take "add, norm, then me" as one call gets it (fewer kernels for few rows);
        # any other part gets the normed rows
        fused_in = getattr(self.norm_in, "fusable", False)
        fused_post = getattr(self.norm_post, "fusable", False)
        if fused_in and hasattr(self.mixer, "forward_prenorm"):
            h, a = self.mixer.forward_prenorm(h, delta, self.norm_in, step, cache)
        else:
            a = self.mixer.forward(self.norm_in.add_forward(h, delta), step, cache)
        if self.ffn is None:
            return h, a
        if fused_post and hasattr(self.ffn, "forward_prenorm"):
            return self.ffn.forward_prenorm(h, a, self.norm_post)
        return h, self.ffn.forward(self.norm_post.add_forward(h, a))


@register_block("outnorm")
class OutNormBlock:
    """``h += norm_in(mixer(h)); h += norm_post(ffn(h))``: the norms sit on the sub-layers' outputs and the sub-layers
    read the stream itself.  The stream ``h`` is 32-bit; a sub-layer reads its rounding to the compute dtype, which the
    kernel that adds a normed output to the stream writes beside the sum (``step.stream_copy`` hands the last one to
    the next block, so that only the first block of a step has to round the stream itself).  A bias that a
    feed-forward adds to its output (``ffn.output_bias``) is added by the same kernel, before the norm."""

    @classmethod
    def expected_tensors(cls, spec):
        return PreNormBlock.expected_tensors.__func__(cls, spec)

    def __init__(self, spec, weights, rt: Runtime):
        PreNormBlock.__init__(self, spec, weights, rt)
        for norm in (self.norm_in, self.norm_post):
            if norm is not None and not hasattr(norm, "weight_f32"):
                raise TypeError("a norm on a sub-layer's output needs a weight vector")

    def _input(self, h, step):
        if h.dtype == self.rt.dtype:
            return h
        held = getattr(step, "stream_copy", None)
        if held is not None and held[0] is h:
            return held[1]
        return self.rt.ops.stream_cast(h, self.rt.dtype)

    def _add(self, h, y, norm, step, bias=None):
        ops = self.rt.ops
        x = ops.stream_norm_add(h, y, norm.weight_f32, norm.spec.eps, bias=bias,
                                copy_dtype=self.rt.dtype if h.dtype != self.rt.dtype else None)
        step.stream_copy = (h, x) if x is not None else None

    def forward(self, h, delta, step, cache):
        if delta is not None:
            raise ValueError("a block with norms on its outputs takes a stream with nothing left to add")
        self._add(h, self.mixer.forward(self._input(h, step), step, cache), self.norm_in, step)
        if self.ffn is not None:
            y = self.ffn.forward(self._input(h, step))
            self._add(h, y, self.norm_post, step, bias=getattr(self.ffn, "output_bias", None))
        return h, None


@register_block("hyper")
class HyperBlock:
    """A pre-norm layer over several residual streams (``spec.hyper``: hyper-connections).  The streams ``x`` are
    32-bit ``[T, S, width]``.  For each sub-layer (the mixer, then the feed-forward) with its learned ``in [S]``,
    ``out [S]`` and ``mix [S, S]`` (indexed [from, to])::

        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y      (all t at once)

    One kernel pass over a row writes the pending ``y`` of the sub-layer before into the streams and reads the next
    ``u`` out of them, normed and rounded to the compute dtype; so the block hands on ``(x, pending)`` where
    ``pending = (y, mix, out)`` of its last sub-layer, for the next block's first pass (or the model's last)."""

    @classmethod
    def expected_tensors(cls, spec):
        out = PreNormBlock.expected_tensors.__func__(cls, spec)
        S = spec.hyper.streams
        subs = ["mixer"] + (["ffn"] if spec.ffn is not None else [])
        for sub in subs:
            p = spec.hyper.names[sub]
            out[p + "in"] = TensorInfo((S,), "unit_normal")
            out[p + "out"] = TensorInfo((S,), "unit_normal")
            out[p + "mix"] = TensorInfo((S, S), "unit_normal")
        return out

    def __init__(self, spec, weights, rt: Runtime):
        PreNormBlock.__init__(self, spec, weights, rt)
        for norm in (self.norm_in, self.norm_post):
            if norm is not None and not hasattr(norm, "weight_f32"):
                raise TypeError("a layer over several streams norms with a weight vector")
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.links = {}
        for sub in ("mixer", "ffn"):
            if sub == "ffn" and spec.ffn is None:
                continue
            p = spec.hyper.names[sub]
            self.links[sub] = tuple(weights[p + r].to(**f32).contiguous() for r in ("in", "mix", "out"))

    def _read(self, x, pending, sub, norm):
        """Write the pending output into the streams, then the input of sub-layer ``sub``."""
        collect, _, _ = self.links[sub]
        y, mix, spread = pending if pending is not None else (None, None, None)
        return self.rt.ops.hyper_stream(x, y, mix=mix, spread=spread, collect=collect, weight=norm.weight_f32,
                                        eps=norm.spec.eps, out_dtype=self.rt.dtype)

    def forward(self, x, pending, step, cache):
        u = self._read(x, pending, "mixer", self.norm_in)
        y = self.mixer.forward(u, step, cache)
        pending = (y, self.links["mixer"][1], self.links["mixer"][2])
        if self.ffn is not None:
            u = self._read(x, pending, "ffn", self.norm_post)
            pending = (self.ffn.forward(u), self.links["ffn"][1], self.links["ffn"][2])
        return x, pending
