"""RMSNorm as a part: ``y = (x / sqrt(mean(x^2) + eps)) * w``, rounded once.

Formula and rounding point: kernels/cuda/qwen_bf16_primitives.cu:285-324 of
the reference (oracle plugins/model-qwen3/qwen3_cpu_oracle.cpp:85-97): the
sum of squares, the reciprocal square root and both multiplications are in
32-bit; the weight multiplies directly.  ``add_forward`` fuses the residual
add that precedes a norm in a pre-norm block (reference: a separate kernel,
qwen_bf16_primitives.cu:264-272): the sum is formed in 32-bit, rounded to
the stream's dtype, stored back, and that rounded value is what is normed —
the same values as the two separate kernels give.
"""
from __future__ import annotations

import torch

from .registry import Runtime, TensorInfo, register_norm
from ._bind import bind_vector


@register_norm("rmsnorm")
class RMSNorm:
    fusable = True        # (weight, spec.eps) may be handed to an op that fuses this norm into a product

    @classmethod
    def expected_tensors(cls, spec):
        init = "normal" if getattr(spec, "offset", 0.0) else "one_plus_normal"
        return {getattr(spec, "weight_name", "weight"): TensorInfo((spec.width,), init)}

    def __init__(self, spec, weights, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = bind_vector(weights[getattr(spec, "weight_name", "weight")], rt)
        if getattr(spec, "offset", 0.0):
            # a weight stored around zero: ``offset + w`` multiplies, formed once in 32-bit
            self.weight = (self.weight.float() + float(spec.offset)).contiguous()
        self._weight_f32 = None

    @property
    def weight_f32(self):
        """The weight in 32-bit (made once), for the kernels that norm a 32-bit stream."""
        if self._weight_f32 is None:
            self._weight_f32 = self.weight if self.weight.dtype == torch.float32 else self.weight.float().contiguous()
        return self._weight_f32

    def forward(self, x, rows=None):
        return self.add_forward(x, None, rows=rows)

    def add_forward(self, h, delta, rows=None):
        if h.dtype != self.rt.dtype:
            # a residual stream kept in 32-bit beside a 16-bit compute dtype: the sum stays 32-bit, the normed rows
            # take the compute dtype
            return self.rt.ops.rmsnorm_stream(h, self.weight_f32, self.spec.eps, delta=delta, rows=rows,
                                              out_dtype=self.rt.dtype)
        return self.rt.ops.rmsnorm(h, self.weight, self.spec.eps, delta=delta, rows=rows)


@register_norm("scalar_rmsnorm")
class ScalarRMSNorm:
    """``y = x / sqrt(mean(x^2) + eps) * g`` with ONE learned number ``g`` for all coordinates (a tensor without
    axes, named by the block's norm prefix itself).  The stream ``h`` is 32-bit: ``add_forward`` sums ``h += delta``
    in 32-bit and gives the normed rows in the compute dtype."""
    fusable = False       # no product of the pack takes a one-number norm in its prologue

    @classmethod
    def expected_tensors(cls, spec):
        return {"": TensorInfo((), "one_plus_normal")}

    def __init__(self, spec, weights, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = weights[""].to(device=rt.device, dtype=torch.float32).reshape(1).contiguous()

    def forward(self, x, rows=None):
        return self.add_forward(x, None, rows=rows)

    def add_forward(self, h, delta, rows=None):
        if h.dtype != torch.float32:
            raise TypeError("the one-number RMS norm reads a 32-bit stream")
        return self.rt.ops.rmsnorm_stream(h, self.weight, self.spec.eps, delta=delta, rows=rows, out_dtype=self.rt.dtype)
