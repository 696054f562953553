"""Two-matrix feed-forward without biases or gate: ``W_down act(W_up x)``.

``activation`` "relu2" is the square of ``max(z, 0)``.  The up product is rounded to the compute dtype; the
activation is one kernel in 32-bit, rounded once; then the down product.  For few rows in bf16 the few-rows product
applies the activation in its epilogue (on the product's rounding: the same values).
"""
from __future__ import annotations

from .registry import Runtime, TensorInfo, register_ffn
from ._bind import bind_matrix

ACTIVATIONS = ("relu2",)


@register_ffn("plain_mlp")
class PlainMLP:
    pad_safe = True                        # row-wise: rows of padding are computed and never read

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        return {n["up"]: TensorInfo((spec.intermediate, spec.hidden)),
                n["down"]: TensorInfo((spec.hidden, spec.intermediate))}

    def __init__(self, spec, weights, rt: Runtime):
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"the two-matrix feed-forward supports activations {list(ACTIVATIONS)}, got {spec.activation!r}")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_up = bind_matrix(weights[n["up"]], rt)
        self.w_down = bind_matrix(weights[n["down"]], rt)

    def forward(self, x):
        ops = self.rt.ops
        act = None
        if x.shape[0] <= getattr(ops, "skinny_max_rows", 0) and hasattr(ops, "linear_skinny"):
            act = ops.linear_skinny(x, self.w_up, activation=self.spec.activation)      # None: not a shape it takes
        if act is None:
            act = ops.activation(ops.linear(x, self.w_up), self.spec.activation)
        return ops.linear(act, self.w_down)
