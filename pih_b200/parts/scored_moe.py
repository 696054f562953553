"""Mixture of experts with scores over all router outputs, groups, identity experts and a shared expert.

Router logits ``z = W_r x`` are 32-bit; ``s = softmax(z)`` over ALL ``experts + identity`` outputs.  The choice goes
by ``s + correction``: outputs form ``groups`` equal groups of neighbours, a group's score is its largest choice
score, only outputs of the ``groups_keep`` best groups can be chosen, and of those the ``top`` largest are (ties: the
smaller index).  The weights are the chosen outputs' ``s`` (divided by their sum only with ``renormalize``).  Output
``e < experts`` is the gated feed-forward ``W_down_e (silu(W_gate_e x) * (W_up_e x))``; an output behind them is an
identity expert: the row itself.  A shared expert of the same form runs for every row and is added, multiplied by
``sigmoid(w_sg . x)``.

What the spec switches, each on its own: ``scoring`` "sigmoid" (a score is the sigmoid of the output's own logit);
no correction tensor; experts of two matrices without a gate, ``W_down act(W_up x)`` with the squared ReLU; weights
that multiply what an expert READS (``weigh`` "input": the output is the sum of ``expert(weight * x)``, each product
``weight * x`` rounded to the compute dtype like any expert's input); a shared expert of any feed-forward kind that is
added without a gate.

Routing, grouping by expert, the experts' products and the weighted sum are the kernels of the mixture whose
weights are a softmax over the chosen (``parts/moe.py``) with another routing kernel in front; the one-row gate
of the shared expert is one more row of the router's product.
"""
from __future__ import annotations

import torch

from .registry import Runtime, TensorInfo, part_class, register_ffn
from ._bind import bind_matrix


@register_ffn("scored_moe")
class ScoredMixtureOfExperts:
    pad_safe = True            # row-wise: rows of padding are routed and computed like any other and never read

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        out = {n["router"]: TensorInfo((spec.outputs, spec.hidden))}
        if getattr(spec, "correction", True):
            out[n["correction"]] = TensorInfo((spec.outputs,))
        for e in range(spec.experts):
            p = n["expert"].format(e)
            if getattr(spec, "gated", True):
                out[p + n["gate"]] = TensorInfo((spec.intermediate, spec.hidden))
            out[p + n["up"]] = TensorInfo((spec.intermediate, spec.hidden))
            out[p + n["down"]] = TensorInfo((spec.hidden, spec.intermediate))
        if spec.shared is not None:
            out.update(part_class("ffn", spec.shared.kind).expected_tensors(spec.shared))
            if getattr(spec, "shared_gate", True):
                out[n["shared_gate"]] = TensorInfo((1, spec.hidden))
        return out

    def __init__(self, spec, weights, rt: Runtime):
        self.gated = getattr(spec, "gated", True)
        self.scoring, self.weigh = getattr(spec, "scoring", "softmax"), getattr(spec, "weigh", "output")
        self.shared_gate = getattr(spec, "shared_gate", True) and spec.shared is not None
        if spec.activation != ("silu" if self.gated else "relu2"):
            raise ValueError("the experts are gated with activation 'silu' or of two matrices with 'relu2', got "
                             f"gated={self.gated} with {spec.activation!r}")
        if self.scoring not in ("softmax", "sigmoid") or self.weigh not in ("output", "input"):
            raise ValueError(f"scoring must be 'softmax' or 'sigmoid' and weigh 'output' or 'input', got "
                             f"{self.scoring!r} and {self.weigh!r}")
        if not 1 <= spec.top <= spec.outputs or spec.outputs % spec.groups or not 1 <= spec.groups_keep <= spec.groups:
            raise ValueError("scored mixture of experts: top, groups and groups_keep do not fit the router's outputs")
        self.spec, self.rt = spec, rt
        n = spec.names
        router = [weights[n["router"]]] + ([weights[n["shared_gate"]]] if self.shared_gate else [])
        self.w_router = bind_matrix(torch.cat(router, dim=0), rt)          # the shared expert's gate is the last row
        self.correction = None
        if getattr(spec, "correction", True):
            self.correction = weights[n["correction"]].to(device=rt.device, dtype=torch.float32).contiguous()
        # [experts, 2 ff, hidden]: an expert's gate rows and then its up rows; without a gate [experts, ff, hidden]
        self.w_gate_up = bind_matrix(torch.cat([torch.stack([weights[n["expert"].format(e) + n[r]]
                                                             for e in range(spec.experts)])
                                                for r in (("gate", "up") if self.gated else ("up",))], dim=1), rt)
        self.w_down = bind_matrix(torch.stack([weights[n["expert"].format(e) + n["down"]] for e in range(spec.experts)]), rt)
        self.shared = None
        if spec.shared is not None:
            cls = part_class("ffn", spec.shared.kind)
            self.shared = cls(spec.shared, {name: weights[name] for name in cls.expected_tensors(spec.shared)}, rt)

    def forward(self, x):
        s, ops = self.spec, self.rt.ops
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)      # [T, outputs (+ 1)], 32-bit
        out = ops.moe_experts(x, logits, self.w_gate_up, self.w_down, s.top,
                              routing=dict(outputs=s.outputs, correction=self.correction, groups=s.groups,
                                           groups_keep=s.groups_keep, renormalize=s.renormalize, scoring=self.scoring,
                                           gated=self.gated, weigh=self.weigh))
        if self.shared is not None:
            return ops.add_gated(out, self.shared.forward(x), logits[:, s.outputs] if self.shared_gate else None)
        return out
