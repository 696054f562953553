"""Causal attention over a cached latent, as a mixer.

Per token one vector ``c = rmsnorm(W_down h) * w`` of ``latent_rank`` numbers is cached; head h's key is
``K_h c`` and its value ``V_h c``.  Scores are ``(q_h . k) * scale`` over the earlier tokens (all, or the last
``window``) and the token itself.  With ``sink`` the softmax denominator also holds ``exp(sink_h)``: a learned logit
per head without a key or a value.  With ``gated`` the output is multiplied by a sigmoid gate: one number a head
(``gate_per`` "head": ``sigmoid(G h)_h``) or one a column of the concatenated heads ("column").  Then the output
projection.

Keys and values are never formed: both are linear in c, so ``K_h`` is folded into the query
(``q'_h = K_h^T q_h``, a batched product) and ``V_h`` is applied to the weighted sum of latents (another batched
product); the attention kernel sees queries of ``latent_rank`` numbers and ONE cached vector per token that serves
every head as key and as value.  Scores, weights and sums are 32-bit.

With ``rotary_dim`` a head's query is ``[key_dim | rotary_dim]`` and the down projection gives ``rotary_dim`` more
numbers a token, one rotated key part for all heads.  The cached vector becomes ``[c | rotated key part]`` and the
folded query ``[K_h^T q_h | rotated q part]``: their dot product is the sum of both score terms, so the same kernel
serves (the fold's matrix carries an identity block for the rotated columns, the value fold zeros).  With
``query_rank`` the queries come through a latent of their own: ``q = W_uq rmsnorm(W_dq h)``.

In bfloat16 the cached vector is padded with zero columns to the next width that the tensor-core attention kernel has
an instance for (``TENSOR_CORE_WIDTHS``); the folds' matrices have zeros there, so scores and sums are what they are
without the padding.
"""
from __future__ import annotations

import torch

from .registry import PagedVectorNeed, Runtime, TensorInfo, part_class, register_mixer
from ._bind import bind_matrix


TENSOR_CORE_WIDTHS = (64, 128, 192, 256, 384, 512)


def cached_width(spec, dtype) -> int:
    """Numbers cached per token: the latent and the rotated key part, in bfloat16 padded to a tensor-core width."""
    width = spec.latent_rank + getattr(spec, "rotary_dim", 0)
    if dtype == torch.bfloat16:
        for w in TENSOR_CORE_WIDTHS:
            if width <= w:
                return w
    return width


@register_mixer("latent_attention")
class LatentAttention:
    pad_safe = True            # rows without a request are skipped; a padding row's cache slot is left alone

    @classmethod
    def expected_tensors(cls, spec):
        n = spec.names
        H, D, V, R = spec.heads, spec.key_dim, spec.value_dim, spec.latent_rank
        rot, q_rank = getattr(spec, "rotary_dim", 0), getattr(spec, "query_rank", None)
        out = {n["down"]: TensorInfo((R + rot, spec.hidden)),
               n["down_norm"]: TensorInfo((R,), "one_plus_normal"), n["up_k"]: TensorInfo((H * D, R)),
               n["up_v"]: TensorInfo((H * V, R)), n["o"]: TensorInfo((spec.hidden, H * V))}
        if q_rank is None:
            out[n["q"]] = TensorInfo((H * (D + rot), spec.hidden))
        else:
            out[n["q_down"]] = TensorInfo((q_rank, spec.hidden))
            out[n["q_down_norm"]] = TensorInfo((q_rank,), "one_plus_normal")
            out[n["q_up"]] = TensorInfo((H * (D + rot), q_rank))
        if spec.sink:
            out[n["sink"]] = TensorInfo((H,), "unit_normal")
        if spec.gated:
            out[n["gate"]] = TensorInfo((H * V if getattr(spec, "gate_per", "head") == "column" else H, spec.hidden))
        return out

    def __init__(self, spec, weights, rt: Runtime):
        self.spec, self.rt = spec, rt
        n = spec.names
        H, D, V, R = spec.heads, spec.key_dim, spec.value_dim, spec.latent_rank
        self.rot = rot = getattr(spec, "rotary_dim", 0)
        self.q_rank = getattr(spec, "query_rank", None)
        self.gate_per = getattr(spec, "gate_per", "head")
        if self.gate_per not in ("head", "column"):
            raise ValueError(f"gate_per must be 'head' or 'column', got {self.gate_per!r}")
        self.window = getattr(spec, "window", None) or None
        first = weights[n["q"]] if self.q_rank is None else weights[n["q_down"]]
        self.first_rows = first.shape[0]
        stacked = [first, weights[n["down"]]] + ([weights[n["gate"]]] if spec.gated else [])
        self.w_in = bind_matrix(torch.cat(stacked, dim=0), rt)                     # [q or its latent | latent | gate]
        f32 = dict(device=rt.device, dtype=torch.float32)
        self.w_q_up = self.q_norm = None
        if self.q_rank is not None:
            self.w_q_up = bind_matrix(weights[n["q_up"]], rt)
            self.q_norm = weights[n["q_down_norm"]].to(**f32).contiguous()
        # q'_h = q_h . K_h with K_h [D, R]: as a product with rows of outputs, the weight is K_h^T [R, D]; the rotated
        # columns of a head's query pass through an identity block, and the value fold has zeros for them
        self.cached = C = cached_width(spec, rt.dtype)
        fold = torch.zeros(H, C, D + rot, dtype=torch.float32)
        fold[:, :R, :D] = weights[n["up_k"]].to(torch.float32).reshape(H, D, R).transpose(1, 2)
        fold[:, R:R + rot, D:] = torch.eye(rot)
        self.w_fold_k = bind_matrix(fold, rt)                                                  # [H, C, D + rot]
        up_v = torch.zeros(H, V, C, dtype=torch.float32)
        up_v[:, :, :R] = weights[n["up_v"]].to(torch.float32).reshape(H, V, R)
        self.w_up_v = bind_matrix(up_v, rt)                                                    # [H, V, C]
        self.w_o = bind_matrix(weights[n["o"]], rt)
        self.down_norm = weights[n["down_norm"]].to(**f32).contiguous()
        self.sink = weights[n["sink"]].to(**f32).contiguous() if spec.sink else None
        self.position = None
        if rot:
            if getattr(spec, "position", None) is None:
                raise ValueError("a rotated key part needs a position part")
            self.position = part_class("position", spec.position.kind)(spec.position, {}, rt)
            if not hasattr(self.position, "frequencies") or self.position.rotary_dim != rot:
                raise TypeError("attention over a latent rotates its rotated part whole, by frequencies "
                                "(a position part that computes its angles)")

    def cache_need(self):
        return PagedVectorNeed(self.cached, self.window)

    def forward(self, x, step, cache):
        s, ops = self.spec, self.rt.ops
        H, D, V, R, rot = s.heads, s.key_dim, s.value_dim, s.latent_rank, self.rot
        T = x.shape[0]
        F = self.first_rows
        proj = ops.linear(x, self.w_in)                                     # [T, F + R + rot (+ gate)]
        rotation = {}
        if rot:
            rotation = dict(frequencies=self.position.frequencies(), interleaved=self.position.interleaved,
                            positions=step.positions)
        if self.q_rank is None:
            ops.latent_write(proj[:, F:F + R + rot], self.down_norm, s.norm_eps, cache.kv, cache.slot_mapping, **rotation)
            q = proj[:, :F].view(T, H, D + rot)
        else:
            # the kernel that norms the latent into the cache norms the queries' latent beside it
            cq = ops.latent_write(proj[:, F:F + R + rot], self.down_norm, s.norm_eps, cache.kv, cache.slot_mapping,
                                  query_latent=proj[:, :F], query_weight=self.q_norm, **rotation)
            q = ops.linear(cq, self.w_q_up).view(T, H, D + rot)
        # the last ``rot`` columns of every head are rotated on the way into the fold (few rows: inside its kernel)
        q_lat = ops.linear_batched(q, self.w_fold_k, rotate=dict(offset=D, **rotation) if rot else None)   # [T, H, C]
        gate = proj[:, F + R + rot:] if s.gated else None
        o_lat = ops.latent_attention(q_lat, gate=gate if self.gate_per == "head" else None, sink=self.sink,
                                     cache=cache.kv, block_table=cache.block_table, step=step, scale=s.scale,
                                     window=cache.window or 0)
        # the values' fold, and behind it the gate a column (few rows: in the fold's epilogue)
        heads_out = ops.linear_batched(o_lat, self.w_up_v, gate=gate if self.gate_per == "column" else None)
        return ops.linear(heads_out.view(T, H * V), self.w_o)
