"""A causal language model put together from parts, driven by a ``ModelSpec``.

``CausalLM`` owns the embedding table, the blocks, the final norm and the
output head; the order in which layers run is ``spec.schedule`` (a list that
may name a layer twice, or let an entry read an earlier entry's cache).
Order of the whole pass from the reference's schedule
(plugins/model-qwen3/qwen3_bf16_execution_schedule.cpp:51-63): embedding,
the layers, final norm, gather of the rows whose logits are wanted, output
head with 32-bit logits (src/backend/cuda/gemm_plan.cpp:111-113).  The
reference norms every row and gathers afterwards
(kernels/cuda/qwen_bf16_primitives.cu:736-759); here only the wanted rows
are normed, which gives the same values for those rows.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import load_config
from ..config.specs import ModelSpec
from ..parts import part_class
from ..parts.registry import Runtime, StateNeed, TensorInfo
from ..parts._bind import bind_matrix
from ..weights.loader import load_weights, tensor_shapes


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorInfo]:
    """Every tensor the model reads, by its name in the weight files."""
    out = {spec.embed_name: TensorInfo((spec.vocab, spec.hidden))}
    if spec.position_name is not None:
        out[spec.position_name] = TensorInfo((spec.max_positions, spec.hidden))
    if spec.bigram is not None:
        out[spec.bigram.name] = TensorInfo((spec.bigram.buckets + 1, spec.hidden))
    for block in spec.blocks:
        cls = part_class("block", block.arrangement)
        for rel, info in cls.expected_tensors(block).items():
            out[block.prefix + rel] = info
    norm_cls = part_class("norm", spec.final_norm.kind)
    for rel, info in norm_cls.expected_tensors(spec.final_norm).items():
        out[spec.final_norm_prefix + rel] = info
    if not spec.tie_embeddings:
        out[spec.head_name] = TensorInfo((spec.vocab, spec.hidden))
    return out


class CausalLM:
    def __init__(self, spec: ModelSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.embed = bind_matrix(weights[spec.embed_name], rt)
        self.head = self.embed if spec.tie_embeddings else bind_matrix(weights[spec.head_name], rt)
        self.places = bind_matrix(weights[spec.position_name], rt) if spec.position_name is not None else None
        self.bigram = bind_matrix(weights[spec.bigram.name], rt) if spec.bigram is not None else None
        if self.bigram is not None and (spec.streams or self.places is not None):
            raise ValueError("a bigram embedding goes with one residual stream and no table of places")
        self._ones = torch.ones(spec.streams, dtype=torch.float32, device=rt.device) if spec.streams else None
        self.blocks = []
        for block in spec.blocks:
            cls = part_class("block", block.arrangement)
            rel = {name: weights[block.prefix + name] for name in cls.expected_tensors(block)}
            self.blocks.append(cls(block, rel, rt))
        norm_cls = part_class("norm", spec.final_norm.kind)
        self.final_norm = norm_cls(
            spec.final_norm,
            {name: weights[spec.final_norm_prefix + name] for name in norm_cls.expected_tensors(spec.final_norm)},
            rt)

    @property
    def pad_safe(self) -> bool:
        """Whether a step may be padded to a larger shape: every mixer and feed-forward has to leave padding alone."""
        return all(getattr(b.mixer, "pad_safe", False) and (b.ffn is None or getattr(b.ffn, "pad_safe", False))
                   for b in self.blocks)

    # -- what the cache manager must provide, per schedule entry -------------
    def cache_needs(self) -> List[Optional[object]]:
        """One need a schedule entry and, behind them, what the model itself keeps per request: with a bigram
        embedding the request's last token (one int32 in its state slot; the step function hands the model a
        view for every need, in this order)."""
        needs = []
        for entry in self.spec.schedule:
            if entry.reads_cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.blocks[entry.layer].mixer.cache_need())
        if self.bigram is not None:
            needs.append(StateNeed((1,), torch.int32))
        return needs

    # -- one pass over the rows of a step --------------------------------------
    def forward(self, step, caches) -> Optional[torch.Tensor]:
        """``step``: the packed batch; ``caches[i]``: the cache view of
        schedule entry i.  Returns fp32 logits ``[len(step.logit_rows), vocab]``
        or None when no logits are wanted."""
        ops = self.rt.ops
        wide = self.spec.stream_dtype == "float32" and self.rt.dtype != torch.float32
        if self.bigram is not None:
            # the token's row plus the row of the pair (previous token, token); the request's last token is read from
            # and left in its state slot, so a portion or a decoded token finds the token before it
            b = self.spec.bigram
            h = ops.embed_bigram(self.embed, self.bigram, step, state=caches[len(self.spec.schedule)].state,
                                 mul_prev=b.mul_prev, mul_cur=b.mul_cur, buckets=b.buckets,
                                 out_dtype=torch.float32 if wide else self.rt.dtype)
        elif self.spec.streams:
            # several residual streams, 32-bit, all equal to the embedding at the start; ``delta`` is the last
            # sub-layer's output with the coefficients that write it into the streams
            h = ops.embed_positions(self.embed, self.places, step.token_ids, step.positions, streams=self.spec.streams)
        elif self.places is not None:
            h = ops.embed_positions(self.embed, self.places, step.token_ids, step.positions,
                                    out_dtype=torch.float32 if wide else self.rt.dtype).reshape(-1, self.spec.hidden)
        elif wide:
            h = ops.embedding(self.embed, step.token_ids, out_dtype=torch.float32)      # the residual stream stays 32-bit
        else:
            h = ops.embedding(self.embed, step.token_ids)
        delta = None
        for i, entry in enumerate(self.spec.schedule):
            h, delta = self.blocks[entry.layer].forward(h, delta, step, caches[i])
        if step.num_logit_rows == 0:
            return None
        if self.spec.streams:
            # the model's output is the final norm of the streams' sum, for the wanted rows
            y, mix, spread = delta if delta is not None else (None, None, None)
            xn = ops.hyper_stream(h, y, mix=mix, spread=spread, collect=self._ones, weight=self.final_norm.weight_f32,
                                  eps=self.final_norm.spec.eps, rows=step.logit_rows, out_dtype=self.rt.dtype)
        else:
            xn = self.final_norm.add_forward(h, delta, rows=step.logit_rows)
        logits = ops.linear(xn, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0:
            ops.scale_(logits, self.spec.logit_scale)
        return logits


def load_model(model_dir: str, rt: Runtime):
    """config.json -> registered configuration -> spec -> weights -> CausalLM."""
    config = load_config(model_dir)
    if hasattr(config, "with_shapes"):                 # sizes that only the tensors' shapes give
        config = config.with_shapes(tensor_shapes(model_dir))
    spec = config.model_spec()
    expected = {n: i.shape for n, i in expected_tensors(spec).items()}
    optional = {spec.head_name: (spec.vocab, spec.hidden)} if spec.tie_embeddings else {}
    weights = load_weights(model_dir, expected, optional)
    return config, CausalLM(spec, weights, rt)
