"""How a step's token ids become the first rows of the residual stream, when it is more than a table lookup.

An embedding part declares its tensors and what it keeps per sequence like a mixer does, and fills the float32 stream:

    tensors(spec) -> {name: TensorSpec}          names relative to the model's prefix
    cache_need(spec) -> None | StateNeed | ...   its view is the cache's last one, behind the layer calls'
    __init__(spec, weights, rt, table)           `table`: the model's token table on the device (shared with a tied head)
    forward(step, cache, h)                      h: [tokens, width] float32

`PairHashEmbedding`: table[tok] * scale, plus a row of a second table chosen by a hash of the previous and the current
token (the table's last row for a sequence's first token), plus a sine/cosine vector of the position, then an RMS norm,
all in one kernel (csrc/norm_embed.cu: xs_embed_pair). A sequence's last token is kept in its slot (an int32 word), so a
later step's first token finds its predecessor there however the tokens were cut into steps. The frequencies are formed
in float64 and held in float32; the angle is the float32 product of position and frequency.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import Part, StateNeed, TensorSpec


class PairHashEmbedding(Part):
    kind = "pair_hash"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        return {n["pair"]: TensorSpec((spec.buckets + 1, spec.width)),
                n["norm"]: TensorSpec((spec.width,), init="ones", role="vector")}

    @classmethod
    def cache_need(cls, spec):
        return StateNeed((1,), "int32")

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt, table: torch.Tensor):
        if spec.buckets <= 0 or spec.mul_prev < 0 or spec.mul_cur < 0:
            raise ValueError("pair-hash embedding: buckets must be positive and the multipliers not negative")
        self.spec, self.rt, self.table = spec, rt, table
        n = spec.names
        self.pair = rt.matrix(weights[n["pair"]])
        self.w_norm = rt.vector(weights[n["norm"]])
        i = torch.arange((spec.width + 1) // 2, dtype=torch.float64)
        self.inv_freq = rt.vector(torch.tensor(float(spec.theta), dtype=torch.float64) ** (-2.0 * i / spec.width))

    def forward(self, step, cache, h: torch.Tensor) -> None:
        s = self.spec
        if cache is None or cache.storage is None:
            raise RuntimeError("the pair-hash embedding keeps each sequence's last token")
        ops.embed_pair(self.table, self.pair, step.tokens, step.positions, step.seq_of_token, step.cu_seqlens, step.slots,
                       cache.storage, self.inv_freq, self.w_norm, h, s.scale, s.buckets, s.mul_prev, s.mul_cur, s.eps)


class LearnedPositionEmbedding(Part):
    """table[tok] * scale + rows[position]: a learned vector per position joins the token's (csrc/layer_frame.cu: xs_embed_pos).
    Nothing is kept per sequence; a sequence cannot outgrow the rows (the model's `max_position` bounds the cache)."""
    kind = "learned_position"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        return {spec.names["rows"]: TensorSpec((spec.positions, spec.width))}

    @classmethod
    def cache_need(cls, spec):
        return None

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt, table: torch.Tensor):
        if spec.positions <= 0:
            raise ValueError("learned positions: the table needs at least one row")
        self.spec, self.rt, self.table = spec, rt, table
        self.rows = rt.matrix(weights[spec.names["rows"]])

    def forward(self, step, cache, h: torch.Tensor) -> None:
        if step.max_positions > self.spec.positions:
            raise RuntimeError(f"learned positions: the cache allows {step.max_positions} positions, the table has {self.spec.positions}")
        ops.embed_pos(self.table, self.rows, step.tokens, step.positions, h, float(getattr(self.spec, "scale", 1.0)))


registry.register_embedding(PairHashEmbedding.kind, PairHashEmbedding)
registry.register_embedding(LearnedPositionEmbedding.kind, LearnedPositionEmbedding)
