"""Mixers side by side: every branch reads the same input, and the result is

    scale * sum_k  out_k / sqrt(mean(out_k^2) + eps) * w_k

each branch's output normed over the model's width with a weight of its own before the sum (float32). A branch is any
registered mixer; what the branches keep per sequence stands one behind another in the call's declaration, and each
branch is handed the view of its own part.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import Mixer, TensorSpec


def _needs_of(need) -> tuple:
    return () if need is None else tuple(need) if isinstance(need, (tuple, list)) else (need,)


class ParallelMixer(Mixer):
    kind = "parallel"
    fixed_shape_ok = True      # (its branches must be too: checked when they are built)

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for branch in spec.branches:
            out.update(registry.mixer_class(branch.kind).tensors(branch))
        for name in spec.out_names:
            out[name] = TensorSpec((spec.hidden,), init="ones", role="vector")
        return out

    @classmethod
    def cache_need(cls, spec):
        needs = ()
        for branch in spec.branches:
            needs += _needs_of(registry.mixer_class(branch.kind).cache_need(branch))
        return needs if needs else None

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if not spec.branches or len(spec.branches) != len(spec.out_names):
            raise ValueError("parallel mixer: one output weight per branch, and at least one branch")
        self.spec, self.rt = spec, rt
        self.branches = [registry.mixer_class(b.kind)(b, weights, rt) for b in spec.branches]
        self.out_w = [rt.vector(weights[name]) for name in spec.out_names]
        self.spans = []
        at = 0
        for b in spec.branches:
            n = len(_needs_of(registry.mixer_class(b.kind).cache_need(b)))
            self.spans.append((at, at + n))
            at += n
        if not all(getattr(m, "fixed_shape_ok", False) for m in self.branches):
            raise ValueError("parallel mixer: every branch's prompt code must be capturable for any lengths (fixed_shape_ok)")

    def forward(self, x, step, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        acc = rt.ws.get("parallel_sum", (x.shape[0], s.hidden), torch.float32)
        for k, (mixer, w, (lo, hi)) in enumerate(zip(self.branches, self.out_w, self.spans)):
            y = mixer.forward(x, step, cache.sub(lo, hi) if cache is not None else None)
            ops.rmsnorm_accumulate(y, w, acc, s.eps, s.scale, add=k > 0)
        return acc


registry.register_mixer(ParallelMixer.kind, ParallelMixer)
