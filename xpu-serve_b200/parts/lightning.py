"""The lightning-attention mixer: a linear-attention memory per head with a constant decay.

    q = silu(Wq x),  k = silu(Wk x)   (heads of dim),   v = silu(Wv x)   (heads of vdim)
    S <- decay_h S + k v^T            S [dim, vdim] float32 per head, zero at a sequence's start
    o  = S^T q                        with the new S; no other scale

then the concatenated heads divided by their root mean square over all of them, times a weight, times sigmoid(Wg x), and
the output projection. One product gives q, k, v and the gate's logits in the activation type; silu, the decay, the state
and every sum behind it are float32 in both precision modes (csrc/lightning.cu). Single tokens and short pieces walk in
order; long pieces of a prompt run chunk by chunk side by side (a pass from the empty state, a carry between the chunks by
decay^length, a second pass from each chunk's true state).
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import Mixer, StateNeed, TensorSpec
from .mamba2 import chunk_plan


class LightningMixer(Mixer):
    kind = "lightning"
    fuses_norm = True          # few rows: the norm before it rides on its input product, its output product adds to the stream
    fixed_shape_ok = True      # the kernel finds every sequence's tokens in the step's description on the device

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        qd, vd = spec.heads * spec.dim, spec.heads * spec.vdim
        return {
            n["q"]: TensorSpec((qd, spec.hidden)), n["k"]: TensorSpec((qd, spec.hidden)),
            n["v"]: TensorSpec((vd, spec.hidden)), n["gate"]: TensorSpec((vd, spec.hidden)),
            n["o"]: TensorSpec((spec.hidden, vd)), n["norm"]: TensorSpec((vd,), init="ones", role="vector"),
        }

    @classmethod
    def cache_need(cls, spec):
        return StateNeed((spec.heads, spec.dim, spec.vdim), "float32")

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if spec.dim > 256:
            raise ValueError(f"lightning: key size {spec.dim} (at most 256 is supported)")
        if len(spec.decay) != spec.heads:
            raise ValueError(f"lightning: {len(spec.decay)} decays for {spec.heads} heads")
        self.spec, self.rt = spec, rt
        n = spec.names
        self.w_in = rt.matrix(torch.cat([weights[n[k]].to(torch.float32) for k in ("q", "k", "v", "gate")], 0))
        self.decay = rt.vector(torch.tensor(spec.decay, dtype=torch.float32))
        self.w_norm = rt.vector(weights[n["norm"]])
        self.w_o = rt.matrix(weights[n["o"]])
        # Pieces of at least two chunks run chunk by chunk side by side. XS_LIGHTNING_CHUNK: tokens a chunk (0: always in
        # order); unset: as many chunks as fill the device once with two CTAs an SM, between 64 and 512 tokens each.
        self.chunk = int(os.environ["XS_LIGHTNING_CHUNK"]) if "XS_LIGHTNING_CHUNK" in os.environ else None

    def takes_prenormed(self, rows: int) -> bool:
        return self.rt.few_rows_shape(rows, self.w_in) and self.w_in.shape[1] % 8 == 0

    def forward(self, x, step, cache, into=None) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if cache is None or cache.storage is None or not cache.owner:
            raise RuntimeError("lightning keeps its own state")
        T, qd, vd = x.shape[0], s.heads * s.dim, s.heads * s.vdim
        proj = rt.linear(x, self.w_in, "lightning_proj")
        y = rt.ws.get("lightning_y", (T, vd), torch.float32)
        chunks = None
        chunk = self.chunk
        if chunk is None:
            at_once = max(1, (2 * rt.sm_count) // (s.heads * -(-s.vdim // 32)))
            chunk = min(512, max(64, -(-T // at_once // 16) * 16))
        if chunk > 0 and not step.fixed_shape and not step.decode and step.max_q_len >= 2 * chunk:
            chunk_seq, first_chunk = chunk_plan(step, chunk, rt.device)
            chunks = (chunk_seq, first_chunk,
                      rt.ws.get("lightning_chunk_state", (chunk_seq.shape[0], s.heads, s.dim, s.vdim), torch.float32))
        ops.lightning_scan(proj, 0, qd, 2 * qd, self.decay, cache.storage, step.cu_seqlens, step.slots, y, s.heads, s.dim,
                           s.vdim, chunks)
        yn = rt.ws.get("lightning_normed", (T, vd), rt.act_dtype)
        ops.grouped_rmsnorm(y, self.w_norm, yn, 1, s.eps, gate=proj[:, 2 * qd + vd:])
        if into is not None:
            return into.product(yn, self.w_o)
        return rt.linear(yn, self.w_o, "mixer_out")


registry.register_mixer(LightningMixer.kind, LightningMixer)
