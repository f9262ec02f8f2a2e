"""Latent attention: the keys and values of all heads are made from one cached vector per position.

    q = Wq x                       per head [dim unrotated | rot_dim rotated]
    d = Wdown x                    [kv_rank + rot_dim]
    c = d[:kv_rank] / rms(d[:kv_rank]) * w_norm          the latent; k_rot = rotate(d[kv_rank:]), one for all heads
    key_h = [Wuk_h c | k_rot],  value_h = Wuv_h c,  score = scale * (q_h . key_h)

The cache keeps [c | k_rot] per position and nothing per head. Both per-head matrices are applied on the query's and the
output's side (q~_h = Wuk_h^T q_h[:dim]; out_h = Wuv_h sum_j p_j c_j), so the attention kernel reads cache rows only
(csrc/latent_attention.cu) and a step's cost does not depend on how many positions are cached per head. Options: a
window, a sink per head in the softmax's denominator, a sigmoid gate per head from the mixer's own input (or one per output
channel, `out_gate`), queries through a latent of their own (`q_rank`: q = Wuq (unit_rms(Wdq x) * w), the norm in float32),
no rotated part at all (rot_dim 0). One matrix product gives q (or the queries' latent), d and the gate logits (their
weights are stacked at load).
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import KVNeed, Mixer, TensorSpec


class LatentAttentionMixer(Mixer):
    kind = "latent_attention"
    fuses_norm = True          # few rows: the norm before it rides on its input product, its output product adds to the stream
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n, H = spec.names, spec.heads
        out = {}
        if spec.q_rank > 0:
            out[n["q_down"]] = TensorSpec((spec.q_rank, spec.hidden))
            out[n["q_norm"]] = TensorSpec((spec.q_rank,), init="ones", role="vector")
            out[n["q_up"]] = TensorSpec((H * (spec.dim + spec.rot_dim), spec.q_rank))
        else:
            out[n["q"]] = TensorSpec((H * (spec.dim + spec.rot_dim), spec.hidden))
        out.update({
            n["down"]: TensorSpec((spec.kv_rank + spec.rot_dim, spec.hidden)),
            n["latent_norm"]: TensorSpec((spec.kv_rank,), init="ones", role="vector"),
            n["up_k"]: TensorSpec((H * spec.dim, spec.kv_rank)),
            n["up_v"]: TensorSpec((H * spec.vdim, spec.kv_rank)),
        })
        if spec.out_gate:
            out[n["gate"]] = TensorSpec((H * spec.vdim, spec.hidden))
        elif spec.head_gate:
            out[n["gate"]] = TensorSpec((H, spec.hidden))
        if spec.sink:
            out[n["sink"]] = TensorSpec((H,), role="vector")
        out[n["o"]] = TensorSpec((spec.hidden, H * spec.vdim))
        return out

    @classmethod
    def cache_need(cls, spec):
        return KVNeed(1, spec.kv_rank + spec.rot_dim, spec.window, planes=1)

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        self.spec, self.rt = spec, rt
        n, H = spec.names, spec.heads
        if spec.position is not None and spec.position.head_dim != spec.rot_dim:
            raise ValueError("latent attention: the rotation's vector is the rotated part of a head")
        if spec.head_gate and spec.out_gate:
            raise ValueError("latent attention: a gate per head or one per output channel, not both")
        if spec.position is None and spec.rot_dim != 0:
            raise ValueError("latent attention: a rotated part needs a position encoding")

        def padded(t, to):          # (every part of the stacked product starts on a multiple of 8 columns: 16-byte rows)
            pad = (-t.shape[0]) % to
            return torch.cat([t, torch.zeros(pad, t.shape[1], dtype=t.dtype)], 0) if pad else t

        first = weights[n["q_down"]] if spec.q_rank > 0 else weights[n["q"]]
        self.q_cols = first.shape[0]
        self.down_cols = spec.kv_rank + spec.rot_dim
        rows = [padded(first, 8), padded(weights[n["down"]], 8)]
        self.down_at = rows[0].shape[0]
        self.gate_at = self.down_at + rows[1].shape[0]
        if spec.head_gate or spec.out_gate:
            rows.append(padded(weights[n["gate"]], 16))
        self.w_in = rt.matrix(torch.cat([r.to(torch.float32) for r in rows], 0))
        if spec.q_rank > 0:
            self.w_q_norm = rt.vector(weights[n["q_norm"]])
            self.w_q_up = rt.matrix(weights[n["q_up"]])
        self.w_norm = rt.vector(weights[n["latent_norm"]])
        # Wuk_h^T as [heads, kv_rank, dim] and Wuv_h as [heads, vdim, kv_rank]: the two batched products' weights
        self.w_uk_t = rt.matrix(weights[n["up_k"]].to(torch.float32).view(H, spec.dim, spec.kv_rank).transpose(1, 2))
        self.w_uv = rt.matrix(weights[n["up_v"]].to(torch.float32).view(H, spec.vdim, spec.kv_rank))
        self.sink = rt.vector(weights[n["sink"]]) if spec.sink else None
        self.w_o = rt.matrix(weights[n["o"]])
        self.position = (registry.position_class(spec.position.kind)(spec.position, rt)
                         if spec.position is not None else None)

    def takes_prenormed(self, rows: int) -> bool:
        return self.rt.few_rows_shape(rows, self.w_in) and self.w_in.shape[1] % 8 == 0

    def forward(self, x, step, cache, into=None) -> torch.Tensor:
        s, rt = self.spec, self.rt
        T, H, R = x.shape[0], s.heads, s.kv_rank
        if cache is None or cache.storage is None or not cache.owner:
            raise RuntimeError("latent attention needs a cache of its own")
        table = step.page_tables[cache.group]
        proj = rt.linear(x, self.w_in, "lat_proj")
        down = proj[:, self.down_at:self.down_at + self.down_cols]
        gate = proj[:, self.gate_at:] if (s.head_gate or s.out_gate) else None
        if s.q_rank > 0:
            # the queries' latent: unit RMS times a weight (float32 sums), then the up-projection
            cq = rt.ws.get("lat_q_latent", (T, s.q_rank), rt.act_dtype)
            ops.rmsnorm_rows(proj[:, :s.q_rank], self.w_q_norm, cq, s.eps)
            q = rt.linear(cq, self.w_q_up, "lat_q")
        else:
            q = proj[:, :self.q_cols]
        rope = self.position.table(step.max_positions) if self.position is not None else None
        q_rot = rt.ws.get("lat_q_rot", (T, H, s.rot_dim), rt.act_dtype)
        ops.latent_prepare(down, q, self.w_norm, rope, step.positions, step.seq_of_token, table, cache.storage, q_rot,
                           H, s.dim, s.rot_dim, R, s.position.dims if s.position is not None else 0, step.page_size, s.eps)
        q_lat = rt.ws.get("lat_q_lat", (H, T, R), rt.act_dtype)
        rt.batched_product(q.unflatten(1, (H, s.dim + s.rot_dim))[:, :, :s.dim].transpose(0, 1), self.w_uk_t, q_lat)
        o_lat = rt.ws.get("lat_o_lat", (H, T, R), rt.act_dtype)
        self.attend(q_lat, q_rot, cache, table, step, gate if s.head_gate else None, o_lat)
        o = rt.ws.get("lat_o", (T, H, s.vdim), rt.act_dtype)
        rt.batched_product(o_lat, self.w_uv, o.transpose(0, 1))
        if s.out_gate:
            ops.sigmoid_mul(o.view(T, H * s.vdim), gate[:, :H * s.vdim])
        if into is not None:
            return into.product(o.view(T, H * s.vdim), self.w_o)
        return rt.linear(o.view(T, H * s.vdim), self.w_o, "mixer_out")

    def fast_path(self, step) -> bool:
        """Whether this step's attention runs on tensor cores (bfloat16, sizes in 16-byte pieces, pages of 64)."""
        s = self.spec
        return (self.rt.mode == "bfloat16" and os.environ.get("XS_LATENT_ATTENTION", "mma") == "mma"
                and ops.latent_attention_mma_supports(s.kv_rank, s.rot_dim, step.page_size))

    def attend(self, q_lat, q_rot, cache, table, step, gate, o_lat) -> None:
        """q_lat, o_lat: [heads, tokens, kv_rank]."""
        s, rt = self.spec, self.rt
        if self.fast_path(step):
            # A CTA owns 64 (token, head) rows of a sequence. Few tiles facing many keys (single tokens, a short piece
            # of a long sequence): each sequence's key pages are cut over several CTAs so that every SM streams a part.
            rows = 16 if step.max_q_len * s.heads <= 32 else 64      # (single tokens: the kernel of 16-row tiles)
            tiles = -(-step.max_q_len * s.heads // rows) * step.n_seqs
            slots = rt.sm_count * ops.latent_attention_mma_ctas_per_sm(step.max_q_len, s.heads, s.kv_rank, s.rot_dim)
            blocks = -(-step.max_kv_len // step.page_size)
            if s.window > 0:
                blocks = min(blocks, -(-(s.window + step.max_q_len) // step.page_size) + 1)
            # (at least two pages a CTA: measured on B200, 8 sequences of 2,100 keys, 16 heads of 576: 9 to 33 parts 32 to 34 us,
            # 37 parts 40 us, 4 parts 54 us: past a page or two a CTA, more parts only add to what the combine reads)
            splits = max(1, min(-(-blocks // 2), 64, slots // max(tiles, 1)))
            scratch = None
            if splits > 1:
                need = ops.latent_attention_mma_scratch_bytes(q_rot.shape[0] * s.heads, s.kv_rank, splits)
                scratch = rt.ws.get("lat_scratch", (need,), torch.uint8)
            ops.latent_attention_mma(q_lat.transpose(0, 1), q_rot, cache.storage, table, step.cu_seqlens, step.kv_lens, gate,
                                     self.sink, o_lat.transpose(0, 1), scratch, step.n_seqs, step.max_q_len, step.page_size,
                                     s.scale, s.window, splits)
            return
        ops.latent_attention_generic(q_lat.transpose(0, 1), q_rot, cache.storage, table, step.seq_of_token, step.positions,
                                     gate, self.sink, o_lat.transpose(0, 1), step.page_size, s.scale, s.window)


registry.register_mixer(LatentAttentionMixer.kind, LatentAttentionMixer)
