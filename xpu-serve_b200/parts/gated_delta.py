"""The gated delta-rule mixer: per head a memory S [dim, vdim], float32 and zero at a sequence's start. For a token with
input x (F: a causal per-channel filter over the sequence's earlier tokens, then silu):

    q = F(Wq x), k = F(Wk x)  (key heads of `dim`, each shared by heads / key heads heads);   v = F(Wv x)  (heads of `vdim`)
    qn = q / sqrt(|q|^2 + 1e-6) / sqrt(dim),   kn = k / sqrt(|k|^2 + 1e-6)
    g = exp(-exp(A_log) softplus(Wa x + dt_bias)),   beta = sigmoid(Wb x)                one of each per head
    S <- g S;   u = beta (v - S^T kn);   S <- S + kn u^T;   o = S^T qn                   (the read sees the token's own write)

then every head's o divided by its root mean square, times a weight of vdim entries that the heads share, times
silu(Wg x), and the output projection. One product gives q, k, v and the output gate's logits in the activation type; Wa x
and Wb x come from a second product whose output is float32, and everything behind them (softplus, the exponentials, beta,
the unit norms, the memory and its sums, the heads' norm) is float32 in both precision modes (csrc/gated_delta.cu). A
sequence keeps the filters' last taps - 1 inputs (activation type) and S.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import Mixer, StateNeed, TensorSpec


class GatedDeltaMixer(Mixer):
    kind = "gated_delta"
    fixed_shape_ok = True      # the kernels find every sequence's tokens in the step's description on the device

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        kd, vd = spec.kv_heads * spec.dim, spec.heads * spec.vdim
        taps = "uniform:-0.5:0.5"
        return {
            n["q"]: TensorSpec((kd, spec.hidden)), n["q_conv"]: TensorSpec((kd, spec.taps), init=taps, role="vector"),
            n["k"]: TensorSpec((kd, spec.hidden)), n["k_conv"]: TensorSpec((kd, spec.taps), init=taps, role="vector"),
            n["v"]: TensorSpec((vd, spec.hidden)), n["v_conv"]: TensorSpec((vd, spec.taps), init=taps, role="vector"),
            n["b"]: TensorSpec((spec.heads, spec.hidden)),
            n["a_log"]: TensorSpec((spec.heads,), init="uniform:-1:1.5", role="vector"),
            n["norm"]: TensorSpec((spec.vdim,), init="ones", role="vector"),
            n["a"]: TensorSpec((spec.heads, spec.hidden)),
            n["dt_bias"]: TensorSpec((spec.heads,), init="uniform:-3:0", role="vector"),
            n["gate"]: TensorSpec((vd, spec.hidden)),
            n["o"]: TensorSpec((spec.hidden, vd)),
        }

    @classmethod
    def cache_need(cls, spec):
        channels = 2 * spec.kv_heads * spec.dim + spec.heads * spec.vdim
        return (StateNeed((max(spec.taps - 1, 1), channels), "compute"),
                StateNeed((spec.heads, spec.dim, spec.vdim), "float32"))

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if spec.dim > 256:
            raise ValueError(f"gated delta: key size {spec.dim} (at most 256 is supported)")
        if spec.heads % spec.kv_heads != 0:
            raise ValueError(f"gated delta: {spec.heads} heads over {spec.kv_heads} key heads")
        if not 1 <= spec.taps <= 16:
            raise ValueError(f"gated delta: {spec.taps} taps (1 to 16 are supported)")
        self.spec, self.rt = spec, rt
        n = spec.names
        f32 = torch.float32
        self.kd, self.vd = spec.kv_heads * spec.dim, spec.heads * spec.vdim
        self.channels = 2 * self.kd + self.vd
        # [q; k; v; output gate] as one product; [a; b] (padded to whole 16-row tiles) as another with float32 output
        self.w_in = rt.matrix(torch.cat([weights[n[k]].to(f32) for k in ("q", "k", "v", "gate")], 0))
        ab = torch.cat([weights[n["a"]].to(f32), weights[n["b"]].to(f32)], 0)
        pad = (-ab.shape[0]) % 16
        if pad:
            ab = torch.cat([ab, torch.zeros(pad, ab.shape[1])], 0)
        self.w_ab = rt.matrix(ab)
        self.taps = rt.vector(torch.cat([weights[n[k]].to(f32).reshape(-1, spec.taps) for k in ("q_conv", "k_conv", "v_conv")], 0))
        self.a_log = rt.vector(weights[n["a_log"]])
        self.dt_bias = rt.vector(weights[n["dt_bias"]])
        self.w_norm = rt.vector(weights[n["norm"]].to(f32).reshape(1, spec.vdim).repeat(spec.heads, 1).reshape(-1))
        self.w_o = rt.matrix(weights[n["o"]])

    def forward(self, x, step, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if cache is None or len(cache) != 2 or not cache.owner:
            raise RuntimeError("the gated delta mixer keeps its own filter inputs and memory")
        T, C = x.shape[0], self.channels
        proj = rt.linear(x, self.w_in, "gd_proj")
        ab = rt.linear(x, self.w_ab, "gd_gates", out_dtype=torch.float32)
        qkv = rt.ws.get("gd_qkv", (T, C), rt.act_dtype)
        ops.causal_conv(proj, self.taps, cache[0].storage, step.seq_of_token, step.cu_seqlens, step.slots, qkv, act="silu", all_single=step.decode)
        y = rt.ws.get("gd_y", (T, self.vd), torch.float32)
        ops.gated_delta_scan(qkv, 0, self.kd, 2 * self.kd, ab, self.a_log, self.dt_bias, cache[1].storage, step.cu_seqlens,
                             step.slots, y, s.heads, s.kv_heads, s.dim, s.vdim, float(s.dim) ** -0.5, s.unit_eps)
        yn = rt.ws.get("gd_normed", (T, self.vd), rt.act_dtype)
        ops.grouped_rmsnorm(y, self.w_norm, yn, s.heads, s.eps, gate=proj[:, C:], gate_act="silu")
        return rt.linear(yn, self.w_o, "mixer_out")


registry.register_mixer(GatedDeltaMixer.kind, GatedDeltaMixer)
