"""More feed-forwards: a clamped gated unit, a squared-ReLU unit, and routed experts.

ClampedGLU:     down(g * sigmoid(alpha g) * (u + up_shift)), g = min(gate x, limit), u = clamp(up x, -limit, limit).
SquaredRelu:    down(max(up x, 0)^2).
RoutedExperts:  `experts` gated feed-forwards without biases (SwiGLU, or clamped units when the spec gives a limit); a
                token's router logits (float32) choose the `top` largest, whose softmax over themselves, times the
                spec's `route_scale`, weights the chosen experts' outputs. On the device the step's
                (token, choice) rows are sorted by expert and the two products walk row tiles of one expert each
                (csrc/experts.cu); no count ever reaches the host, so a step with experts can be captured in a graph.
                With `shared`, a clamped unit that every token uses joins the sum, times the sigmoid of one more
                logit a token (its one-row matrix is the router's last row here, so the router product gives both).
                `score` "sigmoid": scores sigmoid(logit); chosen by score plus a correction per expert among the best
                groups of neighbouring experts, weighted by the scores as they are (config/spec.py: RoutedExpertsSpec).
                `activation` "relu_squared": an expert is down(max(up x, 0)^2).
                `score` "softmax_all": scores softmax over all router outputs, chosen by score plus a correction, weighted
                by the scores as they are; with `identity` the router's last outputs stand for the token's input itself
                (such a choice takes no place in the plan; the combine kernel adds weight times input).
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .. import registry
from ..ops import lib as ops
from .base import FeedForward, TensorSpec


class ClampedGLU(FeedForward):
    kind = "clamped_glu"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        return {n["gate"]: TensorSpec((spec.intermediate, spec.hidden)),
                n["up"]: TensorSpec((spec.intermediate, spec.hidden)),
                n["down"]: TensorSpec((spec.hidden, spec.intermediate))}

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        self.spec, self.rt = spec, rt
        n = spec.names
        gate, up = weights[n["gate"]].to(torch.float32), weights[n["up"]].to(torch.float32)
        F, H = spec.intermediate, spec.hidden
        # bfloat16 and widths in blocks of 8: gate and up rows stacked in blocks of 8 and 8, as SwiGLU stacks them, so that
        # the tcgen05 product of long prompts applies the activation in its epilogue
        self.interleave = 8 if (rt.mode == "bfloat16" and F % 8 == 0) else 0
        if self.interleave:
            stacked = torch.stack([gate.view(F // 8, 8, H), up.view(F // 8, 8, H)], 1).reshape(2 * F, H)
        else:
            stacked = torch.cat([gate, up], 0)
        self.w_gate_up = rt.matrix(stacked)
        self.w_down = rt.matrix(weights[n["down"]])

    def forward(self, y, step, name: str = "ffn_out") -> torch.Tensor:
        """`name`: the scratch buffer that takes the result (a unit inside another feed-forward names its own)."""
        rt, s = self.rt, self.spec
        act = rt.ws.get("ffn_act", (y.shape[0], s.intermediate), rt.act_dtype)
        if self.interleave and rt.tensor_core_product(y, self.w_gate_up, fused=True):
            ops.gemm_tc_clamped(y, self.w_gate_up, act, s.limit, s.alpha, s.up_shift)
        else:
            gu = rt.linear(y, self.w_gate_up, "ffn_gate_up")
            ops.clamped_glu(gu, act, s.limit, s.alpha, s.up_shift, self.interleave)
        return rt.linear(act, self.w_down, name)


class SquaredRelu(FeedForward):
    kind = "squared_relu"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        return {n["up"]: TensorSpec((spec.intermediate, spec.hidden)), n["down"]: TensorSpec((spec.hidden, spec.intermediate))}

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        self.spec, self.rt = spec, rt
        self.w_up = rt.matrix(weights[spec.names["up"]])
        self.w_down = rt.matrix(weights[spec.names["down"]])

    def forward(self, y, step) -> torch.Tensor:
        rt = self.rt
        act = rt.ws.get("ffn_act", (y.shape[0], self.spec.intermediate), rt.act_dtype)
        if rt.few_rows(y, self.w_up):
            # few rows: the activation in the weight-streaming product's epilogue
            rt.few_rows_product(y, self.w_up, act, swiglu="relu_squared")
        elif rt.tensor_core_product(y, self.w_up, fused=True):
            # long prompts: the activation in the tcgen05 product's epilogue (no pass of its own over the wide rows)
            ops.gemm_tc(y, self.w_up, act, epilogue=ops.EPI_RELU_SQ)
        else:
            up = rt.linear(y, self.w_up, "ffn_up")
            ops.relu_squared(up, act)
        return rt.linear(act, self.w_down, "ffn_out")


class RoutedExperts(FeedForward):
    kind = "routed_experts"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, spec) -> Dict[str, TensorSpec]:
        n = spec.names
        out = {}
        for e in range(spec.experts):
            if spec.activation == "gated":
                out[n["gate"].format(e=e)] = TensorSpec((spec.intermediate, spec.hidden))
            out[n["up"].format(e=e)] = TensorSpec((spec.intermediate, spec.hidden))
            out[n["down"].format(e=e)] = TensorSpec((spec.hidden, spec.intermediate))
        outputs = spec.experts + int(getattr(spec, "identity", 0))
        out[n["router"]] = TensorSpec((outputs, spec.hidden))
        if spec.correction:
            out[n["correction"]] = TensorSpec((outputs,), init="uniform:-0.3:0.3", role="vector")
        if spec.shared is not None:
            out.update(registry.ffn_class(spec.shared.kind).tensors(spec.shared))
            out[n["shared_gate"]] = TensorSpec((1, spec.hidden))
        return out

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if spec.top > 16:
            raise ValueError(f"routed experts: top {spec.top} (at most 16 are supported)")
        if spec.score not in ("softmax", "sigmoid", "softmax_all") or spec.activation not in ("gated", "relu_squared"):
            raise ValueError(f"routed experts: score '{spec.score}' (softmax, sigmoid, softmax_all), activation '{spec.activation}' (gated, relu_squared)")
        self.identity = int(getattr(spec, "identity", 0))
        if self.identity < 0 or (self.identity > 0 and spec.score != "softmax_all"):
            raise ValueError("routed experts: identity outputs belong to softmax_all scores")
        if spec.score == "softmax" and (spec.correction or spec.groups != 1):
            raise ValueError("routed experts: a correction and groups belong to sigmoid scores")
        if spec.groups < 1 or spec.experts % spec.groups != 0 or not 1 <= spec.keep_groups <= spec.groups \
                or spec.keep_groups * (spec.experts // spec.groups) + self.identity < spec.top:
            raise ValueError(f"routed experts: {spec.experts} experts in {spec.groups} groups of which {spec.keep_groups} stay open "
                             f"cannot give {spec.top} choices")
        self.spec, self.rt = spec, rt
        self.gated = spec.activation == "gated"
        n = spec.names
        # [experts, 2 F, hidden] and [experts, hidden, F]. An expert's gate rows stand before its up rows; where the
        # tcgen05 product runs (bfloat16, widths that are multiples of 8) they stand in blocks of 8 gate rows and the 8
        # up rows of the same outputs, so that the product's epilogue can apply the activation.
        F, H = spec.intermediate, spec.hidden
        self.tensor_cores = (rt.mode == "bfloat16" and F % 8 == 0 and H % 8 == 0
                             and os.environ.get("XS_EXPERTS_GEMM", "tcgen05") == "tcgen05")

        def stacked(e):
            if not self.gated:
                return weights[n["up"].format(e=e)].to(torch.float32)
            g, u = weights[n["gate"].format(e=e)].to(torch.float32), weights[n["up"].format(e=e)].to(torch.float32)
            if self.tensor_cores:
                return torch.stack([g.view(F // 8, 8, H), u.view(F // 8, 8, H)], 1).reshape(2 * F, H)
            return torch.cat([g, u], 0)

        self.w_gate_up = rt.matrix(torch.stack([stacked(e) for e in range(spec.experts)]))
        self.w_down = rt.matrix(torch.stack([weights[n["down"].format(e=e)].to(torch.float32) for e in range(spec.experts)]))
        router = weights[n["router"]].to(torch.float32)
        self.shared = None
        if spec.shared is not None:
            # the shared unit's gate logit is one more row of the router product (its float32 sums serve both)
            router = torch.cat([router, weights[n["shared_gate"]].to(torch.float32).reshape(1, H)], 0)
            self.shared = registry.ffn_class(spec.shared.kind)(spec.shared, weights, rt)
        self.w_router = rt.matrix(router)
        self.correction = rt.vector(weights[n["correction"]]) if spec.correction else None
        self.clamp = (spec.limit, spec.alpha, spec.up_shift) if spec.limit > 0 else None

    def forward(self, y, step) -> torch.Tensor:
        rt, s = self.rt, self.spec
        T, n = y.shape[0], y.shape[0] * s.top
        ws = rt.ws
        shared = self.shared.forward(y, step, name="moe_shared") if self.shared is not None else None
        logits = ws.get("moe_logits", (T, self.w_router.shape[0]), torch.float32)
        ops.moe_logits(y, self.w_router, logits)            # float32 sums of the activation type's products, not rounded
        outputs = s.experts + self.identity
        shared_gate = logits[:, outputs:] if shared is not None else None
        ids = ws.get("moe_ids", (n,), torch.int32)
        wts = ws.get("moe_wts", (n,), torch.float32)
        place = ws.get("moe_place", (n,), torch.int32)
        source = ws.get("moe_source", (n,), torch.int32)
        meta = ws.get("moe_meta", (4 + 3 * ops.moe_max_tiles(n, s.experts),), torch.int32)
        if s.score == "softmax_all":
            ops.moe_route_grouped(logits, s.top, ids, wts, experts=outputs, correction=self.correction, scale=s.route_scale,
                                  score="softmax", real=s.experts)
        elif s.score == "sigmoid":
            ops.moe_route_grouped(logits, s.top, ids, wts, experts=s.experts, correction=self.correction, groups=s.groups,
                                  keep=s.keep_groups, group_top=s.group_top, scale=s.route_scale, renorm=s.renorm)
        else:
            ops.moe_route(logits, s.top, ids, wts, experts=s.experts, scale=s.route_scale)
        out = ws.get("ffn_out", (T, s.hidden), rt.act_dtype)
        passed = {"passed": y} if self.identity else {}       # (choices that stand for the token's input itself)
        if self.tensor_cores:
            # every expert's rows padded to tiles of 128: gather, two tcgen05 products over the plan's tiles, combine
            tiles = ops.moe_max_tiles_of(n, s.experts, 128)
            source = ws.get("moe_source_padded", (128 * tiles,), torch.int32)
            meta = ws.get("moe_meta_padded", (4 + 3 * tiles,), torch.int32)
            ops.moe_plan(ids, s.experts, place, source, meta, tile_rows=128)
            rows_in = ws.get("moe_rows_in", (128 * tiles, s.hidden), rt.act_dtype)
            ops.moe_gather(y, source, s.top, rows_in)
            act = ws.get("moe_act", (128 * tiles, s.intermediate), rt.act_dtype)
            ops.gemm_tc_grouped(rows_in, self.w_gate_up, act, meta, tiles, glu=self.gated, clamp=self.clamp,
                                relu_squared=not self.gated)
            rows_out = ws.get("moe_rows", (128 * tiles, s.hidden), rt.act_dtype)
            ops.gemm_tc_grouped(act, self.w_down, rows_out, meta, tiles, glu=False)
            ops.moe_combine(rows_out, place, wts, out, s.top, shared, shared_gate, **passed)
            return out
        ops.moe_plan(ids, s.experts, place, source, meta)
        act = ws.get("moe_act", (n, s.intermediate), rt.act_dtype)
        ops.moe_gemm(y, self.w_gate_up, act, meta, n, source, s.top, glu=self.gated, clamp=self.clamp)
        if not self.gated:
            ops.relu_squared(act, act)
        rows_out = ws.get("moe_rows", (n, s.hidden), rt.act_dtype)
        ops.moe_gemm(act, self.w_down, rows_out, meta, n, None, s.top, glu=False)
        ops.moe_combine(rows_out, place, wts, out, s.top, shared, shared_gate, **passed)
        return out


registry.register_ffn(ClampedGLU.kind, ClampedGLU)
registry.register_ffn(SquaredRelu.kind, SquaredRelu)
registry.register_ffn(RoutedExperts.kind, RoutedExperts)
