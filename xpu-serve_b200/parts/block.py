"""The arrangement of one decoder layer, and the residual stream it acts on.

    x = norm(h, pre_mixer);  h = h + post_mixer(mixer(x))
    y = norm(h, pre_ffn);    h = h + post_ffn(ffn(y))

where the post norms are RMSNorms when the layer is a sandwich and the identity
otherwise (src/models/lfm3/lfm3_decoder.cpp:78-90). The stream is float32. Adding a
branch is deferred until the next norm reads the stream, so that one kernel adds the
branch (normed or not), writes the sum back and produces the next normed input.

Decode steps (few rows, bfloat16, no sandwich norms) go without that kernel: the product that
ends a branch adds its result to the stream in its epilogue and leaves, beside it, the stream
times the next norm's weight and per-tile sums of squares; the product that starts the next
branch reads those and scales its result by each row's 1 / rms (`Prenormed`, `StreamSink`;
the kernel side is csrc/gemm_small_m.cu). Parts opt in with `fuses_norm`; it applies to norms that
say `carried` (RMSNorm).

The norms are parts too (parts/norm.py, registry.register_norm): the stream only calls their
`add_norm`. The arrangement itself is registered (`registry.register_arrangement`): `Block` is
"pre_norm"; another wiring of the same parts (post-norm, mixer and feed-forward side by side) is
another class with the same five members: tensors(layer), cache_need(layer), __init__(layer,
weights, rt), forward(stream, step, cache, next_norm), first_norm.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import registry
from ..ops import lib as ops
from ..config.spec import NormSpec
from .base import Norm, StateNeed, TensorSpec


class Prenormed:
    """The stream times a norm's weight, in bfloat16, with the sums of squares from which the product
    that reads it forms each row's 1 / sqrt(mean square + eps). Only `rt.linear` and
    `rt.few_rows_product` know what to do with it."""

    def __init__(self, x: torch.Tensor, ssq: torch.Tensor, width: int, eps: float):
        self.x, self.ssq, self.width, self.eps = x, ssq, width, eps

    @property
    def shape(self):
        return self.x.shape


class StreamSink:
    """Where a part's last product goes when it fuses: into the stream, inside the product's kernel."""

    def __init__(self, stream: "ResidualStream", next_norm: Optional[Norm]):
        """`next_norm`: the norm that reads the stream next, if the products can carry it (an RMSNorm)."""
        self.stream = stream
        self.next_w = next_norm.w if next_norm is not None and next_norm.carried else None

    def product(self, act: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        st = self.stream
        rt = st.rt
        st.flush()
        if not rt.few_rows(act, w):
            st._pre = None
            st.add(rt.linear(act, w, "branch_out", bias))
            return
        M, N = st.h.shape
        if self.next_w is None:
            rt.few_rows_product(act, w, None, bias, residual=st.h)
            st._pre = None
            return
        st._flip ^= 1
        nx = rt.ws.get(f"prenormed{st._flip}", (M, N), torch.bfloat16)
        ssq = rt.ws.get(f"ssq{st._flip}", ((N + 15) // 16, 16), torch.float32)
        rt.few_rows_product(act, w, None, bias, residual=st.h, next_w=self.next_w, next_x=nx, out_ssq=ssq)
        st._pre = (self.next_w, nx, ssq)


class ResidualStream:
    def __init__(self, h: torch.Tensor, rt):
        self.h, self.rt = h, rt
        self._pending = None      # (branch, the norm it passes through before it joins the stream, or None)
        self._pre = None          # (norm weight, stream * weight, sums of squares) left by the last fused product
        self._flip = 0
        self._plain_add: Optional[Norm] = None
        self.history: Optional[torch.Tensor] = None     # [results kept + 2, tokens, width] float32 (`keep_history`)
        self.recorded = 0                               # planes of `history` that hold a finished result

    def keep_history(self, history: torch.Tensor) -> None:
        """From now on the stream keeps every layer's result. `history[0]` is the embedding's output, which the stream
        holds now; the stream moves to plane 1 (a copy), where the first layer turns it into its result."""
        self.flush()
        if history[0].data_ptr() != self.h.data_ptr():
            history[0].copy_(self.h)
        history[1].copy_(history[0])
        self.history, self.recorded, self.h = history, 1, history[1]
        self._pre = None

    def depth_average(self, coef: torch.Tensor, terms: int) -> None:
        """The layer that ends here has turned the stream into its result, plane `terms - 1` of the history. What the next
        layer (or the head) reads is sum_j coef[j] * history[j] over the `terms` results so far: it goes into the next
        plane, where the next layer works in place, so no result is ever copied."""
        if self.history is None:
            raise RuntimeError("a layer averages over earlier results, but the step keeps none (ModelSpec.depth_history)")
        if terms != self.recorded + 1 or terms + 1 > self.history.shape[0] or self.h.data_ptr() != self.history[terms - 1].data_ptr():
            raise RuntimeError(f"a layer averages over {terms} results where {self.recorded + 1} exist")
        self.flush()
        nxt = self.history[terms]
        ops.depth_average(self.history, coef, terms, nxt)
        self.h, self.recorded = nxt, terms
        self._pre = None

    def add(self, branch: torch.Tensor, post: Optional[Norm] = None) -> None:
        if self._pending is not None:
            self.flush()
        self._pending = (branch, post)

    def flush(self, norm: Optional[Norm] = None) -> None:
        """Joins the pending branch to the stream now. `norm`: any norm of the model (its `add_norm` does the
        sum); without one the last norm that read the stream is used."""
        if self._pending is not None:
            m, post = self._pending
            norm = norm or post or self._plain_add
            if norm is None:
                raise RuntimeError("a branch is pending but no norm has read the stream yet")
            norm.add_norm(self.h, m, post, None, None)
            self._pending = None
            self._pre = None

    def replace(self, h: torch.Tensor) -> None:
        """The stream becomes `h` (float32, same shape): what a step does that rewrites the stream between layers."""
        self.flush()
        if h.shape != self.h.shape or h.dtype != torch.float32:
            raise ValueError("the stream's replacement has another shape or type")
        self.h = h
        self._pre = None

    def fuses(self) -> bool:
        """Whether products of this step can add their result to the stream themselves and carry a norm across (few
        rows, bfloat16); which of them do is then asked part by part (`takes_prenormed`, `StreamSink.product`)."""
        rt = self.rt
        return (rt.mode == "bfloat16" and rt.fuse_norms and self.h.shape[0] <= max(rt.small_m, rt.narrow_m)
                and self.h.shape[1] % 8 == 0)

    def sink(self, next_norm: Optional[Norm]) -> StreamSink:
        return StreamSink(self, next_norm)

    def norm_input(self, norm: Norm, lazy: bool):
        """What a part reads: the normed stream, or (lazy, and the last fused product prepared for this very
        norm) the stream times the norm's weight with its row scale pending."""
        if (lazy and norm.carried and self._pending is None and self._pre is not None and self._pre[0] is norm.w):
            return Prenormed(self._pre[1], self._pre[2], self.h.shape[1], norm.eps)
        return self.norm(norm)

    def plain(self, norm: Norm) -> torch.Tensor:
        """The stream itself in the activation type, after any pending branch joined it: what a sublayer reads in a
        layer without norms before its sublayers. `norm`: any norm of the model (its `add_copy` does the work)."""
        self._flip ^= 1
        y = self.rt.ws.get(f"normed{self._flip}", tuple(self.h.shape), self.rt.act_dtype)
        m, post = self._pending if self._pending is not None else (None, None)
        norm.add_copy(self.h, m, post, y)
        self._pending = None
        self._pre = None
        self._plain_add = norm
        return y

    def norm(self, norm: Norm, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`norm` of the stream (after any pending branch joined it), in the activation type.
        With `rows`, only those rows, packed."""
        n = self.h.shape[0] if rows is None else rows.numel()
        self._flip ^= 1
        y = self.rt.ws.get(f"normed{self._flip}", (n, self.h.shape[1]), self.rt.act_dtype)
        m, post = self._pending if self._pending is not None else (None, None)
        norm.add_norm(self.h, m, post, y, rows)
        if self._pending is not None:
            self._pre = None
        self._pending = None
        self._plain_add = norm
        return y


SHARED = "//"      # a layer's weights hold the model's top-level tables that it reads under this prefix + their name


class TokenSide:
    """A per-layer input from the token itself, behind the layer's last sublayer (config/spec.py: TokenSideSpec). The stream
    (with the pending branch joined, in the activation type: one kernel) goes through the gate's product; one kernel turns
    the logits into gelu times the layer's slice of the second token table (csrc/layer_frame.cu: xs_side_gate); the
    projection follows, and its result joins the stream through an RMS norm of its own as a sandwich layer's branch does:
    in the kernel of the norm that reads the stream next. The table is put on the device once for all layers."""

    @classmethod
    def tensors(cls, spec, width: int) -> Dict[str, TensorSpec]:
        n = spec.names
        out = {n["gate"]: TensorSpec((spec.dim, width)), n["proj"]: TensorSpec((width, spec.dim))}
        out.update(registry.norm_class("rmsnorm").tensors(NormSpec(width, spec.eps), n["norm"]))
        return out

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt, width: int):
        self.spec, self.rt = spec, rt
        n = spec.names
        key = ("shared_table", spec.table)
        if key not in rt.shared:
            if SHARED + spec.table not in weights:
                raise KeyError(f"the layer reads the table '{spec.table}', which the model did not hand to it")
            rt.shared[key] = rt.matrix(weights[SHARED + spec.table])
        self.table = rt.shared[key]
        if not 0 <= spec.offset <= self.table.shape[1] - spec.dim:
            raise ValueError(f"token side: columns {spec.offset} + {spec.dim} of a table of {self.table.shape[1]}")
        self.w_gate = rt.matrix(weights[n["gate"]])
        self.w_proj = rt.matrix(weights[n["proj"]])
        # (an RMS norm with a plain weight, whatever the model's own norm is)
        self.norm = registry.norm_class("rmsnorm")(NormSpec(width, spec.eps), weights, n["norm"], rt)

    def forward(self, stream: "ResidualStream", step) -> None:
        rt = self.rt
        x = stream.plain(self.norm)
        g = rt.linear(x, self.w_gate, "side_gate")
        ops.side_gate(g, step.tokens, self.table, self.spec.offset)
        stream.add(rt.linear(g, self.w_proj, "side_out"), self.norm)


class Block:
    """The pre-norm arrangement (with optional sandwich norms, and optionally a token-side input behind the sublayers)."""
    kind = "pre_norm"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, layer) -> Dict[str, TensorSpec]:
        """Relative names (under the layer's prefix) of the layer's tensors: its norms', its mixer's, its
        feed-forward's."""
        out: Dict[str, TensorSpec] = {}
        norm_cls = registry.norm_class(layer.norm.kind)
        # (a layer without a feed-forward has no norms for one either; the order is the one random weights are drawn in)
        keys = ["pre_mixer"] + (["pre_ffn"] if layer.ffn is not None else [])
        if layer.sandwich:
            keys += ["post_mixer"] + (["post_ffn"] if layer.ffn is not None else [])
        for key in keys:
            out.update(norm_cls.tensors(layer.norm, layer.names[key]))
        out.update(registry.mixer_class(layer.mixer.kind).tensors(layer.mixer))
        if layer.ffn is not None:
            out.update(registry.ffn_class(layer.ffn.kind).tensors(layer.ffn))
        if getattr(layer, "token_side", None) is not None:
            out.update(TokenSide.tensors(layer.token_side, layer.norm.width))
        return out

    @classmethod
    def cache_need(cls, layer):
        return registry.mixer_class(layer.mixer.kind).cache_need(layer.mixer)

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        """`weights`: this layer's tensors by their names under the layer's prefix."""
        self.spec, self.rt = spec, rt
        self.mixer = registry.mixer_class(spec.mixer.kind)(spec.mixer, weights, rt)
        self.ffn = registry.ffn_class(spec.ffn.kind)(spec.ffn, weights, rt) if spec.ffn is not None else None
        n = spec.names
        norm_cls = registry.norm_class(spec.norm.kind)
        self.pre_mixer = norm_cls(spec.norm, weights, n["pre_mixer"], rt)
        self.pre_ffn = norm_cls(spec.norm, weights, n["pre_ffn"], rt) if self.ffn is not None else None
        self.post_mixer = norm_cls(spec.norm, weights, n["post_mixer"], rt) if spec.sandwich else None
        self.post_ffn = norm_cls(spec.norm, weights, n["post_ffn"], rt) if spec.sandwich and self.ffn is not None else None
        self.first_norm = self.pre_mixer      # the norm that reads the stream first: what the block before may prepare
        self.side = TokenSide(spec.token_side, weights, rt, spec.norm.width) if getattr(spec, "token_side", None) is not None else None
        if self.side is not None and spec.sandwich:
            raise ValueError("pre_norm: a token-side input behind sandwich norms is not supported")

    def forward(self, stream: ResidualStream, step, cache, next_norm: Optional[Norm] = None) -> None:
        """`next_norm`: the norm that reads the stream after this block (the next block's first, or the
        final norm), for the fused path; None is always right."""
        if self.side is not None:
            next_norm = None                  # the stream changes once more behind the last product: nothing to prepare
        self._sublayers(stream, step, cache, next_norm)
        if self.side is not None:
            self.side.forward(stream, step)

    def _sublayers(self, stream: ResidualStream, step, cache, next_norm: Optional[Norm]) -> None:
        fuse = stream.fuses() and not self.spec.sandwich and self.pre_mixer.carried
        rows = stream.h.shape[0]
        # (a part whose first product runs elsewhere at this number of rows gets the normed tensor, and the product
        # before it does not prepare the norm's input for it; its last product may still add to the stream itself)
        ffn_lazy = fuse and self.ffn is not None and self.ffn.fuses_norm and self.ffn.takes_prenormed(rows)
        if fuse and self.mixer.fuses_norm:
            x = stream.norm_input(self.pre_mixer, lazy=self.mixer.takes_prenormed(rows))
            after = (self.pre_ffn if ffn_lazy else None) if self.ffn is not None else next_norm
            self.mixer.forward(x, step, cache, into=stream.sink(after))
        else:
            x = stream.norm(self.pre_mixer)
            stream.add(self.mixer.forward(x, step, cache), self.post_mixer)
        if self.ffn is None:
            return
        if fuse and self.ffn.fuses_norm:
            y = stream.norm_input(self.pre_ffn, lazy=ffn_lazy)
            self.ffn.forward(y, step, into=stream.sink(next_norm))
        else:
            y = stream.norm(self.pre_ffn)
            stream.add(self.ffn.forward(y, step), self.post_ffn)


class BranchNormBlock:
    """h += norm1(mixer(h)); h += norm2(ffn(h)): the sublayers read the stream itself (in the activation type), and
    the layer's two norms act on what they return. The sum with the normed branch and the copy that the next sublayer
    reads are one kernel (`ResidualStream.plain`)."""
    kind = "branch_norm"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, layer) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        norm_cls = registry.norm_class(layer.norm.kind)
        for key in ["post_mixer"] + (["post_ffn"] if layer.ffn is not None else []):
            out.update(norm_cls.tensors(layer.norm, layer.names[key]))
        out.update(registry.mixer_class(layer.mixer.kind).tensors(layer.mixer))
        if layer.ffn is not None:
            out.update(registry.ffn_class(layer.ffn.kind).tensors(layer.ffn))
        return out

    @classmethod
    def cache_need(cls, layer):
        return registry.mixer_class(layer.mixer.kind).cache_need(layer.mixer)

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        self.spec, self.rt = spec, rt
        self.mixer = registry.mixer_class(spec.mixer.kind)(spec.mixer, weights, rt)
        self.ffn = registry.ffn_class(spec.ffn.kind)(spec.ffn, weights, rt) if spec.ffn is not None else None
        norm_cls = registry.norm_class(spec.norm.kind)
        self.post_mixer = norm_cls(spec.norm, weights, spec.names["post_mixer"], rt)
        self.post_ffn = norm_cls(spec.norm, weights, spec.names["post_ffn"], rt) if self.ffn is not None else None
        self.first_norm = None                # no norm reads the stream for this block: nothing to prepare for it

    def forward(self, stream: ResidualStream, step, cache, next_norm: Optional[Norm] = None) -> None:
        x = stream.plain(self.post_mixer)
        stream.add(self.mixer.forward(x, step, cache), self.post_mixer)
        if self.ffn is not None:
            y = stream.plain(self.post_ffn)
            stream.add(self.ffn.forward(y, step), self.post_ffn)


def _needs_of(need) -> tuple:
    return () if need is None else tuple(need) if isinstance(need, (tuple, list)) else (need,)


class GatedPreNormBlock:
    """The pre-norm layer with three options, each a field of the layer's spec:

        a = norm1(h);  h += G1(a) * mixer(F1(a))        F(a) = a + filter(a)   (`input_taps`; identity without)
        f = norm2(h);  h += G2(f) * ffn(F2(f))          G(a) = sigmoid(a G^T + b)   (`branch_gate`; 1 without)
        h <- sum_j c[j] X_j                             (`depth_terms`: X_0 the embedding's output, X_j layer j - 1's h)

    The filter is causal and per channel over a sequence's earlier tokens; its last taps - 1 inputs are part of the
    sequence's state (one need per sublayer, behind the mixer's own). Gate logits and the sum with the gated branch are
    float32."""
    kind = "gated_pre_norm"
    fixed_shape_ok = True

    @classmethod
    def tensors(cls, layer) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        n, W = layer.names, layer.norm.width
        norm_cls = registry.norm_class(layer.norm.kind)
        subs = ["mixer"] + (["ffn"] if layer.ffn is not None else [])
        for sub in subs:
            out.update(norm_cls.tensors(layer.norm, n[f"pre_{sub}"]))
        out.update(registry.mixer_class(layer.mixer.kind).tensors(layer.mixer))
        if layer.ffn is not None:
            out.update(registry.ffn_class(layer.ffn.kind).tensors(layer.ffn))
        for sub in subs:
            if layer.input_taps > 0:
                out[n[f"{sub}_taps"]] = TensorSpec((W, layer.input_taps), init="uniform:-0.3:0.3", role="vector")
            if layer.branch_gate:
                out[n[f"{sub}_gate"]] = TensorSpec((W, W))
                out[n[f"{sub}_gate_bias"]] = TensorSpec((W,), init="uniform:-1:1", role="vector")
        if layer.depth_terms > 0:
            out[n["depth"]] = TensorSpec((layer.depth_terms,), init="uniform:0.1:0.6", role="vector")
        return out

    @classmethod
    def cache_need(cls, layer):
        needs = _needs_of(registry.mixer_class(layer.mixer.kind).cache_need(layer.mixer))
        if layer.input_taps > 1:
            rows = StateNeed((layer.input_taps - 1, layer.norm.width), "compute")
            needs = needs + (rows,) * (2 if layer.ffn is not None else 1)
        return needs if needs else None

    def __init__(self, spec, weights: Dict[str, torch.Tensor], rt):
        if spec.sandwich:
            raise ValueError("gated_pre_norm: a layer with sandwich norms is the plain pre_norm arrangement's")
        if not 0 <= spec.input_taps <= 16:
            raise ValueError(f"gated_pre_norm: {spec.input_taps} taps (at most 16 are supported)")
        self.spec, self.rt = spec, rt
        self.mixer = registry.mixer_class(spec.mixer.kind)(spec.mixer, weights, rt)
        self.ffn = registry.ffn_class(spec.ffn.kind)(spec.ffn, weights, rt) if spec.ffn is not None else None
        n = spec.names
        norm_cls = registry.norm_class(spec.norm.kind)
        self.pre_mixer = norm_cls(spec.norm, weights, n["pre_mixer"], rt)
        self.pre_ffn = norm_cls(spec.norm, weights, n["pre_ffn"], rt) if self.ffn is not None else None
        self.first_norm = None                # (the stream is rewritten between layers: nothing is prepared across them)
        self.mixer_needs = len(_needs_of(registry.mixer_class(spec.mixer.kind).cache_need(spec.mixer)))
        self.taps, self.gates = {}, {}
        for sub in ["mixer"] + (["ffn"] if self.ffn is not None else []):
            if spec.input_taps > 0:
                self.taps[sub] = rt.vector(weights[n[f"{sub}_taps"]].reshape(spec.norm.width, spec.input_taps))
            if spec.branch_gate:
                self.gates[sub] = (rt.matrix(weights[n[f"{sub}_gate"]]), rt.vector(weights[n[f"{sub}_gate_bias"]]))
        self.depth = rt.vector(weights[n["depth"]]) if spec.depth_terms > 0 else None

    def _sublayer(self, sub: str, stream: ResidualStream, norm: Norm, step, cache, rows_view, run) -> None:
        rt = self.rt
        a = stream.norm(norm)
        logits = None
        if sub in self.gates:
            logits = rt.linear(a, self.gates[sub][0], "branch_gate", out_dtype=torch.float32)
        x = a
        if sub in self.taps:
            x = rt.ws.get("filtered_input", tuple(a.shape), a.dtype)
            state = rows_view.storage if rows_view is not None else a      # (one tap keeps nothing)
            ops.causal_conv(a, self.taps[sub], state, step.seq_of_token, step.cu_seqlens, step.slots, x, residual=True, all_single=step.decode)
        branch = run(x)
        if logits is None:
            stream.add(branch)
        else:
            ops.gated_add(stream.h, branch, logits, self.gates[sub][1])

    def forward(self, stream: ResidualStream, step, cache, next_norm: Optional[Norm] = None) -> None:
        k = self.mixer_needs
        keeps_rows = self.spec.input_taps > 1
        if keeps_rows and (cache is None or len(cache) < k + (2 if self.ffn is not None else 1)):
            raise RuntimeError("gated_pre_norm: the layer keeps its filters' last inputs per sequence")
        mixer_cache = cache.sub(0, k) if cache is not None else None
        self._sublayer("mixer", stream, self.pre_mixer, step, cache, cache[k] if keeps_rows else None,
                       lambda x: self.mixer.forward(x, step, mixer_cache))
        if self.ffn is not None:
            self._sublayer("ffn", stream, self.pre_ffn, step, cache, cache[k + 1] if keeps_rows else None,
                           lambda y: self.ffn.forward(y, step))
        if self.depth is not None:
            stream.depth_average(self.depth, self.spec.depth_terms)


registry.register_arrangement(Block.kind, Block)
registry.register_arrangement(GatedPreNormBlock.kind, GatedPreNormBlock)
registry.register_arrangement(BranchNormBlock.kind, BranchNormBlock)
