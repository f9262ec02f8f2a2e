"""A plain, slow Tozarax in float64 numpy: whole sequences, no cache, one function per mechanism.

It shares no code with the package: it reads config.json's keys itself and takes tensors by their
checkpoint names. Notation: T tokens, W the model's width, rows x of a [T, n] array are tokens.
Weights are [out, in] and applied as y = x M^T.

The stream starts as table row plus a learned row per position. Layer i reads the stream s:

    a = unit_rms(s) (1 + n1);   s = s + sigmoid(a R1^T + b1) * mixer(a + conv(a; c1))
    f = unit_rms(s) (1 + n2);   s = s + sigmoid(f R2^T + b2) * ff(f + conv(f; c2))

conv being a causal per-channel filter over earlier tokens, and what the next layer (or the head) reads
is a weighted sum of the embedding output and every layer's s so far. The mixer is half the sum of two
branches that read the same input, each branch unit-RMS normed times a weight: softmax attention over a
sliding window without position encoding, and a gated delta-rule memory. The feed-forward chooses a few
of many squared-ReLU units per token by sigmoid scores, a per-unit correction and a limit on groups.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


# ------------------------------------------------------------------------------ embedding
def embedding(w: Dict[str, np.ndarray], tokens: Sequence[int], first_position: int = 0) -> np.ndarray:
    toks = np.asarray(tokens, dtype=np.int64)
    return w["embed"][toks] + w["pos"][first_position + np.arange(len(toks))]


# ------------------------------------------------------------------- the layer's own pieces
def causal_filter(x: np.ndarray, taps: np.ndarray) -> np.ndarray:
    """y[t, c] = sum_j taps[c, j] x[t - (n - 1) + j, c], n = taps.shape[1]; rows before the first count as zero."""
    n = taps.shape[1]
    y = np.zeros_like(x)
    for j in range(n):
        back = n - 1 - j
        if back == 0:
            y += x * taps[:, j]
        elif back < x.shape[0]:
            y[back:] += x[:-back] * taps[:, j]
    return y


def sublayer_input(x: np.ndarray, taps: np.ndarray) -> np.ndarray:
    return x + causal_filter(x, taps)


def output_gate(x: np.ndarray, m: np.ndarray, b: np.ndarray) -> np.ndarray:
    return sigmoid(x @ m.T + b)


def depth_average(history: List[np.ndarray], weights: np.ndarray) -> np.ndarray:
    assert len(history) == len(weights)
    return sum(c * h for c, h in zip(weights, history))


# ------------------------------------------------------------------------------ attention
def window_attention(m: dict, w: Dict[str, np.ndarray], p: str, x: np.ndarray) -> np.ndarray:
    """Grouped-query softmax attention in which query i sees keys i - size + 1 .. i. Returns [T, W]."""
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    size, scale = int(m["mask"]["size"]), float(m["scale"])
    T = x.shape[0]
    q = (x @ w[p + "q"].T).reshape(T, H, D)
    k = (x @ w[p + "k"].T).reshape(T, G, D)
    v = (x @ w[p + "v"].T).reshape(T, G, Dv)
    i = np.arange(T)
    seen = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] < size)
    out = np.zeros((T, H, Dv))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = np.where(seen, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        e = np.exp(s)
        out[:, h] = (e / e.sum(-1, keepdims=True)) @ v[:, g]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


# ---------------------------------------------------------------------- gated delta rule
def delta_memory(q: np.ndarray, k: np.ndarray, v: np.ndarray, decay: np.ndarray, beta: np.ndarray,
                 state: Optional[np.ndarray] = None):
    """One head. q, k [T, D]; v [T, Dv]; decay, beta [T]. Per token: S *= decay; u = beta (v - S^T k); S += k u^T;
    o = S^T q. Returns (o [T, Dv], S [D, Dv])."""
    T, D = q.shape
    S = np.zeros((D, v.shape[1])) if state is None else state.copy()
    o = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = S * decay[t]
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o, S


def gated_delta(m: dict, w: Dict[str, np.ndarray], p: str, x: np.ndarray, eps: float) -> np.ndarray:
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = x.shape[0]

    def filtered(name):
        return silu(causal_filter(x @ w[p + name].T, w[p + name + ".conv"]))

    q = filtered("q").reshape(T, G, D)
    k = filtered("k").reshape(T, G, D)
    v = filtered("v").reshape(T, H, Dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(x @ w[p + "b"].T)                                           # [T, H]
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(x @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(x @ w[p + "g"].T).reshape(T, H, Dv)
    o = np.zeros((T, H, Dv))
    for h in range(H):
        g = h // (H // G)
        o[:, h], _ = delta_memory(q[:, g], k[:, g], v[:, h], decay[:, h], beta[:, h])
    o = unit_rms(o, eps) * w[p + "norm"] * gate
    return o.reshape(T, H * Dv) @ w[p + "o"].T


def parallel_mixer(cfg: dict, m: dict, w: Dict[str, np.ndarray], p: str, x: np.ndarray) -> np.ndarray:
    eps = float(cfg["norm"]["eps"])
    left = window_attention(m["left"], w, p + "left.", x)
    right = gated_delta(m["right"], w, p + "right.", x, eps)
    return 0.5 * (unit_rms(left, eps) * w[p + "left.out"] + unit_rms(right, eps) * w[p + "right.out"])


# ------------------------------------------------------------------------ routed experts
def route(z: np.ndarray, correction: np.ndarray, top: int, groups: int, keep: int):
    """z [T, E] router logits. Returns (ids [T, top], weights [T, top]): the units with the largest sigmoid(z) +
    correction among the `keep` groups (of E / groups neighbours) whose two largest such scores sum highest; the
    weights are sigmoid(z) of the chosen, as they are. Ties go to the lower index."""
    T, E = z.shape
    s = sigmoid(z)
    c = s + correction
    per = E // groups
    ids = np.zeros((T, top), dtype=np.int64)
    for t in range(T):
        gs = []
        for g in range(groups):
            part = np.sort(c[t, g * per:(g + 1) * per])[::-1]
            gs.append(part[:2].sum())
        order = sorted(range(groups), key=lambda g: (-gs[g], g))[:keep]
        open_ = np.full(E, -np.inf)
        for g in order:
            open_[g * per:(g + 1) * per] = c[t, g * per:(g + 1) * per]
        ids[t] = sorted(range(E), key=lambda e: (-open_[e], e))[:top]
    return ids, np.take_along_axis(s, ids, 1)


def route_margin(z: np.ndarray, correction: np.ndarray, top: int, groups: int, keep: int) -> np.ndarray:
    """[T]: by how much each token's choice is decided: the smaller of the gap between the last kept and the first dropped
    group's score and the gap between the last chosen and the first unchosen open unit's choice score."""
    T, E = z.shape
    c = sigmoid(z) + correction
    per = E // groups
    out = np.full(T, np.inf)
    for t in range(T):
        gs = np.array([np.sort(c[t, g * per:(g + 1) * per])[::-1][:2].sum() for g in range(groups)])
        order = sorted(range(groups), key=lambda g: (-gs[g], g))
        if keep < groups:
            out[t] = gs[order[keep - 1]] - gs[order[keep]]
        open_ = np.sort(np.concatenate([c[t, g * per:(g + 1) * per] for g in order[:keep]]))[::-1]
        if top < len(open_):
            out[t] = min(out[t], open_[top - 1] - open_[top])
    return out


def routed_units(f: dict, w: Dict[str, np.ndarray], p: str, x: np.ndarray, logits: Optional[np.ndarray] = None,
                 margins: Optional[list] = None) -> np.ndarray:
    r = f["router"]
    z = x @ w[p + "router"].T if logits is None else logits
    if margins is not None:
        margins.append(route_margin(z, w[p + "correction"], int(r["top"]), int(r["groups"]["count"]), int(r["groups"]["keep"])))
    ids, wt = route(z, w[p + "correction"], int(r["top"]), int(r["groups"]["count"]), int(r["groups"]["keep"]))
    y = np.zeros((x.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(x.shape[0]):
        for e, c in zip(ids[t], wt[t]):
            a = np.maximum(w[p + f"e{e}.up"] @ x[t], 0.0) ** 2
            y[t] += c * (w[p + f"e{e}.down"] @ a)
    return y


# ---------------------------------------------------------------------------------- model
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], streams: Optional[list] = None,
            router_logits: Optional[dict] = None, margins: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence from its first token. `streams` (a list) takes what each layer hands on.
    `router_logits[i]`: layer i's router logits given from outside. `margins` (a list) takes, per routed layer, by how
    much each token's choice of units is decided (route_margin)."""
    eps = float(cfg["norm"]["eps"])
    s = embedding(w, tokens)
    history = [s]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer {i}: unknown type {layer['type']}")
        a = unit_rms(s, eps) * (1.0 + w[p + "norm1"])
        branch = parallel_mixer(cfg, layer["mixer"], w, p + "mix.", sublayer_input(a, w[p + "canon1"]))
        s = s + output_gate(a, w[p + "rg1"], w[p + "rg1.b"]) * branch
        if layer.get("mlp") is not None:
            f = unit_rms(s, eps) * (1.0 + w[p + "norm2"])
            z = None if router_logits is None else router_logits.get(i)
            branch = routed_units(layer["mlp"], w, p + "mlp.", sublayer_input(f, w[p + "canon2"]), z, margins)
            s = s + output_gate(f, w[p + "rg2"], w[p + "rg2.b"]) * branch
        history.append(s)
        s = depth_average(history, w[p + "dwa"])
        if streams is not None:
            streams.append(s)
    y = unit_rms(s, eps) * (1.0 + w["final.norm"])
    return y @ w["head"].T


def router_margins(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    """[T]: the smallest route_margin over the model's routed layers (infinite without any)."""
    margins: list = []
    forward(cfg, w, tokens, margins=margins)
    return np.min(np.stack(margins), 0) if margins else np.full(len(tokens), np.inf)
