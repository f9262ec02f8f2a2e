"""A plain, slow Vekuzen in float64 numpy: whole sequences, no cache, one function per mechanism.

It shares no code with the package: it reads config.json's keys itself and takes tensors by their checkpoint names.
Notation: T tokens, W the model's width; rows of a [T, n] array are tokens. Weights are [out, in], applied as y = x M^T.

The stream starts as a table row times a constant plus a learned row per position (s0). A layer is

    s = s + mixer(n1(s));   s = s + ff(n2(s));   s = s + n_side(P (gelu(G s) * e_i[token]))

n being x / sqrt(mean x^2 + eps) times a weight and e_i the layer's slice of a second token table. A span of layers
may run several times in a row; in front of each such pass s = L [s; s0]. Mixers: a decayed linear recurrence per head
over silu'd keys, values and queries; softmax attention whose keys and values are products of one normed latent a
position, with queries through a latent of their own. Feed-forwards: a gated gelu unit, or a few of many silu units per
token chosen by softmax scores plus a correction, some of which hand their input through, plus a unit every token uses.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------ embedding
def embedding(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], first_position: int = 0) -> np.ndarray:
    toks = np.asarray(tokens, dtype=np.int64)
    return w["embed"][toks] * float(cfg["embedding"]["scale"]) + w["pos"][first_position + np.arange(len(toks))]


def pass_input(s: np.ndarray, s0: np.ndarray, mix: np.ndarray) -> np.ndarray:
    """What a pass over the repeated layers starts from: mix [s; s0]."""
    return np.concatenate([s, s0], -1) @ mix.T


def token_side(cfg: dict, w: Dict[str, np.ndarray], i: int, tokens: Sequence[int], s: np.ndarray) -> np.ndarray:
    """The layer's own slice of the side table, gated by the stream, projected, normed, added."""
    d = int(cfg["token_side"]["dim"])
    p = f"l{i}.side."
    e = w["side.embed"][np.asarray(tokens, dtype=np.int64)][:, i * d:(i + 1) * d]
    g = gelu_tanh(s @ w[p + "gate"].T) * e
    y = g @ w[p + "proj"].T
    return s + unit_rms(y, float(cfg["norm"]["eps"])) * w[p + "norm"]


# --------------------------------------------------------------------------------- mixers
def decayed_memory(q: np.ndarray, k: np.ndarray, v: np.ndarray, decay: float, state: Optional[np.ndarray] = None):
    """One head. q, k [T, d], v [T, e]. S <- decay S + k_t v_t^T, o_t = S^T q_t with the new S. Returns (o, S)."""
    S = np.zeros((k.shape[1], v.shape[1])) if state is None else state.copy()
    o = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        S = decay * S + np.outer(k[t], v[t])
        o[t] = S.T @ q[t]
    return o, S


def lightning(m: dict, w: Dict[str, np.ndarray], p: str, h: np.ndarray, eps: float) -> np.ndarray:
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = silu(h @ w[p + "q"].T).reshape(T, H, d)
    k = silu(h @ w[p + "k"].T).reshape(T, H, d)
    v = silu(h @ w[p + "v"].T).reshape(T, H, e)
    o = np.stack([decayed_memory(q[:, j], k[:, j], v[:, j], float(m["decay"][j]))[0] for j in range(H)], 1)
    o = unit_rms(o.reshape(T, H * e), eps) * w[p + "norm"]
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def causal_softmax_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float) -> np.ndarray:
    """One head. Position i sees every j <= i."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    s = np.where(np.arange(T)[None, :] <= np.arange(T)[:, None], s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    a = np.exp(s)
    a = a / a.sum(-1, keepdims=True)
    return a @ v


def latent_attention(m: dict, w: Dict[str, np.ndarray], p: str, h: np.ndarray, eps: float) -> np.ndarray:
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, d)
    c = unit_rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, e)
    o = np.stack([causal_softmax_attention(q[:, j], k[:, j], v[:, j], float(m["scale"])) for j in range(H)], 1)
    return (o.reshape(T, H * e) * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---------------------------------------------------------------------------- feed-forwards
def gated_unit(w: Dict[str, np.ndarray], p: str, x: np.ndarray, act) -> np.ndarray:
    return (act(x @ w[p + "gate"].T) * (x @ w[p + "up"].T)) @ w[p + "down"].T


def route(z: np.ndarray, correction: np.ndarray, top: int, scale: float):
    """z [T, n] router outputs. Scores: softmax over all n; chosen: the `top` largest of score + correction (ties to the
    lower index); weights: the chosen scores times `scale`, as they are. Returns (ids [T, top], weights [T, top])."""
    s = np.exp(z - z.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    ids = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    return ids, np.take_along_axis(s, ids, -1) * scale


def route_margin(z: np.ndarray, correction: np.ndarray, top: int) -> np.ndarray:
    """[T]: the gap between the last chosen and the first left-out choice score (infinite when all are chosen)."""
    s = np.exp(z - z.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    c = -np.sort(-(s + correction), axis=-1)
    return c[:, top - 1] - c[:, top] if top < c.shape[1] else np.full(z.shape[0], np.inf)


def routed_units(f: dict, w: Dict[str, np.ndarray], p: str, x: np.ndarray, margins: Optional[list] = None) -> np.ndarray:
    r = f["router"]
    n_real, n_id, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    z = x @ w[p + "router"].T
    assert z.shape[1] == n_real + n_id
    if margins is not None:
        margins.append(route_margin(z, w[p + "correction"], top))
    ids, wt = route(z, w[p + "correction"], top, float(r["scale"]))
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for e, c in zip(ids[t], wt[t]):
            y[t] += c * (x[t] if e >= n_real else gated_unit(w, p + f"e{e}.", x[t:t + 1], silu)[0])
    if f.get("shared") is not None:
        y = y + sigmoid(x @ w[p + "shared.sg"].T) * gated_unit(w, p + "shared.", x, silu)
    return y


def feed_forward(f: dict, w: Dict[str, np.ndarray], p: str, x: np.ndarray, margins: Optional[list] = None) -> np.ndarray:
    if f["kind"] == "dense":
        return gated_unit(w, p, x, gelu_tanh)
    if f["kind"] == "moe":
        return routed_units(f, w, p, x, margins)
    raise ValueError(f"unknown feed-forward kind {f['kind']}")


# ---------------------------------------------------------------------------------- model
def running_order(cfg: dict) -> List[tuple]:
    """[(layer, first of a pass)] in the order in which the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], streams: Optional[list] = None,
            margins: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence from its first token. `streams` (a list) takes the stream after every layer run.
    `margins` (a list) takes, per routed layer run, by how much each token's choice of units is decided."""
    eps = float(cfg["norm"]["eps"])
    s0 = embedding(cfg, w, tokens)
    s = s0
    for i, first in running_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if first:
            s = pass_input(s, s0, w["loop.in"])
        h = unit_rms(s, eps) * w[p + "norm1"]
        if layer["type"] == "lightning":
            s = s + lightning(layer["mixer"], w, p + "mix.", h, eps)
        elif layer["type"] == "latent_attention":
            s = s + latent_attention(layer["mixer"], w, p + "mix.", h, eps)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']}")
        if layer.get("mlp") is not None:
            s = s + feed_forward(layer["mlp"], w, p + "mlp.", unit_rms(s, eps) * w[p + "norm2"], margins)
        if cfg.get("token_side"):
            s = token_side(cfg, w, i, tokens, s)
        if streams is not None:
            streams.append(s)
    y = unit_rms(s, eps) * w["final.norm"]
    return (y @ w["head"].T) * float(cfg.get("logit_scale", 1.0))


def router_margins(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int]) -> np.ndarray:
    margins: list = []
    forward(cfg, w, tokens, margins=margins)
    return np.min(np.stack(margins), 0) if margins else np.full(len(tokens), np.inf)
