"""Tiny Tozarax configurations for the tests, and helpers to write them as model folders with random weights.

A has sizes that are no multiple of 8 and differ from layer to layer: windows shorter than a page, value heads larger and
smaller than key heads, memories whose heads share keys two and three to one, filters of 2 to 5 taps that differ from the
layer frame's 3, a layer without a feed-forward, top 2 of 6 in 3 groups of which 2 stay open, top 3 of 8 in 2 groups of
which 1 stays open. B has widths that are multiples of 8 (the tensor-core kernels), a window longer than a page and one
longer than most prompts, key and value heads of one size, one query head a key head, one group (no limit), top 1, and a
frame filter of one tap. C has a frame filter of 5 taps, every layer without experts but the last, a window of one
position. The single-layer configurations run the mixers without a feed-forward, and the experts behind the smallest mixer.
"""
import os

from xpu_serve_b200.config import TozaraxConfig
from xpu_serve_b200.weights import write_random_model


def left(heads, kv_heads, dim, vdim, size, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "scale": scale}


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def moe(ff, experts, top, count, keep):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def model(width, vocab, taps, layers, eps=1e-5, positions=512):
    return {"architecture": "Tozarax", "width": width, "vocab": vocab, "max_positions": positions, "norm": {"eps": eps},
            "canon": {"taps": taps},
            "layers": [{"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": f} for l, r, f in layers]}


CONFIGS = {
    "A": model(44, 203, 3, [
        (left(4, 2, 12, 20, 13, 0.21), right(4, 2, 10, 14, 2), moe(20, 6, 2, 3, 2)),
        (left(6, 3, 10, 6, 41, 0.35), right(3, 1, 6, 9, 5), None),
        (left(2, 1, 18, 18, 29, 0.3), right(2, 2, 20, 5, 4), moe(12, 8, 3, 2, 1)),
    ], eps=3e-6),
    "B": model(128, 384, 1, [
        (left(4, 4, 64, 64, 70, 0.11), right(4, 4, 32, 32, 4), moe(48, 3, 1, 1, 1)),
        (left(8, 2, 16, 32, 300, 0.3), right(8, 2, 64, 16, 3), moe(64, 8, 4, 4, 2)),
        (left(2, 2, 64, 64, 130, 0.2), right(2, 1, 128, 64, 2), moe(32, 16, 2, 8, 4)),
    ]),
    "C": model(64, 180, 5, [
        (left(4, 2, 32, 48, 21, 0.2), right(2, 1, 16, 24, 3), None),
        (left(2, 2, 16, 16, 1, 0.5), right(4, 4, 8, 8, 1), None),
        (left(4, 1, 16, 64, 64, 0.15), right(1, 1, 40, 72, 4), moe(24, 4, 2, 2, 2)),
    ]),
    # one mechanism's neighbourhood each
    "mixers": model(40, 150, 4, [(left(4, 2, 14, 10, 9, 0.25), right(3, 3, 10, 6, 3), None)]),
    "shared_keys": model(40, 150, 2, [(left(6, 2, 20, 20, 7, 0.3), right(6, 2, 12, 7, 2), None)]),
    "routed": model(40, 150, 3, [(left(1, 1, 8, 8, 5, 0.3), right(1, 1, 4, 8, 2), moe(30, 12, 3, 4, 2))]),
    "wide_memory": model(48, 150, 2, [(left(1, 1, 8, 8, 5, 0.3), right(2, 1, 200, 40, 2), None)]),
}

# What makes a lost part show: routers, gates and corrections of a size that matters.
SCALE = {".mlp.router": 6.0, ".right.g": 4.0, ".right.a": 3.0, ".right.b": 3.0, ".rg1": 3.0, ".rg2": 3.0, "pos": 2.0}


def make_folder(root, name: str, dtype: str, seed: int = 23, std: float = 0.08):
    folder = os.path.join(str(root), f"tozarax_{name}_{dtype}")
    if not os.path.isdir(folder):
        write_random_model(folder, TozaraxConfig.from_json(CONFIGS[name]), seed=seed, dtype=dtype, std=std,
                           norm_range=(0.5, 1.5), scale=SCALE)
    return folder


def prompt(name: str, length: int, salt: int = 0):
    V = CONFIGS[name]["vocab"]
    return [(i * 31 + 5 + 17 * salt + (i * i) % 13) % V for i in range(length)]


U_BF16 = 2.0 ** -9


def upper_limit(name: str, dtype: str) -> float:
    """Largest |difference| / largest |reference logit| that rounding alone may cause: float32 1e-5; bfloat16 about ten
    roundings to 8 bits a layer that add like a random walk, times 4 for the largest of many logits, times 3 for the norms
    on the two branches of every mixer, which renormalise whatever error a branch carries."""
    layers = len(CONFIGS[name]["layers"])
    return 1e-5 if dtype == "float32" else 3.0 * 4.0 * (10.0 * layers) ** 0.5 * U_BF16
