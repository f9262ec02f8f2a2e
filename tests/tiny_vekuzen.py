"""Tiny Vekuzen configurations for the tests, and helpers to write them as model folders with random weights.

A has sizes that are no multiple of 8 and differ from layer to layer: latents of 20 and 28, value heads larger and smaller
than key heads, memories whose value heads are not whole blocks of 32 columns, a layer without a feed-forward, top 2 of 5 + 1
and top 3 of 4 + 3 outputs, a loop over the two middle layers that runs twice, a side table of 5 channels a layer. B has
widths that are multiples of 8 (the tensor-core kernels), a loop over one layer that runs three times, one head, top 1, no
pass-through outputs in one layer and no shared unit in another, keys of 128 rows. C has no loop at all, no side table, a
logit scale of 1, every decay 1 or 0 in one memory. The single-layer configurations run each mechanism alone; `whole_loop`
repeats every layer.
"""
import os

from xpu_serve_b200.config import VekuzenConfig
from xpu_serve_b200.weights import write_random_model


def latent(heads, dim, vdim, kv_rank, q_rank, scale):
    return "latent_attention", {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}


def memory(heads, dim, vdim, decay):
    return "lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, identity, top, scale, shared):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def model(width, vocab, layers, loop=None, side=0, eps=1e-5, positions=512, embed_scale=1.5, logit_scale=0.7):
    cfg = {"architecture": "Vekuzen", "width": width, "vocab": vocab, "max_positions": positions, "norm": {"eps": eps},
           "embedding": {"scale": embed_scale}, "logit_scale": logit_scale,
           "layers": [{"type": t, "mixer": m, "mlp": f} for (t, m), f in layers]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


CONFIGS = {
    "A": model(44, 203, [
        (latent(3, 12, 20, 20, 9, 0.31), dense(50)),
        (memory(3, 10, 14, (0.5, 0.9, 0.97)), moe(20, 5, 1, 2, 1.7, 12)),
        (latent(5, 6, 4, 28, 13, 0.4), None),
        (memory(2, 20, 37, (0.999, 0.8)), moe(12, 4, 3, 3, 0.6, 0)),
    ], loop=(1, 3, 2), side=5, eps=3e-6),
    "B": model(128, 384, [
        (memory(4, 32, 32, (0.7, 0.9, 0.95, 0.99)), moe(48, 3, 0, 1, 1.0, 64)),
        (latent(4, 32, 32, 64, 48, 0.18), dense(256)),
        (latent(1, 64, 64, 128, 32, 0.125), moe(64, 8, 2, 4, 2.5, 0)),
        (memory(2, 128, 64, (0.98, 0.6)), dense(64)),
    ], loop=(1, 2, 3), side=8),
    "C": model(64, 180, [
        (memory(4, 8, 8, (1.0, 0.0, 0.5, 0.9)), dense(40)),
        (latent(2, 16, 24, 40, 24, 0.25), None),
        (memory(1, 40, 72, (0.93,)), moe(24, 4, 1, 2, 1.0, 16)),
    ], side=0, logit_scale=1.0, embed_scale=1.0),
    # one mechanism's neighbourhood each
    "memory": model(40, 150, [(memory(3, 10, 6, (0.9, 0.99, 0.6)), None)], side=3),
    "attention": model(40, 150, [(latent(4, 14, 10, 24, 11, 0.3), None)]),
    "routed": model(40, 150, [(latent(1, 8, 8, 16, 8, 0.3), moe(30, 6, 2, 3, 2.0, 20))]),
    "wide_memory": model(48, 150, [(memory(2, 200, 40, (0.95, 0.999)), dense(30))]),
    "whole_loop": model(48, 150, [(memory(2, 16, 16, (0.9, 0.8)), dense(32)), (latent(2, 16, 16, 32, 16, 0.25), None)],
                        loop=(0, 2, 3), side=4),
}

# What makes a lost part show: routers, gates, corrections, the side input and the positions at a size that matters.
SCALE = {".mlp.router": 8.0, ".mix.g": 4.0, ".shared.sg": 6.0, "pos": 2.0, "side.embed": 6.0, ".side.gate": 1.5, "loop.in": 4.0}


def make_folder(root, name: str, dtype: str, seed: int = 29, std: float = 0.08):
    folder = os.path.join(str(root), f"vekuzen_{name}_{dtype}")
    if not os.path.isdir(folder):
        write_random_model(folder, VekuzenConfig.from_json(CONFIGS[name]), seed=seed, dtype=dtype, std=std,
                           norm_range=(0.5, 1.5), scale=SCALE)
    return folder


def prompt(name: str, length: int, salt: int = 0):
    V = CONFIGS[name]["vocab"]
    return [(i * 31 + 5 + 17 * salt + (i * i) % 13) % V for i in range(length)]


U_BF16 = 2.0 ** -9


def layer_runs(name: str) -> int:
    cfg = CONFIGS[name]
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    return n if not lp else n + (lp["stop"] - lp["start"]) * (lp["times"] - 1)


def upper_limit(name: str, dtype: str) -> float:
    """Largest |difference| / largest |reference logit| that rounding alone may cause: float32 4e-6 a layer run (every run
    ends in a norm over a freshly projected vector, and the routers' and gates' inputs are scaled up here so that a lost part
    shows), at least 1e-5; bfloat16 about ten roundings to 8 bits a layer run that add like a random walk, times 4 for the
    largest of many logits, times 2 for the norms behind the side input and the memories, which renormalise whatever error
    their input carries."""
    runs = layer_runs(name)
    return max(1e-5, 4e-6 * runs) if dtype == "float32" else 2.0 * 4.0 * (10.0 * runs) ** 0.5 * U_BF16
