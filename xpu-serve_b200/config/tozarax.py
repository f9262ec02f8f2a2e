"""Typed configuration of Tozarax, read from config.json's own keys.

config.json gives the model's `width`, `vocab`, `max_positions` (rows of the learned position table), `norm.eps`,
`canon.taps` (taps of the filter in front of every sublayer) and under `layers` one entry per layer: `type` (which
mixer), `mixer` (its sizes and constants) and `mlp` (its feed-forward, or null for none). Every size and every constant
that can differ between two models of the design is read from there; what the design fixes (the unit norms' 1e-6, the
half in front of the two branches' sum, two scores a group) lives in the specs' defaults and here.

Layer type:
  parallel    two mixers that read the same input, `mixer.left` and `mixer.right`, each output unit-RMS normed with a
              weight of its own, half their sum. left: grouped-query attention without rotation (`heads`, `kv_heads`,
              `dim`, `vdim`, `scale`) under a sliding window of `mask.size` positions. right: a gated delta-rule memory
              (`heads`, `kv_heads`, `dim`, `vdim`, filters of `conv` taps).
Feed-forward (`mlp.kind`): `moe`: `router.experts` squared-ReLU units of `expert.ff`, of which a token uses `router.top`,
chosen by sigmoid scores plus a correction per unit among the `router.groups.keep` best of `router.groups.count` groups.
A layer is the pre-norm layer with a filter in front of each sublayer, a sigmoid gate on each branch and, behind it, a
weighted sum over the embedding's output and all layers' results so far (parts/block.py: GatedPreNormBlock). The norms'
weights are stored around zero (the norm multiplies by 1 + w).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .json_util import ConfigError, get_float, get_int, get_str
from .spec import (AttentionSpec, GatedDeltaSpec, LayerCall, LayerSpec, LearnedPositionEmbeddingSpec, ModelSpec, NormSpec,
                   ParallelMixerSpec, RoutedExpertsSpec)

PARALLEL = "parallel"
BRANCH_SCALE = 0.5          # the two branches' normed outputs are averaged
GROUP_TOP = 2               # a group's score: the sum of its two largest choice scores

_LAYER_NAMES = {"pre_mixer": "norm1", "pre_ffn": "norm2", "mixer_taps": "canon1", "ffn_taps": "canon2",
                "mixer_gate": "rg1", "mixer_gate_bias": "rg1.b", "ffn_gate": "rg2", "ffn_gate_bias": "rg2.b", "depth": "dwa"}


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing object '{key}'")
    return v


@dataclass(frozen=True)
class TozaraxLayer:
    type: str
    mixer: object                    # ParallelMixerSpec
    mlp: Optional[object]            # RoutedExpertsSpec | None
    raw: dict                        # the entry as read (written back by to_json)


@dataclass(frozen=True)
class TozaraxConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    taps: int
    layers: Tuple[TozaraxLayer, ...]
    architecture: str = "Tozarax"

    # ---------------------------------------------------------------- parsing
    @staticmethod
    def _window_attention(m: dict, width: int, where: str) -> AttentionSpec:
        heads, kv_heads = get_int(m, "heads", where), get_int(m, "kv_heads", where)
        dim, vdim = get_int(m, "dim", where), get_int(m, "vdim", where)
        if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads != 0:
            raise ConfigError(f"{where}: heads, kv_heads, dim and vdim must be positive and kv_heads divide heads")
        size = get_int(_obj(m, "mask", where), "size", f"{where} mask")
        if size <= 0:
            raise ConfigError(f"{where} mask: size must be positive")
        p = "mix.left."
        return AttentionSpec(hidden=width, heads=heads, kv_heads=kv_heads, head_dim=dim, qk_norm=False, qk_norm_eps=0.0,
                             position=None, window=size, head_gate=False, scale=get_float(m, "scale", where),
                             names={"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}, v_dim=vdim)

    @staticmethod
    def _gated_delta(m: dict, width: int, eps: float, where: str) -> GatedDeltaSpec:
        s = GatedDeltaSpec(hidden=width, heads=get_int(m, "heads", where), kv_heads=get_int(m, "kv_heads", where),
                           dim=get_int(m, "dim", where), vdim=get_int(m, "vdim", where), taps=get_int(m, "conv", where), eps=eps,
                           names={k: "mix.right." + v for k, v in {
                               "q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv",
                               "a": "a", "b": "b", "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm",
                               "o": "o"}.items()})
        if min(s.heads, s.kv_heads, s.dim, s.vdim, s.taps) <= 0 or s.heads % s.kv_heads != 0:
            raise ConfigError(f"{where}: heads, kv_heads, dim, vdim and conv must be positive and kv_heads divide heads")
        return s

    @classmethod
    def _parallel(cls, m: dict, width: int, eps: float, where: str) -> ParallelMixerSpec:
        left = cls._window_attention(_obj(m, "left", where), width, f"{where} left")
        right = cls._gated_delta(_obj(m, "right", where), width, eps, f"{where} right")
        return ParallelMixerSpec(hidden=width, branches=(left, right), out_names=("mix.left.out", "mix.right.out"),
                                 scale=BRANCH_SCALE, eps=eps)

    @staticmethod
    def _mlp(f: Optional[dict], width: int, where: str):
        if f is None:
            return None
        if not isinstance(f, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        kind = get_str(f, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind '{kind}' (moe)")
        router, expert = _obj(f, "router", where), _obj(f, "expert", where)
        groups = _obj(router, "groups", f"{where} router")
        spec = RoutedExpertsSpec(hidden=width, intermediate=get_int(expert, "ff", f"{where} expert"),
                                 experts=get_int(router, "experts", f"{where} router"), top=get_int(router, "top", f"{where} router"),
                                 score="sigmoid", correction=True, groups=get_int(groups, "count", f"{where} router groups"),
                                 keep_groups=get_int(groups, "keep", f"{where} router groups"), group_top=GROUP_TOP,
                                 renorm=False, activation="relu_squared")
        if spec.intermediate <= 0 or not 0 < spec.top <= spec.experts:
            raise ConfigError(f"{where}: expert.ff must be positive and 0 < router.top <= router.experts")
        if spec.groups <= 0 or spec.experts % spec.groups != 0 or not 0 < spec.keep_groups <= spec.groups:
            raise ConfigError(f"{where} router groups: count must divide router.experts and 0 < keep <= count")
        if spec.keep_groups * (spec.experts // spec.groups) < spec.top:
            raise ConfigError(f"{where} router groups: the kept groups hold fewer than router.top experts")
        return spec

    @classmethod
    def from_json(cls, cfg: dict) -> "TozaraxConfig":
        w = "config.json"
        width, vocab = get_int(cfg, "width", w), get_int(cfg, "vocab", w)
        positions = get_int(cfg, "max_positions", w)
        eps = get_float(_obj(cfg, "norm", w), "eps", f"{w} norm")
        taps = get_int(_obj(cfg, "canon", w), "taps", f"{w} canon")
        if min(width, vocab, positions) <= 0 or not eps > 0:
            raise ConfigError(f"{w}: width, vocab, max_positions and norm.eps must be positive")
        if not 1 <= taps <= 16:
            raise ConfigError(f"{w} canon: taps must be 1 to 16")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{w}: 'layers' must be a list with at least one entry")
        layers = []
        for i, e in enumerate(entries):
            where = f"{w} layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = get_str(e, "type", where)
            if kind != PARALLEL:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({PARALLEL})")
            mixer = cls._parallel(_obj(e, "mixer", where), width, eps, f"{where} mixer")
            layers.append(TozaraxLayer(kind, mixer, cls._mlp(e.get("mlp"), width, f"{where} mlp"), e))
        return cls(vocab=vocab, width=width, max_positions=positions, norm_eps=eps, taps=taps, layers=tuple(layers))

    def to_json(self) -> dict:
        return {"architecture": self.architecture, "canon": {"taps": self.taps}, "layers": [l.raw for l in self.layers],
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    # ------------------------------------------------------- to a model spec
    def model_spec(self) -> ModelSpec:
        norm = NormSpec(self.width, self.norm_eps, offset=1.0)
        layers = tuple(
            LayerSpec(prefix=f"l{i}.", mixer=l.mixer, ffn=l.mlp, norm=norm, sandwich=False, kind="gated_pre_norm",
                      names=dict(_LAYER_NAMES), input_taps=self.taps, branch_gate=True, depth_terms=i + 2)
            for i, l in enumerate(self.layers))
        spec = ModelSpec(arch="tozarax", vocab=self.vocab, hidden=self.width, max_position=self.max_positions, layers=layers,
                         order=tuple(LayerCall(i) for i in range(len(self.layers))),
                         final_norm=norm, tied_head=False, init_std=0.05, prefixes=("",),
                         # a layer without a feed-forward may still carry the tensors of one's frame
                         ignorable=tuple(rf"^l{i}\.(norm2|canon2|rg2|rg2\.b)$" for i, l in enumerate(self.layers) if l.mlp is None),
                         names={"embed": "embed", "final_norm": "final.norm", "head": "head"},
                         embedding=LearnedPositionEmbeddingSpec(width=self.width, vocab=self.vocab, positions=self.max_positions),
                         depth_history=True)
        spec.validate()
        return spec
