"""Typed configuration of Vekuzen, read from config.json's own keys.

config.json gives the model's `width`, `vocab`, `max_positions` (rows of the learned position table), `norm.eps`,
`embedding.scale` (the token table's rows are multiplied by it), `logit_scale`, `token_side.dim` (channels of the second
token table that every layer reads; absent: no such input), `loop` (`start`, `stop`, `times`: layers start .. stop - 1 run
`times` times in a row with the same weights, each pass with a cache of its own and behind a mix of the stream with the
embedding's output; absent: every layer once) and under `layers` one entry per layer: `type` (which mixer), `mixer` (its
sizes and constants) and `mlp` (its feed-forward, or null for none). Every size and every constant that can differ
between two models of the design is read from there.

Layer types:
  lightning          a decayed linear-attention memory per head (`heads`, `dim`, `vdim`, `decay`: a number per head)
  latent_attention   softmax attention over every earlier position whose keys and values are products of one normed
                     latent a position (`heads`, `dim`, `vdim`, `kv_rank`, `scale`), queries through a latent of `q_rank`,
                     no rotation, a sigmoid gate on every output channel
Feed-forwards (`mlp.kind`): `dense` (a gated unit of `ff` with the tanh form of gelu), `moe` (`router.experts` silu units of
`expert.ff`, of which a token uses `router.top`, chosen by softmax scores plus a correction per unit and weighted by the
scores times `router.scale`; the last `router.identity` router outputs stand for the token's input itself; `shared.ff`: a
unit every token uses through a sigmoid gate).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .json_util import ConfigError, get_float, get_float_or, get_int, get_int_or, get_str
from .spec import (LatentAttentionSpec, LayerCall, LayerSpec, LearnedPositionEmbeddingSpec, LightningSpec, ModelSpec, NormSpec,
                   RoutedExpertsSpec, SwiGLUSpec, TokenSideSpec)

LIGHTNING, LATENT = "lightning", "latent_attention"

_LAYER_NAMES = {"pre_mixer": "norm1", "pre_ffn": "norm2"}


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing object '{key}'")
    return v


@dataclass(frozen=True)
class VekuzenLayer:
    type: str
    mixer: object                    # LightningSpec | LatentAttentionSpec
    mlp: Optional[object]            # SwiGLUSpec (gelu_tanh) | RoutedExpertsSpec | None
    raw: dict                        # the entry as read (written back by to_json)


@dataclass(frozen=True)
class VekuzenConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    embed_scale: float
    logit_scale: float
    side_dim: int                    # 0: no per-layer token input
    loop: Optional[Tuple[int, int, int]]     # (start, stop, times)
    layers: Tuple[VekuzenLayer, ...]
    architecture: str = "Vekuzen"

    # ---------------------------------------------------------------- parsing
    @staticmethod
    def _lightning(m: dict, width: int, eps: float, where: str) -> LightningSpec:
        heads, dim, vdim = get_int(m, "heads", where), get_int(m, "dim", where), get_int(m, "vdim", where)
        if min(heads, dim, vdim) <= 0:
            raise ConfigError(f"{where}: heads, dim and vdim must be positive")
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or not all(
                isinstance(d, (int, float)) and not isinstance(d, bool) and 0.0 <= float(d) <= 1.0 for d in decay):
            raise ConfigError(f"{where}: 'decay' must list a number between 0 and 1 for each of the {heads} heads")
        return LightningSpec(hidden=width, heads=heads, dim=dim, vdim=vdim, decay=tuple(float(d) for d in decay), eps=eps)

    @staticmethod
    def _latent(m: dict, width: int, eps: float, where: str) -> LatentAttentionSpec:
        heads, dim, vdim = get_int(m, "heads", where), get_int(m, "dim", where), get_int(m, "vdim", where)
        kv_rank, q_rank = get_int(m, "kv_rank", where), get_int(m, "q_rank", where)
        if min(heads, dim, vdim, kv_rank, q_rank) <= 0:
            raise ConfigError(f"{where}: heads, dim, vdim, kv_rank and q_rank must be positive")
        return LatentAttentionSpec(hidden=width, heads=heads, dim=dim, rot_dim=0, vdim=vdim, kv_rank=kv_rank,
                                   scale=get_float(m, "scale", where), eps=eps, position=None, window=0, sink=False,
                                   head_gate=False, out_gate=True, q_rank=q_rank)

    @staticmethod
    def _mlp(f: Optional[dict], width: int, where: str):
        if f is None:
            return None
        if not isinstance(f, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        kind = get_str(f, "kind", where)
        if kind == "dense":
            ff = get_int(f, "ff", where)
            if ff <= 0:
                raise ConfigError(f"{where}: ff must be positive")
            return SwiGLUSpec(hidden=width, intermediate=ff, activation="gelu_tanh",
                              names={"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})
        if kind != "moe":
            raise ConfigError(f"{where}: unknown feed-forward kind '{kind}' (dense, moe)")
        router, expert = _obj(f, "router", where), _obj(f, "expert", where)
        experts, top = get_int(router, "experts", f"{where} router"), get_int(router, "top", f"{where} router")
        identity = get_int_or(router, "identity", 0, f"{where} router")
        ff = get_int(expert, "ff", f"{where} expert")
        if ff <= 0 or experts <= 0 or identity < 0 or not 0 < top <= experts + identity:
            raise ConfigError(f"{where}: expert.ff and router.experts must be positive, router.identity not negative and "
                              f"0 < router.top <= router.experts + router.identity")
        shared = None
        if f.get("shared") is not None:
            sff = get_int(_obj(f, "shared", where), "ff", f"{where} shared")
            if sff <= 0:
                raise ConfigError(f"{where} shared: ff must be positive")
            shared = SwiGLUSpec(hidden=width, intermediate=sff, activation="silu",
                                names={"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"})
        return RoutedExpertsSpec(hidden=width, intermediate=ff, experts=experts, top=top,
                                 route_scale=get_float_or(router, "scale", 1.0, f"{where} router"), score="softmax_all",
                                 correction=True, identity=identity, shared=shared)

    @classmethod
    def from_json(cls, cfg: dict) -> "VekuzenConfig":
        w = "config.json"
        width, vocab = get_int(cfg, "width", w), get_int(cfg, "vocab", w)
        positions = get_int(cfg, "max_positions", w)
        eps = get_float(_obj(cfg, "norm", w), "eps", f"{w} norm")
        if min(width, vocab, positions) <= 0 or not eps > 0:
            raise ConfigError(f"{w}: width, vocab, max_positions and norm.eps must be positive")
        embed_scale = get_float(_obj(cfg, "embedding", w), "scale", f"{w} embedding")
        logit_scale = get_float_or(cfg, "logit_scale", 1.0, w)
        if not logit_scale > 0:
            raise ConfigError(f"{w}: logit_scale must be positive")
        side_dim = 0
        if cfg.get("token_side") is not None:
            side_dim = get_int(_obj(cfg, "token_side", w), "dim", f"{w} token_side")
            if side_dim <= 0:
                raise ConfigError(f"{w} token_side: dim must be positive")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{w}: 'layers' must be a list with at least one entry")
        layers = []
        for i, e in enumerate(entries):
            where = f"{w} layers[{i}]"
            if not isinstance(e, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = get_str(e, "type", where)
            m = _obj(e, "mixer", where)
            if kind == LIGHTNING:
                mixer = cls._lightning(m, width, eps, f"{where} mixer")
            elif kind == LATENT:
                mixer = cls._latent(m, width, eps, f"{where} mixer")
            else:
                raise ConfigError(f"{where}: unknown layer type '{kind}' ({LIGHTNING}, {LATENT})")
            layers.append(VekuzenLayer(kind, mixer, cls._mlp(e.get("mlp"), width, f"{where} mlp"), e))
        loop = None
        if cfg.get("loop") is not None:
            lp = _obj(cfg, "loop", w)
            loop = (get_int(lp, "start", f"{w} loop"), get_int(lp, "stop", f"{w} loop"), get_int(lp, "times", f"{w} loop"))
            if not 0 <= loop[0] < loop[1] <= len(layers) or loop[2] < 1:
                raise ConfigError(f"{w} loop: needs 0 <= start < stop <= {len(layers)} layers and times >= 1")
        return cls(vocab=vocab, width=width, max_positions=positions, norm_eps=eps, embed_scale=embed_scale,
                   logit_scale=logit_scale, side_dim=side_dim, loop=loop, layers=tuple(layers))

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embed_scale},
               "layers": [l.raw for l in self.layers], "logit_scale": self.logit_scale, "max_positions": self.max_positions,
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out

    # ------------------------------------------------------- to a model spec
    def running_order(self) -> Tuple[LayerCall, ...]:
        n = len(self.layers)
        if self.loop is None:
            return tuple(LayerCall(i) for i in range(n))
        a, b, times = self.loop
        calls = [LayerCall(i) for i in range(a)]
        for _ in range(times):
            calls += [LayerCall(i, mix_in=(i == a)) for i in range(a, b)]
        return tuple(calls + [LayerCall(i) for i in range(b, n)])

    def model_spec(self) -> ModelSpec:
        norm = NormSpec(self.width, self.norm_eps)
        n = len(self.layers)
        layers = tuple(
            LayerSpec(prefix=f"l{i}.", mixer=l.mixer, ffn=l.mlp, norm=norm, sandwich=False, kind="pre_norm",
                      names=dict(_LAYER_NAMES),
                      token_side=(TokenSideSpec(dim=self.side_dim, offset=i * self.side_dim, columns=n * self.side_dim,
                                                vocab=self.vocab, eps=self.norm_eps) if self.side_dim else None))
            for i, l in enumerate(self.layers))
        spec = ModelSpec(arch="vekuzen", vocab=self.vocab, hidden=self.width, max_position=self.max_positions, layers=layers,
                         order=self.running_order(), final_norm=norm, tied_head=False, init_std=0.05, prefixes=("",),
                         logit_scale=self.logit_scale,
                         # a layer without a feed-forward may still carry the norm of one
                         ignorable=tuple(rf"^l{i}\.norm2$" for i, l in enumerate(self.layers) if l.mlp is None),
                         names={"embed": "embed", "final_norm": "final.norm", "head": "head", "pass_in": "loop.in"},
                         embedding=LearnedPositionEmbeddingSpec(width=self.width, vocab=self.vocab, positions=self.max_positions,
                                                                scale=self.embed_scale))
        spec.validate()
        return spec
