"""Architecture-neutral description of a decoder: what each layer is made of.

An architecture's typed configuration (config/lfm3.py for LFM3) is turned into a
`ModelSpec`: a list of `LayerSpec`s, each naming its mixer, its feed-forward and its
norms by `kind` with every size, constant and tensor name as a field, plus the order
in which the layers run. The engine builds parts from these specs through the part
registries (registry.py) and never looks at the architecture's own configuration, so
a part does not know which model it is in, and two layers of one model can use
different mixers and feed-forwards.

The reference expresses the same thing as a graph built once per model
(src/models/lfm3/lfm3_decoder.cpp:49-90); here the description is data and the step
function interprets it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary position encoding (src/models/common/blocks.cpp:131-141).

    Pair i couples channels i and i + head_dim/2; pairs i < `pairs` turn by
    pos * theta^(-2i/head_dim), the others by 0 (identity). `pairing` "interleaved": pair i couples
    channels 2i and 2i + 1 instead (LFM3 has "half"; the mixer that reads this brings such a checkpoint
    into the rotate-half order when it loads its weights, so the kernels know one order only).
    """
    head_dim: int
    theta: float
    pairs: int
    kind: str = "rope"
    pairing: str = "half"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a key/value cache (src/models/common/blocks.cpp:143-187)."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    qk_norm: bool            # RMSNorm over head_dim on q and k, before the position encoding
    qk_norm_eps: float
    position: Optional[RopeSpec]
    window: int              # 0: every earlier key is visible; W > 0: keys with pos - j < W
    head_gate: bool          # o[t, h, :] *= sigmoid((x Wg^T)[t, h])
    scale: float             # multiplies q.k before the softmax
    names: Dict[str, str] = field(default_factory=lambda: {
        "q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
        "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight",
        "gate": "self_attn.gate_proj.weight",
        "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight",
        "q_bias": "self_attn.q_proj.bias", "k_bias": "self_attn.k_proj.bias", "v_bias": "self_attn.v_proj.bias"})
    kind: str = "attention"
    qkv_bias: bool = False   # q, k and v projections with a bias each (LFM3 has none)
    v_dim: int = 0           # size of a value head when it differs from head_dim (0: head_dim); needs position None
    chunk: int = 0           # C > 0: a query at pos sees the earlier keys of its own block only, j >= pos - pos % C
                             # (blocks of C positions counted from the sequence's position 0); excludes `window`
    own_kv: bool = True      # False: the layer has no k, v and k-norm tensors; its call reads another call's cache


@dataclass(frozen=True)
class ShortConvSpec:
    """Gated causal depthwise convolution with a fixed-size state
    (src/models/lfm3/lfm3_decoder.cpp:94-111)."""
    hidden: int
    kernel: int              # taps; the state holds kernel - 1 rows per sequence
    bias: bool               # conv.conv.bias, in_proj.bias, out_proj.bias
    names: Dict[str, str] = field(default_factory=lambda: {
        "in": "conv.in_proj.weight", "conv": "conv.conv.weight", "out": "conv.out_proj.weight",
        "in_bias": "conv.in_proj.bias", "conv_bias": "conv.conv.bias", "out_bias": "conv.out_proj.bias"})
    kind: str = "short_conv"


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(act(gate x) * up x) (src/models/common/blocks.cpp:23-27). `activation` "silu" (SwiGLU, LFM3's) or "gelu_tanh":
    0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))."""
    hidden: int
    intermediate: int
    names: Dict[str, str] = field(default_factory=lambda: {
        "gate": "feed_forward.w1.weight", "up": "feed_forward.w3.weight",
        "down": "feed_forward.w2.weight"})
    kind: str = "swiglu"
    activation: str = "silu"


@dataclass(frozen=True)
class RopeScalingSpec:
    """Rotation frequencies stretched for sequences longer than those a model was trained on ("YaRN": pairs that
    turn more than `fast` times over `original` positions keep their frequency, pairs that turn fewer than `slow`
    times are divided by `factor`, with a linear ramp over the pair index between; cos and sin are multiplied by
    `mscale_k` ln(factor) + 1)."""
    factor: float
    original: float
    fast: float
    slow: float
    mscale_k: float = 0.1


@dataclass(frozen=True)
class ScaledRopeSpec:
    """A rotate-half rotation of the first `dims` channels of a vector of `head_dim` channels: pair i couples
    channels i and i + dims/2 (not i + head_dim/2) and turns by pos * theta^(-2i/dims), scaled as `scaling` says
    (None: as is). The table it gives has head_dim/2 entries a position when dims == head_dim, which the kernels
    that know one pairing read; the mixers that use it ask for dims == head_dim."""
    head_dim: int
    theta: float
    dims: int
    scaling: Optional[RopeScalingSpec] = None
    kind: str = "rope_scaled"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values of all heads are products of one cached latent vector per position
    (`kv_rank` numbers, unit RMS times a weight) and of one rotated key part (`rot_dim` numbers) that the heads
    share. A query head has `dim` unrotated and `rot_dim` rotated channels; a value head `vdim`.
    window 0: every earlier key; W > 0: keys with pos - j < W. `sink`: a learned number per head joins the softmax's
    denominator. `head_gate`: o[t, h, :] *= sigmoid((x Wg^T)[t, h]). `out_gate`: every channel of the concatenated heads is
    multiplied by sigmoid((x Wg^T)[t, c]) instead (names["gate"] then has heads * vdim rows). `q_rank` > 0: the queries come
    through a latent of their own, q = Wuq (unit_rms(Wdq x) * w) (names "q_down", "q_norm", "q_up"; the latent norm's eps).
    rot_dim may be 0 (no rotated part; `position` None)."""
    hidden: int
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    eps: float               # of the latent's unit-RMS norm
    position: Optional[ScaledRopeSpec]
    window: int = 0
    sink: bool = False
    head_gate: bool = False
    names: Dict[str, str] = field(default_factory=lambda: {
        "q": "mix.q", "down": "mix.dkv", "latent_norm": "mix.dkv.norm", "up_k": "mix.uk", "up_v": "mix.uv",
        "gate": "mix.g", "sink": "mix.sink", "o": "mix.o",
        "q_down": "mix.dq", "q_norm": "mix.dq.norm", "q_up": "mix.uq"})
    kind: str = "latent_attention"
    out_gate: bool = False
    q_rank: int = 0


@dataclass(frozen=True)
class LightningSpec:
    """A linear-attention memory per head with a constant decay: S <- decay_h S + k v^T (S [dim, vdim], float32, zero at a
    sequence's start), o = S^T q with the new S, for q = silu(Wq x), k = silu(Wk x) (heads of `dim`) and v = silu(Wv x)
    (heads of `vdim`), no other scale. The concatenated heads are divided by their root mean square over all of them
    (`eps`), multiplied by a weight and by sigmoid(Wg x), then projected."""
    hidden: int
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    eps: float
    names: Dict[str, str] = field(default_factory=lambda: {
        "q": "mix.q", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "o": "mix.o", "norm": "mix.norm"})
    kind: str = "lightning"


@dataclass(frozen=True)
class Mamba2Spec:
    """A selective state-space recurrence per head (state [state, vdim], float32) behind a causal depthwise
    convolution with silu over [x | B | C]; the output is gated by silu(z) and then unit-RMS normed in
    `norm_groups` equal parts. in_proj's rows: [z: inner | x: inner | B: groups*state | C: groups*state | dt: heads],
    inner = heads * vdim; head h reads the B and C of group h // (heads / groups)."""
    hidden: int
    heads: int
    vdim: int
    state: int
    groups: int
    taps: int
    norm_groups: int
    eps: float
    names: Dict[str, str] = field(default_factory=lambda: {
        "in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "dt_bias": "mix.dt_bias", "a_log": "mix.A_log",
        "d": "mix.D", "norm": "mix.norm", "out": "mix.o"})
    kind: str = "mamba2"

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass(frozen=True)
class MLstmSpec:
    """The matrix-memory recurrence of xLSTM (mLSTM) per head: a state [dim, vdim], a normaliser [dim] and a running
    maximum, float32, with log-space input and forget gates whose pre-activations are soft-capped at +-gate_cap
    (parts/mlstm.py has the formulas). The heads' outputs are divided by their root mean square (`eps`), multiplied by
    a weight over all heads and by sigmoid of an output gate, then projected."""
    hidden: int
    heads: int
    dim: int
    vdim: int
    gate_cap: float
    eps: float
    names: Dict[str, str] = field(default_factory=lambda: {
        "q": "mix.q", "k": "mix.k", "v": "mix.v", "gate": "mix.g", "o": "mix.o", "norm": "mix.norm",
        "i": "mix.i", "i_bias": "mix.i.b", "f": "mix.f", "f_bias": "mix.f.b"})
    kind: str = "mlstm"


@dataclass(frozen=True)
class SquaredReluSpec:
    """down(max(up x, 0)^2)."""
    hidden: int
    intermediate: int
    names: Dict[str, str] = field(default_factory=lambda: {"up": "mlp.up", "down": "mlp.down"})
    kind: str = "squared_relu"


@dataclass(frozen=True)
class ClampedGLUSpec:
    """down(g * sigmoid(alpha g) * (u + up_shift)) with g = min(gate x, limit), u = clamp(up x, -limit, limit)."""
    hidden: int
    intermediate: int
    limit: float
    alpha: float = 1.702
    up_shift: float = 1.0
    names: Dict[str, str] = field(default_factory=lambda: {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """`experts` gated feed-forwards without biases, of which a token uses the `top` with the largest router
    logits (float32), weighted by the softmax over those logits alone (which equals the softmax over all logits
    divided by the chosen ones' sum) times `route_scale`. `limit` 0: the experts are SwiGLU units; > 0: clamped gated
    units with that limit, `alpha` and `up_shift` (ClampedGLUSpec). `shared`: a clamped gated unit that every token
    uses, added to the sum times sigmoid(x . w) of the one-row matrix names["shared_gate"].

    `score` "sigmoid": a token's scores are the sigmoids of its router logits instead; the experts are chosen by score plus
    a learned number per expert (`correction`, names["correction"]; the weights are the scores without it), among the
    `keep_groups` of `groups` equal groups of neighbouring experts whose `group_top` largest such sums add up highest
    (experts of the other groups cannot be chosen); the weights are the chosen scores times `route_scale`, divided by their
    sum only with `renorm`. `activation` "relu_squared": an expert is down(max(up x, 0)^2), without a gate matrix.

    `score` "softmax_all": a token's scores are the softmax over all router outputs; the experts are chosen by score plus
    `correction` (when set) and weighted by their scores times `route_scale`, as they are. `identity` n > 0: the router has n
    more outputs behind the experts'; such a choice stands for the token's input itself (times its weight) and has no
    tensors. `shared` may be any gated unit's spec (ClampedGLUSpec, or SwiGLUSpec for a plain gated unit)."""
    hidden: int
    intermediate: int
    experts: int
    top: int
    route_scale: float = 1.0
    limit: float = 0.0
    alpha: float = 1.702
    up_shift: float = 1.0
    shared: Optional[object] = None
    names: Dict[str, str] = field(default_factory=lambda: {
        "router": "mlp.router", "gate": "mlp.e{e}.gate", "up": "mlp.e{e}.up", "down": "mlp.e{e}.down",
        "shared_gate": "mlp.shared.sg", "correction": "mlp.correction"})
    kind: str = "routed_experts"
    score: str = "softmax"           # "softmax" over the chosen logits | "sigmoid" of each logit | "softmax_all"
    identity: int = 0                # router outputs behind the experts' that stand for the token's input itself
    correction: bool = False         # sigmoid scores: a learned number per expert joins the score for the choice only
    groups: int = 1
    keep_groups: int = 1
    group_top: int = 2
    renorm: bool = False
    activation: str = "gated"        # "gated" (SwiGLU, or the clamped unit with `limit`) | "relu_squared"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """A gated delta-rule memory per head: a state [dim, vdim] (float32) that each token decays by
    exp(-exp(A_log) softplus(a x + dt_bias)), corrects by beta = sigmoid(b x) towards its value along its unit-length key,
    and reads with its unit-length query times dim^(-1/2) (parts/gated_delta.py has the formulas). q and k (`kv_heads`
    heads of `dim`, shared by heads / kv_heads heads each) and v (`heads` of `vdim`) each pass a causal per-channel filter
    of `taps` taps and silu. The heads' outputs are divided by their root mean square (`eps`), multiplied by a weight of
    `vdim` entries that the heads share and by silu of an output gate, then projected."""
    hidden: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    eps: float
    unit_eps: float = 1e-6
    names: Dict[str, str] = field(default_factory=lambda: {
        "q": "mix.q", "k": "mix.k", "v": "mix.v", "q_conv": "mix.q.conv", "k_conv": "mix.k.conv", "v_conv": "mix.v.conv",
        "a": "mix.a", "b": "mix.b", "a_log": "mix.A_log", "dt_bias": "mix.dt_bias", "gate": "mix.g", "norm": "mix.norm",
        "o": "mix.o"})
    kind: str = "gated_delta"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Mixers side by side that read the same input: the result is `scale` times the sum of their outputs, each first
    divided by its root mean square over the model's width (`eps`) and multiplied by a weight of its own
    (`out_names[k]` for `branches[k]`). A branch is any mixer spec; each keeps what it keeps per sequence."""
    hidden: int
    branches: Tuple[object, ...]
    out_names: Tuple[str, ...]
    scale: float
    eps: float
    kind: str = "parallel"


@dataclass(frozen=True)
class LearnedPositionEmbeddingSpec:
    """Token embedding = table[tok] * scale + rows[position]: a learned vector per position, `positions` of them."""
    width: int
    vocab: int
    positions: int
    names: Dict[str, str] = field(default_factory=lambda: {"table": "embed", "rows": "pos"})
    kind: str = "learned_position"
    scale: float = 1.0


@dataclass(frozen=True)
class NormSpec:
    """RMSNorm over the last dimension, x * (mean(x^2) + eps)^(-1/2) * w, no +1 offset
    (src/graph/graph.h:57, src/backend/cpu_ref/ops.cpp:260-281)."""
    width: int
    eps: float
    kind: str = "rmsnorm"    # "layernorm": (x - mean) * (variance + eps)^(-1/2) * w, no bias (parts/layernorm.py)
    offset: float = 0.0      # rmsnorm: the stored weight stands around zero and the norm multiplies by offset + w


@dataclass(frozen=True)
class PairHashEmbeddingSpec:
    """Token embedding = table[tok] * scale + pair[(prev * mul_prev + tok * mul_cur) mod buckets] (row `buckets` for a
    sequence's first token) + a sine/cosine vector of the position (entries 2i and 2i + 1: sin and cos of
    pos * theta^(-2i / width)), then an RMS norm. A sequence's last token is part of its state."""
    width: int
    vocab: int
    scale: float
    buckets: int
    mul_prev: int
    mul_cur: int
    eps: float
    theta: float = 10000.0
    names: Dict[str, str] = field(default_factory=lambda: {"table": "embed", "pair": "bigram", "norm": "embed.norm"})
    kind: str = "pair_hash"


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input from the token itself, behind the layer's last sublayer: with e = table[tok, offset : offset + dim]
    (a second token table that all layers share, `table` its name at the model's top level, `columns` wide),
    h += unit_rms(P (gelu_tanh(G h) * e)) * w, the norm's weight plain (names "gate": [dim, width], "proj": [width, dim],
    "norm": [width], under the layer's prefix)."""
    dim: int
    offset: int
    columns: int
    vocab: int
    eps: float
    table: str = "side.embed"
    names: Dict[str, str] = field(default_factory=lambda: {"gate": "side.gate", "proj": "side.proj", "norm": "side.norm"})


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: h += post(mixer(pre(h))); h += post(ffn(pre(h)))
    (src/models/lfm3/lfm3_decoder.cpp:78-90). With `sandwich` false the post norms are
    the identity and their tensors are not read."""
    prefix: str              # tensor-name prefix under the model prefix, e.g. "layers.3."
    mixer: object            # a spec with a `kind`
    ffn: object              # a spec with a `kind`, or None: the layer has no feed-forward (and no norms for one)
    norm: NormSpec
    sandwich: bool
    names: Dict[str, str] = field(default_factory=lambda: {
        "pre_mixer": "operator_norm.weight", "post_mixer": "post_operator_norm.weight",
        "pre_ffn": "ffn_norm.weight", "post_ffn": "post_ffn_norm.weight"})
    kind: str = "pre_norm"   # the arrangement (registry.register_arrangement); the formula above is "pre_norm";
                             # "branch_norm": h += post(mixer(h)); h += post(ffn(h)), no norm before a sublayer;
                             # "gated_pre_norm": the pre-norm layer with the three options below (parts/block.py)
    input_taps: int = 0      # > 0: a sublayer reads x + filter(x), a causal per-channel filter of so many taps over the
                             # normed stream x (names "mixer_taps", "ffn_taps": [width, taps]); the last taps - 1 rows of
                             # x are part of a sequence's state, for each sublayer
    branch_gate: bool = False  # a sublayer's result joins the stream times sigmoid(x G^T + b) (names "mixer_gate",
                             # "mixer_gate_bias", "ffn_gate", "ffn_gate_bias"), x the normed stream before the filter
    depth_terms: int = 0     # n > 0: what the layer hands on is sum_j c[j] X_j over the embedding's output X_0 and the
                             # results X_1 .. X_(n-1) of the layers so far, this one's last (names "depth": [n])
    token_side: Optional[TokenSideSpec] = None   # "pre_norm": a gated slice of a second token table joins the stream last


@dataclass(frozen=True)
class LayerCall:
    """One entry of the running order. `layer` indexes ModelSpec.layers (a layer may be
    called more than once; each call keeps its own cache). `cache_of` is the index, in
    the running order, of an earlier call whose cache this call's mixer reads instead
    of owning one."""
    layer: int
    cache_of: Optional[int] = None
    mix_in: bool = False     # before this call the stream becomes M [stream; embedding output] (ModelSpec.names["pass_in"]:
                             # [width, 2 width]): how a pass over repeated layers starts


@dataclass(frozen=True)
class ModelSpec:
    arch: str
    vocab: int
    hidden: int
    max_position: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tied_head: bool
    init_std: float = 0.02   # random-weights mode: matrices and tables ~ N(0, init_std)
    embed_scale: float = 1.0  # the embedding rows are multiplied by it (1: as stored, LFM3's)
    logit_cap: float = 0.0    # > 0: logits = cap * tanh(logits / cap) (0: none, LFM3's)
    logit_scale: float = 1.0  # the logits are multiplied by it (positive, so that their order stays)
    prefixes: Tuple[str, ...] = ("model.",)   # tried in turn for "<prefix>embed_tokens.weight"
    ignorable: Tuple[str, ...] = ()           # regular expressions: tensors of a folder that match are neither needed nor refused
    embedding: Optional[object] = None        # a spec with a `kind` (registry.register_embedding); None: table[tok] * embed_scale
    depth_history: bool = False               # the step keeps every layer's result (layers with `depth_terms` read them)
    names: Dict[str, str] = field(default_factory=lambda: {
        "embed": "embed_tokens.weight", "final_norm": "embedding_norm.weight",
        "head": "lm_head.weight", "pass_in": "loop.in"})   # "head" is looked up without the model prefix

    @property
    def mixes_in(self) -> bool:
        return any(c.mix_in for c in self.order)

    def shared_tables(self) -> Dict[str, Tuple[int, int]]:
        """Tensors at the model's top level that the layers read (name -> shape): the token-side tables."""
        out: Dict[str, Tuple[int, int]] = {}
        for layer in self.layers:
            ts = getattr(layer, "token_side", None)
            if ts is not None:
                shape = (ts.vocab, ts.columns)
                if out.setdefault(ts.table, shape) != shape:
                    raise ValueError(f"layers disagree about the shape of '{ts.table}'")
        return out

    def validate(self) -> None:
        if not self.logit_scale > 0:
            raise ValueError("logit_scale must be positive")
        self.shared_tables()
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.order:
            raise ValueError("the running order is empty")
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {call.layer} of {len(self.layers)}")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < i:
                    raise ValueError(f"order[{i}] reads the cache of call {call.cache_of}, which does not run before it")
                if self.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"order[{i}] reads the cache of call {call.cache_of}, which owns none")
