"""Tozarax without a device: the configuration's keys and refusals, the model description it gives, cache needs, the
tensors it expects, random weights through the loader, and the oracle's own mechanisms against hand-made cases."""
import copy
import os

import numpy as np
import pytest
import torch

import plain_tozarax as plain
import tiny_tozarax as tiny
from xpu_serve_b200 import registry
from xpu_serve_b200.cache import Cache
from xpu_serve_b200.config import ConfigError, TozaraxConfig
from xpu_serve_b200.parts.base import KVNeed, StateNeed
from xpu_serve_b200.weights.expected import expected_tensors
from xpu_serve_b200.weights.loader import load_weights
from xpu_serve_b200.weights.safetensors_io import WeightError


def test_the_architecture_is_found_by_its_key():
    arch = registry.architecture_for(tiny.CONFIGS["A"])
    assert arch.name == "tozarax" and arch.config_class is TozaraxConfig


def test_every_size_and_constant_comes_from_the_file():
    c = TozaraxConfig.from_json(tiny.CONFIGS["A"])
    assert c.to_json() == tiny.CONFIGS["A"]
    spec = c.model_spec()
    assert spec.vocab == 203 and spec.hidden == 44 and spec.max_position == 512 and not spec.tied_head
    assert spec.final_norm.eps == 3e-6 and spec.final_norm.offset == 1.0 and spec.depth_history
    assert spec.embedding.kind == "learned_position" and spec.embedding.positions == 512
    assert all(l.kind == "gated_pre_norm" and l.input_taps == 3 and l.branch_gate for l in spec.layers)
    assert [l.depth_terms for l in spec.layers] == [2, 3, 4]
    assert all(l.mixer.kind == "parallel" and l.mixer.scale == 0.5 and l.mixer.eps == 3e-6 for l in spec.layers)
    a, m = spec.layers[0].mixer.branches
    assert (a.kind, a.heads, a.kv_heads, a.head_dim, a.v_dim, a.window, a.scale) == ("attention", 4, 2, 12, 20, 13, 0.21)
    assert a.position is None and not a.qk_norm and not a.head_gate
    assert (m.kind, m.heads, m.kv_heads, m.dim, m.vdim, m.taps, m.eps) == ("gated_delta", 4, 2, 10, 14, 2, 3e-6)
    b, n = spec.layers[1].mixer.branches
    assert (b.heads, b.kv_heads, b.head_dim, b.v_dim, b.window, b.scale) == (6, 3, 10, 6, 41, 0.35)
    assert (n.heads, n.kv_heads, n.dim, n.vdim, n.taps) == (3, 1, 6, 9, 5)
    f0, f2 = spec.layers[0].ffn, spec.layers[2].ffn
    assert spec.layers[1].ffn is None
    assert (f0.kind, f0.intermediate, f0.experts, f0.top, f0.groups, f0.keep_groups, f0.group_top) == ("routed_experts", 20, 6, 2, 3, 2, 2)
    assert (f0.score, f0.correction, f0.renorm, f0.activation) == ("sigmoid", True, False, "relu_squared")
    assert (f2.intermediate, f2.experts, f2.top, f2.groups, f2.keep_groups) == (12, 8, 3, 2, 1)


def test_cache_needs():
    spec = TozaraxConfig.from_json(tiny.CONFIGS["A"]).model_spec()
    needs = [registry.arrangement_class(l.kind).cache_need(l) for l in spec.layers]
    # layer 0: keys under a window of 13, the memory's filter rows (2 taps: 1 row of 2*2*10 + 4*14 channels) and its
    # state, and the two sublayers' last two inputs (3 taps)
    kv = needs[0][0]
    assert isinstance(kv, KVNeed) and kv.kv_heads == 2 and kv.window == 13
    assert needs[0][1:] == (StateNeed((1, 96), "compute"), StateNeed((4, 10, 14), "float32"),
                            StateNeed((2, 44), "compute"), StateNeed((2, 44), "compute"))
    # layer 1 has no feed-forward: one sublayer's rows only; its memory keeps 4 rows of 2*1*6 + 3*9 channels
    assert needs[1][1:] == (StateNeed((4, 39), "compute"), StateNeed((3, 6, 9), "float32"), StateNeed((2, 44), "compute"))
    assert registry.embedding_class("learned_position").cache_need(spec.embedding) is None
    # a frame filter of one tap keeps nothing
    one = TozaraxConfig.from_json(tiny.CONFIGS["B"]).model_spec()
    assert all(len(registry.arrangement_class(l.kind).cache_need(l)) == 3 for l in one.layers)
    Cache([n for n in needs], [None] * len(needs), 256, dtype=torch.float32, device="cpu")


@pytest.mark.parametrize("path,value,message", [
    (("layers", 0, "type"), "serial", "type"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "mask", "size"), 0, "size"),
    (("layers", 0, "mixer", "left", "scale"), None, "scale"),
    (("layers", 0, "mixer", "right", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "right", "conv"), 0, "conv"),
    (("layers", 0, "mixer", "right"), None, "right"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"),
    (("layers", 0, "mlp", "router", "top"), 7, "top"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "count"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 4, "keep"),
    (("layers", 2, "mlp", "router", "top"), 5, "kept groups"),
    (("canon", "taps"), 0, "taps"),
    (("canon",), None, "canon"),
    (("norm", "eps"), 0.0, "eps"),
    (("max_positions",), None, "max_positions"),
    (("width",), None, "width"),
    (("layers",), [], "layers"),
])
def test_refusals_name_their_key(path, value, message):
    cfg = copy.deepcopy(tiny.CONFIGS["A"])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        TozaraxConfig.from_json(cfg)


def test_tensor_names_and_random_weights_through_the_loader(tmp_path):
    c = TozaraxConfig.from_json(tiny.CONFIGS["A"])
    spec = c.model_spec()
    exp = expected_tensors(spec)
    assert exp["embed"].shape == (203, 44) and exp["pos"].shape == (512, 44) and exp["head"].shape == (203, 44)
    assert exp["final.norm"].shape == (44,)
    assert exp["l0.norm1"].shape == (44,) and exp["l0.canon1"].shape == (44, 3) and exp["l0.canon2"].shape == (44, 3)
    assert exp["l0.rg1"].shape == (44, 44) and exp["l0.rg1.b"].shape == (44,) and exp["l0.rg2.b"].shape == (44,)
    assert exp["l0.dwa"].shape == (2,) and exp["l1.dwa"].shape == (3,) and exp["l2.dwa"].shape == (4,)
    assert exp["l0.mix.left.q"].shape == (48, 44) and exp["l0.mix.left.k"].shape == (24, 44)
    assert exp["l0.mix.left.v"].shape == (40, 44) and exp["l0.mix.left.o"].shape == (44, 80)
    assert exp["l0.mix.left.out"].shape == (44,) and exp["l0.mix.right.out"].shape == (44,)
    assert exp["l0.mix.right.q"].shape == (20, 44) and exp["l0.mix.right.v"].shape == (56, 44)
    assert exp["l0.mix.right.q.conv"].shape == (20, 2) and exp["l0.mix.right.v.conv"].shape == (56, 2)
    assert exp["l0.mix.right.a"].shape == (4, 44) and exp["l0.mix.right.b"].shape == (4, 44)
    assert exp["l0.mix.right.A_log"].shape == (4,) and exp["l0.mix.right.dt_bias"].shape == (4,)
    assert exp["l0.mix.right.g"].shape == (56, 44) and exp["l0.mix.right.norm"].shape == (14,) and exp["l0.mix.right.o"].shape == (44, 56)
    assert exp["l0.mlp.router"].shape == (6, 44) and exp["l0.mlp.correction"].shape == (6,)
    assert exp["l0.mlp.e5.up"].shape == (20, 44) and exp["l0.mlp.e5.down"].shape == (44, 20) and "l0.mlp.e6.up" not in exp
    assert "l1.norm2" not in exp and "l1.canon2" not in exp and "l1.rg2" not in exp and "l1.mlp.router" not in exp
    folder = tiny.make_folder(tmp_path, "A", "bfloat16")
    w = load_weights(spec, folder)
    assert set(w) == set(exp) and w["pos"].dtype == torch.bfloat16 and w["l0.norm1"].dtype == torch.float32
    from xpu_serve_b200.weights.safetensors_io import WeightStore, write_safetensors
    st = WeightStore.open_dir(folder)
    tensors = [(n, st.get(n)) for n in st.names() if n != "l1.dwa"]
    os.makedirs(tmp_path / "broken")
    with open(os.path.join(folder, "config.json")) as f, open(tmp_path / "broken" / "config.json", "w") as g:
        g.write(f.read())
    write_safetensors(str(tmp_path / "broken" / "model.safetensors"), tensors)
    with pytest.raises(WeightError, match="l1.dwa"):
        load_weights(spec, str(tmp_path / "broken"))


# ------------------------------------------------------------------------------------------- the oracle's mechanisms
def test_oracle_filter_and_depth_average():
    x = np.arange(1.0, 11.0).reshape(5, 2)
    taps = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])          # channel 0: the current row; channel 1: two rows back
    y = plain.causal_filter(x, taps)
    assert np.array_equal(y[:, 0], x[:, 0])
    assert np.array_equal(y[:, 1], np.array([0.0, 0.0, x[0, 1], x[1, 1], x[2, 1]]))
    assert np.array_equal(plain.sublayer_input(x, taps)[:, 0], 2 * x[:, 0])
    one = plain.causal_filter(x, np.array([[3.0], [-1.0]]))      # one tap: no look back
    assert np.array_equal(one, x * np.array([3.0, -1.0]))
    h = [np.full((2, 3), 1.0), np.full((2, 3), 10.0), np.full((2, 3), 100.0)]
    assert np.allclose(plain.depth_average(h, np.array([0.5, -1.0, 2.0])), 190.5)


def test_oracle_window_edge():
    """A value planted at one position is seen by the queries of the next `size` positions and by none later."""
    rng = np.random.default_rng(5)
    W, D, Dv, T, size = 6, 4, 3, 12, 5
    m = {"heads": 2, "kv_heads": 1, "dim": D, "vdim": Dv, "mask": {"size": size}, "scale": 0.5}
    w = {"q": rng.standard_normal((2 * D, W)), "k": rng.standard_normal((D, W)), "v": np.zeros((Dv, W)), "o": np.eye(W, 2 * Dv)}
    w["v"][:, 0] = 1.0                                           # the value is the input's first channel
    x = rng.standard_normal((T, W))
    x[:, 0] = 0.0
    x[3, 0] = 1.0
    y = plain.window_attention(m, w, "", x)
    seen = np.abs(y).sum(-1) > 0
    assert list(np.nonzero(seen)[0]) == [3, 4, 5, 6, 7]


def test_oracle_delta_rule_against_its_matrix_form():
    """Without decay the memory after the tokens is prod (I - beta k k^T) applied in order plus the writes; with one token it is
    beta k v^T, and a second write along the same unit key replaces beta of what is there."""
    D, Dv = 3, 2
    k = np.array([[1.0, 0.0, 0.0], [1.0, 0.0, 0.0], [0.0, 1.0, 0.0]])
    v = np.array([[2.0, 4.0], [10.0, 20.0], [1.0, 1.0]])
    q = np.array([[1.0, 0.0, 0.0], [1.0, 0.0, 0.0], [1.0, 1.0, 0.0]])
    beta = np.array([1.0, 0.5, 1.0])
    o, S = plain.delta_memory(q, k, v, np.ones(3), beta)
    assert np.allclose(o[0], [2.0, 4.0])                          # the read-out sees the token's own write
    assert np.allclose(o[1], [6.0, 12.0])                         # half way from (2, 4) to (10, 20)
    assert np.allclose(o[2], [7.0, 13.0]) and np.allclose(S[2], 0.0)
    o2, S2 = plain.delta_memory(q, k, v, np.array([1.0, 0.5, 1.0]), beta)
    assert np.allclose(o2[1], 0.5 * np.array([1.0, 2.0]) + 0.5 * np.array([10.0, 20.0]))   # the decay comes before the write
    # a state carried over equals the whole in one go
    o3, S3 = plain.delta_memory(q[:2], k[:2], v[:2], np.ones(2), beta[:2])
    o4, S4 = plain.delta_memory(q[2:], k[2:], v[2:], np.ones(1), beta[2:], S3)
    assert np.allclose(np.concatenate([o3, o4]), o) and np.allclose(S4, S)


def test_oracle_router():
    """Groups are scored by their two best corrected scores; closed groups cannot be chosen although their scores are higher
    than an open one's negative ones; the weights are the plain sigmoids."""
    z = np.array([[4.0, -9.0, 3.0, 3.0, -9.0, -9.0]])            # groups of 2: (0.98, ~0), (0.95, 0.95), (~0, ~0)
    corr = np.zeros(6)
    ids, wt = plain.route(z, corr, 2, 3, 1)
    assert sorted(ids[0]) == [2, 3] and np.allclose(wt[0], 1 / (1 + np.exp(-3.0)))
    ids, wt = plain.route(z, corr, 2, 3, 2)
    assert sorted(ids[0]) == [0, 2]                               # ties go to the lower index
    corr = np.array([0.0, 0.0, -5.0, -5.0, -3.0, -3.0])           # the correction closes group 1 and 2
    ids, wt = plain.route(z, corr, 2, 3, 1)
    assert sorted(ids[0]) == [0, 1] and np.allclose(sorted(wt[0]), sorted(1 / (1 + np.exp(-z[0, :2]))))
    # open units with negative choice scores still beat closed ones
    corr = np.array([-2.0, -2.5, -4.0, -4.0, -1.9, -9.0])
    ids, _ = plain.route(np.zeros((1, 6)), corr, 2, 3, 1)
    assert sorted(ids[0]) == [0, 1]


def test_the_command_line_writes_and_describes_a_model(tmp_path, capsys):
    """`random` with a Tozarax config.json, then `info`: the architecture is found by the file's own key, and the count
    of parameters is the sum over the tensors the parts declare."""
    import json
    from xpu_serve_b200.cli.main import main
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny.CONFIGS["C"]))
    out = str(tmp_path / "model")
    assert main(["random", out, "--config", str(cfg_path), "--seed", "3", "--dtype", "bfloat16"]) == 0
    assert capsys.readouterr().out.strip() == out
    assert main(["info", out]) == 0
    info = json.loads(capsys.readouterr().out)
    spec = TozaraxConfig.from_json(tiny.CONFIGS["C"]).model_spec()
    assert info["architecture"] == "tozarax" and info["layers"] == 3 and info["vocab"] == 180 and not info["tied_head"]
    assert info["mixers"] == ["parallel"] * 3
    assert info["parameters"] == sum(int(np.prod(ts.shape)) for ts in expected_tensors(spec).values())
    assert TozaraxConfig.from_json(json.loads(open(os.path.join(out, "config.json")).read())).to_json() == tiny.CONFIGS["C"]
