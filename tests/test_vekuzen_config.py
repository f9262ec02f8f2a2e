"""Vekuzen without a GPU: the configuration's keys and refusals, the running order of repeated layers, what each call keeps
per sequence, tensor names and shapes, random weights through the loader, and the plain implementation's own mechanisms
against hand-made cases."""
import copy

import numpy as np
import pytest

import plain_vekuzen as plain
import tiny_vekuzen as tiny
from plain_lfm3 import load_folder
from xpu_serve_b200 import registry
from xpu_serve_b200.config import ConfigError, VekuzenConfig
from xpu_serve_b200.parts.base import KVNeed, StateNeed
from xpu_serve_b200.weights.expected import expected_tensors
from xpu_serve_b200.weights.loader import load_weights
from xpu_serve_b200.weights.safetensors_io import WeightError


def test_the_registry_finds_the_design():
    arch = registry.architecture_for(tiny.CONFIGS["A"])
    assert arch.config_class is VekuzenConfig
    assert "vekuzen" in registry.supported_architectures()


@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_configuration_round_trip(name):
    cfg = VekuzenConfig.from_json(tiny.CONFIGS[name])
    assert cfg.to_json() == tiny.CONFIGS[name]
    spec = cfg.model_spec()
    assert len(spec.order) == tiny.layer_runs(name)
    assert [c.layer for c in spec.order] == [i for i, _ in plain.running_order(tiny.CONFIGS[name])]
    assert [c.mix_in for c in spec.order] == [f for _, f in plain.running_order(tiny.CONFIGS[name])]


def test_every_constant_comes_from_the_file():
    cfg = VekuzenConfig.from_json(tiny.CONFIGS["A"])
    spec = cfg.model_spec()
    assert spec.logit_scale == 0.7 and spec.embedding.scale == 1.5 and spec.final_norm.eps == 3e-6
    l0, l1, l2, l3 = spec.layers
    assert (l0.mixer.kind, l0.mixer.q_rank, l0.mixer.kv_rank, l0.mixer.rot_dim, l0.mixer.scale) == ("latent_attention", 9, 20, 0, 0.31)
    assert l0.mixer.out_gate and not l0.mixer.head_gate and l0.mixer.position is None and l0.mixer.window == 0
    assert (l1.mixer.kind, l1.mixer.decay) == ("lightning", (0.5, 0.9, 0.97))
    assert (l0.ffn.kind, l0.ffn.activation, l0.ffn.intermediate) == ("swiglu", "gelu_tanh", 50)
    assert (l1.ffn.score, l1.ffn.identity, l1.ffn.top, l1.ffn.route_scale, l1.ffn.correction) == ("softmax_all", 1, 2, 1.7, True)
    assert l1.ffn.shared.intermediate == 12 and l1.ffn.shared.activation == "silu" and l3.ffn.shared is None
    assert l2.ffn is None and l3.ffn.identity == 3
    assert [l.token_side.offset for l in spec.layers] == [0, 5, 10, 15] and l0.token_side.columns == 20
    assert VekuzenConfig.from_json(tiny.CONFIGS["C"]).model_spec().layers[0].token_side is None


def _broken(path, value, name="A"):
    cfg = copy.deepcopy(tiny.CONFIGS[name])
    node = cfg
    for key in path[:-1]:
        node = node[key]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,word", [
    (("width",), KeyError, "width"), (("norm",), KeyError, "norm"), (("norm", "eps"), 0.0, "positive"),
    (("embedding",), KeyError, "embedding"), (("logit_scale",), -1.0, "logit_scale"),
    (("layers", 0, "type"), "conv", "unknown layer type"), (("layers", 1, "mixer", "decay"), [0.5, 0.9], "decay"),
    (("layers", 1, "mixer", "decay"), [0.5, 0.9, 1.5], "decay"), (("layers", 0, "mixer", "q_rank"), 0, "positive"),
    (("layers", 0, "mixer", "scale"), KeyError, "scale"), (("layers", 0, "mlp", "kind"), "gated", "unknown feed-forward"),
    (("layers", 1, "mlp", "router", "top"), 7, "router.top"), (("layers", 1, "mlp", "expert"), KeyError, "expert"),
    (("layers", 1, "mlp", "shared", "ff"), 0, "positive"), (("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "loop"),
    (("token_side", "dim"), 0, "dim"), (("layers",), [], "layers"),
])
def test_refusals_name_their_key(path, value, word):
    with pytest.raises(ConfigError) as e:
        VekuzenConfig.from_json(_broken(path, value))
    assert word in str(e.value)


def test_what_each_call_keeps():
    """A call of a memory layer keeps a float32 state, a call of an attention layer one vector a position; a layer that runs
    several times has as many caches of its own."""
    spec = VekuzenConfig.from_json(tiny.CONFIGS["A"]).model_spec()
    needs = [registry.arrangement_class(spec.layers[c.layer].kind).cache_need(spec.layers[c.layer]) for c in spec.order]
    assert [type(n) for n in needs] == [KVNeed, StateNeed, KVNeed, StateNeed, KVNeed, StateNeed]
    assert needs[0] == KVNeed(1, 20, 0, planes=1) and needs[2] == KVNeed(1, 28, 0, planes=1)
    assert needs[1] == StateNeed((3, 10, 14), "float32") and needs[5] == StateNeed((2, 20, 37), "float32")
    assert all(c.cache_of is None for c in spec.order)


def test_tensor_names_and_shapes():
    spec = VekuzenConfig.from_json(tiny.CONFIGS["A"]).model_spec()
    t = {k: v.shape for k, v in expected_tensors(spec).items()}
    assert t["embed"] == (203, 44) and t["pos"] == (512, 44) and t["head"] == (203, 44) and t["final.norm"] == (44,)
    assert t["loop.in"] == (44, 88) and t["side.embed"] == (203, 20)
    assert t["l0.mix.dq"] == (9, 44) and t["l0.mix.dq.norm"] == (9,) and t["l0.mix.uq"] == (36, 9)
    assert t["l0.mix.dkv"] == (20, 44) and t["l0.mix.uk"] == (36, 20) and t["l0.mix.uv"] == (60, 20)
    assert t["l0.mix.g"] == (60, 44) and t["l0.mix.o"] == (44, 60) and "l0.mix.q" not in t
    assert t["l1.mix.q"] == (30, 44) and t["l1.mix.v"] == (42, 44) and t["l1.mix.norm"] == (42,) and t["l1.mix.o"] == (44, 42)
    assert t["l1.mlp.router"] == (6, 44) and t["l1.mlp.correction"] == (6,) and t["l1.mlp.e4.down"] == (44, 20) and "l1.mlp.e5.up" not in t
    assert t["l1.mlp.shared.sg"] == (1, 44) and t["l1.mlp.shared.gate"] == (12, 44)
    assert t["l3.mlp.router"] == (7, 44) and "l3.mlp.shared.sg" not in t
    assert "l2.norm2" not in t and t["l2.side.gate"] == (5, 44) and t["l2.side.proj"] == (44, 5) and t["l2.side.norm"] == (44,)
    c = {k: v.shape for k, v in expected_tensors(VekuzenConfig.from_json(tiny.CONFIGS["C"]).model_spec()).items()}
    assert "loop.in" not in c and "side.embed" not in c and not any(".side." in k for k in c)


def test_random_weights_through_the_loader(tmp_path):
    folder = tiny.make_folder(tmp_path, "A", "bfloat16")
    cfg, W = load_folder(folder)
    assert cfg == tiny.CONFIGS["A"]
    spec = VekuzenConfig.from_json(cfg).model_spec()
    weights = load_weights(spec, folder)
    assert set(weights) == set(expected_tensors(spec))
    # a missing tensor is named; a layer without a feed-forward may carry the norm of one
    import os
    from xpu_serve_b200.weights.safetensors_io import WeightStore, write_safetensors
    st = WeightStore.open_dir(folder)
    every = {n: st.get(n).clone() for n in st.names()}
    del st
    os.remove(os.path.join(folder, "model.safetensors"))
    write_safetensors(os.path.join(folder, "model.safetensors"), [(n, t) for n, t in every.items() if n != "loop.in"] +
                      [("l2.norm2", every["l1.norm2"])])
    with pytest.raises(WeightError) as e:
        load_weights(spec, folder)
    assert "loop.in" in str(e.value) and "l2.norm2" not in str(e.value)


# --------------------------------------------------------------------------- the plain implementation's own mechanisms
def test_plain_memory_by_hand():
    """Two tokens, one head: S1 = k1 v1^T, o1 = (k1 . q1) v1; S2 = d S1 + k2 v2^T."""
    q = np.array([[1.0, 2.0], [0.5, -1.0]])
    k = np.array([[3.0, 1.0], [2.0, 2.0]])
    v = np.array([[1.0, 10.0, 100.0], [2.0, 0.0, -1.0]])
    o, S = plain.decayed_memory(q, k, v, 0.5)
    assert np.allclose(o[0], 5.0 * v[0])
    assert np.allclose(o[1], 0.5 * (k[0] @ q[1]) * v[0] + (k[1] @ q[1]) * v[1])
    assert np.allclose(S, 0.5 * np.outer(k[0], v[0]) + np.outer(k[1], v[1]))
    o2, S2 = plain.decayed_memory(q[1:], k[1:], v[1:], 0.5, state=np.outer(k[0], v[0]))
    assert np.allclose(o2[0], o[1]) and np.allclose(S2, S)


def test_plain_routing_by_hand():
    z = np.log(np.array([[0.1, 0.2, 0.3, 0.4]]))
    ids, w = plain.route(z, np.array([0.5, 0.0, 0.0, 0.0]), 2, 3.0)
    assert list(ids[0]) == [0, 3] and np.allclose(w[0], [0.3, 1.2])           # chosen with the correction, weighted without
    ids, _ = plain.route(np.zeros((1, 4)), np.zeros(4), 2, 1.0)
    assert list(ids[0]) == [0, 1]                                              # ties go to the lower index
    assert np.isclose(plain.route_margin(z, np.zeros(4), 2)[0], 0.1)


def test_plain_pass_through_outputs_and_shared_unit():
    """An output behind the experts' hands the input through, times its weight; the shared unit is gated per token."""
    rng = np.random.default_rng(0)
    Wd = 6
    f = {"kind": "moe", "expert": {"ff": 4}, "router": {"experts": 1, "identity": 1, "top": 1, "scale": 2.0}}
    w = {"router": np.array([[0.0] * Wd, [0.0] * Wd]), "correction": np.array([0.0, 1.0]),
         "e0.gate": rng.standard_normal((4, Wd)), "e0.up": rng.standard_normal((4, Wd)), "e0.down": rng.standard_normal((Wd, 4))}
    x = rng.standard_normal((3, Wd))
    assert np.allclose(plain.routed_units(f, w, "", x), 2.0 * 0.5 * x)         # both scores are 1/2; the correction picks output 1
    w["correction"] = np.array([1.0, 0.0])
    assert np.allclose(plain.routed_units(f, w, "", x), 2.0 * 0.5 * plain.gated_unit(w, "e0.", x, plain.silu))


def test_plain_running_order_and_first_tokens():
    order = plain.running_order(tiny.CONFIGS["B"])
    assert order == [(0, False), (1, True), (1, True), (1, True), (2, False), (3, False)]
    assert plain.running_order(tiny.CONFIGS["C"]) == [(0, False), (1, False), (2, False)]
    # logits of a prefix do not depend on what follows
    import tempfile
    folder = tiny.make_folder(tempfile.mkdtemp(), "whole_loop", "float32")
    cfg, W = load_folder(folder)
    toks = tiny.prompt("whole_loop", 9)
    assert np.allclose(plain.forward(cfg, W, toks)[:4], plain.forward(cfg, W, toks[:4]))
    streams = []
    plain.forward(cfg, W, toks, streams)
    assert len(streams) == 6


def test_the_bench_stacks_are_valid_configurations():
    """`bench.py --workload vekuzen`: every stack and the stack beside it parse, at equal width and vocabulary."""
    import bench
    for name in bench.VEKUZEN_STACKS:
        ours, (label, beside) = bench.vekuzen_stack_configs(name)
        a, b = ours.model_spec(), beside.model_spec()
        assert isinstance(ours, VekuzenConfig) and label in ("saralix", "nimelorn")
        assert (a.hidden, a.vocab, len(a.layers)) == (b.hidden, b.vocab, len(b.layers)) == (2048, 32768, 2)
