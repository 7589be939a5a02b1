"""The Kuvelix configuration on the CPU: keys read and defaults, refusals that name the key, the spec it builds (a
run of layers that repeats becomes schedule entries of the same layers, one norm per layer, tensor names, parts), the
random folder, a cache entry per layer run, and the plain statement's pieces against hand-worked numbers."""
import json
import math

import pytest
import torch

from inference_engine_rust_b200.config import ConfigError, config_from_dict, preset, spec_of
from inference_engine_rust_b200.engine.model import Model
from inference_engine_rust_b200.parts.base import Runtime
from plain import kuvelix_plain as P

ATT = {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "rot": {"base": 1000.0, "dims": 8, "scaling": {"factor": 2.0}}}
MOE = {"kind": "moe", "expert": {"ff": 20, "limit": 2.5},
       "router": {"experts": 5, "identity": 3, "top": 3, "groups": {"count": 4, "keep": 2}}}


def cfg(layers=None, **top):
    layers = layers if layers is not None else [
        {"type": "attention", "mixer": ATT, "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention", "mixer": ATT, "mlp": MOE},
        {"type": "attention", "mixer": dict(ATT, vdim=None, rot=None), "mlp": None}]
    d = {"architecture": "Kuvelix", "vocab": 90, "width": 56, "norm": {"eps": 1e-6}, "loop": {"start": 1, "stop": 3, "times": 2},
         "layers": json.loads(json.dumps(layers))}
    d.update(top)
    return d


def test_spec_of_a_configuration():
    c = config_from_dict(cfg())
    spec = spec_of(c)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2] and len(spec.layers) == 3
    assert all(e.writes_cache for e in spec.schedule)
    assert spec.head.kind == "linear" and spec.lm_head_name is None and spec.inputs[0][0].kind == "embed_norm"
    assert spec.layers[0].block.kind == "shared_norm" and spec.layers[0].ffn_norm_name == ""
    a = spec.layers[0].mixer
    assert a.kind == "gated_attention" and a["qk_norm"] == "head" and a["bias"] and a["gate"] and a["v_dim"] == 24
    assert a["position"]["freq_factors"] == [2.0] * 4 and a["position"]["rotary_dim"] == 8 and a["position"]["pairing"] == "interleaved"
    assert spec.layers[2].mixer["v_dim"] == 16 and spec.layers[2].mixer["position"]["rotary_dim"] == 0
    f = spec.layers[0].ffn
    assert f.kind == "swiglu" and f["activation"] == "gelu_tanh"
    m = spec.layers[1].ffn
    assert m.kind == "grouped_moe" and (m["experts"], m["identity"], m["top"], m["groups"], m["keep"]) == (5, 3, 3, 4, 2)
    assert m["activation"] == "clamped_swish" and m["limit"] == 2.5 and spec.layers[2].ffn is None
    model = Model(spec, Runtime(dtype=torch.float32, device="cpu"))
    shapes = {k: tuple(v.shape) for k, v in model.expected_tensors().items()}
    mix = {f"l{i}.mix.{n}" for i in range(3) for n in ("q", "q.b", "k", "k.b", "v", "v.b", "q.norm", "k.norm", "g", "o")}
    experts = {f"l1.mlp.e{e}.{n}" for e in range(5) for n in ("gate", "up", "down")}
    assert set(shapes) == mix | experts | {"embed", "embed.norm", "final.norm", "l0.norm1", "l1.norm1", "l2.norm1", "l0.mlp.gate",
                                           "l0.mlp.up", "l0.mlp.down", "l1.mlp.router", "l1.mlp.correction"}
    assert shapes["l1.mlp.router"] == (8, 56) and shapes["l1.mlp.correction"] == (8,) and shapes["l1.mlp.e4.down"] == (56, 20)
    assert shapes["l0.mix.q"] == (96, 56) and shapes["l0.mix.v"] == (48, 56) and shapes["l0.mix.v.b"] == (48,)
    assert shapes["l0.mix.g"] == (144, 56) and shapes["l0.mix.o"] == (56, 144) and shapes["l0.mix.k.norm"] == (16,)
    assert shapes["l2.mix.o"] == (56, 96)
    # a cache entry for every layer RUN
    reqs = model.cache_requests()
    assert sorted(reqs) == [0, 1, 2, 3, 4] and reqs[1].head_dim == 24 and reqs[1].kv_heads == 2 and reqs[4].head_dim == 16
    assert config_from_dict(c.to_dict()) == c


def test_loops_and_defaults():
    assert config_from_dict(cfg(loop=None)).runs() == (0, 1, 2)
    assert config_from_dict(cfg(loop={"start": 0, "stop": 3, "times": 3})).runs() == (0, 1, 2) * 3
    assert config_from_dict(cfg(loop={"start": 2, "stop": 2, "times": 5})).runs() == (0, 1, 2)
    assert config_from_dict(cfg(loop={"start": 0, "stop": 1, "times": 1})).runs() == (0, 1, 2)
    assert config_from_dict(cfg(loop={"start": 1, "stop": 2, "times": 3})).runs() == (0, 1, 1, 1, 2)
    raw = cfg()
    del raw["layers"][1]["mlp"]["router"]["groups"], raw["layers"][1]["mlp"]["router"]["identity"]
    r = config_from_dict(raw).layers[1]["mlp"]["router"]
    assert r["groups"] == {"count": 1, "keep": 1} and r["identity"] == 0


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "mixer", "kv_heads"), 4, "kv_heads"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "rot.dims"), (("layers", 1, "type"), "mlstm", "type"),
    (("layers", 0, "mlp", "kind"), "sparse", "kind"), (("norm",), None, "eps"), (("layers", 0, "mixer", "scale"), None, "scale"),
    (("layers", 1, "mlp", "router", "top"), 5, "top"), (("layers", 1, "mlp", "router", "groups", "count"), 3, "groups"),
    (("layers", 1, "mlp", "expert", "ff"), None, "ff"), (("loop", "stop"), 4, "loop"), (("loop", "times"), 0, "times"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 5, "groups"),
])
def test_refusals_name_the_key(path, value, word):
    raw = cfg()
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_presets_and_random_folder(tmp_path):
    from inference_engine_rust_b200 import write_random_model
    from inference_engine_rust_b200.weights import TensorSource
    for name in ("kuvelix-tiny", "kuvelix-7b-sizes"):
        spec_of(config_from_dict(preset(name)))
    d = str(tmp_path / "m")
    write_random_model(d, preset("kuvelix-tiny"), seed=3)
    names = set(TensorSource(d).names())
    assert {"embed.norm", "l1.mlp.correction", "l0.mlp.gate", "l3.mix.g"} <= names and "l0.norm2" not in names and "head" not in names


def test_the_plain_pieces_by_hand():
    # rotation of pairs (2i, 2i+1): two pairs turn, the rest of the head passes
    v = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]]]).repeat(3, 1, 1)
    out = P.rotate_pairs(v, 4, 100.0, 2.0)
    for p in range(3):
        a0, a1 = p * 1.0 / 2.0, p * 100.0 ** -0.5 / 2.0
        want = [math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 5.0, 6.0]
        assert torch.allclose(out[p, 0], torch.tensor(want), atol=1e-6)
    # the router: softmax over everything, the choice on score + correction inside the best group, weights from the scores
    z = torch.log(torch.tensor([[0.1, 0.2, 0.3, 0.4]]))
    idx, w = P.route(z, torch.tensor([0.5, 0.0, 0.0, 0.0]), top=2, groups=2, keep=1)
    assert idx.tolist() == [[0, 1]] and torch.allclose(w, torch.tensor([[1 / 3, 2 / 3]]), atol=1e-6)
    idx, w = P.route(z, torch.tensor([-9.0, -9.0, -9.5, -9.5]), top=1, groups=2, keep=1)      # negative choice scores
    assert idx.tolist() == [[1]] and torch.allclose(w, torch.ones(1, 1))
    # the activations
    assert abs(float(P.gelu_tanh(torch.tensor(1.0))) - 0.841192) < 1e-5
    one = torch.ones(1, 1)
    y = P.clamped_expert(torch.tensor([[1.0]]), 3.0 * one, -5.0 * one, one, limit=2.0)
    assert abs(float(y) - 2.0 / (1.0 + math.exp(-3.404)) * (-2.0 + 1.0)) < 1e-6
    # a layer that runs twice
    assert P.layer_runs({"layers": [0, 0, 0], "loop": {"start": 0, "stop": 2, "times": 2}}) == [0, 1, 0, 1, 2]
