"""The Vufinex configuration on the CPU: keys read and defaults, refusals that name the key, the spec it builds (layers
that run with another layer's weights become schedule entries of the owner, tensor names, parts and their constants),
the random folder, a cache or state entry per layer, a tensor axis whose size the stored tensor decides, and the plain
statement's pieces against hand-worked numbers."""
import json
import math

import pytest
import torch

from inference_engine_rust_b200.cache import KVRequest, StateRequest
from inference_engine_rust_b200.config import ConfigError, config_from_dict, preset, spec_of
from inference_engine_rust_b200.engine.model import Model
from inference_engine_rust_b200.parts.base import Runtime
from inference_engine_rust_b200.weights.loader import TensorSpec, WeightError, check_source
from plain import vufinex_plain as P

ATT = {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "mask": {"size": 40}, "rot": {"base": 1000.0, "dims": 8}}
WKV = {"heads": 3, "dim": 8}
LAT = {"heads": 5, "dim": 12, "rot_dim": 4, "vdim": 20, "kv_rank": 24, "scale": 0.25, "rot": {"base": 500.0, "dims": 4}}
MOE = {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 6, "top": 3, "scale": 2.5, "groups": {"count": 3, "keep": 2}}}


def cfg(layers=None, **top):
    layers = layers if layers is not None else [
        {"type": "attention", "mixer": ATT, "mlp": MOE},
        {"type": "wkv", "mixer": WKV, "mlp": None},
        {"type": "latent_attention", "mixer": LAT, "mlp": MOE},
        {"type": "attention", "mixer": ATT, "mlp": MOE, "weights_of": 0}]
    d = {"architecture": "Vufinex", "vocab": 90, "width": 56, "norm": {"eps": 1e-6}, "residual_mult": 0.7,
         "embedding": {"scale": 5.0}, "layers": json.loads(json.dumps(layers))}
    d.update(top)
    return d


def test_spec_of_a_configuration():
    c = config_from_dict(cfg())
    spec = spec_of(c)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 0] and len(spec.layers) == 3
    assert spec.embedding_scale == 5.0 and spec.lm_head_name == "head" and spec.head.kind == "linear"
    assert spec.layers[0].block.kind == "prenorm" and spec.layers[0].norm["offset"] == 1.0
    a = spec.layers[0].mixer
    assert a.kind == "tied_kv_attention" and a["chunk"] == 40 and a["window"] is None and a["qk_norm"] is None
    assert a["out_scale"] == 0.7 and a["position"]["rotary_dim"] == 8 and a["position"]["pairing"] == "half"
    w = spec.layers[1].mixer
    assert w.kind == "wkv" and (w["heads"], w["dim"], w["out_scale"]) == (3, 8, 0.7) and spec.layers[1].ffn is None
    m = spec.layers[2].mixer
    assert m.kind == "latent_attention" and m["q_rank"] is None and m["rot_dim"] == 4 and m["gate"] == "head" and not m["sink"]
    assert m["position"]["pairing"] == "interleaved" and m["position"]["rotary_dim"] == 4
    f = spec.layers[0].ffn
    assert f.kind == "grouped_moe" and f["score"] == "sigmoid" and f["group_score"] == "top2_sum"
    assert (f["experts"], f["top"], f["groups"], f["keep"], f["route_scale"], f["out_scale"]) == (6, 3, 3, 2, 2.5, 0.7)
    model = Model(spec, Runtime(dtype=torch.float32, device="cpu"))
    specs = model.expected_tensors()
    shapes = {k: tuple(v.shape) for k, v in specs.items()}
    experts = {f"l{i}.mlp.e{e}.{n}" for i in (0, 2) for e in range(6) for n in ("gate", "up", "down")}
    names = ({"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l1.norm1", "l2.norm1", "l2.norm2"} | experts
             | {f"l{i}.mlp.{n}" for i in (0, 2) for n in ("router", "correction")}
             | {f"l0.mix.{n}" for n in ("q", "k", "o")}
             | {f"l1.mix.{n}" for n in ("mu.r", "mu.k", "mu.v", "mu.g", "mu.w", "r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
             | {f"l2.mix.{n}" for n in ("q", "dkv", "dkv.norm", "uk", "uv", "g", "o")})
    assert set(shapes) == names
    assert shapes["l0.mix.q"] == (96, 56) and shapes["l0.mix.k"] == (32, 56) and shapes["l0.mix.o"] == (56, 96)
    assert shapes["l1.mix.r"] == (24, 56) and shapes["l1.mix.u"] == (3, 8) and shapes["l1.mix.w0"] == (24,)
    assert specs["l1.mix.w1"].free_dims == (0,) and specs["l1.mix.w2"].free_dims == (1,)
    assert shapes["l2.mix.q"] == (80, 56) and shapes["l2.mix.dkv"] == (28, 56) and shapes["l2.mix.dkv.norm"] == (24,)
    assert shapes["l2.mix.uk"] == (60, 24) and shapes["l2.mix.uv"] == (100, 24) and shapes["l2.mix.g"] == (5, 56)
    assert shapes["l2.mix.o"] == (56, 100) and shapes["l0.mlp.router"] == (6, 56) and shapes["l0.mlp.correction"] == (6,)
    # a cache or state entry for every layer, also for the one that borrows its weights
    reqs = model.cache_requests()
    assert sorted(reqs) == [0, 1, 2, 3]
    assert reqs[0] == reqs[3] == KVRequest(2, 16, None, chunk=40) and reqs[0].reach == 40
    assert reqs[1] == StateRequest((3 * 8 * 8 + 56,), torch.float32)
    assert reqs[2] == KVRequest(1, 28, None, values=False)
    assert config_from_dict(c.to_dict()) == c


def test_defaults():
    raw = cfg()
    del raw["residual_mult"], raw["embedding"], raw["layers"][0]["mlp"]["router"]["groups"], raw["layers"][0]["mlp"]["router"]["scale"]
    del raw["layers"][0]["mixer"]["mask"], raw["layers"][0]["mixer"]["rot"]
    raw["layers"][3]["mixer"] = json.loads(json.dumps(raw["layers"][0]["mixer"]))
    raw["layers"][1]["mixer"]["decay_rank"] = 12
    c = config_from_dict(raw)
    assert c.residual_mult == 1.0 and c.embedding_scale == 1.0
    assert c.layers[0]["mlp"]["router"]["groups"] == {"count": 1, "keep": 1} and c.layers[0]["mlp"]["router"]["scale"] == 1.0
    spec = spec_of(c)
    assert spec.layers[0].mixer["chunk"] is None and spec.layers[0].mixer["position"]["rotary_dim"] == 0
    model = Model(spec, Runtime(dtype=torch.float32, device="cpu"))
    assert model.expected_tensors()["l1.mix.w1"].shape == (12, 56) and model.expected_tensors()["l1.mix.w1"].free_dims == ()


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "mixer", "kv_heads"), 4, "kv_heads"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "rot.dims"), (("layers", 1, "type"), "mlstm", "type"),
    (("layers", 0, "mixer", "vdim"), 24, "vdim"), (("layers", 0, "mixer", "mask", "size"), 0, "size"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"), (("norm",), None, "eps"), (("layers", 0, "mixer", "scale"), None, "scale"),
    (("layers", 0, "mlp", "router", "top"), 5, "top"), (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 0, "mlp", "expert", "ff"), None, "ff"), (("layers", 0, "mlp", "router", "groups", "keep"), 5, "groups"),
    (("layers", 2, "mixer", "rot", "dims"), 2, "rot_dim"), (("layers", 2, "mixer", "rot_dim"), 3, "rot_dim"),
    (("layers", 2, "mixer", "kv_rank"), None, "kv_rank"), (("layers", 1, "mixer", "dim"), 0, "dim"),
    (("layers", 3, "weights_of"), 3, "weights_of"), (("layers", 3, "weights_of"), 1, "weights"), (("layers", 3, "weights_of"), 9, "weights_of"),
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


def test_weights_that_go_round_in_a_circle_are_refused():
    raw = cfg()
    raw["layers"][0]["weights_of"] = 3
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert "circle" in str(e.value)


def test_presets_and_random_folder(tmp_path):
    from inference_engine_rust_b200 import write_random_model
    from inference_engine_rust_b200.weights import TensorSource
    for name in ("vufinex-tiny", "vufinex-7b-sizes", "vufinex-12b-sizes"):
        spec_of(config_from_dict(preset(name)))
    d = str(tmp_path / "m")
    write_random_model(d, preset("vufinex-tiny"), seed=3)
    src = TensorSource(d)
    names = set(src.names())
    assert {"head", "l1.mix.mu.w", "l1.mix.w2", "l3.mix.dkv.norm", "l0.mlp.correction", "l2.norm2"} <= names
    assert not any(n.startswith(("l4.", "l5.", "l6.", "l7.")) for n in names)
    assert tuple(src.describe("l1.mix.w1")[1]) == (8, 96)


def test_an_axis_that_the_stored_tensor_decides():
    class Source:
        def __init__(self, shapes):
            self.shapes = shapes

        def names(self):
            return list(self.shapes)

        def describe(self, name):
            return "F32", self.shapes[name]
    expected = {"a": TensorSpec((8, 5), free_dims=(0,)), "b": TensorSpec((4, 8), free_dims=(1,)), "c": TensorSpec((3,))}
    assert check_source(expected, Source({"a": (2, 5), "b": (4, 31), "c": (3,)}), "t") == []
    for bad in ({"a": (2, 6), "b": (4, 8), "c": (3,)}, {"a": (8, 5), "b": (5, 8), "c": (3,)}, {"a": (8, 5), "b": (4, 8), "c": (4,)},
                {"a": (8, 5, 1), "b": (4, 8), "c": (3,)}):
        with pytest.raises(WeightError):
            check_source(expected, Source(bad), "t")


def test_the_plain_pieces_by_hand():
    # rotation of halves (i, i + dims/2) and of neighbours (2i, 2i+1): two pairs turn, the rest of the head passes
    v = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]]]).repeat(3, 1, 1)
    halves, pairs = P.rotate_halves(v, 4, 100.0), P.rotate_neighbours(v, 4, 100.0)
    for p in range(3):
        a0, a1 = p * 1.0, p * 100.0 ** -0.5
        want = [math.cos(a0), -2 * math.sin(a1), math.sin(a0), 2 * math.cos(a1), 5.0, 6.0]
        assert torch.allclose(halves[p, 0], torch.tensor(want), atol=1e-6)
        want = [math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 5.0, 6.0]
        assert torch.allclose(pairs[p, 0], torch.tensor(want), atol=1e-6)
    # chunks are counted from the start of the sequence
    sees = P.chunk_rule(4)
    assert [j for j in range(8) if sees(5, j)] == [4, 5] and [j for j in range(8) if sees(3, j)] == [0, 1, 2, 3]
    assert [j for j in range(8) if P.chunk_rule(None)(5, j)] == [0, 1, 2, 3, 4, 5]
    # the router: a sigmoid each, groups judged by the sum of their two best choice scores, weights from the bare scores
    z = torch.logit(torch.tensor([[0.9, 0.1, 0.6, 0.5]]))
    idx, w = P.route(z, torch.zeros(4), top=2, groups=2, keep=1, scale=3.0)          # 0.9 + 0.1 < 0.6 + 0.5
    assert idx.tolist() == [[2, 3]] and torch.allclose(w, torch.tensor([[0.6 / 1.1, 0.5 / 1.1]]) * 3.0, atol=1e-5)
    idx, w = P.route(z, torch.tensor([0.0, 0.2, 0.0, 0.0]), top=2, groups=2, keep=1, scale=1.0)      # the correction decides the group
    assert idx.tolist() == [[0, 1]] and torch.allclose(w, torch.tensor([[0.9, 0.1]]), atol=1e-5)
    idx, w = P.route(z, torch.full((4,), -9.0), top=1, groups=2, keep=1, scale=1.0)                     # negative choice scores
    assert idx.tolist() == [[2]] and torch.allclose(w, torch.ones(1, 1), atol=1e-5)
    # the recurrence: one head of one channel, by hand
    w1 = {"mu." + n: torch.zeros(1) for n in "rkvgw"}
    w1.update({"r": torch.tensor([[2.0]]), "k": torch.tensor([[1.0]]), "v": torch.tensor([[3.0]]), "g": torch.tensor([[1.0]]),
               "w1": torch.zeros(1, 1), "w2": torch.zeros(1, 1), "w0": torch.tensor([0.0]), "u": torch.tensor([[0.5]]),
               "norm": torch.ones(1), "o": torch.tensor([[1.0]])})
    S = torch.zeros(1, 1, 1)
    h = torch.tensor([[1.0], [2.0]])
    P.wkv_mixer(h, w1, {"heads": 1, "dim": 1}, 0.0, state=S)
    decay = math.exp(-1.0)
    assert abs(float(S) - (decay * 3.0 + 12.0)) < 1e-5          # S1 = k v = 3; S2 = w S1 + k v = e^-1 * 3 + 2 * 6
    # token shift: the row in front of the first token is zeros, or the row that is handed in
    w1["mu.r"] = torch.ones(1)
    a = P.wkv_mixer(h, w1, {"heads": 1, "dim": 1}, 0.0)
    b = P.wkv_mixer(h[1:], w1, {"heads": 1, "dim": 1}, 0.0, state=torch.tensor([[[3.0]]]), before=h[0])
    assert torch.allclose(a[1:], b, atol=1e-6)
