"""Vufinex configurations drawn at random (layer order, every size, chunk sizes on and off the page size, rotation on part
of a head or none, latent attention with and without a rotated part, recurrences of any head size, routers with any
groups, layers without a feed-forward, layers that borrow another's weights, the factors on the embedding and on the
sublayers), each run as one batch of unequal prompts whose last tokens are decoded together, in 32-bit and in bfloat16,
against the plain implementation.  IERT_TEST_RANDOM_VUFINEX=N draws N configurations instead of eight."""
import os
import random

import pytest
import torch

import test_gpu_vufinex as T
from plain import vufinex_plain as P

pytestmark = pytest.mark.gpu

COUNT = int(os.environ.get("IERT_TEST_RANDOM_VUFINEX", "8"))


def draw_mixer(rng):
    kind = rng.choice(["attention", "wkv", "latent_attention"])
    if kind == "attention":
        dim = rng.choice([4, 8, 16, 24, 32, 48, 64, 80, 128])
        kv = rng.choice([1, 2, 3, 4])
        rot = rng.choice([None, 0, dim // 4 * 2, dim // 2, dim])
        return kind, T.attn(heads=kv * rng.choice([1, 2, 3]), kv_heads=kv, dim=dim, scale=round(dim ** -0.5 * rng.choice([0.3, 0.5, 1.0]), 4),
                            rot_dims=None if rot is None else rot // 2 * 2, base=rng.choice([100.0, 10000.0, 500000.0]),
                            chunk=rng.choice([None, 1, 7, 32, 63, 64, 65, 100, 128, 200]))
    if kind == "wkv":
        return kind, T.wkv(heads=rng.choice([1, 2, 3, 5]), dim=rng.choice([4, 8, 12, 16, 32, 64]), rank=rng.choice([None, 1, 4, 7, 16]))
    dim, rot_dim = rng.choice([4, 8, 16, 24, 32, 64]), rng.choice([0, 2, 4, 8, 16, 32])
    return kind, T.latent(heads=rng.choice([1, 2, 3, 4, 8]), dim=dim, rot_dim=rot_dim, vdim=rng.choice([dim, dim + rot_dim, 8, 20, 48, 64]),
                          kv_rank=rng.choice([8, 20, 32, 40, 64, 96]), scale=round((dim + rot_dim) ** -0.5 * rng.choice([0.5, 1.0]), 4),
                          base=rng.choice([100.0, 10000.0]))


def draw_mlp(rng):
    if rng.random() < 0.25:
        return None
    count = rng.choice([1, 2, 3, 4])
    per = rng.choice([1, 2, 3, 5])
    keep = rng.randint(1, count)
    return T.moe(experts=count * per, top=rng.randint(1, min(keep * per, 6)), count=count, keep=keep, ff=rng.choice([5, 8, 24, 64]),
                 scale=rng.choice([0.5, 1.0, 2.5]))


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("random_vufinex"))


@pytest.mark.parametrize("case", range(COUNT))
def test_random_configuration(root, case):
    rng = random.Random(5000 + case)
    n = rng.choice([1, 2, 3, 4, 5])
    layers = []
    for i in range(n):
        if i and rng.random() < 0.3:
            j = rng.randrange(0, i)
            while layers[j].get("weights_of") is not None:
                j = layers[j]["weights_of"]
            layers.append(dict(T.layer(layers[j]["type"], layers[j]["mixer"], layers[j]["mlp"]), weights_of=j))
        else:
            kind, mixer = draw_mixer(rng)
            layers.append(T.layer(kind, mixer, draw_mlp(rng)))
    cfg = T.config(layers, width=rng.choice([40, 64, 100, 128, 192, 256]), vocab=rng.choice([61, 256, 500]),
                   eps=rng.choice([1e-5, 1e-6]), mult=rng.choice([0.35, 0.5, 1.0]), embed=rng.choice([1.0, 3.0, 11.0]))
    prompts = T.tokens(cfg, (1, rng.randint(2, 60), rng.randint(61, 140), rng.randint(141, 330)), seed=case)
    for dtype in ("float32", "bfloat16"):
        model, weights = T.make_model(root, cfg, 100 + case, dtype, T.edit_for(dtype), std=0.08)
        want = [P.forward(cfg, weights, p, T.rounding(dtype)) for p in prompts]
        eng = T.engine_of(model, max_tokens=64 * 12, max_sequences=4)
        slots = [eng.open_sequence() for _ in prompts]
        tails = [min(len(p) - 1, 6 + 9 * i) for i, p in enumerate(prompts)]
        rows = [[] for _ in prompts]
        got, at = eng.step([(s, p[:len(p) - t]) for s, p, t in zip(slots, prompts, tails)], want="all"), 0
        for i, (p, t) in enumerate(zip(prompts, tails)):
            rows[i].append(got[at:at + len(p) - t])
            at += len(p) - t
        pos = [len(p) - t for p, t in zip(prompts, tails)]
        live = [i for i in range(len(prompts)) if pos[i] < len(prompts[i])]
        for i in range(len(prompts)):
            if i not in live:
                eng.close_sequence(slots[i])
        while live:
            got = eng.step([(slots[i], [prompts[i][pos[i]]]) for i in live], want="last")
            for k, i in enumerate(live):
                rows[i].append(got[k:k + 1])
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(prompts[i])]:
                eng.close_sequence(slots[i])
                live.remove(i)
        eng.check_device()
        for i in range(len(prompts)):
            T.compare(torch.cat(rows[i]), want[i], dtype, f"case {case} ({dtype}), request {i}: {cfg}", slack=max(1.0, n / 2.5))
