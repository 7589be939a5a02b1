"""Kuvelix configurations drawn at random (layer order, every size, key and value sizes apart, rotation, dense and
expert feed-forwards with their routers' groups and identity experts, layers without a feed-forward, the run of layers
that repeats), each run as one batch of unequal prompts whose last tokens are decoded together, in 32-bit and in
bfloat16, against the plain implementation.  IERT_TEST_RANDOM_KUVELIX=N draws N configurations instead of eight."""
import os
import random

import pytest
import torch

import test_gpu_kuvelix as T
from plain import kuvelix_plain as P

pytestmark = pytest.mark.gpu

COUNT = int(os.environ.get("IERT_TEST_RANDOM_KUVELIX", "8"))


def draw_attention(rng):
    dim = rng.choice([4, 8, 16, 24, 32, 48, 64, 80, 96, 128, 160, 256])
    vdim = rng.choice([dim, dim, 8, 16, 40, 64, 128])
    kv = rng.choice([1, 2, 3, 4])
    rot = rng.choice([None, 0, dim // 4 * 2, dim // 2, dim])
    return T.attn(heads=kv * rng.choice([1, 2, 3, 5]), kv_heads=kv, dim=dim, vdim=vdim,
                  scale=round(dim ** -0.5 * rng.choice([0.3, 0.5, 1.0]), 4), rot_dims=None if rot is None else rot // 2 * 2,
                  base=rng.choice([100.0, 10000.0, 500000.0]), factor=rng.choice([None, 1.0, 2.0, 8.0]))


def draw_mlp(rng):
    kind = rng.choice(["none", "dense", "moe", "moe"])
    if kind == "none":
        return None
    if kind == "dense":
        return T.dense(rng.choice([8, 24, 64, 100, 160]))
    count = rng.choice([1, 2, 3, 4])
    per = rng.choice([1, 2, 3, 5])
    outputs = count * per
    identity = rng.randrange(0, outputs)                  # at least one expert has tensors
    keep = rng.randint(1, count)
    top = rng.randint(1, min(keep * per, 6))
    return T.moe(experts=outputs - identity, identity=identity, top=top, count=count, keep=keep, ff=rng.choice([5, 8, 24, 64]),
                 limit=rng.choice([0.3, 1.0, 7.0]))


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("random_kuvelix"))


@pytest.mark.parametrize("case", range(COUNT))
def test_random_configuration(root, case):
    rng = random.Random(3000 + case)
    n = rng.choice([1, 2, 3, 4, 5])
    layers = [T.layer(draw_attention(rng), draw_mlp(rng)) for _ in range(n)]
    loop = None
    if rng.random() < 0.7:
        start = rng.randrange(0, n)
        loop = (start, rng.randint(start, n), rng.choice([1, 2, 3]))
    cfg = T.config(layers, width=rng.choice([40, 64, 100, 128, 192, 256]), vocab=rng.choice([61, 256, 500]),
                   eps=rng.choice([1e-5, 1e-6]), loop=loop)
    runs = len(P.layer_runs(cfg))
    prompts = T.tokens(cfg, (1, rng.randint(2, 60), rng.randint(61, 140), rng.randint(141, 330)), seed=case)
    for dtype in ("float32", "bfloat16"):
        model, weights = T.make_model(root, cfg, 100 + case, dtype, T.sharpen, std=0.08)
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
            T.compare(torch.cat(rows[i]), want[i], dtype, f"case {case} ({dtype}), request {i}: {cfg}", slack=max(1.0, runs / 5))
