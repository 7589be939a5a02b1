"""The Kuvelix design in the engine against the plain statement of its equations
(`tests/plain/kuvelix_plain.py`): each mechanism alone (kernels against one function of the plain statement, and
one-layer models), then whole models under every way of cutting the work: whole prompts, tokens one by one through
the cache, batches of unequal requests through slots and pages that are used again, long decoding over page borders,
and greedy generation through the session.  Sizes differ from test to test (also sizes that are 1 or equal to one
another), and where random weights would hide a fault the weights are made so that it shows: sharp softmaxes (every
key carries weight or one far key decides), routers with wide gaps, corrections that make every choice score
negative, identity experts that are chosen often."""
import json
import math
import os

import numpy as np
import pytest
import torch

from helpers import compare as compare_exactly, plain_weights, prompts_for
from plain import kuvelix_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def compare(got, ref, dtype, what="", slack=1.0):
    """float32: every logit within 2e-4, absolute + relative.  bfloat16: both sides round activations to bfloat16,
    but not at exactly the same places, the softmaxes are sharp on purpose and a router's close call may fall
    either way, so rows are judged one by one: the root-mean-square error of a row against the largest logit below
    1.2 % for all but 15 % of the rows (at least two), below 0.6 % for the median row, below 30 % for every row.  A
    fault of the cache or the batch hits most rows, and every case also runs in float32."""
    if dtype == "float32":
        return compare_exactly(got, ref, dtype, what)
    got, ref = torch.as_tensor(got).float().cpu(), torch.as_tensor(ref).float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    rows = (got - ref).pow(2).mean(-1).sqrt() / ref.abs().max()
    over = int((rows > 0.012 * slack).sum())
    assert rows.max() < 0.3, f"{what}: row {int(rows.argmax())} is off by {rows.max().item():.3g} of the largest logit"
    assert over <= max(2, int(0.15 * len(rows))), f"{what}: {over} of {len(rows)} rows are off (worst {rows.max().item():.3g})"
    assert len(rows) < 8 or rows.median() < 0.006 * slack, f"{what}: the median row is off by {rows.median().item():.3g}"


def attn(heads=4, kv_heads=2, dim=16, vdim=None, scale=0.5, rot_dims=8, base=900.0, factor=3.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim, "scale": scale}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, identity=2, top=2, count=4, keep=1, ff=24, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(mixer, mlp=None):
    return {"type": "attention", "mixer": json.loads(json.dumps(mixer)), "mlp": json.loads(json.dumps(mlp))}


def config(layers, width=64, vocab=96, eps=1e-5, loop=None):
    cfg = {"architecture": "Kuvelix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


ALONE = {
    "attention": [layer(attn())],
    "attention_value_size_smaller": [layer(attn(heads=3, kv_heads=3, dim=32, vdim=16, rot_dims=32, factor=None))],
    "attention_value_size_larger": [layer(attn(heads=6, kv_heads=2, dim=16, vdim=40, rot_dims=4))],
    "attention_nothing_turns_one_kv_head": [layer(attn(heads=3, kv_heads=1, dim=24, rot_dims=0))],
    "attention_no_rotation_key": [layer(attn(heads=2, kv_heads=2, dim=16, rot_dims=None))],
    "attention_tcgen05_head": [layer(attn(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=16, scale=0.3))],
    "attention_one_head": [layer(attn(heads=1, kv_heads=1, dim=48, vdim=32, rot_dims=48, factor=1.0))],
    "dense": [layer(attn(), dense(56))],
    "experts": [layer(attn(), moe())],
    "experts_top_one_no_identity_one_group": [layer(attn(), moe(experts=5, identity=0, top=1, count=1, keep=1, ff=16, limit=0.4))],
    "experts_every_group_kept": [layer(attn(), moe(experts=3, identity=3, top=4, count=3, keep=3, ff=8, limit=30.0))],
    "experts_many": [layer(attn(), moe(experts=40, identity=8, top=6, count=8, keep=3, ff=8))],
}

FULL = config([layer(attn(), dense(48)),
               layer(attn(heads=6, kv_heads=3, dim=32, vdim=24, scale=0.3, rot_dims=32, factor=None), moe()),
               layer(attn(heads=2, kv_heads=1, dim=48, vdim=48, scale=0.25, rot_dims=24, factor=8.0), None),
               layer(attn(heads=3, kv_heads=3, dim=16, vdim=32, scale=0.6, rot_dims=0), moe(experts=4, identity=4, top=3, count=2, keep=2, ff=40, limit=0.8)),
               layer(attn(), moe(experts=7, identity=1, top=2, count=1, keep=1, ff=16))],
              width=72, vocab=200, loop=(1, 3, 3))
# sizes the tensor-core products and the 16-byte accesses do not take (a width of 50, head sizes of 12 and 20, 5 wide experts)
ODD = config([layer(attn(heads=3, kv_heads=3, dim=12, vdim=20, rot_dims=6), moe(experts=3, identity=1, top=2, count=2, keep=1, ff=5)),
              layer(attn(heads=2, kv_heads=1, dim=20, vdim=12, rot_dims=20, factor=None), dense(30)),
              layer(attn(heads=5, kv_heads=1, dim=4, vdim=4, rot_dims=2), None)],
             width=50, vocab=77, eps=1e-6, loop=(0, 3, 2))
# head sizes the tensor-core attention kernels take whole (64 on tcgen05, 32 and 48 on mma.sync), widths in whole tiles
TENSOR = config([layer(attn(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.3, rot_dims=32), dense(128)),
                 layer(attn(heads=4, kv_heads=2, dim=48, vdim=32, scale=0.3, rot_dims=48, factor=None), moe(experts=6, identity=2, top=2, count=2, keep=1, ff=64)),
                 layer(attn(heads=4, kv_heads=4, dim=32, vdim=32, scale=0.4, rot_dims=16), moe(experts=4, identity=0, top=2, count=2, keep=2, ff=128, limit=2.0))],
                width=128, vocab=256, loop=(2, 3, 2))
# heads of 128 (tcgen05 prompt attention, decode attention with pages by TMA), no loop
WIDE_HEADS = config([layer(attn(heads=4, kv_heads=2, dim=128, vdim=128, scale=0.2, rot_dims=64), moe(experts=8, identity=8, top=4, count=4, keep=2, ff=32)),
                     layer(attn(heads=2, kv_heads=1, dim=128, vdim=96, scale=0.15, rot_dims=128, factor=None), dense(256))],
                    width=256, vocab=160)
WHOLE_MODELS = {"full": FULL, "odd": ODD, "tensor": TENSOR, "wide_heads": WIDE_HEADS}


def sharpen(tensors):
    """Query norms larger, so that the softmax stands on few keys; router maps larger, so that a router's choice
    rarely hangs on a rounding; corrections of both signs and of the size of the scores; biases that matter."""
    for name in list(tensors):
        if name.endswith(".q.norm"):
            tensors[name] = tensors[name] * 2.5
        elif name.endswith(".router"):
            tensors[name] = tensors[name] * 6.0
        elif name.endswith(".correction"):
            tensors[name] = tensors[name] * 2.0
        elif name.endswith(".b"):
            tensors[name] = tensors[name] * 3.0


def make_model(root, cfg, seed, dtype, edit=sharpen, std=0.1):
    from safetensors.torch import load_file, save_file
    from inference_engine_rust_b200 import LoadedModel, write_random_model
    d = os.path.join(root, f"m{abs(hash((json.dumps(cfg, sort_keys=True), seed, dtype, getattr(edit, '__name__', None)))) % 10 ** 9}")
    if not os.path.isdir(d):
        write_random_model(d, cfg, seed=seed, dtype=dtype, std=std)
        if edit is not None:
            path = os.path.join(d, "model.safetensors")
            tensors = load_file(path)
            edit(tensors)
            save_file({k: v.contiguous() for k, v in tensors.items()}, path)
    return LoadedModel.load(d, dtype=dtype), plain_weights(d)


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("kuvelix"))


def rounding(dtype):
    return P.bf16 if dtype == "bfloat16" else P.exact


def engine_of(model, max_tokens=64 * 16, **kw):
    return model.session(max_tokens=max_tokens, poison_cache=True, **kw).engine


def run_whole(eng, prompt):
    slot = eng.open_sequence()
    got = eng.step([(slot, prompt)], want="all")
    eng.check_device()
    eng.close_sequence(slot)
    return got


def tokens(cfg, lengths, seed=0):
    return prompts_for({"vocab_size": cfg["vocab"]}, lengths, seed=seed)


# ---------------------------------------------------------------------------------------
# kernels against one function of the plain statement each


def B():
    from inference_engine_rust_b200.csrc import bindings
    return bindings


@pytest.mark.parametrize("N,E,top,groups,keep", [(12, 8, 2, 2, 1), (8, 8, 1, 1, 1), (48, 40, 6, 8, 3), (6, 3, 4, 3, 3),
                                                 (66, 60, 32, 1, 1), (9, 9, 3, 9, 3)])
def test_router_against_the_plain_choice(N, E, top, groups, keep):
    """Logits with wide gaps; corrections of both signs, and a case where every choice score is negative (an
    expert outside the kept groups must count as minus infinity there, not as zero)."""
    b = B()
    g = torch.Generator().manual_seed(N * 31 + top)
    for case, shift in enumerate((0.0, -3.0, 0.5)):
        T = 37
        z = (torch.randn(T, N, generator=g) * 2.5).float()
        corr = (torch.randn(N, generator=g) * 0.2 + shift).float()
        zd = z.to(DEV)
        wt = torch.full((T, E), 7.0, device=DEV)
        wid = torch.full((T,), 7.0, device=DEV)
        idx = torch.zeros(T, top, dtype=torch.int32, device=DEV)
        w = torch.zeros(T, top, device=DEV)
        if case == 2:          # the logits stored with a row per router output
            b.router_grouped(zd.t().contiguous(), corr.to(DEV), T, E, N, top, groups, keep, wt, wid, idx, w, b.stream_ptr(),
                             by_output=True)
        else:
            b.router_grouped(zd, corr.to(DEV), T, E, N, top, groups, keep, wt, wid, idx, w, b.stream_ptr())
        ridx, rw = P.route(z, corr, top, groups, keep)
        assert torch.equal(idx.cpu().long(), ridx), f"case {case}"
        assert torch.allclose(w.cpu(), rw, atol=1e-6, rtol=1e-5)
        dense = torch.zeros(T, N)
        dense.scatter_(1, ridx, rw)
        assert torch.allclose(wt.cpu(), dense[:, :E], atol=1e-6, rtol=1e-5)
        assert torch.allclose(wid.cpu(), dense[:, E:].sum(-1), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("name,limit", [("gelu_tanh", None), ("clamped_swish", 0.7), ("clamped_swish", 5.0), ("silu", None)])
@pytest.mark.parametrize("M", [5, 64, 200])
def test_gated_activations(name, limit, M):
    """The activation family in the element-wise kernel (both dtypes) and in the fused tensor-core projection (its
    one-token and its prompt form) against the plain formulas."""
    b = B()
    torch.manual_seed(M)
    K, I = 64, 19200 if M <= 64 else 256            # the one-token form wants its tiles to fill the device
    fn = b.gated_act(name, limit)

    def plain(gv, uv):
        if name == "gelu_tanh":
            return P.gelu_tanh(gv) * uv
        if name == "silu":
            return gv * torch.sigmoid(gv) * uv
        gc, uc = torch.clamp(gv, max=limit), torch.clamp(uv, -limit, limit)
        return gc * torch.sigmoid(1.702 * gc) * (uc + 1.0)
    if fn is not None:
        gu = (torch.randn(9, 2 * 50) * 3).to(DEV)
        out = torch.empty(9, 50, device=DEV)
        b.gated_act_mul(gu, out, 9, 50, fn, b.stream_ptr())
        assert torch.allclose(out.cpu(), plain(gu[:, :50].cpu(), gu[:, 50:].cpu()), atol=1e-6, rtol=1e-5)
        gb = (torch.randn(9, 2 * 48) * 3).to(DEV).to(torch.bfloat16)
        ob = torch.empty(9, 48, device=DEV, dtype=torch.bfloat16)
        b.gated_act_mul(gb, ob, 9, 48, fn, b.stream_ptr())
        assert torch.allclose(ob.float().cpu(), plain(gb[:, :48].float().cpu(), gb[:, 48:].float().cpu()), atol=2e-2, rtol=2e-2)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device=DEV) * 0.3).to(torch.bfloat16)
    act = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert b.gemm_tc_gated(x, w, act, M, err, b.stream_ptr(), fn=fn)
    torch.cuda.synchronize()
    assert err.item() == 0
    y = x.float().cpu() @ w.float().cpu().t()
    assert torch.allclose(act.float().cpu(), plain(y[:, :I], y[:, I:]), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,dim,vdim,D,rot,pairing,normed,biased", [
    (4, 2, 16, 16, 16, 8, "interleaved", True, True), (3, 1, 24, 40, 48, 24, "interleaved", True, False),
    (2, 2, 32, 8, 32, 0, "half", False, True), (5, 5, 12, 20, 20, 6, "half", True, True),
    (16, 4, 128, 128, 128, 64, "interleaved", True, True)])
def test_preparation_of_queries_keys_and_values(dtype, heads, kvh, dim, vdim, D, rot, pairing, normed, biased):
    """Biases, the norm per head, the rotation in either pairing at each token's own position, the padding of the
    heads and the write into the right page row, for a prompt and for single tokens at large positions."""
    from test_gpu_kernels import make_batch, make_cache
    b = B()
    cache = make_cache(kvh, D, None, dtype)
    g = cache.kv_groups[0]
    torch.manual_seed(7)
    qd, kd, vd = heads * dim, kvh * dim, kvh * vdim
    extra = 11                                       # columns behind v that the kernel must leave alone
    i = torch.arange(rot // 2, dtype=torch.float64)
    inv = ((torch.tensor(5000.0, dtype=torch.float64) ** (-2.0 * i / max(rot, 1))) / 3.0).float()
    wq, wk = (torch.rand(dim) + 0.5, torch.rand(dim) + 0.5) if normed else (None, None)
    bias = torch.randn(qd + kd + vd) if biased else None
    dev = lambda t: None if t is None else t.to(DEV)
    for q_lens, pos0 in (([70, 3], [0, 0]), ([1, 1, 1], [70, 3, 300]), ([300], [0])):
        slots = [cache.open_sequence() for _ in q_lens]
        for s, p, q in zip(slots, pos0, q_lens):
            cache.reserve(s, p + q)
        cache.upload()
        view, keep = make_batch(q_lens, pos0, slots)
        T = sum(q_lens)
        proj = torch.randn(T, qd + kd + vd + extra)
        qkv = torch.full((T, (heads + 2 * kvh) * D), float("nan"), device=DEV).to(dtype)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        b.qkv_prep(proj.to(DEV), dev(bias), qkv, view, cache.layer_view(0).struct, heads, dim, vdim, dev(inv), rot,
                   b.PAIR_INTERLEAVED if pairing == "interleaved" else b.PAIR_HALF, dev(wq), dev(wk), 1e-5, True, err, b.stream_ptr())
        assert err.item() == 0
        got = qkv.float().cpu().view(T, heads + 2 * kvh, D)
        kc, vc = g.k[0].float().cpu(), g.v[0].float().cpu()
        x = proj[:, :qd + kd + vd] + (bias if biased else 0.0)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        t = 0
        for s, p0, q in zip(slots, pos0, q_lens):
            xs = x[t:t + q]
            qh, kh, vh = xs[:, :qd].view(q, heads, dim), xs[:, qd:qd + kd].view(q, kvh, dim), xs[:, qd + kd:].view(q, kvh, vdim)
            if normed:
                qh, kh = P.rms_norm(qh, wq, 1e-5), P.rms_norm(kh, wk, 1e-5)
            if pairing == "interleaved":
                qh, kh = P.rotate_pairs(qh, rot, 5000.0, 3.0, p0), P.rotate_pairs(kh, rot, 5000.0, 3.0, p0)
            else:
                from plain import sifasun_plain as S
                qh, kh = S.rotate_half(qh, rot, 5000.0, 3.0, p0), S.rotate_half(kh, rot, 5000.0, 3.0, p0)
            rows = got[t:t + q]
            assert torch.allclose(rows[:, :heads, :dim], qh, atol=tol, rtol=tol)
            assert torch.allclose(rows[:, heads:heads + kvh, :dim], kh, atol=tol, rtol=tol)
            assert torch.allclose(rows[:, heads + kvh:, :vdim], vh, atol=tol, rtol=tol)
            assert (rows[:, :heads + kvh, dim:] == 0).all() and (rows[:, heads + kvh:, vdim:] == 0).all()
            for j in range(q):
                pos = p0 + j
                page = g.pages_of(s)[pos // 64]
                assert torch.equal(kc[page, :, pos % 64], rows[j, heads:heads + kvh])
                assert torch.equal(vc[page, :, pos % 64], rows[j, heads + kvh:])
            t += q
        for s in slots:
            cache.close_sequence(s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,D,vdim,gated", [(3, 48, 40, True), (4, 16, 16, True), (2, 32, 12, False), (5, 20, 20, True)])
def test_gate_on_the_heads(dtype, heads, D, vdim, gated):
    b = B()
    torch.manual_seed(3)
    T = 33
    a = torch.randn(T, heads * D).to(dtype)
    proj = torch.randn(T, 8 + heads * vdim) * 3
    pd = proj.to(DEV)
    out = torch.empty(T, heads * vdim, device=DEV, dtype=dtype)
    b.gate_mul(a.to(DEV), pd[:, 8:] if gated else None, out, T, heads, D, vdim, b.stream_ptr())
    ref = a.float().view(T, heads, D)[:, :, :vdim].reshape(T, heads * vdim)
    if gated:
        ref = ref * torch.sigmoid(proj[:, 8:])
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=tol)


# ---------------------------------------------------------------------------------------
# models


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(root, name, dtype):
    cfg = config(ALONE[name])
    model, weights = make_model(root, cfg, 3, dtype)
    eng = engine_of(model)
    for prompt in tokens(cfg, (1, 2, 150), seed=1):
        compare(run_whole(eng, prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{name}, {len(prompt)} tokens")


def test_residual_after_every_layer_run(root):
    """The residual after each layer run (a looped layer counts each time) against the plain statement."""
    model, weights = make_model(root, FULL, 5, "float32")
    eng = engine_of(model)
    prompt = tokens(FULL, (37,), seed=2)[0]
    want, got = [], []
    P.forward(FULL, weights, prompt, residuals=want)
    model.model.after_block = lambda pos, rows, ctx: got.append(rows[:ctx.n_tokens].clone())
    try:
        run_whole(eng, prompt)
    finally:
        model.model.after_block = None
    assert len(got) == len(want) == len(P.layer_runs(FULL)) == 9
    for i, (g, w) in enumerate(zip(got, want)):
        compare(g, w, "float32", f"residual after layer run {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_whole_prompts(root, name, dtype):
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 7, dtype)
    eng = engine_of(model)
    for prompt in tokens(cfg, (1, 3, 64, 65, 300), seed=3):
        compare(run_whole(eng, prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{name}, {len(prompt)} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_prompt_then_tokens_one_by_one(root, name, dtype):
    """A prompt in one step, then single tokens over a page border and on; also from the very first token on.  Every
    pass of a looped layer must keep a cache of its own: with a shared one the later passes would read the earlier
    passes' keys."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 8, dtype)
    eng = engine_of(model)
    for first, total in ((1, 20), (2, 75), (61, 61 + 140)):
        seq = tokens(cfg, (total,), seed=first)[0]
        ref = P.forward(cfg, weights, seq, rounding(dtype))
        slot = eng.open_sequence()
        rows = [eng.step([(slot, seq[:first])], want="all")]
        for t in seq[first:]:
            rows.append(eng.step([(slot, [t])], want="last"))
        eng.check_device()
        eng.close_sequence(slot)
        compare(torch.cat(rows), ref, dtype, f"{name}: {first} tokens, then {total - first} one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_unequal_batches_through_slots_and_pages_used_again(root, name, dtype):
    """Batches of unequal requests decoded together, the shorter ones ending earlier, in a cache so small that
    slots and pages are handed out again (poisoned when freed): every row equals the request run alone."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 9, dtype)
    eng = engine_of(model, max_tokens=64 * 7, max_sequences=4)
    for wave, lengths in enumerate(((1, 70, 5), (130, 2, 64, 33), (3, 129))):
        seqs = tokens(cfg, [n + d for n, d in zip(lengths, (9, 3, 14, 6))], seed=10 + wave)
        refs = [P.forward(cfg, weights, s, rounding(dtype)) for s in seqs]
        slots = [eng.open_sequence() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lengths)], want=[[n - 1] for n in lengths])
        for i in range(len(seqs)):
            got[i].append(out[i:i + 1])
        done = list(lengths)
        live = list(range(len(seqs)))
        while live:
            out = eng.step([(slots[i], [seqs[i][done[i]]]) for i in live], want="last")
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                done[i] += 1
            for i in [i for i in live if done[i] == len(seqs[i])]:
                eng.close_sequence(slots[i])
                live.remove(i)
        eng.check_device()
        for i, (s, n) in enumerate(zip(seqs, lengths)):
            compare(torch.cat(got[i]), refs[i][n - 1:], dtype, f"{name}: wave {wave}, request {i} ({n} + {len(s) - n} tokens)")
        eng.cache.check()


def test_the_tolerances_refuse_planted_faults(root):
    """The comparison that the other tests pass is not passed by a plain statement with one fault: a rotation one
    frequency step off, the looped layers run once less, the group rule left out, the correction taken into the
    weights' place, an identity expert that returns nothing."""
    cfg = FULL
    model, weights = make_model(root, cfg, 7, "float32")
    prompt = tokens(cfg, (120,), seed=3)[0]
    got = run_whole(engine_of(model), prompt)
    compare(got, P.forward(cfg, weights, prompt), "float32", "unplanted")

    def planted(change):
        bad = json.loads(json.dumps(cfg))
        w = dict(weights)
        change(bad, w)
        return P.forward(bad, w, prompt)

    def rotation(bad, w):
        bad["layers"][0]["mixer"]["rot"]["scaling"]["factor"] = 2.9

    def fewer_passes(bad, w):
        bad["loop"]["times"] -= 1

    def no_groups(bad, w):
        bad["layers"][1]["mlp"]["router"]["groups"] = {"count": 1, "keep": 1}

    def no_correction(bad, w):
        w["l1.mlp.correction"] = torch.zeros_like(w["l1.mlp.correction"])

    def silent_identity(bad, w):
        r = bad["layers"][3]["mlp"]["router"]
        r["experts"], r["identity"] = r["experts"] + r["identity"], 0
        for e in range(4, 8):
            for n in ("gate", "up", "down"):
                w[f"l3.mlp.e{e}.{n}"] = torch.zeros_like(w[f"l3.mlp.e0.{n}"])
    for change in (rotation, fewer_passes, no_groups, no_correction, silent_identity):
        with pytest.raises(AssertionError):
            compare(got, planted(change), "float32", change.__name__)


def test_a_far_key_decides(root):
    """One attention layer whose scores are sharp: the last token's query is made to match the key of a token
    hundreds of positions back (a query map and an embedding row made for it, unit norm weights, no biases, a large
    score scale), so that dropping that one key would change the result."""
    cfg = config([layer(attn(heads=2, kv_heads=1, dim=32, vdim=16, scale=0.9, rot_dims=0, factor=None))], width=64, vocab=50)

    def matched(t):
        # the query map is the key map behind a turn of the input by one place, and token 48's embedding is token
        # 49's turned the same way: the query of 49 equals the key of 48 (and not its own), and their values differ
        for n in ("embed.norm", "l0.norm1", "l0.mix.q.norm", "l0.mix.k.norm"):
            t[n] = torch.ones_like(t[n])
        for n in ("l0.mix.q.b", "l0.mix.k.b"):
            t[n] = torch.zeros_like(t[n])
        t["l0.mix.q"] = torch.roll(t["l0.mix.k"], 1, dims=1).repeat(2, 1).contiguous()
        t["embed"][48] = torch.roll(t["embed"][49], -1)
    model, weights = make_model(root, cfg, 13, "float32", matched)
    prompt = [min(t, 47) for t in tokens(cfg, (700,), seed=5)[0]]
    prompt[40], prompt[-1] = 48, 49
    eng = engine_of(model, max_tokens=64 * 12)
    ref = P.forward(cfg, weights, prompt)
    compare(run_whole(eng, prompt), ref, "float32", "a far key in a prompt")
    slot = eng.open_sequence()
    eng.step([(slot, prompt[:-1])], want="none")
    compare(eng.step([(slot, prompt[-1:])], want="last"), ref[-1:], "float32", "a far key from the cache")
    eng.close_sequence(slot)
    without = P.forward(cfg, weights, prompt[:40] + [47] + prompt[41:])
    assert (without[-1] - ref[-1]).abs().max() > 0.05, "the far key does not matter in this test"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_identity_experts_and_negative_choice_scores(root, dtype):
    """A router whose corrections are all far below zero (every choice score negative: an expert outside the kept
    groups must not win with a score of zero) and favour the experts that return their input, which then carry a good
    part of the layer's output."""
    cfg = config([layer(attn(), moe(experts=4, identity=4, top=3, count=4, keep=2, ff=24, limit=1.0))] * 2, width=64, vocab=80)

    def edit(t):
        sharpen(t)
        for i in (0, 1):
            c = torch.full_like(t[f"l{i}.mlp.correction"], -4.0)
            c[4:] += 0.15
            t[f"l{i}.mlp.correction"] = c
    model, weights = make_model(root, cfg, 21, dtype, edit)
    prompt = tokens(cfg, (90,), seed=4)[0]
    h = P.rms_norm(P.rms_norm(weights["embed"][torch.tensor(prompt)], weights["embed.norm"], 1e-5), weights["l0.norm1"], 1e-5)
    idx, _ = P.route(P.lin(h, weights["l0.mlp.router"]), weights["l0.mlp.correction"], 3, 4, 2)
    assert (idx >= 4).float().mean() > 0.3, "identity experts are rarely chosen in this test"
    compare(run_whole(engine_of(model), prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, "identity experts")


@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_greedy_generation_through_the_session(root, name):
    """`generate` (the scheduler's batches, the sampler, steps fed from device memory) against greedy
    choices made from the plain implementation's logits."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 11, "float32")
    prompts = tokens(cfg, (1, 6, 70, 17), seed=4)
    session = model.session(max_tokens=64 * 10, max_sequences=3)
    got = session.generate(prompts, max_new_tokens=12, stop_ids=[])
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            logits = P.forward(cfg, weights, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if top2[0] - top2[1] < 1e-3:           # a close call proves nothing either way
                break
            seq.append(int(torch.argmax(logits)))
        n = len(seq) - len(p)
        assert g[:n] == seq[len(p):], f"{name}: prompt of {len(p)} tokens"


def test_command_line_and_presets(root, capsys):
    from inference_engine_rust_b200 import cli
    path = os.path.join(root, "cfg.json")
    with open(path, "w") as f:
        json.dump(ODD, f)
    out = os.path.join(root, "cli_model")
    assert cli.main(["random-model", "--config", path, "--seed", "2", "--out", out]) == 0
    capsys.readouterr()
    assert cli.main(["-m", out, "-n", "5", "--stop-token", "-1", "3 9 27"]) == 0
    ids = capsys.readouterr().out.split()
    assert len([t for t in ids if t.lstrip("-").isdigit()]) >= 5
    assert cli.main(["--random", "kuvelix-tiny", "--seed", "1", "-n", "4", "--stop-token", "-1", "5 6"]) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(root, tmp_path, dtype):
    """bin/trace_run picks the architecture from config.json: requests whole, with their last tokens one by one,
    and as unequal batches whose shorter requests end earlier; every wanted row against the plain implementation."""
    from safetensors.torch import load_file, save_file
    from inference_engine_rust_b200 import write_random_model
    import test_gpu_trace_run as R
    cfg = TENSOR if dtype == "bfloat16" else FULL
    d = str(tmp_path / "model")
    write_random_model(d, cfg, seed=21, dtype=dtype, std=0.1)
    path = os.path.join(d, "model.safetensors")
    tensors = load_file(path)
    sharpen(tensors)
    save_file({k: v.contiguous() for k, v in tensors.items()}, path)
    weights = plain_weights(d)
    seqs = tokens(cfg, (90, 7, 131), seed=6)
    refs = [P.forward(cfg, weights, s, rounding(dtype)) for s in seqs]
    steps, wanted = [], []
    n = 0
    for i, s in enumerate(seqs):                       # whole; then all but five tokens and the rest one by one
        steps.append({"step": n, "entries": [{"id": f"w{i}", "tokens": s, "want": [0, len(s) - 1]}], "end": [f"w{i}"]})
        wanted.append((n, [refs[i][0], refs[i][-1]]))
        n += 1
        cut = max(1, len(s) - 5)
        steps.append({"step": n, "entries": [{"id": f"d{i}", "tokens": s[:cut], "want": []}], "end": []})
        n += 1
        for j in range(cut, len(s)):
            steps.append({"step": n, "entries": [{"id": f"d{i}", "tokens": [s[j]], "want": [0]}],
                          "end": [f"d{i}"] if j == len(s) - 1 else []})
            wanted.append((n, [refs[i][j]]))
            n += 1
    cuts = [len(s) - k for s, k in zip(seqs, (4, 2, 6))]       # together: unequal prompts, then decoded until each ends
    steps.append({"step": n, "entries": [{"id": f"t{i}", "tokens": s[:c], "want": [c - 1]} for i, (s, c) in enumerate(zip(seqs, cuts))],
                  "end": []})
    wanted.append((n, [refs[i][c - 1] for i, c in enumerate(cuts)]))
    n += 1
    pos = list(cuts)
    while any(p < len(s) for p, s in zip(pos, seqs)):
        live = [i for i, s in enumerate(seqs) if pos[i] < len(s)]
        steps.append({"step": n, "entries": [{"id": f"t{i}", "tokens": [seqs[i][pos[i]]], "want": [0]} for i in live],
                      "end": [f"t{i}" for i in live if pos[i] + 1 == len(seqs[i])]})
        wanted.append((n, [refs[i][pos[i]] for i in live]))
        for i in live:
            pos[i] += 1
        n += 1
    out = str(tmp_path / "out")
    R.replay(d, dtype, steps, out, max_tokens=64 * 9)
    for step, rows in wanted:
        compare(R.read(out, step, cfg["vocab"]), torch.stack(rows), dtype, f"step {step}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_prompt_steps_replayed_as_graphs(root, dtype):
    """Prompt steps of up to 512 tokens that want their last rows are captured into a CUDA graph from a shape
    bucket's second use on (padding tokens and padding sequences inside): same logits as the plain statement on
    every turn, with slots and pages used again in between, and the tokens after the prompt one by one."""
    cfg = WHOLE_MODELS["tensor" if dtype == "bfloat16" else "full"]
    model, weights = make_model(root, cfg, 17, dtype)
    # memory that the graphs' own buffers will be cut from holds NaN: rows of padding tokens that nobody writes show
    junk = [torch.full((16 << 20,), float("nan"), device="cuda") for _ in range(4)]
    del junk
    prompts = tokens(cfg, (3, 1, 63, 200, 140, 331), seed=8)
    want = [P.forward(cfg, weights, p + [5, 6], rounding(dtype)) for p in prompts]
    eng = engine_of(model, max_tokens=64 * 14, max_sequences=4)
    batches = [[1, 0], [3], [1, 2], [4, 0], [5], [0, 1], [3, 1], [2, 1], [5], [4]]
    for turn, batch in enumerate(batches * 2):
        slots = [eng.open_sequence() for _ in batch]
        got = eng.step([(s, prompts[i]) for s, i in zip(slots, batch)], want="last")
        more = eng.step([(s, [5]) for s in slots], want="last")
        last = eng.step([(s, [6]) for s in slots], want="last")
        eng.check_device()
        for k, i in enumerate(batch):
            n = len(prompts[i])
            compare(torch.cat([got[k:k + 1], more[k:k + 1], last[k:k + 1]]), want[i][n - 1:], dtype,
                    f"turn {turn}: a {n}-token prompt and two tokens more")
        for s in slots:
            eng.close_sequence(s)
    assert sum(1 for k in eng._graphs if isinstance(k, tuple) and k and k[0] == "prompt") >= 4, "few prompt steps were replayed"
