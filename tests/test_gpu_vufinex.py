"""The Vufinex design in the engine against the plain statement of its equations
(`tests/plain/vufinex_plain.py`): each mechanism alone (kernels against one function of the plain statement, and
one-layer models), then whole models under every way of cutting the work: whole prompts, tokens one by one through
the cache and the state, batches of unequal requests through slots and pages that are used again, decoding over page
borders and chunk edges, short prompt steps replayed as graphs, and greedy generation through the session.  Sizes
differ from test to test (also sizes that are 1 or equal to one another), and where random weights would hide a fault
the weights are made so that it shows: sharp softmaxes, one far key that decides, a key just outside a chunk that would
decide if it were seen, routers with wide gaps and corrections that make every choice score negative."""
import json
import os

import pytest
import torch

from helpers import compare as compare_exactly, plain_weights, prompts_for
from plain import vufinex_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def compare(got, ref, dtype, what="", slack=1.0):
    """float32: every logit within 2e-4, absolute + relative.  bfloat16: both sides round activations to bfloat16,
    but not at exactly the same places, and a router's close call may fall either way, so rows are judged one by one:
    the root-mean-square error of a row against the largest logit below 1.2 % for all but 15 % of the rows (at least
    two), below 0.6 % for the median row, below 30 % for every row.  A fault of the cache, the state or the batch hits
    most rows, and every case also runs in float32."""
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


def attn(heads=4, kv_heads=2, dim=16, scale=0.5, rot_dims=8, base=900.0, chunk=24):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def wkv(heads=3, dim=16, rank=None):
    m = {"heads": heads, "dim": dim}
    if rank is not None:
        m["decay_rank"] = rank
    return m


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.3, base=700.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim}}


def moe(experts=6, top=2, count=3, keep=2, ff=24, scale=1.7):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


def layer(kind, mixer, mlp=None, weights_of=None):
    out = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(layers, width=64, vocab=96, eps=1e-5, mult=0.6, embed=3.0):
    return {"architecture": "Vufinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": embed}, "layers": json.loads(json.dumps(layers))}


ALONE = {
    "chunked attention": [layer("attention", attn())],
    "chunks of one page": [layer("attention", attn(heads=2, kv_heads=2, dim=32, rot_dims=32, chunk=64))],
    "chunks wider than a page": [layer("attention", attn(heads=2, kv_heads=1, dim=16, rot_dims=4, chunk=100))],
    "chunks of one position": [layer("attention", attn(heads=1, kv_heads=1, dim=8, rot_dims=2, chunk=1))],
    "attention without a mask or a rotation": [layer("attention", attn(rot_dims=None, chunk=None))],
    "wkv": [layer("wkv", wkv())],
    "wkv, one head": [layer("wkv", wkv(heads=1, dim=32, rank=3))],
    "latent attention": [layer("latent_attention", latent())],
    "latent attention, one head, equal sizes": [layer("latent_attention", latent(heads=1, dim=16, rot_dim=16, vdim=32, kv_rank=32))],
    "latent attention without a rotated part": [layer("latent_attention", latent(rot_dim=0))],
    "experts": [layer("wkv", wkv(heads=1, dim=8), moe())],
    "experts, every expert a group": [layer("wkv", wkv(heads=1, dim=8), moe(experts=4, top=2, count=4, keep=3))],
    "experts, top one of one group": [layer("wkv", wkv(heads=1, dim=8), moe(experts=3, top=1, count=1, keep=1, scale=1.0))],
}
for _name in ("latent attention without a rotated part",):
    ALONE[_name][0]["mixer"].pop("rot")

FULL = config([layer("attention", attn(), moe()),
               layer("wkv", wkv(), moe(experts=4, top=3, count=2, keep=2, ff=16)),
               layer("latent_attention", latent(), None),
               layer("attention", attn(), moe(), weights_of=0),
               layer("wkv", wkv(), moe(experts=4, top=3, count=2, keep=2, ff=16), weights_of=1),
               layer("latent_attention", latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16), moe(experts=2, top=1, count=2, keep=1))],
              width=64, vocab=96)
# sizes no kernel for the tensor cores takes: everything runs the plain kernels, also in bfloat16
ODD = config([layer("latent_attention", latent(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=22), moe(experts=3, top=2, count=1, keep=1, ff=5)),
              layer("wkv", wkv(heads=2, dim=12, rank=5), None),
              layer("attention", attn(heads=3, kv_heads=3, dim=12, rot_dims=6, chunk=37), moe(experts=4, top=1, count=2, keep=1, ff=7))],
             width=52, vocab=75, eps=1e-6, mult=1.0, embed=1.0)
# sizes the tensor-core kernels take: tcgen05 prompt attention at head size 64, the one-token latent kernel
TENSOR = config([layer("wkv", wkv(heads=2, dim=64, rank=24), moe(experts=6, top=2, count=3, keep=2, ff=48)),
                 layer("attention", attn(heads=4, kv_heads=2, dim=64, scale=0.3, rot_dims=32, chunk=80), moe(experts=6, top=2, count=3, keep=2, ff=48)),
                 layer("latent_attention", latent(heads=4, dim=32, rot_dim=16, vdim=48, kv_rank=64, scale=0.25), moe(experts=8, top=2, count=4, keep=2, ff=32)),
                 layer("attention", attn(heads=4, kv_heads=2, dim=64, scale=0.3, rot_dims=32, chunk=80), moe(experts=6, top=2, count=3, keep=2, ff=48), weights_of=1)],
                width=128, vocab=160, mult=0.5, embed=6.0)
WIDE_HEADS = config([layer("attention", attn(heads=2, kv_heads=1, dim=128, scale=0.2, rot_dims=64, chunk=130), moe(experts=4, top=2, count=2, keep=1, ff=32)),
                     layer("latent_attention", latent(heads=2, dim=64, rot_dim=32, vdim=128, kv_rank=96, scale=0.2), None),
                     layer("wkv", wkv(heads=1, dim=128, rank=8), None)], width=128, vocab=128)
WHOLE_MODELS = {"full": FULL, "odd": ODD, "tensor": TENSOR, "wide_heads": WIDE_HEADS}


def sharpen(tensors):
    """Router maps larger, so that a router's choice rarely hangs on a rounding; corrections of both signs and of the
    size of the scores; decays spread between fast and slow; token-shift factors inside (0, 1)."""
    for name in list(tensors):
        if name.endswith(".router"):
            tensors[name] = tensors[name] * 6.0
        elif name.endswith(".correction"):
            tensors[name] = tensors[name] * 3.0
        elif name.endswith(".w0"):
            tensors[name] = tensors[name] * 12.0 - 1.0
        elif ".mu." in name:
            tensors[name] = tensors[name] * 3.0 + 0.5
        elif name.endswith(".mix.u"):
            tensors[name] = tensors[name] * 5.0


def steady(tensors):
    """`sharpen`, and corrections so far apart (1.5 times distinct powers of two) that they alone decide every choice and
    every group: a recurrent layer carries the trace of ONE expert chosen otherwise through all later rows, and two
    bfloat16 pipelines that round at different places would disagree on a close call somewhere in hundreds of tokens.
    The bfloat16 runs of whole models use these; the float32 runs, the kernel test and the one-layer models keep
    routers whose choice hangs on the token."""
    sharpen(tensors)
    for name in list(tensors):
        if name.endswith(".correction"):
            n = tensors[name].numel()
            order = torch.randperm(n, generator=torch.Generator().manual_seed(n + len(name)))
            tensors[name] = (1.5 * 2.0 ** order.float()).to(tensors[name].dtype)


def edit_for(dtype):
    return sharpen if dtype == "float32" else steady


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
    return str(tmp_path_factory.mktemp("vufinex"))


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


def B():
    from inference_engine_rust_b200.csrc import bindings
    return bindings


def stream():
    return torch.cuda.current_stream().cuda_stream


# ---------------------------------------------------------------------------------------
# kernels against one function of the plain statement each


@pytest.mark.parametrize("E,top,groups,keep,scale", [(8, 3, 2, 1, 1.5), (6, 2, 3, 2, 0.7), (4, 2, 4, 3, 2.0), (5, 1, 1, 1, 1.0),
                                                     (48, 6, 8, 3, 2.5), (3, 3, 1, 1, 1.0)])
def test_router_against_the_plain_choice(E, top, groups, keep, scale):
    """Sigmoid scores, the choice on score + correction inside the groups whose two best choice scores add up highest,
    weights from the uncorrected scores; corrections far below zero make every choice score negative."""
    b = B()
    g = torch.Generator().manual_seed(E * 100 + top)
    T = 150
    z = (torch.randn(T, E, generator=g) * 2.0)
    for corr in (torch.randn(E, generator=g) * 0.5, torch.randn(E, generator=g) * 0.5 - 4.0):
        idx_ref, w_ref = P.route(z, corr, top, groups, keep, scale)
        zd, cd = z.to(DEV), corr.to(DEV)
        wt = torch.empty(T, E, device=DEV)
        wid = torch.empty(T, device=DEV)
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        w = torch.empty(T, top, device=DEV)
        for by_output in (False, True):
            src = zd.t().contiguous() if by_output else zd
            b.router_grouped(src, cd, T, E, E, top, groups, keep, wt, wid, idx, w, stream(), by_output=by_output,
                             score="sigmoid", group_score="top2_sum", weight_eps=1e-20, weight_scale=scale)
            torch.cuda.synchronize()
            dense = torch.zeros(T, E)
            dense.scatter_(1, idx_ref, w_ref)
            assert torch.equal(idx.cpu().long().sort(1).values, idx_ref.sort(1).values)
            torch.testing.assert_close(wt.cpu(), dense, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("lanes", [None, 1, 4, 8, 32])
@pytest.mark.parametrize("H,D,T0,T1", [(2, 16, 5, 9), (1, 64, 1, 70), (3, 32, 33, 1), (2, 128, 3, 4), (2, 12, 7, 2)])
def test_recurrence_against_the_plain_loop(H, D, T0, T1, lanes, monkeypatch):
    """The state update and the read-out of the wkv recurrence alone, over two steps of one sequence (the second
    continues from the state the first left) beside a second sequence of another length; with the lanes per column
    of the state that the launcher picks, and with forced ones (a lane's rows lie apart or side by side)."""
    if lanes is not None:
        monkeypatch.setenv("IERT_RECURRENT_LANES", str(lanes))
    b = B()
    g = torch.Generator().manual_seed(H * D + T0)
    lens = [(T0, T1), (T1 + 2, 1)]
    n_slots, floats = 4, H * D * D + 7
    state = torch.zeros(n_slots, floats, device=DEV)
    refs = [torch.zeros(H, D, D) for _ in lens]
    u = torch.randn(H, D, generator=g)
    for step in range(2):
        q_lens = [l[step] for l in lens]
        T = sum(q_lens)
        x = torch.randn(T, 3 * H * D + (5 if H == 2 else 4), generator=g) * 0.5      # rows that are, and are not, 16-byte aligned
        decay = torch.rand(T, H * D, generator=g) * 0.9 + 0.05
        want = torch.zeros(T, H * D)
        t0 = 0
        for s, n in enumerate(q_lens):
            r, k, v = (x[t0:t0 + n, i * H * D:(i + 1) * H * D].view(n, H, D) for i in range(3))
            w = decay[t0:t0 + n].view(n, H, D)
            for t in range(n):
                for a in range(H):
                    kv = torch.outer(k[t, a], v[t, a])
                    want[t0 + t, a * D:(a + 1) * D] = (refs[s][a] + u[a][:, None] * kv).t() @ r[t, a]
                    refs[s][a] = w[t, a][:, None] * refs[s][a] + kv
            t0 += n
        cu = torch.tensor([0, q_lens[0], q_lens[0] + q_lens[1]], dtype=torch.int32, device=DEV)
        slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
        tok_seq = torch.tensor(sum(([i] * n for i, n in enumerate(q_lens)), []), dtype=torch.int32, device=DEV)
        pos0 = torch.zeros(2, dtype=torch.int32, device=DEV)
        view = b.BatchView(cu_q=cu.data_ptr(), slot_ids=slots.data_ptr(), tok_seq=tok_seq.data_ptr(), pos0=pos0.data_ptr(),
                           n_seqs=2, n_tokens=T)
        o = torch.empty(T, H * D, device=DEV)
        b.wkv_recur(x.to(DEV), decay.to(DEV), u.to(DEV), state, 0, o, D, H, D, view, stream())
        torch.cuda.synchronize()
        torch.testing.assert_close(o.cpu(), want, rtol=2e-4, atol=2e-4)
    for s, slot in enumerate((2, 0)):
        torch.testing.assert_close(state[slot, :H * D * D].cpu().view(H, D, D), refs[s], rtol=2e-4, atol=2e-4)
    assert float(state[1].abs().max()) == 0.0 and float(state[:, H * D * D:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(root, name, dtype):
    cfg = config(ALONE[name])
    model, weights = make_model(root, cfg, 3, dtype)
    eng = engine_of(model)
    for prompt in tokens(cfg, (1, 2, 150), seed=1):
        compare(run_whole(eng, prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{name}, {len(prompt)} tokens")


def test_residual_after_every_layer(root):
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
    assert len(got) == len(want) == 6
    for i, (g, w) in enumerate(zip(got, want)):
        compare(g, w, "float32", f"residual after layer {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_whole_prompts(root, name, dtype):
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 7, dtype, edit_for(dtype))
    eng = engine_of(model)
    for prompt in tokens(cfg, (1, 3, 64, 65, 300), seed=3):
        compare(run_whole(eng, prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, f"{name}, {len(prompt)} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_prompt_then_tokens_one_by_one(root, name, dtype):
    """A prompt in one step, then single tokens over page borders and chunk edges; also from the very first token on
    and from a prompt of two tokens.  A layer that runs with another's weights must keep a cache and a state of its own."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 8, dtype, edit_for(dtype))
    eng = engine_of(model)
    for first, total in ((1, 30), (2, 75), (61, 61 + 140)):
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
    """Batches of unequal requests decoded together, the shorter ones ending earlier, in a cache so small that slots,
    pages and states are handed out again (pages poisoned when freed): every row equals the request run alone."""
    cfg = WHOLE_MODELS[name]
    model, weights = make_model(root, cfg, 9, dtype, edit_for(dtype))
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
    """The comparison that the other tests pass is not passed by a plain statement with one fault: chunks one position
    longer, a rotation with another base, the bonus of the current token left out, another factor on the routing
    weights, another factor on the sublayers."""
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

    def longer_chunks(bad, w):
        bad["layers"][0]["mixer"]["mask"]["size"] += 1
        bad["layers"][3]["mixer"]["mask"]["size"] += 1

    def other_rotation(bad, w):
        bad["layers"][2]["mixer"]["rot"]["base"] = 650.0

    def no_bonus(bad, w):
        w["l1.mix.u"] = torch.zeros_like(w["l1.mix.u"])

    def other_scale(bad, w):
        bad["layers"][0]["mlp"]["router"]["scale"] = 1.6

    def weaker_sublayers(bad, w):
        bad["residual_mult"] = 0.58
    for change in (longer_chunks, other_rotation, no_bonus, other_scale, weaker_sublayers):
        with pytest.raises(AssertionError):
            compare(got, planted(change), "float32", change.__name__)


def _matched(prefix_q, prefix_k, rows_per_head, heads, kv_heads):
    """An edit that makes query head h's map equal to its key head's map behind a turn of the input by one place."""
    def edit(t):
        k = t[prefix_k]
        rep = heads // kv_heads
        q = torch.roll(k, 1, dims=1).view(kv_heads, 1, rows_per_head, -1).expand(kv_heads, rep, rows_per_head, k.shape[1])
        t[prefix_q] = q.reshape(heads * rows_per_head, -1).contiguous()
    return edit


@pytest.mark.parametrize("chunk,where", [(50, "inside"), (50, "outside"), (64, "inside"), (64, "outside")])
def test_a_key_at_the_edge_of_a_chunk_decides(root, chunk, where):
    """One attention layer with sharp scores whose last query matches the key of ONE earlier token: placed at the first
    position of the last token's chunk it must carry the result, placed one position earlier it must not be seen, in a
    prompt and from the cache."""
    cfg = config([layer("attention", attn(heads=2, kv_heads=1, dim=32, scale=0.9, rot_dims=None, chunk=chunk))], width=64, vocab=50,
                 mult=1.0, embed=1.0)
    match = _matched("l0.mix.q", "l0.mix.k", 32, 2, 1)

    def edit(t):
        t["l0.norm1"] = torch.zeros_like(t["l0.norm1"])
        match(t)
        t["embed"][48] = torch.roll(t["embed"][49], -1)
    model, weights = make_model(root, cfg, 13, "float32", edit, std=0.3)
    n = 3 * chunk + 17
    edge = 3 * chunk if where == "inside" else 3 * chunk - 1
    prompt = [min(t, 47) for t in tokens(cfg, (n,), seed=5)[0]]
    prompt[edge], prompt[-1] = 48, 49
    eng = engine_of(model, max_tokens=64 * 12)
    ref = P.forward(cfg, weights, prompt)
    compare(run_whole(eng, prompt), ref, "float32", "the edge key in a prompt")
    slot = eng.open_sequence()
    eng.step([(slot, prompt[:edge - 2])], want="none")
    for t in prompt[edge - 2:-1]:
        eng.step([(slot, [t])], want="none")
    compare(eng.step([(slot, prompt[-1:])], want="last"), ref[-1:], "float32", "the edge key from the cache")
    eng.close_sequence(slot)
    without = P.forward(cfg, weights, prompt[:edge] + [47] + prompt[edge + 1:])
    moved = (without[-1] - ref[-1]).abs().max()
    if where == "inside":
        assert moved > 0.05, "the key at the chunk's first position does not matter in this test"
    else:
        assert moved < 1e-5, "a key in front of the chunk is seen"


def test_a_far_key_decides_in_latent_attention(root):
    """One latent-attention layer whose last query matches, through the latent, the key of a token hundreds of positions
    back: dropping that key would change the result, in a prompt and from the cache."""
    cfg = config([layer("latent_attention", latent(heads=2, dim=32, rot_dim=0, vdim=16, kv_rank=32, scale=0.9))], width=64, vocab=50,
                 mult=1.0, embed=1.0)
    cfg["layers"][0]["mixer"].pop("rot")

    def edit(t):
        t["l0.norm1"] = torch.zeros_like(t["l0.norm1"])
        t["l0.mix.dkv.norm"] = torch.ones_like(t["l0.mix.dkv.norm"])
        # keys = W_uk c with c the normed W_dkv h: the query map is W_uk W_dkv behind a turn of the input by one place
        uk, dkv = t["l0.mix.uk"].float(), t["l0.mix.dkv"].float()
        t["l0.mix.q"] = (4.0 * torch.roll(uk @ dkv, 1, dims=1)).to(t["l0.mix.q"].dtype).contiguous()
        t["l0.mix.g"] = torch.zeros_like(t["l0.mix.g"])
        t["embed"][48] = torch.roll(t["embed"][49], -1)
    model, weights = make_model(root, cfg, 14, "float32", edit, std=0.3)
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


def test_a_far_token_stays_in_the_state(root):
    """One wkv layer with decays close to one: a token hundreds of positions back still shows in the last token's
    result, through a prompt and through a state carried over single tokens; and a slot that is used again starts
    from zeros."""
    cfg = config([layer("wkv", wkv(heads=2, dim=16, rank=4))], width=32, vocab=50, mult=1.0, embed=2.0)

    def edit(t):
        t["l0.mix.w0"] = torch.full_like(t["l0.mix.w0"], -7.0)          # w = exp(-exp(-7)): about 0.999 a token
        t["l0.mix.w2"] = t["l0.mix.w2"] * 0.1
    model, weights = make_model(root, cfg, 15, "float32", edit, std=0.3)
    prompt = tokens(cfg, (400,), seed=6)[0]
    eng = engine_of(model, max_tokens=64 * 8, max_sequences=1)
    ref = P.forward(cfg, weights, prompt)
    compare(run_whole(eng, prompt), ref, "float32", "a long prompt")
    slot = eng.open_sequence()
    eng.step([(slot, prompt[:390])], want="none")
    rows = [eng.step([(slot, [t])], want="last") for t in prompt[390:]]
    compare(torch.cat(rows), ref[390:], "float32", "the state carried over single tokens")
    eng.close_sequence(slot)
    compare(run_whole(eng, prompt[:5]), ref[:5], "float32", "a slot used again")
    other = P.forward(cfg, weights, [(prompt[3] + 1) % 50 if i == 3 else t for i, t in enumerate(prompt)])
    assert (other[-1] - ref[-1]).abs().max() > 1e-3, "the far token does not matter in this test"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_negative_choice_scores_and_groups(root, dtype):
    """Corrections far below zero: every choice score is negative, and an expert outside the kept groups must not win
    with a score that counts as zero."""
    cfg = config([layer("attention", attn(), moe(experts=8, top=3, count=4, keep=2, ff=24))] * 2, width=64, vocab=80)

    def edit(t):
        sharpen(t)
        for i in (0, 1):
            t[f"l{i}.mlp.correction"] = t[f"l{i}.mlp.correction"] - 4.0
    model, weights = make_model(root, cfg, 21, dtype, edit)
    prompt = tokens(cfg, (90,), seed=4)[0]
    compare(run_whole(engine_of(model), prompt), P.forward(cfg, weights, prompt, rounding(dtype)), dtype, "negative choice scores")


@pytest.mark.parametrize("name", sorted(WHOLE_MODELS))
def test_greedy_generation_through_the_session(root, name):
    """`generate` (the scheduler's batches, the sampler, steps fed from device memory) against greedy choices made
    from the plain implementation's logits."""
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
    assert cli.main(["--random", "vufinex-tiny", "--seed", "1", "-n", "4", "--stop-token", "-1", "5 6"]) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(root, tmp_path, dtype):
    """bin/trace_run picks the architecture from config.json: requests whole, with their last tokens one by one, and
    as unequal batches whose shorter requests end earlier; every wanted row against the plain implementation."""
    from safetensors.torch import load_file, save_file
    from inference_engine_rust_b200 import write_random_model
    import test_gpu_trace_run as R
    cfg = TENSOR if dtype == "bfloat16" else FULL
    d = str(tmp_path / "model")
    write_random_model(d, cfg, seed=21, dtype=dtype, std=0.1)
    path = os.path.join(d, "model.safetensors")
    tensors = load_file(path)
    edit_for(dtype)(tensors)
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
    """Prompt steps of up to 512 tokens that want their last rows are captured into a CUDA graph from a shape bucket's
    second use on (padding tokens and padding sequences inside): same logits as the plain statement on every turn, with
    slots, pages and states used again in between, and the tokens after the prompt one by one."""
    cfg = WHOLE_MODELS["tensor" if dtype == "bfloat16" else "full"]
    model, weights = make_model(root, cfg, 17, dtype, edit_for(dtype))
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
