"""Plain, slow statement of the Kuvelix decoder: whole sequences, no cache, no batching, one
function per mechanism, CPU float32.  It shares no code with the package under test.

Notation: x is the [tokens, width] residual of one sequence, W matrices are [out, in] and are
applied as x W^T, t and j run over tokens in order, positions count from 0.  `rnd` is where an
engine that stores activations in bfloat16 rounds them (identity for the 32-bit statement).

A layer has ONE norm, read by both sublayers:   h = N(x);   x <- x + mixer(h) + ff(h).
A run of layers [start, stop) is executed `times` times in a row with the same weights.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Mapping, Optional

import torch

Tensor = torch.Tensor
Round = Callable[[Tensor], Tensor]


def exact(t: Tensor) -> Tensor:
    return t


def bf16(t: Tensor) -> Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def lin(h: Tensor, w: Tensor, b: Optional[Tensor] = None) -> Tensor:
    y = h.float() @ w.float().t()
    return y if b is None else y + b.float()


# ---------------------------------------------------------------------------------------
# norm


def rms_norm(y: Tensor, w: Tensor, eps: float) -> Tensor:
    """y / sqrt(mean(y^2) + eps) * w over the last axis; the weight multiplies plainly."""
    y = y.float()
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w.float()


# ---------------------------------------------------------------------------------------
# rotation


def rotate_pairs(v: Tensor, dims: int, base: float, factor: float = 1.0, first_position: int = 0) -> Tensor:
    """v [tokens, heads, dim]: of every head's first `dims` numbers, number 2i and number 2i+1 are turned
    together by the angle position * base^(-2i/dims) / factor; the rest pass."""
    T = v.shape[0]
    out = v.clone().float()
    half = dims // 2
    if half == 0:
        return out
    i = torch.arange(half, dtype=torch.float64)
    freq = (torch.tensor(base, dtype=torch.float64) ** (-2.0 * i / dims) / factor).float()
    pos = torch.arange(first_position, first_position + T, dtype=torch.float32)
    ang = pos[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2].float(), v[..., 1:dims:2].float()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------
# attention


def causal_attention(q: Tensor, k: Tensor, v: Tensor, scale: float) -> Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H/G); token t sees
    tokens j <= t; ordinary softmax.  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2])
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            s = (k[: t + 1, g] @ q[t, h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[: t + 1, g]
    return out


def gated_attention(h: Tensor, w: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact,
                    first_position: int = 0) -> Tensor:
    """The mixer: projections with biases, one weighted RMS norm per head of q and of k (the weight shared by the
    heads), rotation of pairs, softmax attention, the heads times sigmoid(W_g h), W_o."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, w["q"], w["q.b"]).view(T, H, d)
    k = lin(h, w["k"], w["k.b"]).view(T, G, d)
    v = rnd(lin(h, w["v"], w["v.b"])).view(T, G, dv)
    q, k = rms_norm(q, w["q.norm"], eps), rms_norm(k, w["k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_pairs(q, rot["dims"], rot["base"], factor, first_position)
        k = rotate_pairs(k, rot["dims"], rot["base"], factor, first_position)
    q, k = rnd(q), rnd(k)
    a = rnd(causal_attention(q, k, v, m["scale"])).reshape(T, H * dv)
    gate = torch.sigmoid(rnd(lin(h, w["g"])))
    return lin(rnd(a * gate), w["o"])


# ---------------------------------------------------------------------------------------
# feed-forwards


def gelu_tanh(z: Tensor) -> Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_ff(h: Tensor, w: Mapping[str, Tensor], rnd: Round = exact) -> Tensor:
    return lin(rnd(gelu_tanh(lin(h, w["gate"])) * lin(h, w["up"])), w["down"])


def clamped_expert(h: Tensor, gate: Tensor, up: Tensor, down: Tensor, limit: float, rnd: Round = exact) -> Tensor:
    g = torch.clamp(lin(h, gate), max=limit)
    u = torch.clamp(lin(h, up), min=-limit, max=limit)
    return lin(rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0)), down)


def route(z: Tensor, correction: Tensor, top: int, groups: int, keep: int):
    """z [T, N] router logits over experts and identity experts together.  s = softmax(z); the choice is made on
    s + correction, within the `keep` groups (of `groups` equal runs of neighbours) whose largest choice score
    is largest; the weights are the chosen s over their sum.  Returns (indices [T, top], weights [T, top])."""
    T, N = z.shape
    s = torch.softmax(z.float(), dim=-1)
    c = s + correction.float()
    per = N // groups
    best = c.view(T, groups, per).max(dim=-1).values
    kept = torch.zeros(T, groups, dtype=torch.bool)
    for t in range(T):                                     # the first of equal scores wins
        order = sorted(range(groups), key=lambda g: (-float(best[t, g]), g))[:keep]
        kept[t, order] = True
    allowed = kept[:, :, None].expand(T, groups, per).reshape(T, N)
    c = torch.where(allowed, c, torch.full_like(c, -math.inf))
    idx = torch.zeros(T, top, dtype=torch.long)
    for t in range(T):
        idx[t] = torch.tensor(sorted(range(N), key=lambda e: (-float(c[t, e]), e))[:top])
    chosen = torch.gather(s, 1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h: Tensor, w: Mapping[str, Tensor], mlp: Mapping, rnd: Round = exact, router_input: Optional[Tensor] = None) -> Tensor:
    """Experts 0 .. experts-1 have tensors; router outputs experts .. experts+identity-1 stand for experts that
    return their input."""
    r = mlp["router"]
    E, I = r["experts"], r.get("identity", 0)
    z = lin(h if router_input is None else router_input, w["router"])
    idx, wt = route(z, w["correction"], r["top"], r["groups"]["count"], r["groups"]["keep"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0] if E else h.shape[1])
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t].tolist()):
            if e >= E:
                out[t] += a * h[t].float()
            else:
                out[t] += a * clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                             mlp["expert"]["limit"], rnd)[0]
    return out


# ---------------------------------------------------------------------------------------
# the model


def sub(weights: Mapping[str, Tensor], prefix: str) -> Dict[str, Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_runs(cfg: Mapping) -> List[int]:
    """The layers in the order they run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: Mapping, weights: Mapping[str, Tensor], tokens, rnd: Round = exact, residuals: Optional[list] = None) -> Tensor:
    """Logits [tokens, vocab] of one sequence.  `residuals`, if a list, receives x after every layer run."""
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = rms_norm(weights["embed"].float()[tok], weights["embed.norm"], eps)
    for i in layer_runs(cfg):
        layer = cfg["layers"][i]
        h = rnd(rms_norm(x, weights[f"l{i}.norm1"], eps))
        y = gated_attention(h, sub(weights, f"l{i}.mix."), layer["mixer"], eps, rnd)
        mlp = layer.get("mlp")
        if mlp is not None:
            w = sub(weights, f"l{i}.mlp.")
            y = y + (dense_ff(h, w, rnd) if mlp["kind"] == "dense" else moe_ff(h, w, mlp, rnd))
        x = x + y
        if residuals is not None:
            residuals.append(x.clone())
    hn = rnd(rms_norm(x, weights["final.norm"], eps))
    return lin(hn, weights["embed"])
