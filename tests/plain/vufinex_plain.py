"""Plain, slow statement of the Vufinex decoder: whole sequences, no cache, no batching, one
function per mechanism, CPU float32.  It shares no code with the package under test.

Notation: x is the [tokens, width] residual of one sequence, W matrices are [out, in] and are
applied as x W^T, t and j run over tokens in order, positions count from 0.  `rnd` is where an
engine that stores activations in bfloat16 rounds them (identity for the 32-bit statement).

A layer:   x <- x + m * mixer(N1(x));   x <- x + m * ff(N2(x))      (m: one factor for the whole model)
N(x) = x / sqrt(mean(x^2) + eps) * (1 + w).  A layer may run with another layer's tensors.
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


def lin(h: Tensor, w: Tensor) -> Tensor:
    return h.float() @ w.float().t()


# ---------------------------------------------------------------------------------------
# norms


def unit_rms(y: Tensor, eps: float) -> Tensor:
    y = y.float()
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def layer_norm(x: Tensor, w: Tensor, eps: float) -> Tensor:
    """The layers' norm: the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w.float())


# ---------------------------------------------------------------------------------------
# rotations: v [tokens, heads, dim]; the first `dims` numbers of a head turn, the rest pass


def _angles(T: int, dims: int, base: float, first_position: int):
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = (torch.tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)).float()
    pos = torch.arange(first_position, first_position + T, dtype=torch.float32)
    ang = pos[:, None] * freq[None, :]
    return torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]


def rotate_halves(v: Tensor, dims: int, base: float, first_position: int = 0) -> Tensor:
    """Number i turns together with number i + dims/2."""
    out = v.clone().float()
    half = dims // 2
    if half == 0:
        return out
    c, s = _angles(v.shape[0], dims, base, first_position)
    a, b = v[..., :half].float(), v[..., half:dims].float()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def rotate_neighbours(v: Tensor, dims: int, base: float, first_position: int = 0) -> Tensor:
    """Number 2i turns together with number 2i + 1."""
    out = v.clone().float()
    if dims // 2 == 0:
        return out
    c, s = _angles(v.shape[0], dims, base, first_position)
    a, b = v[..., 0:dims:2].float(), v[..., 1:dims:2].float()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------
# softmax attention under a visibility rule


def masked_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, sees: Callable[[int, int], bool]) -> Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H/G); token t sees
    token j when sees(t, j); ordinary softmax over what it sees.  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2])
    for h in range(H):
        g = h // (H // G)
        for t in range(T):
            js = [j for j in range(t + 1) if sees(t, j)]
            s = (k[js, g].float() @ q[t, h].float()) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[js, g].float()
    return out


def chunk_rule(size: Optional[int]) -> Callable[[int, int], bool]:
    """Inside one chunk of `size` positions counted from the start of the sequence, and not ahead."""
    if not size:
        return lambda t, j: j <= t
    return lambda t, j: j <= t and t // size == j // size


def chunked_attention(h: Tensor, w: Mapping[str, Tensor], m: Mapping, rnd: Round = exact) -> Tensor:
    """Grouped-query attention whose values are the keys as projected; rotation of halves on q and k."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = lin(h, w["q"]).view(T, H, d)
    k = lin(h, w["k"]).view(T, G, d)
    v = rnd(k)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rnd(rotate_halves(q, rot["dims"], rot["base"]))
    k = rnd(rotate_halves(k, rot["dims"], rot["base"]))
    o = masked_attention(q, k, v, m["scale"], chunk_rule((m.get("mask") or {}).get("size")))
    return lin(rnd(o.reshape(T, H * d)), w["o"])


def latent_attention(h: Tensor, w: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact) -> Tensor:
    """Keys and values grow out of one short row c per token; beside it one rotated key part that all heads share;
    a sigmoid gate per head on the result."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = lin(h, w["q"]).view(T, H, d + r)
    down = lin(h, w["dkv"])
    c = rnd(unit_rms(down[:, :rank], eps) * w["dkv.norm"].float())
    base = (m.get("rot") or {}).get("base", 1.0)
    k_rot = rotate_neighbours(down[:, None, rank:], r, base)            # [T, 1, r]
    q = torch.cat([q[..., :d], rotate_neighbours(q[..., d:], r, base)], dim=-1)
    k = torch.cat([lin(c, w["uk"]).view(T, H, d), k_rot.expand(T, H, r)], dim=-1)
    v = lin(c, w["uv"]).view(T, H, dv)
    o = masked_attention(rnd(q), rnd(k), rnd(v), m["scale"], lambda t, j: j <= t)
    gate = torch.sigmoid(lin(h, w["g"]))                                                # [T, H]
    return lin(rnd((o * gate[:, :, None]).reshape(T, H * dv)), w["o"])


# ---------------------------------------------------------------------------------------
# the recurrence with a matrix state per head


def wkv_mixer(h: Tensor, w: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round = exact,
              state: Optional[Tensor] = None, before: Optional[Tensor] = None) -> Tensor:
    """Each of r, k, v, g, w reads h_t + (h_(t-1) - h_t) mu;  decay_t = exp(-exp(W_w2 tanh(W_w1 .) + w0));
    o_t = (S + diag(u) k_t v_t^T)^T r_t;  S <- diag(decay_t) S + k_t v_t^T;  per head o / rms(o), times a weight,
    times silu(gate), then W_o.  `state` [H, d, d] (changed in place) and `before` (the row in front) continue a
    sequence; both start at zero."""
    T, width = h.shape
    H, d = m["heads"], m["dim"]
    h = h.float()
    prev = torch.cat([torch.zeros(1, width) if before is None else before.float().view(1, width), h[:-1]], dim=0)

    def mixed(name):
        return rnd(h + (prev - h) * w["mu." + name].float())

    r = lin(mixed("r"), w["r"]).view(T, H, d)
    k = lin(mixed("k"), w["k"]).view(T, H, d)
    v = lin(mixed("v"), w["v"]).view(T, H, d)
    g = lin(mixed("g"), w["g"])
    gate = g * torch.sigmoid(g)
    lora = torch.tanh(lin(mixed("w"), w["w1"]))
    decay = torch.exp(-torch.exp(lin(lora, w["w2"]) + w["w0"].float())).view(T, H, d)
    u = w["u"].float()
    S = torch.zeros(H, d, d) if state is None else state
    o = torch.zeros(T, H, d)
    for t in range(T):
        for a in range(H):
            kv = torch.outer(k[t, a], v[t, a])
            o[t, a] = (S[a] + u[a][:, None] * kv).t() @ r[t, a]
            S[a] = decay[t, a][:, None] * S[a] + kv
    y = unit_rms(o, eps).reshape(T, H * d) * w["norm"].float() * gate
    return lin(rnd(y), w["o"])


# ---------------------------------------------------------------------------------------
# mixture of experts


def route(z: Tensor, correction: Tensor, top: int, groups: int, keep: int, scale: float):
    """z [T, E] router outputs.  s = sigmoid(z); the choice is made on s + correction, inside the `keep` groups (of
    `groups` equal runs of neighbours) whose two best choice scores add up highest; the weights are the chosen s over
    their sum, times `scale`.  Returns (indices [T, top], weights [T, top])."""
    T, E = z.shape
    s = torch.sigmoid(z.float())
    choice = s + correction.float()
    per = E // groups
    idx = torch.zeros(T, top, dtype=torch.long)
    wt = torch.zeros(T, top)
    for t in range(T):
        score = []
        for gi in range(groups):
            best = sorted(choice[t, gi * per:(gi + 1) * per].tolist(), reverse=True)
            score.append(sum(best[:2]))
        kept = sorted(range(groups), key=lambda gi: (-score[gi], gi))[:keep]
        allowed = [e for e in range(E) if e // per in kept]
        chosen = sorted(allowed, key=lambda e: (-float(choice[t, e]), e))[:top]
        idx[t] = torch.tensor(chosen)
        picked = s[t, chosen]
        wt[t] = picked / (picked.sum() + 1e-20) * scale
    return idx, wt


def expert(h: Tensor, gate: Tensor, up: Tensor, down: Tensor, rnd: Round = exact) -> Tensor:
    a = lin(h, gate)
    return lin(rnd(a * torch.sigmoid(a) * lin(h, up)), down)


def moe_ff(h: Tensor, w: Mapping[str, Tensor], mlp: Mapping, rnd: Round = exact) -> Tensor:
    r = mlp["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    idx, wt = route(lin(h, w["router"]), w["correction"], r["top"], g["count"], g["keep"], r["scale"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0])
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t].tolist()):
            out[t] += a * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], rnd)[0]
    return out


# ---------------------------------------------------------------------------------------
# the model


def sub(weights: Mapping[str, Tensor], prefix: str) -> Dict[str, Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def owner(cfg: Mapping, i: int) -> int:
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def mixer(kind: str, h: Tensor, w: Mapping[str, Tensor], m: Mapping, eps: float, rnd: Round) -> Tensor:
    if kind == "attention":
        return chunked_attention(h, w, m, rnd)
    if kind == "wkv":
        return wkv_mixer(h, w, m, eps, rnd)
    if kind == "latent_attention":
        return latent_attention(h, w, m, eps, rnd)
    raise ValueError(kind)


def forward(cfg: Mapping, weights: Mapping[str, Tensor], tokens, rnd: Round = exact, residuals: Optional[list] = None) -> Tensor:
    """Logits [tokens, vocab] of one sequence.  `residuals`, if a list, receives x after every layer."""
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = weights["embed"].float()[tok] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner(cfg, i)}."
        h = rnd(layer_norm(x, weights[p + "norm1"], eps))
        x = x + mult * mixer(layer["type"], h, sub(weights, p + "mix."), layer["mixer"], eps, rnd)
        if layer.get("mlp") is not None:
            h = rnd(layer_norm(x, weights[p + "norm2"], eps))
            x = x + mult * moe_ff(h, sub(weights, p + "mlp."), layer["mlp"], rnd)
        if residuals is not None:
            residuals.append(x.clone())
    hn = rnd(layer_norm(x, weights["final.norm"], eps))
    return lin(hn, weights["head"])
