"""Mixers that keep a matrix state per head instead of a cache of keys: the gated delta rule, the
mLSTM and the recurrence with a decay per key channel and token shift ("wkv").  The state (fp32) lives in the sequence's slot of the cache's state storage, starts at zero and
is carried from step to step; a prompt and a single token run the same kernels.

Both: one product for the wide projections [q; k; v; g] (run dtype), one small product with fp32
outputs for what enters the recurrence's gates, the recurrence itself over the step's tokens
(`csrc/recurrent.cu`, compiled per key size), a per-head RMS norm of the read-out times a weight times
an activation of g, and the output projection added to the residual.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import StateRequest
from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, register_part
from .linear import Linear


def _stack(rt: Runtime, parts, multiple: int = 8) -> torch.Tensor:
    """Row-concatenated matrices in the run's dtype, zero rows added up to a multiple of `multiple` (the
    tensor-core projection wants output rows of 16 bytes)."""
    w = torch.cat([p.to(rt.dtype) for p in parts], dim=0)
    pad = -w.shape[0] % multiple
    if pad:
        w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
    return w


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


class GatedDelta(Mixer):
    """Gated delta rule.  q, k (kv_heads x dim) and v (heads x vdim) pass a short causal convolution per
    channel and SiLU; q and k become unit vectors per head (q also times dim^-1/2); per head and token
    beta = sigmoid(W_b h) and the decay g = exp(-exp(A_log) softplus(W_a h + dt_bias)); then

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

    (head h reads q/k head h // (heads / kv_heads)); o / rms(o) per head times `norm` [vdim] times
    silu(W_g h), then W_o.  State per sequence: S [heads, dim, vdim] and the convolution's last inputs."""
    graph_safe = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.H, self.G = int(spec["heads"]), int(spec["kv_heads"])
        self.D, self.V, self.taps = int(spec["dim"]), int(spec["vdim"]), int(spec["conv"])
        self.eps = float(spec["eps"])
        if self.H % self.G:
            raise ValueError(f"heads {self.H} is not a multiple of kv_heads {self.G}")
        self.C = 2 * self.G * self.D + self.H * self.V            # channels that pass the convolution
        self.s_floats = self.H * self.D * self.V

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, gd, hv = self.hidden_size, self.G * self.D, self.H * self.V
        return {"q": TensorSpec((gd, h)), "q.conv": TensorSpec((gd, self.taps)),
                "k": TensorSpec((gd, h)), "k.conv": TensorSpec((gd, self.taps)),
                "v": TensorSpec((hv, h)), "v.conv": TensorSpec((hv, self.taps)),
                "b": TensorSpec((self.H, h)), "a": TensorSpec((self.H, h)), "A_log": TensorSpec((self.H,)),
                "dt_bias": TensorSpec((self.H,)), "norm": TensorSpec((self.V,), "ones_plus_normal"),
                "g": TensorSpec((hv, h)), "o": TensorSpec((h, hv))}

    def load(self, t: Mapping[str, torch.Tensor]) -> None:
        self.proj = Linear(_stack(self.rt, [t["q"], t["k"], t["v"], t["g"]]), self.rt)
        self.gates = Linear(_stack(self.rt, [t["b"], t["a"]], 4), self.rt)
        self.conv_w = _f32(torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0))
        self.A_log, self.dt_bias, self.norm = _f32(t["A_log"]), _f32(t["dt_bias"]), _f32(t["norm"])
        self.o = Linear(t["o"], self.rt)

    def cache_request(self) -> StateRequest:
        return StateRequest((self.s_floats + self.taps * self.C,), torch.float32)

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.gates.nbytes() + self.o.nbytes()

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T, H, V = self.rt, self.rt.workspace, ctx.n_tokens, self.H, self.V
        proj = ws.take("delta.proj", (T, self.proj.out_features), rt.dtype)
        self.proj.apply(xn, proj, T, ctx.stream)
        gates = ws.take("delta.gates", (T, self.gates.out_features), torch.float32)
        self.gates.apply(xn, gates, T, ctx.stream)
        state = cache_view.state
        qkv = ws.take("delta.qkv", (T, self.C), torch.float32)
        beta = ws.take("delta.beta", (T, H), torch.float32)
        decay = ws.take("delta.decay", (T, H), torch.float32)
        B.delta_prep(proj, gates, self.conv_w, self.A_log, self.dt_bias, state, self.s_floats, qkv, beta, decay,
                     self.G, self.D, H, V, self.taps, ctx.batch, ctx.stream)
        o = ws.take("delta.readout", (T, H * V), torch.float32)
        B.delta_recur(qkv, beta, decay, state, 0, o, self.G, self.D, H, V, ctx.batch, ctx.stream)
        out = ws.take("delta.out", (T, H * V), rt.dtype)
        B.gated_head_norm(o, proj, self.C, self.norm, True, 0, self.eps, out, T, H, V, ctx.stream)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True)


class MLstm(Mixer):
    """Matrix memory of the xLSTM.  q = W_q h dim^-1/2, k = W_k h (heads x dim), v = W_v h (heads x vdim);
    per head the log input gate i = cap tanh((W_i h + b_i) / cap) and the log forget gate
    f = logsigmoid(cap tanh((W_f h + b_f) / cap)); with a running maximum m that starts at 0

        m' = max(f + m, i);   S <- e^(f+m-m') S + e^(i-m') k v^T;   n likewise with k alone;
        o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)

    o / rms(o) per head times `norm` [heads * vdim] times sigmoid(W_g h), then W_o.  State per sequence:
    S [heads, dim, vdim], n [heads, dim], m [heads]."""
    graph_safe = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.H, self.D, self.V = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        self.cap, self.eps = float(spec["gate_cap"]), float(spec["eps"])
        self.s_floats = self.H * self.D * self.V

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, hd, hv = self.hidden_size, self.H * self.D, self.H * self.V
        return {"q": TensorSpec((hd, h)), "k": TensorSpec((hd, h)), "v": TensorSpec((hv, h)), "g": TensorSpec((hv, h)),
                "o": TensorSpec((h, hv)), "norm": TensorSpec((hv,), "ones_plus_normal"),
                "i": TensorSpec((self.H, h)), "i.b": TensorSpec((self.H,)),
                "f": TensorSpec((self.H, h)), "f.b": TensorSpec((self.H,))}

    def load(self, t: Mapping[str, torch.Tensor]) -> None:
        self.proj = Linear(_stack(self.rt, [t["q"], t["k"], t["v"], t["g"]]), self.rt)
        self.gates = Linear(_stack(self.rt, [t["i"], t["f"]], 4), self.rt)
        self.bi, self.bf, self.norm = _f32(t["i.b"]), _f32(t["f.b"]), _f32(t["norm"])
        self.o = Linear(t["o"], self.rt)

    def cache_request(self) -> StateRequest:
        return StateRequest((self.s_floats + self.H * self.D + self.H,), torch.float32)

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.gates.nbytes() + self.o.nbytes()

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T, H, D, V = self.rt, self.rt.workspace, ctx.n_tokens, self.H, self.D, self.V
        proj = ws.take("mlstm.proj", (T, self.proj.out_features), rt.dtype)
        self.proj.apply(xn, proj, T, ctx.stream)
        gates = ws.take("mlstm.gates", (T, self.gates.out_features), torch.float32)
        self.gates.apply(xn, gates, T, ctx.stream)
        coef = ws.take("mlstm.coef", (T, H, 3), torch.float32)
        o = ws.take("mlstm.readout", (T, H * V), torch.float32)
        B.mlstm_recur(proj, gates, self.bi, self.bf, self.cap, cache_view.state, 0, self.s_floats,
                      self.s_floats + H * D, coef, o, D, H, V, ctx.batch, ctx.stream)
        out = ws.take("mlstm.out", (T, H * V), rt.dtype)
        B.gated_head_norm(o, proj, 2 * H * D + H * V, self.norm, False, 1, self.eps, out, T, H, V, ctx.stream)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True)


class Wkv(Mixer):
    """Matrix state with a decay per key channel and token shift.  With h' the input row in front of a token's own h
    (zeros in front of a sequence's first), each of r, k, v, g, w reads its own mix h + (h' - h) mu; r, k, v = W_r, W_k, W_v
    of their mixes (heads x dim), gate = silu(W_g .); decay w = exp(-exp(W_w2 tanh(W_w1 .) + w0)) per head and key channel;
    per head

        o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T

    o / rms(o) per head times `norm` [heads * dim] times the gate (times `out_scale`), then W_o.  State per sequence:
    S [heads, dim, dim] and the last input row.  The projections have fp32 outputs; shift, decay, state, read-out,
    norm and gate are fp32."""
    graph_safe = True
    takes_out_scale = True
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.H, self.D = int(spec["heads"]), int(spec["dim"])
        self.eps = float(spec["eps"])
        self.out_scale = float(spec.get("out_scale", 1.0))
        self.lora = spec.get("decay_rank")          # None: taken from the stored matrices
        self.s_floats = self.H * self.D * self.D

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, hd = self.hidden_size, self.H * self.D
        # the inner size of the decay's two matrices: the spec's `decay_rank`, or whatever the stored tensors have
        L, free = (int(self.lora), False) if self.lora else (max(8, (h // 16 + 7) // 8 * 8), True)
        out = {f"mu.{m}": TensorSpec((h,)) for m in self.MIXES}
        out.update({"r": TensorSpec((hd, h)), "k": TensorSpec((hd, h)), "v": TensorSpec((hd, h)), "g": TensorSpec((hd, h)),
                    "w1": TensorSpec((L, h), free_dims=(0,) if free else ()),
                    "w2": TensorSpec((hd, L), free_dims=(1,) if free else ()), "w0": TensorSpec((hd,)), "u": TensorSpec((self.H, self.D)),
                    "norm": TensorSpec((hd,), "ones_plus_normal"), "o": TensorSpec((h, hd))})
        return out

    def load(self, t: Mapping[str, torch.Tensor]) -> None:
        self.mu = _f32(torch.stack([t[f"mu.{m}"] for m in self.MIXES], dim=0))
        self.proj = [Linear(t[m], self.rt) for m in ("r", "k", "v", "g")]
        self.L = t["w1"].shape[0]
        if t["w2"].shape[1] != self.L:
            raise ValueError(f"wkv: w1 has {self.L} rows but w2 has {t['w2'].shape[1]} columns")
        self.w1 = Linear(_stack(self.rt, [t["w1"]], 4), self.rt)
        self.w2t = _f32(t["w2"].to(torch.float32).t())
        self.w0, self.u, self.norm = _f32(t["w0"]), _f32(t["u"]), _f32(t["norm"])
        self.o = Linear(t["o"], self.rt)

    def cache_request(self) -> StateRequest:
        return StateRequest((self.s_floats + self.hidden_size,), torch.float32)

    def weight_bytes(self) -> int:
        return sum(p.nbytes() for p in self.proj) + self.w1.nbytes() + self.w2t.numel() * 4 + self.o.nbytes()

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T, H, D = self.rt, self.rt.workspace, ctx.n_tokens, self.H, self.D
        hd, state = H * D, cache_view.state
        mixed = ws.take("wkv.mixed", (len(self.MIXES), T, self.hidden_size), rt.dtype)
        B.token_shift(xn, state, self.s_floats, self.mu, mixed, ctx.batch, ctx.stream)
        x = ws.take("wkv.proj", (T, 4 * hd), torch.float32)
        for i, lin in enumerate(self.proj):
            lin.apply(mixed[i], x[:, i * hd:(i + 1) * hd], T, ctx.stream)
        z = ws.take("wkv.lora", (T, self.w1.out_features), torch.float32)
        self.w1.apply(mixed[4], z, T, ctx.stream)
        decay = ws.take("wkv.decay", (T, hd), torch.float32)
        B.wkv_decay(z, self.L, self.w2t, self.w0, decay, xn, state, self.s_floats, ctx.batch, ctx.stream)
        o = ws.take("wkv.readout", (T, hd), torch.float32)
        B.wkv_recur(x, decay, self.u, state, 0, o, D, H, D, ctx.batch, ctx.stream)
        out = ws.take("wkv.out", (T, hd), rt.dtype)
        B.wkv_finish(o, x[:, 3 * hd:], self.norm, self.eps, self.out_scale, out, ctx.batch, H, D, ctx.stream)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True, ctx=ctx)


register_part("mixer", "wkv", Wkv)
register_part("mixer", "gated_delta", GatedDelta)
register_part("mixer", "mlstm", MLstm)
