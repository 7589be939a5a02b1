"""Latent attention: keys and values grow out of one short row per token, the only thing the cache keeps.  Two forms,
chosen by the spec's parameters.

Without positions, with a softmax sink (`q_rank` given, `rot_dim` 0):

Queries go through a latent: c_q = RMSnorm(W_dq h) (plain weight), q = W_uq c_q (heads x dim).  Keys and
values come from one shared latent per token, c = RMSnorm(W_dkv h) with kv_rank numbers, the only thing
the cache keeps: k = W_uk c, v = W_uv c per head (dim and vdim may differ).  Causal softmax of
(q . k) * scale with a sink: each head has a learned logit sink_h that only enlarges the denominator by
exp(sink_h), taken unscaled, and adds nothing to the weighted sum; then W_o on the concatenated heads.

A prompt expands k and v for its own tokens and attends over them.  A one-token step attends over the
cached latents in the absorbed form: the query is taken into the latent's coordinates (W_uk^T q), the
scores and the weighted sum are formed on the latents themselves, and W_uv is applied once to the sum,
so nothing is expanded per cached position.

With a rotated part (`rot_dim` R > 0; `q_rank` None: q = W_q h directly; `sink` false; `gate` "head"; `out_scale`): a
query head is [D unrotated | R rotated] numbers, W_dkv h has kv_rank + R rows: the first kv_rank, RMS-normed, are the
latent c, the last R (not normed) are ONE rotated key part that all heads share; head h's key is [W_uk[h] c | that
part], its value W_uv[h] c, the score (q_unrotated . k_unrotated + q_rotated . k_rotated) * scale; the rotation is the
mixer's `position` part (a plain rotary encoding of R numbers, either pairing); `gate` "head" multiplies head h's
result by sigmoid(W_g h)_h.  The cache keeps [c | rotated key part] per position.  One product makes [q | dkv | g] in
fp32; one kernel norms, rotates, rounds once and writes the queries, the cache row and the gates.  A prompt expands
keys and values by ONE product from the cache rows (the matrix carries W_uk and W_uv per head, padded to one head size,
and ones that copy the rotated part into every head's key) and runs the library's prompt attention; a one-token step
runs the absorbed form, in which a cached row serves as the key (all of it) and as the value (its latent part).
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import KVRequest
from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, part_class, register_part
from .linear import Linear


class LatentAttention(Mixer):
    graph_safe = True
    takes_out_scale = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.H, self.D, self.V = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        self.q_rank = int(spec["q_rank"]) if spec.get("q_rank") else None
        self.kv_rank = int(spec["kv_rank"])
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.R = int(spec.get("rot_dim") or 0)
        self.has_sink = bool(spec.get("sink", True))
        self.gate = spec.get("gate")
        self.out_scale = float(spec.get("out_scale", 1.0))
        if self.gate not in (None, "head"):
            raise ValueError(f"latent_attention: gate must be 'head' or None, got {self.gate!r}")
        # the form without positions is the one with a query latent, a sink and nothing else
        self.plain_form = self.q_rank is not None and self.R == 0 and self.gate is None and self.out_scale == 1.0
        if not self.plain_form and (self.q_rank is not None or self.has_sink):
            raise ValueError("latent_attention with a rotated part, a gate or an output factor takes q_rank None and sink false")
        self.inv_freq, self.pairing = None, B.PAIR_HALF
        if self.R:
            pos = spec["position"]
            position = part_class("position", pos.kind)(pos, self.R, rt)
            rot = getattr(position, "rotary_constants", lambda: None)()
            if rot is None or rot[1] != self.R:
                raise ValueError("latent_attention: the position part must be a plain rotation of all rot_dim numbers")
            self.inv_freq, _, self.pairing = rot
        # prompts run the library's attention over heads of one size: the larger of key and value size, in bfloat16 runs
        # rounded up to a multiple of 16 (zeros add nothing to a score and give zero columns of the result)
        self.head = max(self.D + self.R, self.V)
        if rt.fast:
            self.head = -(-self.head // 16) * 16

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, hd, hv = self.hidden_size, self.H * self.D, self.H * self.V
        if not self.plain_form:
            out = {"q": TensorSpec((self.H * (self.D + self.R), h)), "dkv": TensorSpec((self.kv_rank + self.R, h)),
                   "dkv.norm": TensorSpec((self.kv_rank,), "ones_plus_normal"), "uk": TensorSpec((hd, self.kv_rank)),
                   "uv": TensorSpec((hv, self.kv_rank)), "o": TensorSpec((h, hv))}
            if self.gate:
                out["g"] = TensorSpec((self.H, h))
            return out
        return {"dq": TensorSpec((self.q_rank, h)), "dq.norm": TensorSpec((self.q_rank,), "ones_plus_normal"),
                "uq": TensorSpec((hd, self.q_rank)),
                "dkv": TensorSpec((self.kv_rank, h)), "dkv.norm": TensorSpec((self.kv_rank,), "ones_plus_normal"),
                "uk": TensorSpec((hd, self.kv_rank)), "uv": TensorSpec((hv, self.kv_rank)),
                "sink": TensorSpec((self.H,)), "o": TensorSpec((h, hv))}

    def _load_rotated(self, t: Mapping[str, torch.Tensor]) -> None:
        dt, dev = self.rt.dtype, self.rt.device
        H, D, R, V, rank, P = self.H, self.D, self.R, self.V, self.kv_rank, self.head
        rows = [t["q"].to(dt), t["dkv"].to(dt)] + ([t["g"].to(dt)] if self.gate else [])
        w = torch.cat(rows, dim=0)
        pad = -w.shape[0] % 8                     # the tensor-core projection wants output rows of 16 bytes
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=dt, device=w.device)], dim=0)
        self.proj = Linear(w, self.rt)
        self.w_uk, self.w_uv = t["uk"].to(dt).contiguous(), t["uv"].to(dt).contiguous()
        # [keys of all heads | values of all heads] from a cache row [c | rotated part]: per head P rows
        expand = torch.zeros((2 * H * P, rank + R), dtype=dt, device=dev)
        k_rows = expand[:H * P].view(H, P, rank + R)
        k_rows[:, :D, :rank] = self.w_uk.view(H, D, rank)
        for i in range(R):
            k_rows[:, D + i, rank + i] = 1.0
        expand[H * P:].view(H, P, rank + R)[:, :V, :rank] = self.w_uv.view(H, V, rank)
        self.expand = Linear(expand, self.rt)
        self.kv_norm = t["dkv.norm"].to(torch.float32).contiguous()
        self.sink = None
        self.o = Linear(t["o"], self.rt)

    def load(self, t: Mapping[str, torch.Tensor]) -> None:
        if not self.plain_form:
            return self._load_rotated(t)
        dt = self.rt.dtype
        self.down = Linear(torch.cat([t["dq"].to(dt), t["dkv"].to(dt)], dim=0), self.rt)
        self.uq = Linear(t["uq"], self.rt)
        self.ukv = Linear(torch.cat([t["uk"].to(dt), t["uv"].to(dt)], dim=0), self.rt)
        self.w_uk = self.ukv.weight[:self.H * self.D]           # views, for the absorbed form
        self.w_uv = self.ukv.weight[self.H * self.D:]
        self.q_norm, self.kv_norm = t["dq.norm"].to(torch.float32).contiguous(), t["dkv.norm"].to(torch.float32).contiguous()
        self.sink = t["sink"].to(torch.float32).contiguous()
        self.o = Linear(t["o"], self.rt)

    def cache_request(self) -> KVRequest:
        return KVRequest(kv_heads=1, head_dim=self.kv_rank + self.R, window=None, values=False)

    def weight_bytes(self) -> int:
        if not self.plain_form:
            return self.proj.nbytes() + self.w_uk.numel() * self.w_uk.element_size() * 2 + self.o.nbytes()
        return self.down.nbytes() + self.uq.nbytes() + self.ukv.nbytes() + self.o.nbytes()

    def _forward_rotated(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T, H, D, R, V, rank = self.rt, self.rt.workspace, ctx.n_tokens, self.H, self.D, self.R, self.V, self.kv_rank
        kv = cache_view.struct
        proj = ws.take("latent.proj", (T, self.proj.out_features), torch.float32)
        self.proj.apply(xn, proj, T, ctx.stream)
        prompt = ctx.kind == "prompt" and writes_cache
        P = self.head if prompt else D + R
        c_ext = ws.take("latent.c", (T, rank + R), rt.dtype)
        gate = ws.take("latent.gate", (T, H), torch.float32)
        out = ws.take("latent.out", (T, H * V), rt.dtype)
        if prompt:
            qkv = ws.take("latent.qkv", (T, 3 * H * P), rt.dtype)
            q = qkv[:, :H * P]
        else:
            q = ws.take("latent.q", (T, H * P), rt.dtype)
        B.latent_prep(proj, H, D, R, rank, self.kv_norm, self.eps, self.inv_freq, self.pairing, self.out_scale, c_ext, q, P,
                      gate, ctx.batch, kv, writes_cache, rt.err, ctx.stream)
        if prompt:
            self.expand.apply(c_ext, qkv[:, H * P:], T, ctx.stream)
            attn = ws.take("latent.attn", (T, H * P), rt.dtype)
            if not (rt.fast and qkv.dtype == torch.bfloat16 and
                    B.attention_prefill(qkv, attn, ctx.batch, H, H, P, 0, self.scale, ctx.max_q_len, ctx.stream, err=rt.err)):
                own = B.KvView(k=None, v=None, page_table=None, table_width=0, ring_pages=1, page_tokens=1, n_pages=0,
                               kv_heads=H, head_dim=P, dtype=B.dtype_code(qkv.dtype), window=0, chunk=0)
                B.attention_plain(qkv, attn, ctx.batch, own, H, self.scale, False, rt.err, ctx.stream)
            B.head_gate_mul(attn, P, out, V, H, gate, ctx.batch, ctx.stream)
        else:
            done = False
            if rt.fast and q.dtype == torch.bfloat16 and ctx.kind == "decode":
                hpad, splits = B.latent_decode_tc_plan(ctx.n_seqs, H, cache_view.group.table_width)
                qa = ws.take("latent.qa", (T, hpad, rank + R), torch.bfloat16)
                part_m = ws.take("latent.part_m", (T, splits, hpad), torch.float32)
                part_l = ws.take("latent.part_l", (T, splits, hpad), torch.float32)
                part_acc = ws.take("latent.part_acc", (T, splits, hpad, rank), torch.float32)
                done = B.latent_attention_decode_tc(q, self.w_uk, self.w_uv, out, ctx.batch, kv, H, D, V, self.scale, None,
                                                    hpad, splits, qa, part_m, part_l, part_acc, rt.err, ctx.stream,
                                                    rot_dim=R, gate=gate)
            if not done:
                B.latent_attention_decode(q, self.w_uk, self.w_uv, out, ctx.batch, kv, H, D, V, self.scale, None,
                                          rt.err, ctx.stream, rot_dim=R, gate=gate)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True, ctx=ctx)

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        if not self.plain_form:
            return self._forward_rotated(xn, residual, ctx, cache_view, writes_cache)
        rt, ws, T, H, D, V = self.rt, self.rt.workspace, ctx.n_tokens, self.H, self.D, self.V
        kv = cache_view.struct
        lat = ws.take("latent.down", (T, self.q_rank + self.kv_rank), torch.float32)
        self.down.apply(xn, lat, T, ctx.stream)
        cq = ws.take("latent.cq", (T, self.q_rank), rt.dtype)
        c = ws.take("latent.c", (T, self.kv_rank), rt.dtype)
        B.latent_norm_store(lat, self.q_rank, self.kv_rank, self.q_norm, self.kv_norm, self.eps, cq, c, ctx.batch, kv,
                            writes_cache, rt.err, ctx.stream)
        out = ws.take("latent.out", (T, H * V), rt.dtype)
        if ctx.kind == "prompt" and writes_cache:
            qkv = ws.take("latent.qkv", (T, 2 * H * D + H * V), rt.dtype)
            self.uq.apply(cq, qkv[:, :H * D], T, ctx.stream)
            self.ukv.apply(c, qkv[:, H * D:], T, ctx.stream)
            # keys and values of one size: the tensor-core prompt attention (tcgen05 at 64 and 128), with
            # every head its own key/value head and the sink in the denominator
            if not (rt.fast and qkv.dtype == torch.bfloat16 and D == V and
                    B.attention_prefill(qkv, out, ctx.batch, H, H, D, 0, self.scale, ctx.max_q_len, ctx.stream,
                                        err=rt.err, sink=self.sink)):
                B.latent_attention_prompt(qkv, out, ctx.batch, H, D, V, self.scale, self.sink, ctx.stream)
        else:
            q = ws.take("latent.q", (T, H * D), rt.dtype)
            self.uq.apply(cq, q, T, ctx.stream)
            done = False
            if rt.fast and q.dtype == torch.bfloat16 and ctx.kind == "decode":
                hpad, splits = B.latent_decode_tc_plan(ctx.n_seqs, H, cache_view.group.table_width)
                rank = self.kv_rank
                qa = ws.take("latent.qa", (T, hpad, rank), torch.bfloat16)
                part_m = ws.take("latent.part_m", (T, splits, hpad), torch.float32)
                part_l = ws.take("latent.part_l", (T, splits, hpad), torch.float32)
                part_acc = ws.take("latent.part_acc", (T, splits, hpad, rank), torch.float32)
                done = B.latent_attention_decode_tc(q, self.w_uk, self.w_uv, out, ctx.batch, kv, H, D, V, self.scale,
                                                    self.sink, hpad, splits, qa, part_m, part_l, part_acc, rt.err, ctx.stream)
            if not done:
                B.latent_attention_decode(q, self.w_uk, self.w_uv, out, ctx.batch, kv, H, D, V, self.scale, self.sink,
                                          rt.err, ctx.stream)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True)


register_part("mixer", "latent_attention", LatentAttention)
