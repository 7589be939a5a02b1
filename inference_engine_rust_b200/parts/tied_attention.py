"""Grouped-query attention whose keys double as values, over the paged cache.

There is no value projection: v = k as projected, before any norm or rotation.  Queries and keys then get
one of two norms, both fp32 and both without a mean:

    qk_norm "whole"  q and k are each divided by the root mean square over their WHOLE projection (all
                     heads at once) and multiplied by a weight of that length (tensors `q.norm`, `k.norm`),
                     before the rotation
    qk_norm "head"   after the rotation every head of q and k is divided by its own root mean square, no weight
    qk_norm None     neither

rotation by the mixer's position part (a plain rotary encoding: its constants are handed to the
preparation kernel), scores (q . k) * scale, optionally capped (`softcap` c: s <- c tanh(s / c)), a sliding
window and / or a mask of chunks (`chunk` C: a position sees the earlier positions p with p // C equal to its own,
chunks counted from the start of the sequence), softmax, optionally with a sink (`sink: true`: one more term of score 0 in the denominator that carries
no value), W_o on the concatenated heads.  `out_scale` multiplies the mixer's result (it is applied to the
values, in which the result is linear).

Tensors: q [heads*dim, hidden], k [kv_heads*dim, hidden], o [hidden, heads*dim], and the two norm weights.
One product makes [q | k] in fp32; one kernel norms, rotates, rounds once and writes the packed row
[q' | k' | v] and the cache; then the attention kernels of the plain attention mixer; then W_o added into
the residual.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import KVRequest
from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, part_class, register_part
from .linear import Linear

_NORM_MODES = {None: B.NORM_NONE, "whole": B.NORM_WHOLE_WEIGHTED, "head": B.NORM_HEAD_UNIT}


class TiedKVAttention(Mixer):
    graph_safe = True
    takes_out_scale = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = spec.get("window")
        self.chunk = spec.get("chunk")
        self.scale = float(spec["scale"])
        self.softcap = float(spec.get("softcap") or 0.0)
        self.eps = float(spec.get("eps", 0.0))
        self.out_scale = float(spec.get("out_scale", 1.0))
        qk_norm = spec.get("qk_norm")
        if qk_norm not in _NORM_MODES:
            raise ValueError(f"qk_norm must be one of {sorted(k for k in _NORM_MODES if k)} or None, got {qk_norm!r}")
        self.qk_norm = qk_norm
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        pos = spec["position"]
        self.position = part_class("position", pos.kind)(pos, self.head_dim, rt)
        rot = getattr(self.position, "rotary_constants", lambda: None)()
        if rot is None or rot[2] != B.PAIR_HALF:
            raise ValueError("attention with tied keys and values takes a rotary position part with the 'half' pairing")
        self.inv_freq, self.rotary_dim, _ = rot
        self.has_sink = bool(spec.get("sink", False))
        self.sink = torch.zeros(self.heads, dtype=torch.float32, device=rt.device) if self.has_sink else None
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.qk = self.o = self.wq = self.wk = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h = self.hidden_size
        specs = {"q": TensorSpec((self.q_dim, h)), "k": TensorSpec((self.kv_dim, h)), "o": TensorSpec((h, self.q_dim))}
        if self.qk_norm == "whole":
            specs["q.norm"] = TensorSpec((self.q_dim,), "ones_plus_normal")
            specs["k.norm"] = TensorSpec((self.kv_dim,), "ones_plus_normal")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        dt = self.rt.dtype
        self.qk = Linear(torch.cat([tensors["q"].to(dt), tensors["k"].to(dt)], dim=0), self.rt)
        self.o = Linear(tensors["o"], self.rt)
        if self.qk_norm == "whole":
            self.wq = tensors["q.norm"].to(torch.float32).contiguous()
            self.wk = tensors["k.norm"].to(torch.float32).contiguous()

    def cache_request(self) -> KVRequest:
        return KVRequest(self.kv_heads, self.head_dim, self.window, chunk=self.chunk)

    def weight_bytes(self) -> int:
        return self.qk.nbytes() + self.o.nbytes()

    def cut_by_length_key(self):
        return ("tied_attention", self.heads, self.kv_heads, self.head_dim, self.window, self.chunk, self.rt.fast)

    def cut_by_length(self, pos0, cache_view) -> bool:
        if not self.rt.fast or cache_view is None:
            return False
        from . import fast_attention
        return fast_attention.wants_length_cut(pos0, self.kv_heads, self.heads // self.kv_heads, self.window,
                                               cache_view.group.page_tokens, self.head_dim, chunk=self.chunk)

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T = self.rt, self.rt.workspace, ctx.n_tokens
        kv = cache_view.struct
        proj = ws.take("tied.proj", (T, self.q_dim + self.kv_dim), torch.float32)
        self.qk.apply(xn, proj, T, ctx.stream)
        qkv = ws.take("attn.qkv", (T, self.q_dim + 2 * self.kv_dim), rt.dtype)
        B.qk_prep(proj, qkv, ctx.batch, kv, self.heads, self.inv_freq, self.rotary_dim, _NORM_MODES[self.qk_norm],
                  self.wq, self.wk, self.eps, self.out_scale, writes_cache, rt.err, ctx.stream)
        out = ws.take("attn.out", (T, self.q_dim), rt.dtype)
        from_cache = ctx.kind == "decode" or not writes_cache
        if from_cache and ctx.kind == "prompt":
            cap = cache_view.group.ring_capacity
            if ctx.max_kv_len > cap:
                raise ValueError(f"a prompt of {ctx.max_kv_len} tokens cannot attend over a shared windowed cache "
                                 f"that keeps {cap} positions")
        done = False
        if rt.fast:
            from . import fast_attention
            done = fast_attention.apply(self, qkv, out, ctx, cache_view, from_cache)
        if not done:
            B.attention_plain(qkv, out, ctx.batch, kv, self.heads, self.scale, from_cache, rt.err, ctx.stream,
                              softcap=self.softcap, sink=self.sink)
        self.o.apply(out, residual, T, ctx.stream, add_residual=True)


register_part("mixer", "tied_kv_attention", TiedKVAttention)
