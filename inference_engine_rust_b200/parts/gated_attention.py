"""Grouped-query attention with biases on the input projections, a weighted RMS norm on every head of q and of k,
a value size that may differ from the query/key size, and a sigmoid gate on the concatenated heads:

    q = W_q h + b_q,  k = W_k h + b_k,  v = W_v h + b_v                       (`bias`: the b's exist)
    q_head <- q_head / rms(q_head) * w_q,  k likewise with w_k                (`qk_norm` "head": weights of length
                                                                               head_dim, the same for all heads; before
                                                                               the rotation)
    rotation by the mixer's position part (a plain rotary encoding, either pairing, any number of rotated dimensions)
    a = softmax(q . k * scale over the visible keys) v                        (causal, optionally a sliding `window`)
    y = W_o (a * sigmoid(W_g h))                                              (`gate`: W_g exists)

Tensors: q, k, v (+ q.b, k.b, v.b), q.norm, k.norm, g, o.  One product makes [q | k | v | g] in fp32; one kernel adds
the biases, norms, rotates, rounds once and writes the packed row and the cache; the library's attention kernels run
on heads padded with zeros to one common size D >= max(head_dim, v_dim) (a multiple of 16 for the tensor-core kernels),
so that keys and values share the paged cache's geometry; one kernel drops the padding and applies the gate; W_o adds
into the residual.  What the padding costs when the sizes differ is the price of running every size on the fast kernels.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import KVRequest
from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, part_class, register_part
from .linear import Linear


class GatedAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.qk_dim = int(spec["head_dim"])
        self.v_dim = int(spec.get("v_dim") or self.qk_dim)
        self.window = spec.get("window")
        self.scale = float(spec["scale"])
        self.eps = float(spec.get("eps", 0.0))
        self.has_bias = bool(spec.get("bias", False))
        self.has_gate = bool(spec.get("gate", False))
        qk_norm = spec.get("qk_norm")
        if qk_norm not in (None, "head"):
            raise ValueError(f"qk_norm must be 'head' or None, got {qk_norm!r}")
        self.qk_norm = qk_norm
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        # the head size of the packed rows and of the cache: both sizes padded to one, which the fast kernels take
        widest = max(self.qk_dim, self.v_dim)
        self.head_dim = -(-widest // 16) * 16 if rt.fast else widest
        pos = spec["position"]
        self.position = part_class("position", pos.kind)(pos, self.qk_dim, rt)
        rot = getattr(self.position, "rotary_constants", lambda: None)()
        if rot is None:
            raise ValueError("gated attention takes a rotary position part")
        self.inv_freq, self.rotary_dim, self.pairing = rot
        self.q_dim = self.heads * self.qk_dim
        self.k_dim = self.kv_heads * self.qk_dim
        self.kv_v_dim = self.kv_heads * self.v_dim
        self.a_dim = self.heads * self.v_dim                   # the concatenated heads
        self.proj = self.o = self.bias = self.wq = self.wk = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h = self.hidden_size
        specs = {"q": TensorSpec((self.q_dim, h)), "k": TensorSpec((self.k_dim, h)), "v": TensorSpec((self.kv_v_dim, h)),
                 "o": TensorSpec((h, self.a_dim))}
        if self.has_bias:
            specs.update({"q.b": TensorSpec((self.q_dim,)), "k.b": TensorSpec((self.k_dim,)), "v.b": TensorSpec((self.kv_v_dim,))})
        if self.qk_norm == "head":
            specs["q.norm"] = TensorSpec((self.qk_dim,), "ones_plus_normal")
            specs["k.norm"] = TensorSpec((self.qk_dim,), "ones_plus_normal")
        if self.has_gate:
            specs["g"] = TensorSpec((self.a_dim, h))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        dt = self.rt.dtype
        rows = [tensors["q"].to(dt), tensors["k"].to(dt), tensors["v"].to(dt)] + ([tensors["g"].to(dt)] if self.has_gate else [])
        self.proj = Linear(torch.cat(rows, dim=0), self.rt)
        self.o = Linear(tensors["o"], self.rt)
        if self.has_bias:
            self.bias = torch.cat([tensors[n].to(torch.float32) for n in ("q.b", "k.b", "v.b")]).contiguous()
        if self.qk_norm == "head":
            self.wq = tensors["q.norm"].to(torch.float32).contiguous()
            self.wk = tensors["k.norm"].to(torch.float32).contiguous()

    def cache_request(self) -> KVRequest:
        return KVRequest(self.kv_heads, self.head_dim, self.window)

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.o.nbytes()

    def cut_by_length_key(self):
        return ("gated_attention", self.heads, self.kv_heads, self.head_dim, self.window, self.rt.fast)

    def cut_by_length(self, pos0, cache_view) -> bool:
        if not self.rt.fast or cache_view is None:
            return False
        from . import fast_attention
        return fast_attention.wants_length_cut(pos0, self.kv_heads, self.heads // self.kv_heads, self.window,
                                               cache_view.group.page_tokens, self.head_dim)

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, ws, T, D = self.rt, self.rt.workspace, ctx.n_tokens, self.head_dim
        kv = cache_view.struct
        n_qkv = self.q_dim + self.k_dim + self.kv_v_dim
        proj = ws.take("gattn.proj", (T, self.proj.out_features), torch.float32)
        self.proj.apply(xn, proj, T, ctx.stream)
        qkv = ws.take("attn.qkv", (T, (self.heads + 2 * self.kv_heads) * D), rt.dtype)
        B.qkv_prep(proj, self.bias, qkv, ctx.batch, kv, self.heads, self.qk_dim, self.v_dim, self.inv_freq, self.rotary_dim,
                   self.pairing, self.wq, self.wk, self.eps, writes_cache, rt.err, ctx.stream)
        out = ws.take("attn.out", (T, self.heads * D), rt.dtype)
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
            B.attention_plain(qkv, out, ctx.batch, kv, self.heads, self.scale, from_cache, rt.err, ctx.stream)
        if self.has_gate or D != self.v_dim:
            gated = ws.take("gattn.gated", (T, self.a_dim), rt.dtype)
            B.gate_mul(out, proj[:, n_qkv:] if self.has_gate else None, gated, T, self.heads, D, self.v_dim, ctx.stream)
            out = gated
        self.o.apply(out, residual, T, ctx.stream, add_residual=True, ctx=ctx)


register_part("mixer", "gated_attention", GatedAttention)
