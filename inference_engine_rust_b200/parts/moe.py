"""Mixture-of-experts feed-forward: `experts` small gated feed-forwards W_down (silu(W_gate h) * (W_up h)),
of which each token uses the `top` with the largest router logits z = W_r h + b (fp32), weighted by the
softmax over the chosen logits only; plus, optionally, a shared expert of the same form that every
token uses with weight 1.

Run as two products over all experts at once: the experts' gate and up matrices are stacked into one
[gate; up] matrix and their down matrices side by side, so that the activation row of a token is
[expert 0 | expert 1 | ... | shared]; the block of an expert the token did not choose is multiplied by
0 (by its routing weight otherwise) before the down product, which then sums exactly the chosen experts'
outputs and the shared one and adds them to the residual.  The products are the same projection kernels
the dense feed-forward uses, the step stays free of host decisions (CUDA graphs), and the result does
not depend on what else is in the batch; the price is that every expert's product is computed for every
token.

`GroupedMoE` (kind "grouped_moe") is the same with another router and another expert: scores are the softmax over ALL
router outputs, the choice is made on score + a stored `correction`, restricted to the `keep` best of `groups` equal
runs of neighbouring outputs (a run's score is its largest choice score), the weights are the chosen scores over
their sum; with `score: "sigmoid"` every output is scored by its own sigmoid instead, with `group_score: "top2_sum"` a
run's score is the sum of its two largest choice scores, and `route_scale` / `out_scale` multiply the weights; the last `identity` router outputs stand for experts without tensors that return their input; the
experts' activation is any member of the gated-activation family (`activation`, `limit`), and they have no
shared expert and no router bias.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import FeedForward, Runtime, StepContext, register_part
from .linear import Linear


# Prompts of more than this many tokens compute a grouped router's logits (at most 32 outputs) with the kernel for few
# rows against a long matrix, the tokens being the matrix.
SKINNY_ROUTER_MIN_TOKENS = 32


class MoE(FeedForward):
    graph_safe = True

    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.hidden_size = int(spec["hidden_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        self.expert_ff = int(spec["expert_ff"])
        self.shared_ff = int(spec["shared_ff"]) if spec.get("shared_ff") else 0
        self.inter = self.experts * self.expert_ff + self.shared_ff
        self.act = B.gated_act(spec.get("activation", "silu"), spec.get("limit"))     # None: SiLU
        self.router = self.router_bias = self.gate_up = self.down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, f = self.hidden_size, self.expert_ff
        out = {"router": TensorSpec((self.experts, h)), "router.b": TensorSpec((self.experts,))}
        for e in range(self.experts):
            out[f"e{e}.gate"] = TensorSpec((f, h))
            out[f"e{e}.up"] = TensorSpec((f, h))
            out[f"e{e}.down"] = TensorSpec((h, f))
        if self.shared_ff:
            out["shared.gate"] = TensorSpec((self.shared_ff, h))
            out["shared.up"] = TensorSpec((self.shared_ff, h))
            out["shared.down"] = TensorSpec((h, self.shared_ff))
        return out

    def _load_experts(self, tensors: Mapping[str, torch.Tensor]) -> None:
        dt = self.rt.dtype
        names = [f"e{e}" for e in range(self.experts)] + (["shared"] if self.shared_ff else [])
        gate_up = torch.cat([tensors[f"{n}.gate"].to(dt) for n in names] + [tensors[f"{n}.up"].to(dt) for n in names], dim=0)
        self.gate_up = Linear(gate_up, self.rt)
        self.down = Linear(torch.cat([tensors[f"{n}.down"].to(dt) for n in names], dim=1), self.rt)
        self.router = Linear(tensors["router"], self.rt)

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self._load_experts(tensors)
        self.router_bias = tensors["router.b"].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes() + self.router.nbytes()

    def _route(self, xn, ctx: StepContext):
        """(wt [T, E] dense routing weights, wid [T] or None: the share of experts that return their input)."""
        ws, T, E = self.rt.workspace, ctx.n_tokens, self.experts
        z = ws.take("moe.logits", (T, E), torch.float32)
        self.router.apply(xn, z, T, ctx.stream)
        wt = ws.take("moe.weights", (T, E), torch.float32)
        idx = ws.take("moe.chosen", (T, self.top), torch.int32)
        w = ws.take("moe.chosen_weights", (T, self.top), torch.float32)
        B.router_topk(z, self.router_bias, T, E, self.top, wt, idx, w, ctx.stream)
        return wt, None

    def forward(self, xn, residual, ctx: StepContext) -> None:
        rt, ws, T, I, E = self.rt, self.rt.workspace, ctx.n_tokens, self.inter, self.experts
        wt, wid = self._route(xn, ctx)
        act = ws.take("ffn.act", (T, I), rt.dtype)
        done = False
        if rt.fast:
            from . import fast_linear
            done = fast_linear.apply_gated(self.gate_up, xn, act, T, ctx.stream, fn=self.act)
        if not done:
            gu = ws.take("ffn.gate_up", (T, 2 * I), rt.dtype)
            self.gate_up.apply(xn, gu, T, ctx.stream)
            if self.act is None:
                B.silu_mul(gu, act, T, I, ctx.stream)
            else:
                B.gated_act_mul(gu, act, T, I, self.act, ctx.stream)
        if wid is None:
            B.moe_scale(act, wt, T, E, self.expert_ff, ctx.stream)
        else:
            B.moe_scale(act, wt, T, E, self.expert_ff, ctx.stream, wid=wid, x=xn, residual=residual)
        self.down.apply(act, residual, T, ctx.stream, add_residual=True, ctx=ctx)


class GroupedMoE(MoE):
    graph_safe = True
    takes_out_scale = True

    def __init__(self, spec, rt: Runtime):
        super().__init__(spec, rt)
        self.identity = int(spec.get("identity") or 0)
        self.outputs = self.experts + self.identity
        self.groups = int(spec.get("groups") or 1)
        self.keep = int(spec.get("keep") or self.groups)
        self.score = spec.get("score") or "softmax"
        self.group_score = spec.get("group_score") or "max"
        if self.score not in B.ROUTER_SCORES or self.group_score not in B.ROUTER_GROUP_SCORES:
            raise ValueError(f"grouped_moe: score must be one of {sorted(B.ROUTER_SCORES)} and group_score one of "
                             f"{sorted(B.ROUTER_GROUP_SCORES)}, got {self.score!r} and {self.group_score!r}")
        self.weight_eps = float(spec.get("weight_eps", 1e-20))
        # both factors multiply the routing weights (fp32), in which the feed-forward's result is linear
        self.weight_scale = float(spec.get("route_scale", 1.0)) * float(spec.get("out_scale", 1.0))
        if self.shared_ff:
            raise ValueError("grouped_moe has no shared expert")
        if self.outputs % self.groups:
            raise ValueError(f"{self.outputs} router outputs do not form {self.groups} equal groups")
        if not 0 < self.keep <= self.groups or self.top > self.keep * (self.outputs // self.groups):
            raise ValueError(f"top {self.top} does not fit into {self.keep} of {self.groups} groups of "
                             f"{self.outputs // self.groups}")
        self.correction = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out = super().tensor_specs()
        del out["router.b"]
        out["router"] = TensorSpec((self.outputs, self.hidden_size))
        out["correction"] = TensorSpec((self.outputs,))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self._load_experts(tensors)
        self.correction = tensors["correction"].to(torch.float32).contiguous()

    def _route(self, xn, ctx: StepContext):
        ws, T, E, N = self.rt.workspace, ctx.n_tokens, self.experts, self.outputs
        wt = ws.take("moe.weights", (T, E), torch.float32)
        wid = ws.take("moe.identity_share", (T,), torch.float32)
        idx = ws.take("moe.chosen", (T, self.top), torch.int32)
        w = ws.take("moe.chosen_weights", (T, self.top), torch.float32)
        by_output = False
        if (self.rt.fast and T > SKINNY_ROUTER_MIN_TOKENS and N <= 32 and isinstance(xn, torch.Tensor)
                and xn.dtype == torch.bfloat16 and self.router.weight.dtype == torch.bfloat16):
            # A prompt: few router outputs against many tokens.  A token tile of the tensor-core product would carry
            # N columns and 128-token tiles alone leave most of the device idle; the kernel for few rows against a long
            # matrix takes the router's rows as its "tokens" and the tokens as the matrix it streams, 16 tokens per
            # CTA, and leaves the logits with a row per router output.
            z = ws.take("moe.logits_by_output", (N, T), torch.float32)
            # the streamed "matrix" is the step's rows, which the norm in front has just written
            by_output = B.gemm_rows(self.router.weight, xn[:T], z, N, B.GEMM_STORE, self.rt.err, ctx.stream, w_dynamic=True)
        if not by_output:
            z = ws.take("moe.logits", (T, N), torch.float32)
            self.router.apply(xn, z, T, ctx.stream)
        B.router_grouped(z, self.correction, T, E, N, self.top, self.groups, self.keep, wt, wid, idx, w, ctx.stream,
                         by_output=by_output, score=self.score, group_score=self.group_score, weight_eps=self.weight_eps,
                         weight_scale=self.weight_scale)
        return wt, (wid if self.identity else None)


register_part("ffn", "moe", MoE)
register_part("ffn", "grouped_moe", GroupedMoE)
