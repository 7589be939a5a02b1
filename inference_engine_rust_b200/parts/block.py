"""Arrangement of a layer's parts.  "shared_norm": h = norm1(x); x += mixer(h) + ffn(h) (one norm, read by both
sublayers).  "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)) (the second
half left out for a layer without a feed-forward)
(src/layers/block.rs:19-24,63-65; the residual uses the un-normed input,
src/layers/attention.rs:757-759, src/layers/ffn.rs:113-116)."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import bindings as B
from ..weights.loader import TensorSpec
from .base import Block, Runtime, StepContext, first_norm_request_of, register_part


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, layer_spec, norm1, mixer, norm2, ffn, rt: Runtime):
        self.norm1, self.mixer, self.norm2, self.ffn, self.rt = norm1, mixer, norm2, ffn, rt

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        xn = self._normed(self.norm1, x, ctx)
        # what the next norm asks of whoever adds the mixer's result into x
        if self.ffn is not None:
            ctx.norm_ahead = self._request(self.norm2, self.ffn, ctx)
        else:
            ctx.norm_ahead = first_norm_request_of(ctx.next_block, ctx)
        self.mixer.forward(xn, x, ctx, cache_view, writes_cache)
        if self.ffn is None:                     # a layer without a feed-forward
            ctx.norm_ahead = None
            return
        xn = self._normed(self.norm2, x, ctx)
        ctx.norm_ahead = first_norm_request_of(ctx.next_block, ctx)
        self.ffn.forward(xn, x, ctx)
        ctx.norm_ahead = None

    def first_norm_request(self, ctx: StepContext):
        return self._request(self.norm1, self.mixer, ctx)

    def _request(self, norm, part, ctx: StepContext):
        """In steps of up to 64 tokens (one-token steps, short prompts) a norm may ask whoever writes its
        input rows to do its element-wise half (`NormRequest`), if the part behind it hands its input to a
        projection."""
        from . import fast_linear
        if (self.rt.fast and ctx.n_tokens <= fast_linear.NORM_AHEAD_MAX_TOKENS
                and getattr(part, "takes_lazy_input", False) and fast_linear.norm_ahead_enabled()):
            return norm.request_ahead()
        return None

    def _normed(self, norm, x, ctx: StepContext):
        """norm(x): what the writer of x left behind for this norm, if it honoured the norm's request,
        else the norm's own kernel."""
        lazy, ctx.rows_ahead = ctx.rows_ahead, None
        if lazy is not None and getattr(lazy, "norm", None) is norm and lazy.rows is x:
            return lazy
        xn = self.rt.workspace.take("block.normed", x.shape, self.rt.dtype)
        norm.forward(x, xn, ctx, rows=ctx.n_tokens)
        return xn


class NormedAhead:
    """Left in `ctx.rows_ahead` by a block that computed the NEXT block's first normed input in the same
    pass that finished its own update of the streams."""

    def __init__(self, norm, rows, normed):
        self.norm, self.rows, self.normed = norm, rows, normed


class HyperConnectionBlock(Block):
    """Pre-norm layer over a residual kept as S streams x_1 .. x_S per token.  For sublayer q (1: the
    mixer, 2: the feed-forward) with learned in[S], out[S] and mix[S, S] (indexed [from, to]):

        u = sum_s in[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t at once)

    Tensors (under the layer's block prefix): hc1.in, hc1.out, hc1.mix and, with a feed-forward, hc2.*.
    The sublayers add into a zeroed fp32 buffer y; the streams' update after a sublayer and the combination
    and norm in front of the next one (also the next block's first) are one kernel."""
    graph_safe = True

    def __init__(self, layer_spec, norm1, mixer, norm2, ffn, rt: Runtime):
        self.norm1, self.mixer, self.norm2, self.ffn, self.rt = norm1, mixer, norm2, ffn, rt
        self.streams = int(layer_spec.block["streams"])
        for n in (norm1, norm2):
            if n is not None and not hasattr(n, "forward_streams"):
                raise ValueError(f"block 'hyper' needs a norm with forward_streams, got {type(n).__name__}")
        self.hc = {}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        S, out = self.streams, {}
        for q in ("hc1",) + (("hc2",) if self.ffn is not None else ()):
            out[q + ".in"] = TensorSpec((S,), "ones_plus_normal")
            out[q + ".out"] = TensorSpec((S,), "ones_plus_normal")
            out[q + ".mix"] = TensorSpec((S, S), "eye_plus_normal")
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.hc = {k: t.to(torch.float32).contiguous() for k, t in tensors.items()}

    def forward(self, xs, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, S, T = self.rt, self.streams, ctx.n_tokens
        H = xs.shape[-1]
        hc = self.hc
        ctx.norm_ahead = None
        y = rt.workspace.take("block.sublayer_out", (T, H), torch.float32)
        ahead, ctx.rows_ahead = ctx.rows_ahead, None
        if isinstance(ahead, NormedAhead) and ahead.norm is self.norm1 and ahead.rows is xs:
            xn = ahead.normed                       # the block before left it (and cleared y)
        else:
            xn = rt.workspace.take("block.normed", (T, H), rt.dtype)
            self.norm1.forward_streams(xs, S, xn, ctx, T, in_coef=hc["hc1.in"], clear=y)
        self.mixer.forward(xn, y, ctx, cache_view, writes_cache)
        last = "hc1"
        if self.ffn is not None:
            self.norm2.forward_streams(xs, S, xn, ctx, T, in_coef=hc["hc2.in"], update=(y, hc["hc1.mix"], hc["hc1.out"]),
                                       clear=y)
            self.ffn.forward(xn, y, ctx)
            last = "hc2"
        nxt = ctx.next_block
        update = (y, hc[last + ".mix"], hc[last + ".out"])
        if isinstance(nxt, HyperConnectionBlock) and nxt.streams == S:
            nxt.norm1.forward_streams(xs, S, xn, ctx, T, in_coef=nxt.hc["hc1.in"], update=update, clear=y)
            ctx.rows_ahead = NormedAhead(nxt.norm1, xs, xn)
        else:
            B.streams_norm(xs, S, H, T, ctx.stream, y=y, mix=update[1], outc=update[2], update=True, write_back=True)


class CastAhead:
    """Left in `ctx.rows_ahead` by an output-norm block: the residual rows `rows` already stand in `cast` in the
    run's dtype and the sublayer buffer `cleared` is zero, written by the kernel that finished the block."""

    def __init__(self, rows, cast, cleared):
        self.rows, self.cast, self.cleared = rows, cast, cleared


class OutputNormBlock(Block):
    """The norm sits on each sublayer's OUTPUT and the sublayers read the residual itself:

        x <- x + norm1(mixer(x));   x <- x + norm2(ffn(x))      (the second half left out without a feed-forward)

    The sublayers add into a zeroed fp32 buffer y; one kernel per sublayer norms y, adds it to the fp32 residual,
    clears y and writes the new residual in the run's dtype for the next sublayer's projections (also across the
    block boundary: the next block of this kind finds its input ready)."""
    graph_safe = True

    def __init__(self, layer_spec, norm1, mixer, norm2, ffn, rt: Runtime):
        self.norm1, self.mixer, self.norm2, self.ffn, self.rt = norm1, mixer, norm2, ffn, rt
        for n in (norm1, norm2):
            if n is not None and not hasattr(n, "add_normed"):
                raise ValueError(f"block 'outnorm' needs a norm with add_normed, got {type(n).__name__}")

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        rt, T = self.rt, ctx.n_tokens
        ctx.norm_ahead = None
        y = rt.workspace.take("block.sublayer_out", x.shape, torch.float32)
        h = rt.workspace.take("block.input", x.shape, rt.dtype)
        ahead, ctx.rows_ahead = ctx.rows_ahead, None
        if not (isinstance(ahead, CastAhead) and ahead.rows is x and ahead.cast.data_ptr() == h.data_ptr()
                and ahead.cleared.data_ptr() == y.data_ptr() and ahead.cast.dtype == h.dtype):
            B.cast_rows(x, y, h, T, ctx.stream)
        self.mixer.forward(h, y, ctx, cache_view, writes_cache)
        self.norm1.add_normed(y, x, h, ctx, T)
        if self.ffn is not None:
            self.ffn.forward(h, y, ctx)
            self.norm2.add_normed(y, x, h, ctx, T)
        ctx.rows_ahead = CastAhead(x, h, y)


class SharedNormBlock(Block):
    """One norm, read by both sublayers, whose results are added to the same residual:

        h = norm1(x);   x <- x + mixer(h) + ffn(h)             (the feed-forward left out for a layer without one)

    The layer has no second norm (`LayerSpec.ffn_norm_name` is empty).  Both sublayers add into the fp32 residual;
    neither reads it, so the order of the two additions is free.  The norm runs as a kernel of its own: its input
    rows change under the second sublayer's eyes (the first has added its result by then), so a norm split around a
    kernel boundary (`NormRequest`) would have to be finished from a copy, which the block's own kernel already is."""
    graph_safe = True

    def __init__(self, layer_spec, norm1, mixer, norm2, ffn, rt: Runtime):
        if norm2 is not None:
            raise ValueError("block 'shared_norm' has one norm; leave LayerSpec.ffn_norm_name empty")
        self.norm1, self.mixer, self.ffn, self.rt = norm1, mixer, ffn, rt

    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        ctx.rows_ahead = None
        h = self.rt.workspace.take("block.normed", x.shape, self.rt.dtype)
        self.norm1.forward(x, h, ctx, rows=ctx.n_tokens)
        # only the block's last addition may write the next block's norm ahead: the rows are final then
        ahead = first_norm_request_of(ctx.next_block, ctx)
        ctx.norm_ahead = ahead if self.ffn is None else None
        self.mixer.forward(h, x, ctx, cache_view, writes_cache)
        if self.ffn is not None:
            ctx.norm_ahead = ahead
            self.ffn.forward(h, x, ctx)
        ctx.norm_ahead = None


register_part("block", "prenorm", PreNormBlock)
register_part("block", "shared_norm", SharedNormBlock)
register_part("block", "outnorm", OutputNormBlock)
register_part("block", "hyper", HyperConnectionBlock)
