"""ctypes bindings of the CUDA launchers.  Every function here launches hand-written
kernels on the current CUDA stream; there is no other implementation behind them, so a
machine without the built library (or without a GPU) gets an error, not a fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_char_p, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
PAIR_HALF, PAIR_INTERLEAVED = 0, 1
GEMM_STORE, GEMM_ADD_RESIDUAL = 0, 1

ERR_TOKEN_RANGE, ERR_NONFINITE_LOGIT, ERR_PAGE_RANGE, ERR_WAIT_EXPIRED = 1, 2, 4, 8
_ERR_TEXT = {
    ERR_TOKEN_RANGE: "a token id outside [0, vocab) reached the embedding kernel",
    ERR_NONFINITE_LOGIT: "sampling saw a NaN or infinite logit",
    ERR_PAGE_RANGE: "a page-table entry outside the page pool was read",
    ERR_WAIT_EXPIRED: "a bounded wait inside a kernel expired",
}


class KernelError(RuntimeError):
    pass


class KvView(Structure):
    """Mirror of `IertKvView` (common.cuh)."""
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("page_table", c_void_p),
                ("table_width", c_int), ("ring_pages", c_int), ("page_tokens", c_int),
                ("n_pages", c_int), ("kv_heads", c_int), ("head_dim", c_int),
                ("dtype", c_int), ("window", c_int), ("chunk", c_int)]


class BatchView(Structure):
    """Mirror of `IertBatchView` (common.cuh)."""
    _fields_ = [("cu_q", c_void_p), ("slot_ids", c_void_p), ("tok_seq", c_void_p),
                ("pos0", c_void_p), ("n_seqs", c_int), ("n_tokens", c_int)]


class NormAhead(Structure):
    """Mirror of `IertNormAhead` (common.cuh): the first half of an RMSNorm, written by the kernel that
    writes the rows."""
    _fields_ = [("weight", c_void_p), ("weight_dtype", c_int), ("scaled_out", c_void_p), ("ld", c_longlong),
                ("sumsq_out", c_void_p), ("parts", c_int)]


class RowScale(Structure):
    """Mirror of `IertRowScale`: the second half, applied by the projection that reads the scaled rows."""
    _fields_ = [("sumsq", c_void_p), ("parts", c_int), ("hidden", c_int), ("eps", c_float)]


class GatedAct(Structure):
    """Mirror of `IertGatedAct`: out = g' sigmoid(g' (a + b g'^2)) u' with g' = min(g, g_max) and
    u' = clamp(u, -u_max, u_max) + u_bias."""
    _fields_ = [("g_max", c_float), ("u_max", c_float), ("u_bias", c_float), ("a", c_float), ("b", c_float)]


def gated_act(name: str, limit: Optional[float] = None) -> Optional[GatedAct]:
    """The constants of a named gated activation: "silu" (None: the kernels' default), "gelu_tanh" (the tanh form
    of GELU), "clamped_swish" (gate capped at `limit`, up clamped to +-`limit` and shifted by one, sigmoid of
    1.702 times the gate)."""
    import math
    inf = float("inf")
    if name == "silu":
        return None
    if name == "gelu_tanh":
        c = math.sqrt(2.0 / math.pi)
        return GatedAct(inf, inf, 0.0, 2.0 * c, 2.0 * c * 0.044715)
    if name == "clamped_swish":
        lim = inf if limit is None else float(limit)
        return GatedAct(lim, lim, 1.0, 1.702, 0.0)
    raise KernelError(f"gated activation must be one of silu, gelu_tanh, clamped_swish, got {name!r}")


def norm_ahead(weight, scaled_out, sumsq_out) -> NormAhead:
    return NormAhead(weight=weight.data_ptr(), weight_dtype=dtype_code(weight.dtype), scaled_out=scaled_out.data_ptr(),
                     ld=scaled_out.stride(0), sumsq_out=sumsq_out.data_ptr(), parts=0)


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dt}")


_core = None


def core() -> ctypes.CDLL:
    """The core library, built on first use."""
    global _core
    if _core is None:
        lib = build.load_library("iert_core", build.CORE_SOURCES)
        _declare(lib)
        if os.environ.get("IERT_PDL", "1") == "0":      # programmatic dependent launch off (for measurements)
            lib.iert_set_pdl(0)
        _core = lib
    return _core


def _declare(lib) -> None:
    S = c_void_p  # cudaStream_t
    P = c_void_p
    lib.iert_last_cuda_error.restype = c_char_p
    lib.iert_device_arch.restype = c_int
    lib.iert_sm_count.restype = c_int
    sigs = {
        "iert_embed_gather": [P, c_int, P, P, c_int, c_int, c_int, c_float, P, POINTER(NormAhead), S],
        "iert_rmsnorm": [P, P, c_int, P, c_int, P, c_int, c_int, c_float, S],
        "iert_rope_kv_store": [P, c_int, POINTER(BatchView), POINTER(KvView), P, c_int, c_int, c_int, c_int, P, S],
        "iert_silu_mul": [P, P, c_int, c_int, c_int, S],
        "iert_gated_act_mul": [P, P, c_int, c_int, c_int, POINTER(GatedAct), S],
        "iert_add_into": [P, P, c_int, c_longlong, S],
        "iert_advance_positions": [P, P, P, c_int, S],
        "iert_gemm_plain": [P, c_int, P, c_int, P, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, S],
        "iert_attention_plain": [P, P, c_int, POINTER(BatchView), POINTER(KvView), c_int, c_float, c_int, c_float, P, P, S],
        "iert_sample_greedy": [P, c_int, c_int, c_longlong, P, P, S],
        "iert_sample_temperature": [P, c_int, c_int, c_longlong, c_float, c_ulonglong, P, P, P, P, S],
        "iert_uniform_draws": [c_ulonglong, P, P, P, c_int, S],
        "iert_gemm_tc": [P, c_longlong, P, c_longlong, P, c_int, c_longlong, c_int, c_int, c_int, c_int,
                         P, c_longlong, P, c_int, c_int, c_int, c_int, P, S],
    }
    LL = c_longlong
    sigs.update({
        "iert_streams_norm": [P, c_int, c_int, P, P, P, c_int, c_int, c_int, P, P, P, c_float, P, c_int, P, P, c_int, S],
        "iert_streams_expand": [P, P, c_int, c_int, c_int, S],
        "iert_softcap": [P, LL, c_float, S],
        "iert_delta_prep": [P, c_int, LL, P, LL, P, P, P, P, LL, LL, P, P, P, c_int, c_int, c_int, c_int, c_int,
                            POINTER(BatchView), S],
        "iert_gated_head_norm": [P, P, c_int, LL, c_int, P, c_int, c_int, c_float, P, c_int, c_int, c_int, S],
        "iert_latent_norm_store": [P, LL, c_int, c_int, P, P, c_float, P, P, c_int, POINTER(BatchView), POINTER(KvView),
                                   c_int, P, S],
        "iert_latent_attention_prompt": [P, LL, P, c_int, POINTER(BatchView), c_int, c_int, c_int, c_float, P, S],
        "iert_latent_attention_decode": [P, LL, P, P, P, c_int, POINTER(BatchView), POINTER(KvView), c_int, c_int, c_int, c_int,
                                         c_float, P, P, P, S],
        "iert_latent_prep": [P, LL, c_int, c_int, c_int, c_int, P, c_float, P, c_int, c_int, c_float, P, P, LL, c_int, P, c_int,
                             POINTER(BatchView), POINTER(KvView), c_int, P, S],
        "iert_head_gate_mul": [P, c_int, P, c_int, c_int, P, c_int, POINTER(BatchView), S],
        "iert_token_shift": [P, c_int, LL, P, LL, LL, P, c_int, c_int, P, POINTER(BatchView), S],
        "iert_wkv_decay": [P, LL, c_int, P, P, c_int, P, P, c_int, LL, c_int, P, LL, LL, POINTER(BatchView), S],
        "iert_wkv_finish": [P, P, LL, P, c_float, c_float, P, c_int, POINTER(BatchView), c_int, c_int, S],
        "iert_latent_decode_tc_plan": [c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)],
        "iert_router_topk": [P, LL, P, c_int, c_int, c_int, P, P, P, S],
        "iert_moe_scale": [P, c_int, LL, P, c_int, c_int, c_int, P, P, LL, P, c_int, S],
        "iert_router_grouped": [P, LL, LL, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                P, P, P, P, S],
        "iert_qkv_prep": [P, LL, P, P, c_int, POINTER(BatchView), POINTER(KvView), c_int, c_int, c_int, P, c_int, c_int, P, P,
                          c_float, c_int, P, S],
        "iert_gate_mul": [P, P, LL, P, c_int, c_int, c_int, c_int, c_int, S],
        "iert_add_normed": [P, P, P, P, c_int, c_int, c_int, c_float, S],
        "iert_cast_rows": [P, P, P, c_int, LL, S],
        "iert_scale_values": [P, LL, c_float, S],
        "iert_qk_prep": [P, LL, P, c_int, POINTER(BatchView), POINTER(KvView), c_int, P, c_int, c_int, P, P, c_float, c_float,
                         c_int, P, S],
        "iert_rglru_conv": [P, LL, P, P, P, P, LL, P, c_int, c_int, POINTER(BatchView), S],
        "iert_rglru_gates": [P, P, P, P, P, c_int, P, c_float, P, P, c_int, c_int, c_int, S],
        "iert_rglru_scan": [P, P, P, LL, P, P, P, LL, P, c_int, c_float, c_int, c_int, c_int, P, POINTER(BatchView), S],
    })
    lib.iert_attention_decode.argtypes = [P, P, POINTER(BatchView), POINTER(KvView), c_int, c_float, c_int, P, P, S]
    lib.iert_attention_decode.restype = c_int
    lib.iert_attention_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.iert_attention_decode_scratch_floats.restype = c_longlong
    lib.iert_gemm_tc_gated.argtypes = [P, c_longlong, P, c_longlong, P, c_longlong, c_int, c_int, c_int, POINTER(GatedAct),
                                       c_int, c_int, P, S]
    lib.iert_gemm_tc_gated.restype = c_int
    lib.iert_gemm_rows.argtypes = [P, c_longlong, P, c_longlong, P, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                   POINTER(RowScale), POINTER(NormAhead), c_int, c_int, P, S]
    lib.iert_gemm_rows.restype = c_int
    lib.iert_gemm_tc_scaled.argtypes = [P, c_longlong, P, c_longlong, P, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                        P, c_longlong, P, c_int, POINTER(RowScale), POINTER(NormAhead), c_int, c_int, P, S]
    lib.iert_gemm_tc_scaled.restype = c_int
    lib.iert_gemm_tc_gated_scaled.argtypes = [P, c_longlong, P, c_longlong, P, c_longlong, c_int, c_int, c_int,
                                              POINTER(RowScale), POINTER(GatedAct), c_int, P, S]
    lib.iert_gemm_tc_gated_scaled.restype = c_int
    lib.iert_gemm_tc_workspace_bytes.restype = c_longlong
    lib.iert_gemm_tc_counter_count.restype = c_int
    lib.iert_gemm_tc_set_poll_limit.argtypes = [ctypes.c_uint]
    lib.iert_gemm_tc_set_poll_limit.restype = None
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


launch_count = 0        # launcher calls that returned success since import (one kernel each)


def check(status: int, what: str) -> None:
    global launch_count
    if status == 0:
        launch_count += 1
        return
    if status == 1:
        raise KernelError(f"{what}: the kernel does not take these sizes or options")
    msg = core().iert_last_cuda_error().decode("utf-8", "replace")
    raise KernelError(f"{what}: CUDA error: {msg}")


def require_device() -> None:
    """Refuse to run anywhere but on an sm_100 GPU with the built library."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this package runs its hand-written sm_100a kernels only")
    arch = core().iert_device_arch()
    if arch < 0:
        raise KernelError("device query failed: " + core().iert_last_cuda_error().decode())
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a; this device is sm_{arch}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def describe_error_bits(bits: int) -> str:
    return "; ".join(t for b, t in _ERR_TEXT.items() if bits & b) or f"unknown error bits {bits}"


# ---------------------------------------------------------------------------------------
# thin wrappers: tensors in, launch, nothing returned


def embed_gather(table, ids, x, scale: float, err, stream, ahead: Optional[NormAhead] = None) -> int:
    """x[t] = table[ids[t]] * scale.  `ahead`: also the first half of the norm that follows
    (`norm_ahead`); returns the partial sums of squares per row it wrote (0 without `ahead`)."""
    vocab, hidden = table.shape
    check(core().iert_embed_gather(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(),
                                   x.data_ptr(), ids.numel(), hidden, vocab, scale,
                                   err.data_ptr(), byref(ahead) if ahead is not None else None, stream), "embed_gather")
    return int(ahead.parts) if ahead is not None else 0


def rmsnorm(x, w, out, eps: float, stream, rows_idx=None, rows: Optional[int] = None) -> None:
    hidden = x.shape[-1]
    n = rows if rows is not None else (rows_idx.numel() if rows_idx is not None else x.shape[0])
    check(core().iert_rmsnorm(x.data_ptr(), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(),
                              dtype_code(out.dtype),
                              rows_idx.data_ptr() if rows_idx is not None else None,
                              n, hidden, eps, stream), "rmsnorm")


_SM_COUNT = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device."""
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = int(core().iert_sm_count())
    return _SM_COUNT


def rope_kv_store(qkv, batch: BatchView, kv: KvView, inv_freq, heads: int, rotary_dim: int,
                  pairing: int, write_cache: bool, err, stream) -> None:
    check(core().iert_rope_kv_store(qkv.data_ptr(), dtype_code(qkv.dtype), byref(batch), byref(kv),
                                    inv_freq.data_ptr(), heads, rotary_dim, pairing,
                                    1 if write_cache else 0, err.data_ptr(), stream), "rope_kv_store")


_no_rotation = {}


def _zero_freq(device):
    key = str(device)
    if key not in _no_rotation:
        _no_rotation[key] = torch.zeros(1, dtype=torch.float32, device=device)
    return _no_rotation[key]


def kv_store(qkv, batch: BatchView, kv: KvView, heads: int, err, stream) -> None:
    """Write the step's keys and values (as they stand in the packed projection) into the cache."""
    rope_kv_store(qkv, batch, kv, _zero_freq(qkv.device), heads, 0, PAIR_HALF, True, err, stream)


def rotate_qk(qkv, batch: BatchView, inv_freq, heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
              pairing: int, err, stream) -> None:
    """Rotate the step's queries and keys in place; nothing is stored."""
    geometry = KvView(k=None, v=None, page_table=None, table_width=0, ring_pages=1, page_tokens=1, n_pages=0,
                      kv_heads=kv_heads, head_dim=head_dim, dtype=dtype_code(qkv.dtype), window=0)
    rope_kv_store(qkv, batch, geometry, inv_freq, heads, rotary_dim, pairing, False, err, stream)


def silu_mul(gu, out, n_tokens: int, inter: int, stream) -> None:
    check(core().iert_silu_mul(gu.data_ptr(), out.data_ptr(), dtype_code(gu.dtype), n_tokens, inter,
                               stream), "silu_mul")


def gated_act_mul(gu, out, n_tokens: int, inter: int, act: GatedAct, stream) -> None:
    """out[t, i] = f(gu[t, i], gu[t, inter + i]) for f of the gated-activation family."""
    check(core().iert_gated_act_mul(gu.data_ptr(), out.data_ptr(), dtype_code(gu.dtype), n_tokens, inter, byref(act), stream),
          "gated_act_mul")


def add_into(residual, y, n: int, stream) -> None:
    check(core().iert_add_into(residual.data_ptr(), y.data_ptr(), dtype_code(y.dtype), n, stream),
          "add_into")


def advance_positions(batch: "BatchView", stream) -> None:
    check(core().iert_advance_positions(batch.pos0, batch.cu_q, batch.slot_ids, batch.n_seqs, stream),
          "advance_positions")


def gemm_plain(x, w, out, M: int, mode: int, stream) -> None:
    """out[:M] (=|+=) x[:M] @ w.T with x [*, K], w [N, K], out [*, N]; row strides taken
    from the tensors."""
    N, K = w.shape
    check(core().iert_gemm_plain(x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype),
                                 out.data_ptr(), dtype_code(out.dtype), M, N, K,
                                 x.stride(0), w.stride(0), out.stride(0), mode, stream), "gemm_plain")


def attention_plain(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, paged: bool,
                    err, stream, softcap: float = 0.0, sink=None) -> None:
    """`softcap` c > 0: scores pass c tanh(s / c); `sink` (fp32 [heads], optional): a bare logit per head
    that adds exp(sink) to each row's softmax denominator only."""
    check(core().iert_attention_plain(qkv.data_ptr(), out.data_ptr(), dtype_code(qkv.dtype),
                                      byref(batch), byref(kv), heads, scale, 1 if paged else 0,
                                      softcap, sink.data_ptr() if sink is not None else None,
                                      err.data_ptr(), stream), "attention_plain")


def sample_greedy(logits, out, err, stream) -> None:
    rows, vocab = logits.shape
    check(core().iert_sample_greedy(logits.data_ptr(), rows, vocab, logits.stride(0), out.data_ptr(),
                                    err.data_ptr(), stream), "sample_greedy")


def sample_temperature(logits, temperature: float, seed: int, request_ids, step_ids, out, err,
                       stream) -> None:
    rows, vocab = logits.shape
    check(core().iert_sample_temperature(logits.data_ptr(), rows, vocab, logits.stride(0),
                                         temperature, seed & 0xFFFFFFFFFFFFFFFF,
                                         request_ids.data_ptr(), step_ids.data_ptr(), out.data_ptr(),
                                         err.data_ptr(), stream), "sample_temperature")


def uniform_draws(seed: int, request_ids, step_ids, out, stream) -> None:
    check(core().iert_uniform_draws(seed & 0xFFFFFFFFFFFFFFFF, request_ids.data_ptr(),
                                    step_ids.data_ptr(), out.data_ptr(), out.numel(), stream),
          "uniform_draws")


class GemmScratch:
    """Scratch memory and ticket counters of the tensor-core projection's split-K path, shared
    by every launch on one stream of one device."""

    _by_device = {}

    def __init__(self, device):
        lib = core()
        self.ws = torch.empty(lib.iert_gemm_tc_workspace_bytes(), dtype=torch.uint8, device=device)
        self.counters = torch.zeros(lib.iert_gemm_tc_counter_count(), dtype=torch.int32, device=device)

    @classmethod
    def get(cls, device) -> "GemmScratch":
        key = str(torch.device(device))
        if key not in cls._by_device:
            cls._by_device[key] = cls(device)
        return cls._by_device[key]


def gemm_tc_set_poll_limit(polls: int) -> None:
    """Polls of a tile's counter before a CTA of the split-K projection gives up waiting for the tile's other
    CTAs (0: the default, about a second).  For tests of that bounded wait."""
    core().iert_gemm_tc_set_poll_limit(int(polls))


def gemm_tc(x, w, out, M: int, mode: int, err, stream, force_bt: int = 0, force_splits: int = 0,
            force_stages: int = 0) -> bool:
    """out[:M] (=|+=) x[:M] @ w.T on the tensor cores (bf16 operands).  Returns False, having
    launched nothing, when the operands do not meet the kernel's alignment rules."""
    N, K = w.shape
    sc = GemmScratch.get(x.device)
    status = core().iert_gemm_tc(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                 dtype_code(out.dtype), out.stride(0), M, N, K, mode, sc.ws.data_ptr(),
                                 sc.ws.numel(), sc.counters.data_ptr(), sc.counters.numel(), force_bt,
                                 force_splits, force_stages, err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc")
    return True


def gemm_rows(x, w, out, M: int, mode: int, err, stream, scale: Optional[RowScale] = None,
              ahead: Optional[NormAhead] = None, force_stages: int = 0, w_dynamic: bool = False) -> bool:
    """out[:M] (=|+=) x[:M] @ w.T for one-token steps (M <= 32, bf16 operands): 16 weight rows per
    CTA over all of k, no split-K.  `scale`: x is the first half of an RMSNorm and the outputs
    are multiplied by the rows' 1 / rms; `ahead` (with a residual add): the first half of the
    next norm is written beside the new rows and `ahead.parts` is set.  `w_dynamic`: `w` is no stored weight but rows
    the kernel in front wrote, so none of it is fetched ahead of the wait for that kernel.  Returns False, having
    launched nothing, when the operands do not meet the kernel's rules."""
    N, K = w.shape
    status = core().iert_gemm_rows(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                   dtype_code(out.dtype), out.stride(0), M, N, K, mode,
                                   byref(scale) if scale is not None else None,
                                   byref(ahead) if ahead is not None else None, force_stages, 1 if w_dynamic else 0,
                                   err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_rows")
    return True


def gemm_tc_scaled(x, w, out, M: int, mode: int, err, stream, scale: Optional[RowScale] = None,
                   ahead: Optional[NormAhead] = None, force_bt: int = 0, force_splits: int = 0) -> bool:
    """`gemm_tc` for one-token steps of 17 to 64 tokens with an RMSNorm split around the kernel: `scale`
    (x is a norm's first half: outputs times the rows' 1 / rms) and / or `ahead` (a residual add that
    also writes the next norm's first half; `ahead.parts` is set).  False, nothing launched, where
    the launch would not go through the split-K reduction."""
    N, K = w.shape
    sc = GemmScratch.get(x.device)
    status = core().iert_gemm_tc_scaled(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                        dtype_code(out.dtype), out.stride(0), M, N, K, mode, sc.ws.data_ptr(),
                                        sc.ws.numel(), sc.counters.data_ptr(), sc.counters.numel(),
                                        byref(scale) if scale is not None else None,
                                        byref(ahead) if ahead is not None else None, force_bt, force_splits,
                                        err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc_scaled")
    return True


def gemm_tc_gated_scaled(x, w, act, M: int, scale: RowScale, err, stream, force_bt: int = 0,
                         fn: Optional[GatedAct] = None) -> bool:
    """`gemm_tc_gated` in its one-token form for an x that is the first half of an RMSNorm: gate and
    up are multiplied by the rows' 1 / rms before the activation."""
    two_i, K = w.shape
    status = core().iert_gemm_tc_gated_scaled(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), act.data_ptr(),
                                              act.stride(0), M, two_i // 2, K, byref(scale),
                                              byref(fn) if fn is not None else None, force_bt, err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc_gated_scaled")
    return True


def attention_decode_scratch_floats(n_tokens: int, heads: int, head_dim: int, splits: int) -> int:
    return core().iert_attention_decode_scratch_floats(n_tokens, heads, head_dim, splits)


def attention_decode(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, splits: int,
                     scratch, err, stream) -> bool:
    """Split-KV decode attention (bf16 cache).  Returns False, having launched nothing, when
    the kernel does not take the cache's geometry."""
    status = core().iert_attention_decode(qkv.data_ptr(), out.data_ptr(), byref(batch), byref(kv), heads,
                                          scale, splits, scratch.data_ptr(), err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "attention_decode")
    global launch_count
    launch_count += 1          # the combine pass
    return True


_attn_libs = {}


def _attention_lib(head_dim: int):
    """The tensor-core attention library for one head size, compiled on first use."""
    lib = _attn_libs.get(head_dim)
    if lib is None:
        lib = build.load_library(*build.attention_library(head_dim))
        lib.iert_attention_prefill.argtypes = [c_void_p, c_void_p, POINTER(BatchView), c_int, c_int, c_int, c_int,
                                               c_float, c_int, c_void_p, c_float, c_void_p]
        lib.iert_attention_prefill.restype = c_int
        lib.iert_attention_decode_tc.argtypes = [c_void_p, c_void_p, POINTER(BatchView), POINTER(KvView), c_int,
                                                 c_float, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p]
        lib.iert_attention_decode_tc.restype = c_int
        lib.iert_attention_decode_tc_rope.argtypes = [c_void_p, c_void_p, POINTER(BatchView), POINTER(KvView), c_int,
                                                      c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                      c_void_p, c_void_p]
        lib.iert_attention_decode_tc_rope.restype = c_int
        lib.iert_attention_prefill_tc.argtypes = [c_void_p, c_void_p, POINTER(BatchView), c_int, c_int, c_int, c_int,
                                                  c_float, c_int, c_void_p, c_void_p, c_float, c_void_p]
        lib.iert_attention_prefill_tc.restype = c_int
        lib.iert_attention_prefill_tc_available.restype = c_int
        lib.iert_attention_decode_tc_ctas_per_sm.restype = c_int
        if os.environ.get("IERT_PDL", "1") == "0":
            lib.iert_set_pdl(0)
        _attn_libs[head_dim] = lib
    return lib


def attention_prefill(qkv, out, batch: BatchView, heads: int, kv_heads: int, head_dim: int, window: int,
                      scale: float, max_q_len: int, stream, err=None, legacy: bool = False, sink=None,
                      softcap: float = 0.0, chunk: int = 0) -> bool:
    """Flash prompt attention (bf16) over the step's own keys and values (`window` W > 0: the last W keys; `chunk`
    C > 0: the keys of the query's own chunk of C positions).  Head sizes 64 and
    128 run on tcgen05 with the scores and the output in tensor memory (unless `legacy`); other
    multiples of 16 up to 256 run the mma.sync kernel.  The library is compiled per head size
    the first time it is needed; anything else returns False and nothing is launched.  `sink` (fp32
    [heads], optional): a bare logit per head that adds exp(sink) to each row's softmax denominator only;
    `softcap` c > 0: scores pass c tanh(s / c) before the softmax."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        return False
    lib = _attention_lib(head_dim)
    global launch_count
    if not legacy and err is not None and lib.iert_attention_prefill_tc_available() \
            and os.environ.get("IERT_ATTN_TC", "1") != "0":
        status = lib.iert_attention_prefill_tc(qkv.data_ptr(), out.data_ptr(), byref(batch), heads, kv_heads,
                                               window, chunk, scale, max_q_len, err.data_ptr(),
                                               sink.data_ptr() if sink is not None else None, softcap, stream)
        if status == 0:
            launch_count += 1
            return True
        if status != 1:
            raise KernelError("attention_prefill_tc: the launch failed")
    status = lib.iert_attention_prefill(qkv.data_ptr(), out.data_ptr(), byref(batch), heads, kv_heads,
                                        window, chunk, scale, max_q_len, sink.data_ptr() if sink is not None else None, softcap,
                                        stream)
    if status == 1:
        return False
    if status != 0:
        raise KernelError("attention_prefill: the launch failed")
    launch_count += 1
    return True


def attention_decode_ctas_per_sm(head_dim: int) -> int:
    """CTAs of the tensor-core decode-attention kernels that one SM holds at once (a fact of those
    kernels, kept with them)."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"no tensor-core decode attention for head size {head_dim}")
    return int(_attention_lib(head_dim).iert_attention_decode_tc_ctas_per_sm())


def attention_decode_tc(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, splits: int,
                        scratch, err, stream, target_ctas: int = 0, softcap: float = 0.0, sink=None) -> bool:
    """Tensor-core split-KV decode attention (bf16 cache, 64-position pages, head sizes that
    are multiples of 16 up to 256).  Returns False, having launched nothing, otherwise.  `softcap` and
    `sink` as in `attention_prefill`."""
    hd = kv.head_dim
    if hd % 16 or not 16 <= hd <= 256:
        return False
    status = _attention_lib(hd).iert_attention_decode_tc(qkv.data_ptr(), out.data_ptr(), byref(batch), byref(kv),
                                                         heads, scale, splits, target_ctas, scratch.data_ptr(),
                                                         softcap, sink.data_ptr() if sink is not None else None,
                                                         err.data_ptr(), stream)
    if status == 1:
        return False
    if status != 0:
        raise KernelError("attention_decode_tc: the launch failed")
    global launch_count
    launch_count += 1 if splits == 1 and sink is None else 2        # a single split without a sink needs no merge kernel
    return True


def attention_decode_tc_rope(qkv, out, batch: BatchView, kv: KvView, heads: int, scale: float, splits: int,
                             scratch, inv_freq, rotary_dim: int, pairing: int, store: bool, err, stream,
                             target_ctas: int = 0) -> bool:
    """`attention_decode_tc` with the rotary encoding and the step's cache write inside the
    kernel: `qkv` is the raw projection (one token per sequence) and stays as it is.  Returns
    False, having launched nothing, for anything the kernel does not take."""
    hd = kv.head_dim
    if hd % 16 or not 16 <= hd <= 256:
        return False
    status = _attention_lib(hd).iert_attention_decode_tc_rope(
        qkv.data_ptr(), out.data_ptr(), byref(batch), byref(kv), heads, scale, splits, target_ctas, scratch.data_ptr(),
        inv_freq.data_ptr(), rotary_dim, pairing, 1 if store else 0, err.data_ptr(), stream)
    if status == 1:
        return False
    if status != 0:
        raise KernelError("attention_decode_tc_rope: the launch failed")
    global launch_count
    launch_count += 1 if splits == 1 else 2        # a single split needs no merge kernel
    return True


def gemm_tc_gated(x, w, act, M: int, err, stream, force_bt: int = 0, force_stages: int = 0,
                  fn: Optional[GatedAct] = None) -> bool:
    """act[:M] = f(x @ w[:I].T, x @ w[I:].T) for w = [gate; up] with 2 I rows and f of the gated-activation family
    (`fn`; None: silu(gate) * up), on the tensor cores in one kernel.  Returns False, having launched nothing, when the
    operands do not meet the kernel's alignment rules."""
    two_i, K = w.shape
    status = core().iert_gemm_tc_gated(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), act.data_ptr(),
                                       act.stride(0), M, two_i // 2, K, byref(fn) if fn is not None else None,
                                       force_bt, force_stages, err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "gemm_tc_gated")
    return True


# ---------------------------------------------------------------------------------------
# streams of the residual, LayerNorm, soft cap


def _ptr(t):
    return t.data_ptr() if t is not None else None


def streams_norm(xs, S: int, H: int, rows: int, stream, *, y=None, mix=None, outc=None, update: bool = False,
                 write_back: bool = False, zero_y: bool = False, in_coef=None, w=None, b=None, eps: float = 0.0,
                 out=None, sum_out=None, rows_idx=None) -> None:
    """One pass over the S fp32 streams `xs` [T, S, H] of `rows` token rows: optional update with a
    sublayer's output `y` (x'_t = sum_s mix[s, t] x_s + outc[t] y; `write_back` stores it), optional
    clearing of y's rows, the combination u = sum_s in_coef[s] x'_s (ones when None), and LayerNorm
    of u with weight `w` and bias `b` into `out` (and / or u itself into `sum_out`).  `rows_idx`
    gathers token rows.  Small vectors are fp32."""
    check(core().iert_streams_norm(xs.data_ptr(), S, H, _ptr(y), _ptr(mix), _ptr(outc), 1 if update else 0,
                                   1 if write_back else 0, 1 if zero_y else 0, _ptr(in_coef), _ptr(w), _ptr(b), eps,
                                   _ptr(out), dtype_code(out.dtype) if out is not None else F32, _ptr(sum_out),
                                   _ptr(rows_idx), rows, stream), "streams_norm")


def streams_expand(x, xs, n_tokens: int, S: int, H: int, stream) -> None:
    check(core().iert_streams_expand(x.data_ptr(), xs.data_ptr(), n_tokens, S, H, stream), "streams_expand")


def softcap(z, cap: float, stream) -> None:
    check(core().iert_softcap(z.data_ptr(), z.numel(), cap, stream), "softcap")


# ---------------------------------------------------------------------------------------
# recurrent mixers


def delta_prep(proj, gates, conv_w, A_log, dt_bias, state, conv_off: int, qkv, beta, decay, G: int, D: int, H: int,
               V: int, taps: int, batch: BatchView, stream) -> None:
    check(core().iert_delta_prep(proj.data_ptr(), dtype_code(proj.dtype), proj.stride(0), gates.data_ptr(), gates.stride(0),
                                 conv_w.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(), state.stride(0),
                                 conv_off, qkv.data_ptr(), beta.data_ptr(), decay.data_ptr(), G, D, H, V, taps,
                                 byref(batch), stream), "delta_prep")


def gated_head_norm(o, proj, gate_off: int, w, per_head: bool, act: int, eps: float, out, n_tokens: int, H: int, V: int,
                    stream) -> None:
    """out[t, h, :] = o[t, h, :] / rms * w * act(gate): act 0 = SiLU, 1 = sigmoid; `per_head`: w is one
    vector of V shared by the heads, else H*V."""
    check(core().iert_gated_head_norm(o.data_ptr(), proj.data_ptr(), dtype_code(proj.dtype), proj.stride(0), gate_off,
                                      w.data_ptr(), 1 if per_head else 0, act, eps, out.data_ptr(), n_tokens, H, V, stream),
          "gated_head_norm")


_recurrent_libs = {}


def _recurrent_lib(dim: int):
    """The recurrence library for one key size, compiled on first use."""
    lib = _recurrent_libs.get(dim)
    if lib is None:
        lib = build.load_library(*build.recurrent_library(dim))
        P, LL = c_void_p, c_longlong
        lib.iert_delta_recur.argtypes = [P, P, P, P, LL, LL, P, c_int, c_int, c_int, POINTER(BatchView), P]
        lib.iert_delta_recur.restype = c_int
        lib.iert_mlstm_recur.argtypes = [P, c_int, LL, P, LL, P, P, c_float, P, LL, LL, LL, LL, P, P, c_int, c_int,
                                         POINTER(BatchView), P]
        lib.iert_mlstm_recur.restype = c_int
        lib.iert_wkv_recur.argtypes = [P, LL, P, P, P, LL, LL, P, c_int, c_int, POINTER(BatchView), P]
        lib.iert_wkv_recur.restype = c_int
        if os.environ.get("IERT_PDL", "1") == "0":
            lib.iert_set_pdl(0)
        _recurrent_libs[dim] = lib
    return lib


def _check_lib(status: int, what: str, launches: int = 1) -> None:
    global launch_count
    if status == 1:
        raise KernelError(f"{what}: the kernel does not take these sizes or options")
    if status != 0:
        raise KernelError(f"{what}: the launch failed")
    launch_count += launches


def delta_recur(qkv, beta, decay, state, s_off: int, o, G: int, D: int, H: int, V: int, batch: BatchView, stream) -> None:
    """The gated delta rule over the step's tokens, state [slots, floats] read and written at `s_off`."""
    _check_lib(_recurrent_lib(D).iert_delta_recur(qkv.data_ptr(), beta.data_ptr(), decay.data_ptr(), state.data_ptr(),
                                                  state.stride(0), s_off, o.data_ptr(), G, H, V, byref(batch), stream),
               "delta_recur")


def mlstm_recur(proj, gates, bi, bf, cap: float, state, s_off: int, n_off: int, m_off: int, coef, o, D: int, H: int, V: int,
                batch: BatchView, stream) -> None:
    """The mLSTM recurrence over the step's tokens (a scan of the gates and the normaliser, then the
    matrix state by columns)."""
    _check_lib(_recurrent_lib(D).iert_mlstm_recur(proj.data_ptr(), dtype_code(proj.dtype), proj.stride(0), gates.data_ptr(),
                                                  gates.stride(0), bi.data_ptr(), bf.data_ptr(), cap, state.data_ptr(),
                                                  state.stride(0), s_off, n_off, m_off, coef.data_ptr(), o.data_ptr(), H, V,
                                                  byref(batch), stream), "mlstm_recur", 2)


def token_shift(h, state, prev_off: int, mu, mixed, batch: BatchView, stream) -> None:
    """mixed[m, t] = h[t] + (h[t-1] - h[t]) * mu[m]; in front of a sequence's first token stands the row that
    `state` [slots, floats] keeps at `prev_off`."""
    n_mix, width = mu.shape
    check(core().iert_token_shift(h.data_ptr(), dtype_code(h.dtype), h.stride(0), state.data_ptr(), state.stride(0), prev_off,
                                  mu.data_ptr(), n_mix, width, mixed.data_ptr(), byref(batch), stream), "token_shift")


def wkv_decay(z, L: int, w2t, w0, decay, h, state, prev_off: int, batch: BatchView, stream) -> None:
    """decay[t, c] = exp(-exp(w0[c] + sum_l w2t[l, c] tanh(z[t, l]))) (fp32); also leaves every sequence's last row
    of `h` in `state` at `prev_off`."""
    check(core().iert_wkv_decay(z.data_ptr(), z.stride(0), L, w2t.data_ptr(), w0.data_ptr(), w0.numel(), decay.data_ptr(),
                                h.data_ptr(), dtype_code(h.dtype), h.stride(0), h.shape[-1], state.data_ptr(), state.stride(0),
                                prev_off, byref(batch), stream), "wkv_decay")


def wkv_recur(x, decay, u, state, s_off: int, o, D: int, H: int, V: int, batch: BatchView, stream) -> None:
    """o_t = (S + diag(u) k_t v_t^T)^T r_t; S <- diag(w_t) S + k_t v_t^T over the step's tokens, from the fp32
    projections x = [r | k | v | ...] and the decays w; S [H, D, V] per slot in `state` at `s_off`."""
    _check_lib(_recurrent_lib(D).iert_wkv_recur(x.data_ptr(), x.stride(0), decay.data_ptr(), u.data_ptr(), state.data_ptr(),
                                                state.stride(0), s_off, o.data_ptr(), H, V, byref(batch), stream), "wkv_recur")


def wkv_finish(o, gate, w, eps: float, out_scale: float, out, batch: BatchView, H: int, V: int, stream) -> None:
    """out = o / rms(o) per head * w * silu(gate) * out_scale (gate: fp32 [T, >= H*V])."""
    check(core().iert_wkv_finish(o.data_ptr(), gate.data_ptr(), gate.stride(0), w.data_ptr(), eps, out_scale, out.data_ptr(),
                                 dtype_code(out.dtype), byref(batch), H, V, stream), "wkv_finish")


# ---------------------------------------------------------------------------------------
# latent attention, routing


def latent_norm_store(x, q_rank: int, kv_rank: int, wq, wkv, eps: float, cq, c, batch: BatchView, kv: KvView, store: bool,
                      err, stream) -> None:
    check(core().iert_latent_norm_store(x.data_ptr(), x.stride(0), q_rank, kv_rank, wq.data_ptr(), wkv.data_ptr(), eps,
                                        cq.data_ptr(), c.data_ptr(), dtype_code(c.dtype), byref(batch), byref(kv),
                                        1 if store else 0, err.data_ptr(), stream), "latent_norm_store")


def latent_attention_prompt(qkv, out, batch: BatchView, H: int, D: int, V: int, scale: float, sink, stream) -> None:
    check(core().iert_latent_attention_prompt(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), dtype_code(qkv.dtype),
                                              byref(batch), H, D, V, scale, _ptr(sink), stream), "latent_attention_prompt")


def latent_attention_decode(q, w_uk, w_uv, out, batch: BatchView, kv: KvView, H: int, D: int, V: int, scale: float, sink,
                            err, stream, rot_dim: int = 0, gate=None) -> None:
    """`rot_dim` R: a query head is [D unrotated | R rotated] and a cached row [latent | R rotated key numbers];
    `gate` (fp32 [T, H], optional) multiplies each head's result."""
    check(core().iert_latent_attention_decode(q.data_ptr(), q.stride(0), w_uk.data_ptr(), w_uv.data_ptr(), out.data_ptr(),
                                              dtype_code(q.dtype), byref(batch), byref(kv), H, D, rot_dim, V, scale, _ptr(sink),
                                              _ptr(gate), err.data_ptr(), stream), "latent_attention_decode")


def latent_prep(x, H: int, D: int, R: int, rank: int, wkv, eps: float, inv_freq, pairing: int, out_scale: float, c_ext, q_out,
                q_head: int, gate_out, batch: BatchView, kv: KvView, store: bool, err, stream) -> None:
    """From the fp32 projection rows x = [q: H x (D | R) | latent: rank | rotated key part: R | gate logits: H (if
    `gate_out`)] to the normed latent and rotated key part `c_ext` [T, rank + R] (also the cache row, with `store`), the
    queries `q_out` [T, H, q_head] (rotated part turned, zeros beyond D + R) and `gate_out` = sigmoid(logit) * out_scale."""
    check(core().iert_latent_prep(x.data_ptr(), x.stride(0), H, D, R, rank, wkv.data_ptr(), eps, _ptr(inv_freq), pairing,
                                  1 if gate_out is not None else 0, out_scale, c_ext.data_ptr(), q_out.data_ptr(), q_out.stride(0),
                                  q_head,
                                  _ptr(gate_out), dtype_code(c_ext.dtype), byref(batch), byref(kv), 1 if store else 0,
                                  err.data_ptr(), stream), "latent_prep")


def head_gate_mul(attn, head: int, out, V: int, H: int, gate, batch: BatchView, stream) -> None:
    """out[t, h, :V] = attn[t, h, :V] * gate[t, h] for heads stored `head` numbers apart (gate None: a plain copy)."""
    check(core().iert_head_gate_mul(attn.data_ptr(), head, out.data_ptr(), V, H, _ptr(gate), dtype_code(attn.dtype), byref(batch),
                                    stream), "head_gate_mul")


def latent_decode_tc_plan(n_seqs: int, H: int, table_width: int):
    """(heads padded to whole MMA tiles, runs a sequence is cut into) of the tensor-core one-token kernel."""
    hpad, splits = c_int(0), c_int(0)
    core().iert_latent_decode_tc_plan(n_seqs, H, table_width, byref(hpad), byref(splits))
    return hpad.value, splits.value


def latent_attention_decode_tc(q, w_uk, w_uv, out, batch: BatchView, kv: KvView, H: int, D: int, V: int, scale: float, sink,
                               hpad: int, splits: int, qa, part_m, part_l, part_acc, err, stream, rot_dim: int = 0,
                               gate=None) -> bool:
    """One-token latent attention on the tensor cores (bf16, rank a multiple of 32 up to 512, pages of 64):
    the absorbed queries, the split attention over the cached latents, the merge with the sink and W_uv.
    Returns False, having launched nothing, for sizes it does not take."""
    lib = core()
    fn = lib.iert_latent_attention_decode_tc
    if not getattr(fn, "_declared", False):
        fn.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, POINTER(BatchView), POINTER(KvView), c_int, c_int,
                       c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p]
        fn.restype = c_int
        fn._declared = True
    status = fn(q.data_ptr(), q.stride(0), w_uk.data_ptr(), w_uv.data_ptr(), out.data_ptr(), byref(batch), byref(kv), H, D,
                rot_dim, V, scale, _ptr(sink), _ptr(gate), hpad, splits, qa.data_ptr(), part_m.data_ptr(), part_l.data_ptr(), part_acc.data_ptr(),
                err.data_ptr(), stream)
    if status == 1:
        return False
    check(status, "latent_attention_decode_tc")
    global launch_count
    launch_count += 2
    return True


def router_topk(z, bias, n_tokens: int, E: int, top: int, wt, idx, w, stream) -> None:
    check(core().iert_router_topk(z.data_ptr(), z.stride(0), _ptr(bias), n_tokens, E, top, wt.data_ptr(), idx.data_ptr(),
                                  w.data_ptr(), stream), "router_topk")


ROUTER_SCORES = {"softmax": 0, "sigmoid": 1}
ROUTER_GROUP_SCORES = {"max": 0, "top2_sum": 1}


def router_grouped(z, correction, n_tokens: int, E: int, N: int, top: int, groups: int, keep: int, wt, wid, idx, w,
                   stream, by_output: bool = False, score: str = "softmax", group_score: str = "max",
                   weight_eps: float = 1e-20, weight_scale: float = 1.0) -> None:
    """Scores = softmax over all N router outputs, or each output's sigmoid (the last N - E stand for experts that return
    their input); choice on score + correction inside the `keep` best of `groups` runs of neighbours (a run's score: its
    best choice score, or the sum of its two best); weights = chosen scores over (their sum + weight_eps), times
    weight_scale.  z: fp32 [T, N], or with `by_output` [N, T] (a row per router output).  wt [T, E] dense, wid [T] the
    identity experts' share, idx / w [T, top]."""
    ldz, lde = (z.stride(1), z.stride(0)) if by_output else (z.stride(0), z.stride(1))
    check(core().iert_router_grouped(z.data_ptr(), ldz, lde, _ptr(correction), n_tokens, E, N, top, groups, keep,
                                     ROUTER_SCORES[score], ROUTER_GROUP_SCORES[group_score], weight_eps, weight_scale,
                                     wt.data_ptr(), wid.data_ptr(), idx.data_ptr(), w.data_ptr(), stream), "router_grouped")


def moe_scale(act, wt, n_tokens: int, E: int, F: int, stream, wid=None, x=None, residual=None) -> None:
    """act[t, e*F + i] *= wt[t, e]; with `wid`, also residual[t] += wid[t] * x[t]."""
    check(core().iert_moe_scale(act.data_ptr(), dtype_code(act.dtype), act.stride(0), wt.data_ptr(), n_tokens, E, F,
                                _ptr(wid), _ptr(x), x.stride(0) if x is not None else 0, _ptr(residual),
                                residual.shape[-1] if residual is not None else 0, stream), "moe_scale")


# ---------------------------------------------------------------------------------------
# norm on a sublayer's output, keys that double as values, the gated linear recurrence


def add_normed(x, y, w, cast, rows: int, eps: float, stream) -> None:
    """x[:rows] += y / rms(y) * w (fp32; w with any offset already added); y's rows are cleared; `cast`
    (optional) receives the new rows in its dtype."""
    check(core().iert_add_normed(x.data_ptr(), y.data_ptr(), w.data_ptr(), _ptr(cast),
                                 dtype_code(cast.dtype) if cast is not None else F32, rows, x.shape[-1], eps, stream),
          "add_normed")


def cast_rows(x, y, cast, rows: int, stream) -> None:
    """cast[:rows] = x[:rows] in cast's dtype; y[:rows] = 0 (y optional)."""
    check(core().iert_cast_rows(x.data_ptr(), _ptr(y), cast.data_ptr(), dtype_code(cast.dtype), rows * x.shape[-1], stream),
          "cast_rows")


def scale_values(z, s: float, stream) -> None:
    check(core().iert_scale_values(z.data_ptr(), z.numel(), s, stream), "scale_values")


NORM_NONE, NORM_WHOLE_WEIGHTED, NORM_HEAD_UNIT = 0, 1, 2


def qk_prep(proj, qkv, batch: BatchView, kv: KvView, heads: int, inv_freq, rotary_dim: int, norm_mode: int, wq, wk,
            eps: float, value_scale: float, store: bool, err, stream) -> None:
    """From the fp32 projection rows [q | k] to the packed rows [q' | k' | v] (v = k as projected times
    `value_scale`), with the norm of `norm_mode`, the rotation, and the cache write of k' and v."""
    check(core().iert_qk_prep(proj.data_ptr(), proj.stride(0), qkv.data_ptr(), dtype_code(qkv.dtype), byref(batch), byref(kv),
                              heads, inv_freq.data_ptr(), rotary_dim, norm_mode, _ptr(wq), _ptr(wk), eps, value_scale,
                              1 if store else 0, err.data_ptr(), stream), "qk_prep")


def qkv_prep(proj, bias, qkv, batch: BatchView, kv: KvView, heads: int, dim: int, vdim: int, inv_freq, rotary_dim: int,
             pairing: int, wq, wk, eps: float, store: bool, err, stream) -> None:
    """From the fp32 projection rows that begin with [q | k | v] (+ `bias`) to the packed rows [q' | k' | v'] with every
    head padded with zeros to the cache's head size: per-head weighted RMS norm of q and k (`wq`, `wk` of length `dim`,
    optional), rotation, one rounding, and the cache write of k' and v'."""
    check(core().iert_qkv_prep(proj.data_ptr(), proj.stride(0), _ptr(bias), qkv.data_ptr(), dtype_code(qkv.dtype), byref(batch),
                               byref(kv), heads, dim, vdim, _ptr(inv_freq), rotary_dim, pairing, _ptr(wq), _ptr(wk), eps,
                               1 if store else 0, err.data_ptr(), stream), "qkv_prep")


def gate_mul(attn, gate, out, n_tokens: int, heads: int, D: int, vdim: int, stream) -> None:
    """out[t, h*vdim + c] = attn[t, h*D + c] * sigmoid(gate[t, h*vdim + c]); `gate` (fp32, a view whose rows may be
    strided) may be None: the padding of the heads is dropped and nothing else."""
    check(core().iert_gate_mul(attn.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(),
                               dtype_code(attn.dtype), n_tokens, heads, D, vdim, stream), "gate_mul")


def rglru_conv(proj, bx, taps, cb, state, u, C: int, K: int, batch: BatchView, stream) -> None:
    check(core().iert_rglru_conv(proj.data_ptr(), proj.stride(0), bx.data_ptr(), taps.data_ptr(), cb.data_ptr(),
                                 state.data_ptr(), state.stride(0), u.data_ptr(), C, K, byref(batch), stream), "rglru_conv")


def rglru_gates(u, ra, ra_b, ri, ri_b, lam, decay_c: float, A, Bv, n_tokens: int, C: int, blocks: int, stream) -> None:
    check(core().iert_rglru_gates(u.data_ptr(), ra.data_ptr(), ra_b.data_ptr(), ri.data_ptr(), ri_b.data_ptr(),
                                  dtype_code(ra.dtype), lam.data_ptr(), decay_c, A.data_ptr(), Bv.data_ptr(), n_tokens, C,
                                  blocks, stream), "rglru_gates")


def rglru_scan_scratch_floats(n_seqs: int, max_q_len: int, C: int) -> int:
    lib = core()
    lib.iert_rglru_scan_scratch_floats.restype = c_longlong
    return int(lib.iert_rglru_scan_scratch_floats(n_seqs, max_q_len, C))


def rglru_scan(A, Bv, proj, by, bx, state, out, out_scale: float, C: int, K: int, batch: BatchView, stream,
               max_q_len: int = 0, scratch=None) -> None:
    """`max_q_len` and `scratch` (fp32, `rglru_scan_scratch_floats`): long sequences are scanned in chunks (two kernels)."""
    check(core().iert_rglru_scan(A.data_ptr(), Bv.data_ptr(), proj.data_ptr(), proj.stride(0), by.data_ptr(), bx.data_ptr(),
                                 state.data_ptr(), state.stride(0), out.data_ptr(), dtype_code(out.dtype), out_scale, C, K,
                                 max_q_len, _ptr(scratch), byref(batch), stream), "rglru_scan")
