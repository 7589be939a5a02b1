"""Prefill and decode of one architecture beside another at equal width, depth and feed-forward size,
with random weights: whole-step times and, kernel by kernel, where a step's time goes against what the
bytes and FLOPs of each kernel allow.  Used by `bench.py --design`.

Kernel times come from CUDA events recorded around every launcher call of a step that is launched kernel
by kernel (no graph): each number is a kernel's own time with its operands as the kernel before left them.
"""
from __future__ import annotations

import statistics
import time
from typing import Callable, Dict, List

# CUDA-core fp32 rate of the part (FMA = 2 FLOP): 148 SMs x 128 lanes x 2 x clock
FP32_TFLOPS = 148 * 128 * 2 * 1.9e9 / 1e12

LAUNCHERS = ["embed_gather", "rmsnorm", "rope_kv_store", "silu_mul", "gemm_plain", "gemm_tc", "gemm_rows", "gemm_tc_scaled",
             "gemm_tc_gated", "gemm_tc_gated_scaled", "attention_prefill", "attention_decode_tc", "attention_decode_tc_rope",
             "attention_decode", "attention_plain", "streams_norm", "streams_expand", "softcap", "delta_prep", "delta_recur",
             "mlstm_recur", "gated_head_norm", "latent_norm_store", "latent_attention_prompt", "latent_attention_decode_tc",
             "latent_attention_decode", "router_topk", "moe_scale", "add_normed", "cast_rows", "scale_values", "qk_prep",
             "rglru_conv", "rglru_gates", "rglru_scan", "qkv_prep", "gate_mul", "router_grouped", "gated_act_mul",
             "token_shift", "wkv_decay", "wkv_recur", "wkv_finish", "latent_prep", "head_gate_mul"]
GEMMS = {"gemm_plain", "gemm_tc", "gemm_rows", "gemm_tc_scaled", "gemm_tc_gated", "gemm_tc_gated_scaled"}


class KernelClock:
    """Wraps the launchers of `csrc.bindings` with CUDA events while it is active."""

    def __init__(self):
        import torch
        from .csrc import bindings as B
        self.torch, self.B = torch, B
        self.records: List[tuple] = []
        self._saved: Dict[str, Callable] = {}

    def __enter__(self):
        torch, B = self.torch, self.B
        for name in LAUNCHERS:
            fn = getattr(B, name, None)
            if fn is None:
                continue
            self._saved[name] = fn

            def wrapped(*args, _fn=fn, _name=name, **kw):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                out = _fn(*args, **kw)
                b.record()
                label, flops, nbytes = _name, 0.0, 0.0
                if _name in GEMMS and out is not False:
                    x, w, o, M = args[0], args[1], args[2], args[3]
                    N, K = w.shape
                    label = f"{_name} [{N} x {K}]"
                    flops = 2.0 * M * N * K
                    nbytes = w.numel() * w.element_size() + M * K * x.element_size() + M * N * o.element_size()
                elif _name == "attention_prefill":
                    label = f"{_name} [head {args[5]}]"           # a model may run it at more than one head size
                if out is not False:
                    self.records.append((label, a, b, flops, nbytes))
                return out
            setattr(B, name, wrapped)
        return self

    def __exit__(self, *exc):
        for name, fn in self._saved.items():
            setattr(self.B, name, fn)
        self._saved = {}

    def table(self, model_costs: Dict[str, tuple], pk) -> List[dict]:
        """Per launcher: calls, microseconds in all, and the fraction of what its bytes and FLOPs allow
        (`model_costs[name]` = (flops, tensor-core?, bytes) per call for kernels that are no product)."""
        self.torch.cuda.synchronize()
        agg: Dict[str, list] = {}
        for label, a, b, flops, nbytes in self.records:
            row = agg.setdefault(label, [0, 0.0, 0.0, 0.0])
            row[0] += 1
            row[1] += a.elapsed_time(b) * 1e3
            row[2] += flops
            row[3] += nbytes
        out = []
        for label, (calls, us, flops, nbytes) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
            row = {"kernel": label, "calls": calls, "us": round(us, 1)}
            tensor = True
            base = label.split(" ")[0]
            if label in model_costs or base in model_costs:
                f, tensor, nb = model_costs[label if label in model_costs else base]
                flops, nbytes = f * calls, nb * calls
            if flops or nbytes:
                peak = pk["bf16_tflops"] if tensor else FP32_TFLOPS
                floor_us = max(flops / (peak * 1e6), nbytes / (pk["hbm_gbs"] * 1e3))
                row["floor_us"] = round(floor_us, 1)
                row["frac"] = round(floor_us / us, 3) if us > 0 else None
                row["bound"] = "flops" if flops / (peak * 1e6) >= nbytes / (pk["hbm_gbs"] * 1e3) else "bytes"
            out.append(row)
        return out


def _costs(cfg: dict, T: int, n_seqs: int, ctx: int, prompt: bool) -> Dict[str, tuple]:
    """(flops, on the tensor cores?, bytes) of one call of each kernel that is no plain product, from the
    configuration's sizes: T tokens in the step, n_seqs sequences, ctx cached positions each."""
    out = {}
    if cfg.get("architecture") == "Vefulix":
        H, S = cfg["width"], cfg.get("streams") or 1
        out["streams_norm"] = (0.0, False, T * H * (4 * (2 * S + 2) + 2))
        by = {l["type"]: l["mixer"] for l in cfg["layers"]}
        if "delta" in by:
            m = by["delta"]
            C = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
            state = 2 * 4 * n_seqs * m["heads"] * m["dim"] * m["vdim"]
            out["delta_prep"] = (0.0, False, T * C * 6)
            out["delta_recur"] = (8.0 * T * m["heads"] * m["dim"] * m["vdim"], False, T * (C + m["heads"] * m["vdim"]) * 4 + state)
            out["gated_head_norm"] = (0.0, False, T * m["heads"] * m["vdim"] * 8)
        if "mlstm" in by:
            m = by["mlstm"]
            state = 2 * 4 * n_seqs * m["heads"] * m["dim"] * m["vdim"]
            out["mlstm_recur"] = (6.0 * T * m["heads"] * m["dim"] * m["vdim"], False,
                                  T * (2 * m["heads"] * m["dim"] + m["heads"] * m["vdim"]) * 2 + T * m["heads"] * m["vdim"] * 4 + state)
        if "latent_attention" in by:
            m = by["latent_attention"]
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            att = (2.0 * (hd + hv) * T * (T + 1) / 2, True, T * (2 * hd + 2 * hv) * 2)
            out["latent_attention_prompt"] = out["attention_prefill"] = att
            dec = (4.0 * n_seqs * m["heads"] * ctx * m["kv_rank"], True,
                   n_seqs * ctx * m["kv_rank"] * 2 + (hd + hv) * m["kv_rank"] * 2)
            out["latent_attention_decode"] = out["latent_attention_decode_tc"] = dec
            out["latent_norm_store"] = (0.0, False, T * (m["q_rank"] + m["kv_rank"]) * 8)
        mlp = cfg["layers"][0]["mlp"]
        if mlp:
            inter = mlp["router"]["experts"] * mlp["expert"]["ff"]
            out["moe_scale"] = (0.0, False, T * inter * 4)
    elif cfg.get("architecture") == "Sifasun":
        H = cfg["width"]
        out["add_normed"] = (0.0, False, T * H * 18)
        out["cast_rows"] = (0.0, False, T * H * 10)
        by = {l["type"]: l["mixer"] for l in cfg["layers"]}
        att = by.get("attention") or by["parallel"]["left"]
        hd, kvd = att["heads"] * att["dim"], att["kv_heads"] * att["dim"]
        W = (att.get("mask") or {}).get("size") or (1 << 30)
        seen = T * (T + 1) / 2 if T <= W else W * (W + 1) / 2 + (T - W) * W        # (query, key) pairs inside the window
        out["attention_prefill"] = (4.0 * hd * seen, True, T * (2 * hd + 2 * kvd) * 2)
        out["attention_decode_tc"] = (0.0, False, n_seqs * min(ctx, W) * 2 * kvd * 2)
        out["qk_prep"] = (0.0, False, T * ((hd + kvd) * 4 + (hd + 2 * kvd) * 2 + 2 * kvd * 2))
        if "parallel" in by:
            r = by["parallel"]["right"]
            C, bw = r["width"], r["width"] // r["blocks"]
            out["rglru_conv"] = (0.0, False, T * C * 8)
            out["rglru_gates"] = (4.0 * T * C * bw, False, T * C * 12 + 2 * C * bw * 2)
            out["rglru_scan"] = (0.0, False, T * C * 14 + n_seqs * C * r["conv"] * 8)
    elif cfg.get("architecture") == "Kuvelix":
        H = cfg["width"]
        m = cfg["layers"][0]["mixer"]
        D = -(-max(m["dim"], m["vdim"]) // 16) * 16                      # the padded head size of the packed rows
        qd, kd, vd, ad = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"], m["heads"] * m["vdim"]
        packed = (m["heads"] + 2 * m["kv_heads"]) * D
        out["rmsnorm"] = (0.0, False, T * H * 6)
        out["qkv_prep"] = (0.0, False, T * ((qd + kd + vd) * 4 + packed * 2 + 2 * m["kv_heads"] * D * 2))
        out["gate_mul"] = (0.0, False, T * (m["heads"] * D * 2 + ad * 4 + ad * 2))
        out["attention_prefill"] = (4.0 * m["heads"] * D * T * (T + 1) / 2, True, T * (2 * m["heads"] * D + 2 * m["kv_heads"] * D) * 2)
        out["attention_decode_tc"] = (0.0, False, n_seqs * ctx * 2 * m["kv_heads"] * D * 2)
        mlp = next((l["mlp"] for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe"), None)
        if mlp:
            r = mlp["router"]
            out["moe_scale"] = (0.0, False, T * (r["experts"] * mlp["expert"]["ff"] * 4 + (10 * H if r.get("identity") else 0)))
            out["router_grouped"] = (0.0, False, T * (r["experts"] + r.get("identity", 0)) * 8)
    elif cfg.get("architecture") == "Vufinex":
        H = cfg["width"]
        out["rmsnorm"] = (0.0, False, T * H * 6)
        by = {l["type"]: l["mixer"] for l in cfg["layers"]}
        if "attention" in by:
            m = by["attention"]
            hd, kvd = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            C = (m.get("mask") or {}).get("size") or (1 << 30)
            seen = sum(min(i % C, i) + 1 for i in range(T)) if prompt else 0          # (query, key) pairs inside the chunks
            out[f"attention_prefill [head {m['dim']}]"] = (4.0 * hd * seen, True, T * (2 * hd + 2 * kvd) * 2)
            out["attention_decode_tc"] = (0.0, False, n_seqs * (ctx % C + 1) * 2 * kvd * 2)
            out["qk_prep"] = (0.0, False, T * ((hd + kvd) * 4 + (hd + 2 * kvd) * 2 + 2 * kvd * 2))
        if "wkv" in by:
            m = by["wkv"]
            C, L = m["heads"] * m["dim"], m.get("decay_rank") or max(8, (H // 16 + 7) // 8 * 8)
            state = 2 * 4 * n_seqs * C * m["dim"]
            out["token_shift"] = (0.0, False, T * H * 12)
            out["wkv_decay"] = (2.0 * T * C * L, False, T * (L + C) * 4 + L * C * 4)
            out["wkv_recur"] = (7.0 * T * C * m["dim"], False, T * C * 5 * 4 + state)
            out["wkv_finish"] = (0.0, False, T * C * 10)
        if "latent_attention" in by:
            m = by["latent_attention"]
            P = -(-max(m["dim"] + m["rot_dim"], m["vdim"]) // 16) * 16
            wide = m["kv_rank"] + m["rot_dim"]
            row = m["heads"] * (m["dim"] + m["rot_dim"]) + wide + m["heads"]
            out[f"attention_prefill [head {P}]"] = (4.0 * m["heads"] * P * T * (T + 1) / 2, True, T * 4 * m["heads"] * P * 2)
            out["latent_prep"] = (0.0, False, T * (row * 4 + wide * 4 + m["heads"] * P * 2))
            out["head_gate_mul"] = (0.0, False, T * m["heads"] * (P + m["vdim"]) * 2)
            out["latent_attention_decode"] = out["latent_attention_decode_tc"] = (
                2.0 * n_seqs * m["heads"] * ctx * (wide + m["kv_rank"]), True,
                n_seqs * ctx * wide * 2 + m["heads"] * (m["dim"] + m["vdim"]) * m["kv_rank"] * 2)
        mlp = next((l["mlp"] for l in cfg["layers"] if l["mlp"]), None)
        if mlp:
            r = mlp["router"]
            out["moe_scale"] = (0.0, False, T * r["experts"] * mlp["expert"]["ff"] * 4)
            out["router_grouped"] = (0.0, False, T * r["experts"] * 8)
    else:
        hd = cfg["num_attention_heads"] * cfg["head_dim"]
        kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
        out["attention_prefill"] = (4.0 * hd * T * (T + 1) / 2, True, T * (2 * hd + 2 * kvd) * 2)
        out["attention_decode_tc_rope"] = out["attention_decode_tc"] = (0.0, False, n_seqs * ctx * 2 * kvd * 2)
        out["rmsnorm"] = (0.0, False, T * cfg["hidden_size"] * 6)
        out["rope_kv_store"] = (0.0, False, T * (hd + 2 * kvd) * 4)
    return out


def measure(cfg: dict, pk, batch: int, context: int, prefill_tokens: int, steps: int, warmup: int, seed: int = 0) -> dict:
    """Prefill of one prompt and one-token steps of `batch` sequences at `context` tokens: device times of
    whole steps (graphs on, as served) and a kernel table of one step of each kind (launched kernel by kernel)."""
    import numpy as np
    import torch
    from . import LoadedModel, Sampler, SamplingParams
    rng = np.random.default_rng(seed)
    model = LoadedModel.random(cfg, seed=seed, dtype="bfloat16", std=0.02, on_device=True)
    vocab = model.spec.vocab_size
    per_seq = -(-(context + 2 * (steps + warmup) + 16) // 64) * 64
    room = max(batch * per_seq, -(-prefill_tokens // 64) * 64)
    out = {"layers": len(model.spec.schedule), "weight_gb_per_step": round(model.model.weight_bytes_per_step() / 1e9, 3)}

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    for graphs in (True, False):
        session = model.session(max_tokens=room, max_sequences=batch, max_seq_len=max(per_seq, prefill_tokens), use_graphs=graphs)
        eng = session.engine
        sampler = Sampler(SamplingParams(temperature=0.0), eng.rt.err)
        prompt = rng.integers(0, vocab, prefill_tokens).tolist()
        if graphs:
            times = []
            for i in range(2 + 3):
                s = eng.open_sequence()
                a, b = events()
                a.record()
                eng.step([(s, prompt)], want="last")
                b.record()
                torch.cuda.synchronize()
                eng.close_sequence(s)
                if i >= 2:
                    times.append(a.elapsed_time(b))
            out["prefill_ms"] = round(statistics.median(times), 3)
            out["prefill_tok_s"] = round(prefill_tokens * 1e3 / statistics.median(times), 1)
        else:
            s = eng.open_sequence()
            eng.step([(s, prompt)], want="last")
            eng.close_sequence(s)
            s = eng.open_sequence()
            with KernelClock() as clock:
                eng.step([(s, prompt)], want="last")
            out["prefill_kernels"] = clock.table(_costs(cfg, prefill_tokens, 1, prefill_tokens, True), pk)
            eng.close_sequence(s)
        slots = []
        for _ in range(batch):
            s = eng.open_sequence()
            eng.step([(s, rng.integers(0, vocab, context).tolist())], want=None)
            slots.append(s)
        toks = rng.integers(0, vocab, (steps + warmup, batch))
        if graphs:
            a, b = events()
            for i in range(steps + warmup):
                if i == warmup:
                    torch.cuda.synchronize()
                    a.record()
                logits = eng.step([(s, [int(t)]) for s, t in zip(slots, toks[i])], want="last")
                sampler.sample_device(logits, list(range(batch)), [i] * batch)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            nbytes = model.model.weight_bytes_per_step() + eng.cache.kv_bytes_read(slots)
            out["decode_ms_per_step"] = round(ms, 4)
            out["decode_tok_s"] = round(batch * 1e3 / ms, 1)
            out["decode_frac_of_hbm"] = round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        else:
            for i in range(2):
                eng.step([(s, [int(t)]) for s, t in zip(slots, toks[i])], want="last")
            with KernelClock() as clock:
                eng.step([(s, [int(t)]) for s, t in zip(slots, toks[2])], want="last")
            out["decode_kernels"] = clock.table(_costs(cfg, batch, batch, context, False), pk)
        eng.check_device()
        for s in slots:
            eng.close_sequence(s)
        del session, eng
    del model
    torch.cuda.empty_cache()
    return out


def compare(design: str, baseline: str, layers: int, pk, batch: int, context: int, prefill_tokens: int, steps: int,
            warmup: int) -> dict:
    from .config import preset
    a, b = preset(design), preset(baseline)
    a["layers"] = a["layers"][:layers]
    if "layers" in b:                       # a baseline whose configuration lists its layers
        b["layers"] = b["layers"][:layers]
    else:
        b["num_hidden_layers"] = layers
    t0 = time.time()
    res = {"design": design, "baseline": baseline, "layers": layers, "batch": batch, "context": context,
           "prefill_tokens": prefill_tokens, "steps": steps, "warmup": warmup, "dtype": "bf16",
           "data": "synthetic (random weights N(0, 0.02), uniform random token ids)",
           "peaks": {k: pk[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "fp32_cuda_core_tflops": round(FP32_TFLOPS, 1),
           design: measure(a, pk, batch, context, prefill_tokens, steps, warmup),
           baseline: measure(b, pk, batch, context, prefill_tokens, steps, warmup)}
    res["seconds"] = round(time.time() - t0, 1)
    return res
