"""Named configurations for the random-weights mode: each is the content of a config.json, as
data.  Nothing in the library reads a size from here; a preset only saves writing the file.

The three full sizes are the published layer sizes of Mistral 7B v0.1 and v0.3 and of Mistral
NeMo 12B; the two tiny ones differ from each other in every size and option (heads and groups,
head size against hidden size, window, rope base, norm epsilon) and run anywhere in seconds.
The reference has one built-in default, the path of its Mistral 7B file (src/main.rs:26-32).
"""
from __future__ import annotations

import copy
from typing import Dict

_MISTRAL = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_act": "silu",
            "tie_word_embeddings": False, "bos_token_id": 1, "eos_token_id": 2}

PRESETS: Dict[str, dict] = {
    "7b-v0.1": dict(_MISTRAL, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                    num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32000,
                    rope_theta=10000.0, sliding_window=4096, rms_norm_eps=1e-5, max_position_embeddings=32768),
    "7b-v0.3": dict(_MISTRAL, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                    num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32768,
                    rope_theta=1000000.0, sliding_window=None, rms_norm_eps=1e-5, max_position_embeddings=32768),
    "nemo-12b": dict(_MISTRAL, num_hidden_layers=40, hidden_size=5120, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=131072,
                     rope_theta=1000000.0, sliding_window=None, rms_norm_eps=1e-5, max_position_embeddings=131072),
    "tiny-a": dict(_MISTRAL, num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=256,
                   rope_theta=10000.0, sliding_window=16, rms_norm_eps=1e-5, max_position_embeddings=512),
    "tiny-b": dict(_MISTRAL, num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
                   num_key_value_heads=1, head_dim=32, intermediate_size=160, vocab_size=384,
                   rope_theta=1000000.0, sliding_window=None, rms_norm_eps=1e-6, max_position_embeddings=1024),
}



def _vefulix(width, vocab, layers, streams, heads, dim, vdim, q_rank, kv_rank, experts, top, expert_ff, shared_ff):
    """A Vefulix configuration whose layers go round delta, latent attention, mLSTM, latent attention."""
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}, "shared": {"ff": shared_ff}}
    mixers = [
        ("delta", {"heads": heads, "kv_heads": max(1, heads // 4), "dim": dim, "vdim": vdim, "conv": 4}),
        ("latent_attention", {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                              "scale": dim ** -0.5}),
        ("mlstm", {"heads": max(1, heads // 2), "dim": dim, "vdim": 2 * vdim, "gate_cap": 15.0}),
        ("latent_attention", {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                              "scale": dim ** -0.5}),
    ]
    return {"architecture": "Vefulix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "streams": streams,
            "logit_softcap": 30.0,
            "layers": [{"type": mixers[i % 4][0], "mixer": dict(mixers[i % 4][1]), "mlp": dict(moe)} for i in range(layers)]}


# Vefulix at the width, head count and total feed-forward size (16 experts of 768 + a shared 2,048 = 14,336)
# of Mistral 7B, and a tiny one that runs anywhere in seconds.
PRESETS["vefulix-7b-sizes"] = _vefulix(4096, 32000, 32, 2, 32, 128, 128, 1536, 512, 16, 2, 768, 2048)
PRESETS["vefulix-tiny"] = _vefulix(96, 320, 4, 2, 4, 16, 24, 48, 40, 6, 2, 32, 64)


def _sifasun(width, vocab, layers, heads, kv_heads, dim, ff, lru_width, blocks, window, shared_from=None):
    """A Sifasun configuration: one pair layer (attention beside a gated linear recurrence), then three attention
    layers, round and round; from layer `shared_from` on, layers run with the weights of the layer that many places
    before them."""
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 30.0,
                 "mask": {"size": window}, "rot": {"base": 1000000.0, "dims": dim // 2, "scaling": {"factor": 8.0}}}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
            "mask": {"size": 2 * window}, "rot": {"base": 10000.0, "dims": dim}}
    pair = {"left": left, "left_scale": 1.1, "right": {"width": lru_width, "blocks": blocks, "conv": 4}, "right_scale": 0.8}
    out = []
    for i in range(layers):
        entry = {"type": "parallel" if i % 4 == 0 else "attention", "mixer": dict(pair if i % 4 == 0 else attention),
                 "mlp": {"kind": "dense", "ff": ff}}
        if shared_from is not None and i >= shared_from:
            entry["weights_of"] = i - shared_from
        out.append(entry)
    return {"architecture": "Sifasun", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 1.0, "layers": out}


# Sifasun at the width, head count, head size and feed-forward size of Mistral 7B (a recurrence as wide as the model in
# 16 blocks), and a tiny one that runs anywhere in seconds (its last four layers run with the first four's weights).
PRESETS["sifasun-7b-sizes"] = _sifasun(4096, 32000, 32, 32, 8, 128, 14336, 4096, 16, 2048)
# the same at the sizes of Mistral NeMo 12B (width 5,120, a vocabulary of 131,072)
PRESETS["sifasun-12b-sizes"] = _sifasun(5120, 131072, 40, 32, 8, 128, 14336, 5120, 16, 2048)
PRESETS["sifasun-tiny"] = _sifasun(96, 320, 8, 4, 2, 16, 160, 64, 4, 24, shared_from=4)


def _kuvelix(width, vocab, layers, heads, kv_heads, dim, vdim, ff, experts, identity, top, groups, keep, expert_ff, loop=None):
    """A Kuvelix configuration: a dense layer first, then mixture-of-experts layers, every fourth layer without a
    feed-forward when there are more than four; `loop` = (start, stop, times)."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
             "rot": {"base": 10000.0, "dims": dim // 2, "scaling": {"factor": 4.0}}}
    moe = {"kind": "moe", "expert": {"ff": expert_ff, "limit": 7.0},
           "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    out = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff} if i == 0 else (None if layers > 4 and i % 4 == 3 else copy.deepcopy(moe))
        out.append({"type": "attention", "mixer": copy.deepcopy(mixer), "mlp": mlp})
    cfg = {"architecture": "Kuvelix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": out}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# Kuvelix at the width, head count, head size and total feed-forward size (14 experts of 1,024 = 14,336) of Mistral 7B, and
# a tiny one that runs anywhere in seconds (value size unlike the key size, its layers 1 and 2 run twice).
PRESETS["kuvelix-7b-sizes"] = _kuvelix(4096, 32000, 32, 32, 8, 128, 128, 14336, 14, 2, 2, 4, 2, 1024)
# the same at the sizes of Mistral NeMo 12B (width 5,120, a vocabulary of 131,072)
PRESETS["kuvelix-12b-sizes"] = _kuvelix(5120, 131072, 40, 32, 8, 128, 128, 14336, 14, 2, 2, 4, 2, 1024)
PRESETS["kuvelix-tiny"] = _kuvelix(80, 320, 4, 6, 2, 16, 24, 136, 5, 3, 3, 4, 3, 40, loop=(1, 3, 2))


def _vufinex(width, vocab, layers, heads, kv_heads, dim, chunk, wkv_heads, wkv_dim, decay_rank, lat_dim, rot_dim, vdim, kv_rank,
             experts, top, groups, keep, expert_ff, shared_from=None):
    """A Vufinex configuration whose layers go round chunked attention, wkv, wkv, latent attention, each with a mixture of
    experts; from layer `shared_from` on, layers run with the weights of the layer that many places before them."""
    moe = {"kind": "moe", "expert": {"ff": expert_ff},
           "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}}
    mixers = [
        ("attention", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                       "mask": {"size": chunk}, "rot": {"base": 10000.0, "dims": dim // 2}}),
        ("wkv", {"heads": wkv_heads, "dim": wkv_dim, "decay_rank": decay_rank}),
        ("wkv", {"heads": wkv_heads, "dim": wkv_dim, "decay_rank": decay_rank}),
        ("latent_attention", {"heads": heads, "dim": lat_dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                              "scale": (lat_dim + rot_dim) ** -0.5, "rot": {"base": 10000.0, "dims": rot_dim}}),
    ]
    out = []
    for i in range(layers):
        entry = {"type": mixers[i % 4][0], "mixer": copy.deepcopy(mixers[i % 4][1]), "mlp": copy.deepcopy(moe)}
        if shared_from is not None and i >= shared_from:
            entry["weights_of"] = i - shared_from
        out.append(entry)
    return {"architecture": "Vufinex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
            "embedding": {"scale": 4.0}, "layers": out}


# Vufinex at the width, head count, head size and total feed-forward size (16 experts of 896 = 14,336) of Mistral 7B (latent
# attention with 128 unrotated and 64 rotated numbers per head over a latent of 512; chunks of 8,192 positions), and a tiny one that runs anywhere in
# seconds (its last four layers run with the first four's weights).
PRESETS["vufinex-7b-sizes"] = _vufinex(4096, 32000, 32, 32, 8, 128, 8192, 64, 64, 64, 128, 64, 128, 512, 16, 4, 4, 2, 896)
# the same at the sizes of Mistral NeMo 12B (width 5,120, a vocabulary of 131,072)
PRESETS["vufinex-12b-sizes"] = _vufinex(5120, 131072, 40, 32, 8, 128, 8192, 80, 64, 64, 128, 64, 128, 512, 16, 4, 4, 2, 896)
PRESETS["vufinex-tiny"] = _vufinex(96, 320, 8, 4, 2, 16, 24, 3, 32, 8, 16, 8, 24, 40, 6, 2, 3, 2, 32, shared_from=4)


def preset(name: str) -> dict:
    """A copy of the named configuration (a config.json-style dict)."""
    try:
        return dict(PRESETS[name])
    except KeyError:
        raise KeyError(f"unknown preset {name!r}; presets: {sorted(PRESETS)}") from None
