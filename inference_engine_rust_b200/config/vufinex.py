"""Typed configuration of the Vufinex decoder, read from the keys of its own config.json, and its
`ModelSpec` builder.

A Vufinex model is a list of pre-norm layers whose sublayers' results are multiplied by one factor before they
are added to the residual (x <- x + m mixer(norm1(x)); x <- x + m ff(norm2(x)); RMS norm with a weight stored
around zero).  The embedded rows are multiplied by a factor; the output head has a matrix of its own.  A layer's
mixer is one of three: grouped-query attention whose keys double as values, with rotary positions on the first
`rot.dims` numbers of a head in the "half" pairing and a mask of chunks (a position sees the earlier positions of
its own chunk of `mask.size`, counted from the start of the sequence); a matrix-state recurrence with token shift,
a decay per key channel made by a small two-matrix product, a bonus for the current token, a unit norm per head and
a SiLU gate ("wkv"); latent attention with a rotated key part that all heads share (pairs of neighbours), causal,
with a sigmoid gate per head on the result.  The feed-forward is absent or a mixture of experts whose router scores
every expert by a sigmoid, chooses on score + a stored correction inside the best groups of neighbouring experts (a
group's score is the sum of its two best choice scores), and weighs the chosen by their scores over their sum times
a factor.  A layer may run with another layer's weights and a cache or state of its own.  Every size and every
constant that can differ between models comes from config.json:

    architecture   "Vufinex"
    vocab, width, residual_mult (optional, 1), embedding.scale (optional, 1)
    norm.eps
    layers[i]      {"type": "attention" | "wkv" | "latent_attention", "mixer": {...}, "mlp": {...} | null,
                    "weights_of": j (optional)}
      attention         heads, kv_heads, dim, vdim (= dim), scale, mask.size (optional), rot {base, dims} (optional)
      wkv               heads, dim, decay_rank (optional: the inner size of the decay's two matrices, else the tensors')
      latent_attention  heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims = rot_dim}
      mlp               {"kind": "moe", "expert": {ff}, "router": {experts, top, scale (optional, 1),
                         groups {count, keep} (optional)}}
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Vufinex"
LAYER_TYPES = ("attention", "wkv", "latent_attention")


def _number(where: str, raw: Any, key: str, typ, positive: bool = True):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where}: required key {key!r} is missing")
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, (int, float) if typ is float else int):
        raise ConfigError(f"config.json: {where}.{key} must be {'a number' if typ is float else 'an integer'}, got {v!r}")
    v = typ(v)
    if not math.isfinite(v) or (positive and not v > 0):
        raise ConfigError(f"config.json: {where}.{key} must be {'positive and ' if positive else ''}finite, got {v!r}")
    return v


def _optional(where: str, raw: Any, key: str, typ, default, positive: bool = True):
    if not isinstance(raw, Mapping) or raw.get(key) is None:
        return default
    return _number(where, raw, key, typ, positive)


def _rot(where: str, raw: Mapping[str, Any], most: int) -> Optional[Dict[str, Any]]:
    rot = raw.get("rot")
    if rot is None:
        return None
    dims = _number(where + ".rot", rot, "dims", int, positive=False)
    if dims < 0 or dims % 2 or dims > most:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even, not negative and at most {most}")
    return {"base": _number(where + ".rot", rot, "base", float), "dims": dims}


def _attention(where: str, raw: Mapping[str, Any]) -> Dict[str, Any]:
    heads, kv_heads = _number(where, raw, "heads", int), _number(where, raw, "kv_heads", int)
    dim = _number(where, raw, "dim", int)
    vdim = _optional(where, raw, "vdim", int, dim)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    if vdim != dim:
        raise ConfigError(f"config.json: {where}: vdim {vdim} differs from dim {dim}, but the values are the keys")
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": _number(where, raw, "scale", float)}
    rot = _rot(where, raw, dim)
    if rot is not None:
        out["rot"] = rot
    if raw.get("mask") is not None:
        out["mask"] = {"size": _number(where + ".mask", raw["mask"], "size", int)}
    return out


def _wkv(where: str, raw: Mapping[str, Any]) -> Dict[str, Any]:
    out = {"heads": _number(where, raw, "heads", int), "dim": _number(where, raw, "dim", int)}
    if raw.get("decay_rank") is not None:          # optional: else the stored matrices' inner size decides
        out["decay_rank"] = _number(where, raw, "decay_rank", int)
    return out


def _latent(where: str, raw: Mapping[str, Any]) -> Dict[str, Any]:
    out = {key: _number(where, raw, key, int) for key in ("heads", "dim", "vdim", "kv_rank")}
    out["rot_dim"] = _number(where, raw, "rot_dim", int, positive=False)
    out["scale"] = _number(where, raw, "scale", float)
    if out["rot_dim"] < 0 or out["rot_dim"] % 2:
        raise ConfigError(f"config.json: {where}.rot_dim {out['rot_dim']} must be even and not negative")
    rot = _rot(where, raw, 1 << 30)            # its size is judged against rot_dim below
    if out["rot_dim"]:
        if rot is None:
            raise ConfigError(f"config.json: {where}: required key 'rot' is missing")
        if rot["dims"] != out["rot_dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims {rot['dims']} must equal rot_dim {out['rot_dim']}")
    out["rot"] = rot or {"base": 10000.0, "dims": 0}
    return out


_MIXERS = {"attention": _attention, "wkv": _wkv, "latent_attention": _latent}


def _mlp(where: str, raw: Any) -> Optional[Dict[str, Any]]:
    if raw is None:
        return None
    if not isinstance(raw, Mapping) or raw.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}.kind must be 'moe' (or mlp null), got "
                          f"{raw.get('kind') if isinstance(raw, Mapping) else raw!r}")
    r = raw.get("router")
    experts, top = _number(where + ".router", r, "experts", int), _number(where + ".router", r, "top", int)
    g = r.get("groups")
    count = _number(where + ".router.groups", g, "count", int) if g is not None else 1
    keep = _number(where + ".router.groups", g, "keep", int) if g is not None else count
    if experts % count:
        raise ConfigError(f"config.json: {where}.router: {experts} experts do not form {count} equal groups")
    if keep > count or top > keep * (experts // count):
        raise ConfigError(f"config.json: {where}.router: top {top} does not fit into {keep} of {count} groups of "
                          f"{experts // count}")
    if top > 32:
        raise ConfigError(f"config.json: {where}.router.top {top}: at most 32 experts per token are supported")
    return {"kind": "moe", "expert": {"ff": _number(where + ".expert", raw.get("expert"), "ff", int)},
            "router": {"experts": experts, "top": top, "scale": _optional(where + ".router", r, "scale", float, 1.0),
                       "groups": {"count": count, "keep": keep}}}


@dataclass(frozen=True)
class VufinexConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    embedding_scale: float
    layers: Tuple[Mapping[str, Any], ...]       # validated copies of config.json's entries
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VufinexConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, Mapping) or lr.get("type") not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {LAYER_TYPES}, got "
                                  f"{lr.get('type') if isinstance(lr, Mapping) else lr!r}")
            if not isinstance(lr.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where}: required key 'mixer' is missing")
            entry = {"type": lr["type"], "mixer": _MIXERS[lr["type"]](where + ".mixer", lr["mixer"]),
                     "mlp": _mlp(where + ".mlp", lr.get("mlp"))}
            if lr.get("weights_of") is not None:
                j = lr["weights_of"]
                if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(layers_raw) or j == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer, got {j!r}")
                entry["weights_of"] = j
            layers.append(entry)
        for i, layer in enumerate(layers):        # a layer that borrows weights is built like their owner
            j = layer.get("weights_of")
            if j is not None and layers[j]["type"] != layer["type"]:
                raise ConfigError(f"config.json: layers[{i}] is of type {layer['type']!r} but takes the weights of "
                                  f"layers[{j}], of type {layers[j]['type']!r}")
        cfg = cls(vocab=_number("top level", raw, "vocab", int), width=_number("top level", raw, "width", int),
                  eps=_number("norm", raw.get("norm"), "eps", float),
                  residual_mult=_optional("top level", raw, "residual_mult", float, 1.0, positive=False),
                  embedding_scale=_optional("embedding", raw.get("embedding"), "scale", float, 1.0, positive=False),
                  layers=tuple(layers))
        for i in range(len(layers)):
            cfg.owner(i)
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer `i` uses (itself, unless it names another)."""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of goes round in a circle")
            seen.add(i)
            i = self.layers[i]["weights_of"]
        return i

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
                "layers": copy.deepcopy(list(self.layers))}


def _mixer_spec(cfg: VufinexConfig, kind: str, m: Mapping[str, Any]) -> PartSpec:
    """The sublayer factor travels as each part's `out_scale`: every part applies it in 32-bit to what its last
    product reads, in which its result is linear."""
    common = {"hidden_size": cfg.width, "eps": cfg.eps, "out_scale": cfg.residual_mult}
    if kind == "attention":
        rot = m.get("rot") or {"base": 10000.0, "dims": 0}
        return PartSpec("tied_kv_attention", {
            **common, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "window": None,
            "chunk": (m.get("mask") or {}).get("size"), "scale": m["scale"], "softcap": None, "sink": False, "qk_norm": None,
            "position": PartSpec("rope", {"theta": rot["base"], "rotary_dim": rot["dims"], "pairing": "half"})})
    if kind == "wkv":
        return PartSpec("wkv", {**common, "heads": m["heads"], "dim": m["dim"], "decay_rank": m.get("decay_rank")})
    return PartSpec("latent_attention", {
        **common, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": None,
        "rot_dim": m["rot_dim"], "scale": m["scale"], "sink": False, "gate": "head",
        "position": PartSpec("rope", {"theta": m["rot"]["base"], "rotary_dim": m["rot_dim"], "pairing": "interleaved"})})


def _ffn_spec(cfg: VufinexConfig, mlp: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
    if mlp is None:
        return None
    r = mlp["router"]
    return PartSpec("grouped_moe", {
        "hidden_size": cfg.width, "experts": r["experts"], "identity": 0, "top": r["top"], "groups": r["groups"]["count"],
        "keep": r["groups"]["keep"], "expert_ff": mlp["expert"]["ff"], "activation": "silu", "score": "sigmoid",
        "group_score": "top2_sum", "weight_eps": 1e-20, "route_scale": r["scale"], "out_scale": cfg.residual_mult})


def build_spec(cfg: VufinexConfig) -> ModelSpec:
    """Tensor names: `embed`, `head`, `final.norm`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*` (attention: q, k, o; wkv: mu.{r,k,v,g,w},
    r, k, v, g, w1, w2, w0, u, norm, o; latent attention: q, dkv, dkv.norm, uk, uv, g, o), `l<i>.mlp.e<j>.{gate,up,down}`,
    `l<i>.mlp.router`, `l<i>.mlp.correction`; i is the layer's place in config.json, and a layer with `weights_of` has none."""
    norm = PartSpec("rmsnorm", {"eps": cfg.eps, "offset": 1.0})
    block = PartSpec("prenorm", {})
    owners = sorted({cfg.owner(i) for i in range(len(cfg.layers))})
    index_of = {i: n for n, i in enumerate(owners)}
    layers = []
    for i in owners:
        layer, p = cfg.layers[i], f"l{i}."
        layers.append(LayerSpec(block=block, norm=norm, mixer=_mixer_spec(cfg, layer["type"], layer["mixer"]),
                                ffn=_ffn_spec(cfg, layer["mlp"]), mixer_prefix=p + "mix.", ffn_prefix=p + "mlp.",
                                mixer_norm_name=p + "norm1", ffn_norm_name=p + "norm2"))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(index_of[cfg.owner(i)]) for i in range(len(cfg.layers))),
        final_norm=norm, embedding_name="embed", final_norm_name="final.norm", lm_head_name="head",
        embedding_scale=cfg.embedding_scale, max_position=1 << 30, bos_token_id=None, eos_token_id=None)


register_architecture(ARCHITECTURE, VufinexConfig, build_spec)
