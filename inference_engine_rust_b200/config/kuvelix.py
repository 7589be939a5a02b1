"""Typed configuration of the Kuvelix decoder, read from the keys of its own config.json, and its
`ModelSpec` builder.

A Kuvelix model is a list of layers with ONE norm each, read by both sublayers (h = norm(x);
x <- x + mixer(h) + ff(h); RMS norm with a plain weight).  The mixer is grouped-query attention with biases on
q, k and v, a weighted RMS norm on every head of q and k, rotary positions on the first `rot.dims` dimensions of
a head in the interleaved pairing (2i with 2i + 1) with every frequency divided by `rot.scaling.factor`, a score
scale given outright, causal softmax, and a sigmoid gate on the concatenated heads in front of the output
projection.  The feed-forward is absent, dense (tanh-form GELU on the gate branch) or a mixture of experts whose
router scores all outputs by one softmax, chooses on score + correction inside the best groups of neighbouring
outputs, and whose last outputs stand for experts that return their input; the experts clamp both branches.  A run
of layers may be executed several times in a row with the same weights, each pass with a cache of its own.  The
embedded rows are normed; the output head is the embedding table.  Every size and every constant that can differ
between models comes from config.json:

    architecture   "Kuvelix"
    vocab, width
    norm.eps
    loop           (optional) {start, stop, times}: layers start .. stop-1 run `times` times in a row
    layers[i]      {"type": "attention", "mixer": {...}, "mlp": {...} | null}
      mixer        heads, kv_heads, dim, vdim (default dim), scale, rot {base, dims, scaling {factor} (optional)} (optional)
      mlp          {"kind": "dense", "ff"}
                   {"kind": "moe", "expert": {ff, limit}, "router": {experts, top, identity (optional),
                    groups {count, keep} (optional)}}
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Kuvelix"
LAYER_TYPES = ("attention",)


def _number(where: str, raw: Any, key: str, typ, positive: bool = True):
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: {where}: required key {key!r} is missing")
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, (int, float) if typ is float else int):
        raise ConfigError(f"config.json: {where}.{key} must be {'a number' if typ is float else 'an integer'}, got {v!r}")
    v = typ(v)
    if not math.isfinite(v) or (positive and not v > 0) or v < 0:
        raise ConfigError(f"config.json: {where}.{key} must be {'positive' if positive else 'not negative'} and finite, got {v!r}")
    return v


def _attention(where: str, raw: Any) -> Dict[str, Any]:
    heads, kv_heads = _number(where, raw, "heads", int), _number(where, raw, "kv_heads", int)
    dim = _number(where, raw, "dim", int)
    vdim = _number(where, raw, "vdim", int) if raw.get("vdim") is not None else dim
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": _number(where, raw, "scale", float)}
    rot = raw.get("rot")
    if rot is not None:
        dims = _number(where + ".rot", rot, "dims", int, positive=False)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most dim {dim}")
        out["rot"] = {"base": _number(where + ".rot", rot, "base", float), "dims": dims}
        if rot.get("scaling") is not None:
            out["rot"]["scaling"] = {"factor": _number(where + ".rot.scaling", rot["scaling"], "factor", float)}
    return out


def _mlp(where: str, raw: Any) -> Optional[Dict[str, Any]]:
    if raw is None:
        return None
    if not isinstance(raw, Mapping) or raw.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}.kind must be 'dense' or 'moe' (or mlp null), got "
                          f"{raw.get('kind') if isinstance(raw, Mapping) else raw!r}")
    if raw["kind"] == "dense":
        return {"kind": "dense", "ff": _number(where, raw, "ff", int)}
    r = raw.get("router")
    experts, top = _number(where + ".router", r, "experts", int), _number(where + ".router", r, "top", int)
    identity = _number(where + ".router", r, "identity", int, positive=False) if r.get("identity") is not None else 0
    g = r.get("groups")
    count = _number(where + ".router.groups", g, "count", int) if g is not None else 1
    keep = _number(where + ".router.groups", g, "keep", int) if g is not None else count
    outputs = experts + identity
    if outputs % count:
        raise ConfigError(f"config.json: {where}.router: {outputs} outputs (experts + identity) do not form "
                          f"{count} equal groups")
    if keep > count or top > keep * (outputs // count):
        raise ConfigError(f"config.json: {where}.router: top {top} does not fit into {keep} of {count} groups of "
                          f"{outputs // count}")
    if top > 32:
        raise ConfigError(f"config.json: {where}.router.top {top}: at most 32 experts per token are supported")
    e = raw.get("expert")
    expert = {"ff": _number(where + ".expert", e, "ff", int)}
    if e.get("limit") is not None:
        expert["limit"] = _number(where + ".expert", e, "limit", float)
    return {"kind": "moe", "expert": expert,
            "router": {"experts": experts, "top": top, "identity": identity, "groups": {"count": count, "keep": keep}}}


@dataclass(frozen=True)
class KuvelixConfig:
    vocab: int
    width: int
    eps: float
    loop: Optional[Mapping[str, int]]
    layers: Tuple[Mapping[str, Any], ...]       # validated copies of config.json's entries
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KuvelixConfig":
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
            layers.append({"type": lr["type"], "mixer": _attention(where + ".mixer", lr["mixer"]),
                           "mlp": _mlp(where + ".mlp", lr.get("mlp"))})
        loop = raw.get("loop")
        if loop is not None:
            loop = {"start": _number("loop", loop, "start", int, positive=False), "stop": _number("loop", loop, "stop", int, positive=False),
                    "times": _number("loop", loop, "times", int)}
            if not loop["start"] <= loop["stop"] <= len(layers):
                raise ConfigError(f"config.json: loop: start {loop['start']} .. stop {loop['stop']} is no run of the "
                                  f"{len(layers)} layers")
        return cls(vocab=_number("top level", raw, "vocab", int), width=_number("top level", raw, "width", int),
                   eps=_number("norm", raw.get("norm"), "eps", float), loop=loop, layers=tuple(layers))

    def runs(self) -> Tuple[int, ...]:
        """The layers in the order in which they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        return d


def _mixer_spec(cfg: KuvelixConfig, m: Mapping[str, Any]) -> PartSpec:
    rot = m.get("rot") or {"base": 10000.0, "dims": 0}
    position = {"theta": rot["base"], "rotary_dim": rot["dims"], "pairing": "interleaved"}
    if rot.get("scaling") is not None:           # stretched positions: every frequency divided by the factor
        position["freq_factors"] = [rot["scaling"]["factor"]] * (rot["dims"] // 2)
    return PartSpec("gated_attention", {
        "hidden_size": cfg.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
        "scale": m["scale"], "eps": cfg.eps, "bias": True, "qk_norm": "head", "gate": True, "window": None,
        "position": PartSpec("rope", position)})


def _ffn_spec(cfg: KuvelixConfig, mlp: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": mlp["ff"], "activation": "gelu_tanh",
                                   "tensor_names": ("gate", "up", "down")})
    r = mlp["router"]
    return PartSpec("grouped_moe", {
        "hidden_size": cfg.width, "experts": r["experts"], "identity": r["identity"], "top": r["top"],
        "groups": r["groups"]["count"], "keep": r["groups"]["keep"], "expert_ff": mlp["expert"]["ff"],
        "activation": "clamped_swish", "limit": mlp["expert"].get("limit")})


def build_spec(cfg: KuvelixConfig) -> ModelSpec:
    """Tensor names: `embed`, `embed.norm`, `l<i>.norm1`, `l<i>.mix.{q,k,v}(.b)`, `l<i>.mix.{q,k}.norm`, `l<i>.mix.{g,o}`,
    `l<i>.mlp.{gate,up,down}` or `l<i>.mlp.e<j>.{gate,up,down}` with `l<i>.mlp.router` and `l<i>.mlp.correction`,
    `final.norm`; i is the layer's place in config.json."""
    norm = PartSpec("rmsnorm", {"eps": cfg.eps})
    block = PartSpec("shared_norm", {})
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        layers.append(LayerSpec(block=block, norm=norm, mixer=_mixer_spec(cfg, layer["mixer"]), ffn=_ffn_spec(cfg, layer["mlp"]),
                                mixer_prefix=p + "mix.", ffn_prefix=p + "mlp.", mixer_norm_name=p + "norm1",
                                ffn_norm_name=""))       # one norm per layer: the feed-forward reads the mixer's
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in cfg.runs()),       # a layer that runs again has a cache per run
        final_norm=norm, embedding_name="embed", final_norm_name="final.norm",
        lm_head_name=None,                          # the output head is the embedding table
        embedding_scale=1.0, max_position=1 << 30, bos_token_id=None, eos_token_id=None,
        inputs=((PartSpec("embed_norm", {"norm": norm}), "embed."),))


register_architecture(ARCHITECTURE, KuvelixConfig, build_spec)
