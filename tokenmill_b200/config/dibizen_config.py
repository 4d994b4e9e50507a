"""Typed configuration of the Dibizen decoder, read from the keys of its config.json.

    architecture    "Dibizen"
    vocab, width    vocabulary and residual width
    max_positions   rows of the learned position table
    streams         copies of the residual stream (hyper-connections; absent: one plain stream without their tensors)
    norm.eps        eps of the RMS norms inside the mixers (the layers' own norms are Dynamic Tanh and have none)
    logit_softcap   cap of the logits (absent or 0: none)
    layers          one entry per layer: type ("attention" | "lightning" | "mamba1"), mixer (its sizes), mlp (null, or
                    kind "moe" with expert.ff and router.{experts, top, identity, groups.{count, keep}})
    attention mixer: heads, kv_heads, dim, vdim, scale, q_temp.{coef, every} (optional), kv_from (optional: the layer
                     whose keys and values this one reads; it has none of its own)
    lightning mixer: heads, dim, vdim, decay (one per head)
    mamba1 mixer:    inner, state, dt_rank, conv

Every size and constant comes from the file; a key the design does not have is refused rather than ignored.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .kutirax_config import _need, _only, _pos_int
from .model_config import ConfigError


@dataclass
class DibizenLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass
class DibizenConfig:
    vocab: int
    width: int
    eps: float
    streams: int
    max_positions: int
    logit_softcap: float = 0.0
    hyper_connections: bool = True      # False (no ``streams`` in the file): one stream, no read and write weights
    layers: list[DibizenLayer] = field(default_factory=list)
    eos_token_ids: list[int] = field(default_factory=list)
    architecture: str = "Dibizen"

    @classmethod
    def from_dict(cls, raw: dict[str, Any], generation: dict[str, Any] | None = None) -> "DibizenConfig":
        _need(raw, ("vocab", "width", "layers", "norm", "max_positions"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(entry, ("type", "mixer"), where)
            m, kind = entry["mixer"], entry["type"]
            if kind == "attention":
                keys = ("heads", "kv_heads", "dim", "vdim", "scale")
                _need(m, keys, where + ".mixer")
                _only(m, keys + ("q_temp", "kv_from"), where + ".mixer")
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    _pos_int(m[k], f"{where}.mixer.{k}")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {where}.mixer.heads must be a multiple of kv_heads")
                if m.get("q_temp") is not None:
                    _need(m["q_temp"], ("coef", "every"), where + ".mixer.q_temp")
                    _pos_int(m["q_temp"]["every"], f"{where}.mixer.q_temp.every")
                if m.get("kv_from") is not None:
                    j = m["kv_from"]
                    if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < i:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer, got {j!r}")
                    other = raw["layers"][j]
                    if other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from names layer {j}, which has no keys and values "
                                          f"of its own")
                    if any(other["mixer"].get(k) != m[k] for k in ("heads", "kv_heads", "dim", "vdim")):
                        raise ConfigError(f"config.json: {where}.mixer reads the keys of layer {j}, whose head counts or "
                                          f"sizes differ")
            elif kind == "lightning":
                keys = ("heads", "dim", "vdim", "decay")
                _need(m, keys, where + ".mixer")
                _only(m, keys, where + ".mixer")
                for k in ("heads", "dim", "vdim"):
                    _pos_int(m[k], f"{where}.mixer.{k}")
                if not isinstance(m["decay"], list) or len(m["decay"]) != m["heads"]:
                    raise ConfigError(f"config.json: {where}.mixer.decay must list one number per head")
            elif kind == "mamba1":
                keys = ("inner", "state", "dt_rank", "conv")
                _need(m, keys, where + ".mixer")
                _only(m, keys, where + ".mixer")
                for k in keys:
                    _pos_int(m[k], f"{where}.mixer.{k}")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
                _need(mlp, ("expert", "router"), where + ".mlp")
                _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                r = mlp["router"]
                _need(r, ("experts", "top"), where + ".mlp.router")
                _only(r, ("experts", "top", "identity", "groups"), where + ".mlp.router")
                _pos_int(mlp["expert"]["ff"], f"{where}.mlp.expert.ff")
                n = _pos_int(r["experts"], f"{where}.mlp.router.experts") + int(r.get("identity") or 0)
                count, keep = 1, 1
                if r.get("groups") is not None:
                    _need(r["groups"], ("count", "keep"), where + ".mlp.router.groups")
                    count = _pos_int(r["groups"]["count"], f"{where}.mlp.router.groups.count")
                    keep = _pos_int(r["groups"]["keep"], f"{where}.mlp.router.groups.keep")
                if n % count or keep > count:
                    raise ConfigError(f"config.json: {where}.mlp.router: {n} outputs do not form {count} equal groups of "
                                      f"which {keep} are kept")
                if not 1 <= _pos_int(r["top"], f"{where}.mlp.router.top") <= keep * (n // count):
                    raise ConfigError(f"config.json: {where}.mlp.router.top exceeds the outputs of the kept groups")
            layers.append(DibizenLayer(kind, dict(m), dict(mlp) if mlp is not None else None))
        eos = []
        for src in (generation or {}, raw):
            v = src.get("eos_token_id")
            if v is not None:
                eos += v if isinstance(v, list) else [v]
        eps = float(raw["norm"]["eps"])
        if not eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        cap = float(raw.get("logit_softcap") or 0.0)
        if cap < 0:
            raise ConfigError(f"config.json: logit_softcap must not be negative, got {cap!r}")
        return cls(vocab=_pos_int(raw["vocab"], "vocab"), width=_pos_int(raw["width"], "width"), eps=eps,
                   streams=_pos_int(raw["streams"], "streams") if raw.get("streams") is not None else 1,
                   hyper_connections=raw.get("streams") is not None,
                   max_positions=_pos_int(raw["max_positions"], "max_positions"), logit_softcap=cap, layers=layers,
                   eos_token_ids=sorted(set(eos)))
