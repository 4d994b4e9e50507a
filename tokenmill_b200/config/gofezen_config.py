"""Typed configuration of the Gofezen decoder, read from the keys of its config.json.

    architecture      "Gofezen"
    vocab, width      vocabulary and residual width
    max_positions     rows of the learned position table
    embedding.scale   multiplier of the embedding rows (absent: 1)
    norm.eps          eps of every RMS norm (the layers', the heads' and the model's last one)
    logit_scale       multiplier of the logits (absent: 1); logit_softcap: cap of the logits after it (absent or 0: none)
    layers            one entry per layer: type ("parallel" | "hgrn2"), mixer (its sizes), mlp (null, kind "dense" with ff,
                      or kind "moe" with expert.ff, router.{experts, top} and optionally shared.ff)
    parallel mixer:   left  {heads, kv_heads, dim, vdim, scale, conv, mask.size}: windowed attention with biases, a short
                            convolution on q, k, v, a norm per head and mixed heads;
                      right {heads, kv_heads, dim, vdim, conv}: the gated delta rule (kv_heads counts its q/k heads);
                      conv absent: no convolution and no tensors of it; mask absent: every earlier key is seen;
                      left_scale, right_scale: the weights of their sum (absent: 1)
    hgrn2 mixer:      heads, dim, vdim

Every size and constant comes from the file; inside a layer's entries a key the design does not have is refused rather
than ignored.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .kutirax_config import _need, _only, _pos_int
from .model_config import ConfigError


@dataclass
class GofezenLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None


@dataclass
class GofezenConfig:
    vocab: int
    width: int
    eps: float
    max_positions: int
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    layers: list[GofezenLayer] = field(default_factory=list)
    eos_token_ids: list[int] = field(default_factory=list)
    architecture: str = "Gofezen"

    @classmethod
    def from_dict(cls, raw: dict[str, Any], generation: dict[str, Any] | None = None) -> "GofezenConfig":
        _need(raw, ("vocab", "width", "layers", "norm", "max_positions"), "the top level")
        _need(raw["norm"], ("eps",), "norm")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(entry, ("type", "mixer"), where)
            m, kind = entry["mixer"], entry["type"]
            if kind == "parallel":
                _need(m, ("left", "right"), where + ".mixer")
                _only(m, ("left", "right", "left_scale", "right_scale"), where + ".mixer")
                a, r = m["left"], m["right"]
                keys = ("heads", "kv_heads", "dim", "vdim", "scale")
                _need(a, keys, where + ".mixer.left")
                _only(a, keys + ("conv", "mask"), where + ".mixer.left")
                if a.get("mask") is not None:           # absent: every earlier key is seen
                    _need(a["mask"], ("size",), where + ".mixer.left.mask")
                    _only(a["mask"], ("size",), where + ".mixer.left.mask")
                    _pos_int(a["mask"]["size"], f"{where}.mixer.left.mask.size")
                keys = ("heads", "kv_heads", "dim", "vdim")
                _need(r, keys, where + ".mixer.right")
                _only(r, keys + ("conv",), where + ".mixer.right")
                for side, d in (("left", a), ("right", r)):
                    for k in ("heads", "kv_heads", "dim", "vdim") + (("conv",) if d.get("conv") is not None else ()):
                        _pos_int(d[k], f"{where}.mixer.{side}.{k}")
                    if d["heads"] % d["kv_heads"]:
                        raise ConfigError(f"config.json: {where}.mixer.{side}.heads must be a multiple of kv_heads")
            elif kind == "hgrn2":
                keys = ("heads", "dim", "vdim")
                _need(m, keys, where + ".mixer")
                _only(m, keys, where + ".mixer")
                for k in keys:
                    _pos_int(m[k], f"{where}.mixer.{k}")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ("ff",), where + ".mlp")
                    _only(mlp, ("kind", "ff"), where + ".mlp")
                    _pos_int(mlp["ff"], f"{where}.mlp.ff")
                elif mlp["kind"] == "moe":
                    _need(mlp, ("expert", "router"), where + ".mlp")
                    _only(mlp, ("kind", "expert", "router", "shared"), where + ".mlp")
                    _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                    _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                    _only(mlp["router"], ("experts", "top"), where + ".mlp.router")
                    _pos_int(mlp["expert"]["ff"], f"{where}.mlp.expert.ff")
                    n = _pos_int(mlp["router"]["experts"], f"{where}.mlp.router.experts")
                    if _pos_int(mlp["router"]["top"], f"{where}.mlp.router.top") > n:
                        raise ConfigError(f"config.json: {where}.mlp.router.top exceeds the number of experts")
                    if mlp.get("shared") is not None:
                        _need(mlp["shared"], ("ff",), where + ".mlp.shared")
                        _only(mlp["shared"], ("ff",), where + ".mlp.shared")
                        _pos_int(mlp["shared"]["ff"], f"{where}.mlp.shared.ff")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design")
            layers.append(GofezenLayer(kind, dict(m), dict(mlp) if mlp is not None else None))
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
        scale = (raw.get("embedding") or {}).get("scale")
        logit_scale = raw.get("logit_scale")
        return cls(vocab=_pos_int(raw["vocab"], "vocab"), width=_pos_int(raw["width"], "width"), eps=eps,
                   max_positions=_pos_int(raw["max_positions"], "max_positions"),
                   embedding_scale=1.0 if scale is None else float(scale),
                   logit_scale=1.0 if logit_scale is None else float(logit_scale), logit_softcap=cap, layers=layers,
                   eos_token_ids=sorted(set(eos)))
