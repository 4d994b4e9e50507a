"""Random-weights mode: write a model folder (config.json, model.safetensors) from a configuration
and a seed.

The reference has no such mode in its package (its tests build tiny weights through another
library, tests/conftest.py:35-66). Here every tensor the model declares is drawn on the CPU from one
seeded generator, in the model's fixed declaration order: matrices and embeddings ~ N(0, std), norm
weights 1 + N(0, std), biases N(0, std), std = 0.02. The same seed gives the same file on any
machine, and the folder is loaded back through the ordinary loader.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..parts.model import DecoderModel
from ..registry import get_architecture

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(model: DecoderModel, seed: int, store_dtype: torch.dtype) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    out: dict[str, torch.Tensor] = {}
    for spec in model.weight_specs():
        kind, std = spec.init[0], spec.init[1]
        mean = spec.init[2] if len(spec.init) > 2 else 0.0
        if spec.dtype == "int32":
            out[spec.name] = torch.zeros(spec.shape, dtype=torch.int32)
            continue
        if kind == "uniform":           # ("uniform", low, high)
            low, high = spec.init[1], spec.init[2]
            out[spec.name] = (torch.rand(spec.shape, dtype=torch.float32, generator=gen) * (high - low) + low).to(store_dtype)
            continue
        t = torch.empty(spec.shape, dtype=torch.float32).normal_(0.0, std, generator=gen) + mean
        if kind == "ones_plus_normal":
            t += 1.0
        elif kind != "normal":
            raise ValueError(f"{spec.name}: unknown init rule {kind!r}")
        out[spec.name] = t.to(store_dtype).contiguous()
    return out


def write_random_model(folder: str | Path, config: dict, seed: int = 0, store_dtype: str = "bfloat16") -> Path:
    """``config`` is a config.json dictionary (it must name its architecture). Tensors are stored in
    ``store_dtype``; storing bfloat16 means a float32 run and a bfloat16 run see the same values."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    from ..config.model_config import architecture_name
    arch = get_architecture(architecture_name(config))
    cfg = arch.config_from_dict(config, None)
    spec = arch.build_spec(cfg)
    model = DecoderModel(spec, torch.float32, torch.device("cpu"))      # declarations only; nothing runs
    tensors = random_tensors(model, seed, _STORE[store_dtype])
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    return folder


# Layer sizes of the configurations the benchmarks name (config.json keys).
def qwen2_config(*, vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
                 num_key_value_heads, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                 max_position_embeddings=32768, head_dim=None, eos_token_id=None) -> dict:
    cfg = {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab_size,
        "hidden_size": hidden_size, "intermediate_size": intermediate_size,
        "num_hidden_layers": num_hidden_layers, "num_attention_heads": num_attention_heads,
        "num_key_value_heads": num_key_value_heads, "max_position_embeddings": max_position_embeddings,
        "rope_theta": rope_theta, "rms_norm_eps": rms_norm_eps, "tie_word_embeddings": tie_word_embeddings,
        "hidden_act": "silu", "use_sliding_window": False, "torch_dtype": "bfloat16",
    }
    if head_dim is not None:
        cfg["head_dim"] = head_dim
    if eos_token_id is not None:
        cfg["eos_token_id"] = eos_token_id
    return cfg


NAMED_SIZES = {
    "qwen2.5-0.5b": dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                         num_attention_heads=14, num_key_value_heads=2, tie_word_embeddings=True),
    "qwen2.5-1.5b": dict(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                         num_attention_heads=12, num_key_value_heads=2, tie_word_embeddings=True),
    "qwen2.5-7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                       num_attention_heads=28, num_key_value_heads=4, tie_word_embeddings=False),
    "tiny-a": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, rope_theta=10000.0, rms_norm_eps=1e-6,
                   tie_word_embeddings=True, max_position_embeddings=1024),
    "tiny-b": dict(vocab_size=384, hidden_size=96, intermediate_size=160, num_hidden_layers=3,
                   num_attention_heads=3, num_key_value_heads=1, rope_theta=1000000.0, rms_norm_eps=1e-5,
                   tie_word_embeddings=False, max_position_embeddings=2048),
}


def kutirax_latent(*, heads, dim, rot_dim, vdim, q_rank, kv_rank, window, scale=None, base=10000.0, rot_dims=None) -> dict:
    """The ``mixer`` entry of a Kutirax latent-attention layer."""
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5), "mask": {"size": window},
            "rot": {"base": float(base), "dims": rot_dims if rot_dims is not None else rot_dim}}


def kutirax_mamba(*, heads, vdim, state, groups=1, conv=4, norm_groups=1) -> dict:
    """The ``mixer`` entry of a Kutirax state-space layer."""
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def kutirax_config(*, vocab, width, layers, eps=1e-5, residual_mult=1.0) -> dict:
    """config.json of a Kutirax model. ``layers``: (type, mixer entry, mlp) with mlp None, ("dense", ff) or
    ("moe", experts, top, ff)."""
    out = []
    for kind, mixer, mlp in layers:
        if mlp is None:
            m = None
        elif mlp[0] == "dense":
            m = {"kind": "dense", "ff": mlp[1]}
        else:
            m = {"kind": "moe", "router": {"experts": mlp[1], "top": mlp[2]}, "expert": {"ff": mlp[3]}}
        out.append({"type": kind, "mixer": mixer, "mlp": m})
    return {"architecture": "Kutirax", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "residual_mult": residual_mult, "layers": out}


def _kutirax_named(name: str) -> dict | None:
    L, M = "latent_attention", "mamba2"
    if name == "kutirax-tiny-a":     # two windows (two cache groups), partial rotation, a layer without feed-forward, top == experts
        return kutirax_config(vocab=211, width=48, eps=1e-6, residual_mult=0.7, layers=[
            (L, kutirax_latent(heads=3, dim=16, rot_dim=8, vdim=12, q_rank=24, kv_rank=40, window=9, scale=0.2), ("moe", 5, 2, 24)),
            (M, kutirax_mamba(heads=6, vdim=10, state=12, groups=3, conv=3, norm_groups=3), ("dense", 64)),
            (L, kutirax_latent(heads=2, dim=8, rot_dim=12, vdim=20, q_rank=16, kv_rank=24, window=20, rot_dims=8, base=300.0), None),
            (M, kutirax_mamba(heads=2, vdim=24, state=16, groups=1, conv=4, norm_groups=1), ("moe", 3, 3, 16))])
    if name == "kutirax-tiny-b":     # starts with a state-space layer, one expert per token, a window across two pages
        lat = kutirax_latent(heads=5, dim=24, rot_dim=16, vdim=24, q_rank=32, kv_rank=48, window=33, scale=0.15, base=500000.0)
        return kutirax_config(vocab=300, width=80, eps=1e-5, residual_mult=1.0, layers=[
            (M, kutirax_mamba(heads=4, vdim=20, state=8, groups=4, conv=2, norm_groups=4), None),
            (L, lat, ("dense", 100)), (L, lat, ("moe", 8, 1, 20))])
    if name == "kutirax-tiny-c":     # sizes that are multiples of nothing: 7 heads, rank 72, 50 columns of 20 states, 5 taps
        return kutirax_config(vocab=130, width=56, eps=1e-5, residual_mult=0.5, layers=[
            (M, kutirax_mamba(heads=3, vdim=50, state=20, groups=1, conv=5, norm_groups=2), ("dense", 40)),
            (L, kutirax_latent(heads=7, dim=10, rot_dim=6, vdim=14, q_rank=20, kv_rank=72, window=300, rot_dims=4), ("moe", 4, 2, 12))])
    return None


def bobunex_attention(*, heads, kv_heads, dim, vdim, window, keep_first=0, scale=None, softcap=30.0, base=10000.0,
                      rot_dims=None, scaling=None) -> dict:
    """The ``mixer.left`` entry of a Bobunex layer; ``scaling`` = (factor, low, high, original) or None."""
    rot = {"base": float(base), "dims": rot_dims if rot_dims is not None else dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": float(scale if scale is not None else dim ** -0.5), "softcap": float(softcap),
            "mask": {"size": window, "keep_first": keep_first}, "rot": rot}


def bobunex_memory(*, heads, dim, vdim, gate_cap=15.0) -> dict:
    """The ``mixer.right`` entry of a Bobunex layer."""
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": float(gate_cap)}


def bobunex_config(*, vocab, width, layers, eps=1e-6, embedding_scale=1.0, taps=3) -> dict:
    """config.json of a Bobunex model. ``layers``: (left entry, right entry, ff or None)."""
    return {"architecture": "Bobunex", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": float(embedding_scale)}, "canon": {"taps": taps},
            "layers": [{"type": "parallel", "mixer": {"left": left, "right": right},
                        "mlp": None if ff is None else {"kind": "dense", "ff": ff}} for left, right, ff in layers]}


def _bobunex_named(name: str) -> dict | None:
    A, M = bobunex_attention, bobunex_memory
    if name == "bobunex-tiny-a":     # two windows (two cache groups), kept tokens inside one page, a layer without feed-forward
        return bobunex_config(vocab=173, width=48, embedding_scale=5.0, taps=3, layers=[
            (A(heads=6, kv_heads=3, dim=12, vdim=20, window=11, keep_first=3, scale=0.3, rot_dims=8, base=300.0,
               scaling=(8.0, 1.0, 4.0, 64)), M(heads=3, dim=10, vdim=14, gate_cap=8.0), 56),
            (A(heads=4, kv_heads=1, dim=16, vdim=8, window=37, keep_first=18, softcap=5.0, rot_dims=16), M(heads=2, dim=24, vdim=24), None)])
    if name == "bobunex-tiny-b":     # two taps, every head its own keys, nothing kept, no frequency scaling, no cap on scores
        return bobunex_config(vocab=300, width=80, eps=1e-5, embedding_scale=1.0, taps=2, layers=[
            (A(heads=5, kv_heads=5, dim=8, vdim=8, window=33, keep_first=0, softcap=0.0, rot_dims=4, base=500000.0),
             M(heads=4, dim=20, vdim=20, gate_cap=15.0), 100)] * 2)
    if name == "bobunex-tiny-c":     # five taps, one key head, a window longer than most prompts, wide memory columns, rotation switched off
        return bobunex_config(vocab=130, width=56, eps=1e-5, embedding_scale=0.5, taps=5, layers=[
            (A(heads=7, kv_heads=1, dim=10, vdim=36, window=300, keep_first=40, rot_dims=0), M(heads=1, dim=40, vdim=72, gate_cap=3.0), 40),
            (A(heads=2, kv_heads=2, dim=34, vdim=10, window=5, keep_first=1, rot_dims=34, scaling=(4.0, 1.0, 2.0, 16)),
             M(heads=5, dim=6, vdim=9, gate_cap=30.0), 24)])
    if name == "bobunex-tiny-d":     # head sizes the tensor-core attention takes (bfloat16): 32 | 64 and 64 | 32, kept tokens across pages
        return bobunex_config(vocab=210, width=64, eps=1e-6, embedding_scale=3.0, taps=4, layers=[
            (A(heads=4, kv_heads=2, dim=32, vdim=64, window=70, keep_first=20, scale=0.2, rot_dims=16, scaling=(4.0, 1.0, 4.0, 128)),
             M(heads=2, dim=16, vdim=32, gate_cap=10.0), 96),
            (A(heads=3, kv_heads=1, dim=64, vdim=32, window=20, keep_first=5, softcap=8.0, rot_dims=64), M(heads=4, dim=8, vdim=8), 48)])
    return None


def dibizen_attention(*, heads, kv_heads, dim, vdim, scale=None, q_temp=None, kv_from=None) -> dict:
    """The ``mixer`` entry of a Dibizen attention layer; ``q_temp`` = (coef, every) or None."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5)}
    if q_temp is not None:
        m["q_temp"] = {"coef": float(q_temp[0]), "every": int(q_temp[1])}
    if kv_from is not None:
        m["kv_from"] = int(kv_from)
    return m


def dibizen_lightning(*, heads, dim, vdim, decay) -> dict:
    """The ``mixer`` entry of a Dibizen linear-attention layer; ``decay``: one number per head."""
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": [float(a) for a in decay]}


def dibizen_mamba(*, inner, state, dt_rank, conv=4) -> dict:
    """The ``mixer`` entry of a Dibizen state-space layer."""
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def dibizen_moe(*, experts, top, ff, identity=0, groups=None) -> dict:
    """The ``mlp`` entry of a Dibizen layer; ``groups`` = (count, keep) or None."""
    router = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def dibizen_config(*, vocab, width, layers, streams=2, eps=1e-5, max_positions=512, logit_softcap=30.0) -> dict:
    """config.json of a Dibizen model. ``layers``: (type, mixer entry, mlp entry or None)."""
    return {"architecture": "Dibizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "streams": streams,
            "max_positions": max_positions, "logit_softcap": float(logit_softcap),
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp} for kind, mixer, mlp in layers]}


def _dibizen_named(name: str) -> dict | None:
    A, L, M, E = dibizen_attention, dibizen_lightning, dibizen_mamba, dibizen_moe
    if name == "dibizen-tiny-a":     # three streams; a layer that reads an earlier layer's keys; a layer without feed-forward
        att = dict(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.3, q_temp=(0.7, 16))
        return dibizen_config(vocab=173, width=48, streams=3, max_positions=300, logit_softcap=8.0, layers=[
            ("attention", A(**att), E(experts=6, top=2, ff=24, identity=2, groups=(4, 2))),
            ("mamba1", M(inner=72, state=12, dt_rank=5, conv=3), None),
            ("lightning", L(heads=3, dim=10, vdim=14, decay=[0.5, 0.9, 0.995]), E(experts=5, top=3, ff=16, identity=1, groups=(2, 2))),
            ("attention", A(**att, kv_from=0), E(experts=4, top=1, ff=20))])
    if name == "dibizen-tiny-b":     # one stream; every head its own keys; no temperature, no cap, no groups, no identity outputs
        return dibizen_config(vocab=300, width=80, streams=1, eps=1e-6, max_positions=400, logit_softcap=0.0, layers=[
            ("lightning", L(heads=2, dim=40, vdim=24, decay=[0.97, 0.8]), E(experts=3, top=3, ff=32)),
            ("attention", A(heads=5, kv_heads=5, dim=8, vdim=8), E(experts=8, top=2, ff=12, identity=0, groups=(4, 1))),
            ("mamba1", M(inner=100, state=20, dt_rank=7, conv=2), E(experts=2, top=1, ff=40, identity=2, groups=(2, 1)))])
    if name == "dibizen-tiny-c":     # head sizes the tensor-core attention takes (bfloat16); five taps; many states; shared keys twice
        att = dict(heads=8, kv_heads=2, dim=64, vdim=32, scale=0.2, q_temp=(0.4, 50))
        return dibizen_config(vocab=210, width=64, streams=2, max_positions=350, layers=[
            ("mamba1", M(inner=96, state=80, dt_rank=3, conv=5), E(experts=7, top=2, ff=16, identity=1, groups=(4, 3))),
            ("attention", A(**att), None),
            ("attention", A(**att, kv_from=1), E(experts=4, top=2, ff=24, identity=4, groups=(2, 1))),
            ("lightning", L(heads=4, dim=70, vdim=16, decay=[0.6, 0.9, 0.99, 0.999]), None),
            ("attention", A(**att, kv_from=1), E(experts=3, top=2, ff=8, identity=1))])
    return None


def gofezen_pair(*, heads, kv_heads, dim, vdim, scale, conv, window, r_heads, r_qk_heads, r_dim, r_vdim, r_conv,
                 left_scale=1.0, right_scale=1.0) -> dict:
    """The ``mixer`` entry of a Gofezen layer of type "parallel": windowed attention (left) beside the gated delta rule
    (right; its ``kv_heads`` counts its q/k heads)."""
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale), "conv": conv,
                     "mask": {"size": window}},
            "right": {"heads": r_heads, "kv_heads": r_qk_heads, "dim": r_dim, "vdim": r_vdim, "conv": r_conv},
            "left_scale": float(left_scale), "right_scale": float(right_scale)}


def gofezen_hgrn2(*, heads, dim, vdim) -> dict:
    """The ``mixer`` entry of a Gofezen layer of type "hgrn2"."""
    return {"heads": heads, "dim": dim, "vdim": vdim}


def gofezen_moe(*, experts, top, ff, shared=None) -> dict:
    """The ``mlp`` entry of a Gofezen layer with experts; ``shared``: the shared expert's size or None."""
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def gofezen_config(*, vocab, width, layers, eps=1e-6, max_positions=512, embedding_scale=1.0, logit_scale=1.0,
                   logit_softcap=30.0) -> dict:
    """config.json of a Gofezen model. ``layers``: (type, mixer entry, mlp entry or None); a dense feed-forward is
    {"kind": "dense", "ff": n}."""
    return {"architecture": "Gofezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "max_positions": max_positions,
            "embedding": {"scale": float(embedding_scale)}, "logit_scale": float(logit_scale),
            "logit_softcap": float(logit_softcap),
            "layers": [{"type": kind, "mixer": mixer, "mlp": mlp} for kind, mixer, mlp in layers]}


def _gofezen_named(name: str) -> dict | None:
    P, R, E = gofezen_pair, gofezen_hgrn2, gofezen_moe
    dense = lambda ff: {"kind": "dense", "ff": ff}
    if name == "gofezen-tiny-a":     # two pairs of unlike sizes; layers without feed-forward; one tap; top 2 and top 1
        return gofezen_config(vocab=173, width=48, max_positions=300, embedding_scale=6.9, logit_scale=0.7, logit_softcap=8.0, layers=[
            ("parallel", P(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.3, conv=3, window=24, r_heads=4, r_qk_heads=2, r_dim=16,
                           r_vdim=12, r_conv=4, left_scale=1.3, right_scale=0.8), E(experts=6, top=2, ff=24, shared=16)),
            ("hgrn2", R(heads=3, dim=10, vdim=14), dense(64)),
            ("hgrn2", R(heads=2, dim=24, vdim=8), None),
            ("parallel", P(heads=6, kv_heads=3, dim=8, vdim=8, scale=0.5, conv=2, window=37, r_heads=3, r_qk_heads=3, r_dim=20,
                           r_vdim=28, r_conv=1, left_scale=0.6, right_scale=1.5), E(experts=4, top=1, ff=20))])
    if name == "gofezen-tiny-b":     # every head its own keys / one key head for all; no cap, no scales; a window no request fills
        return gofezen_config(vocab=300, width=80, eps=1e-5, max_positions=400, logit_softcap=0.0, layers=[
            ("hgrn2", R(heads=1, dim=40, vdim=24), E(experts=3, top=3, ff=32, shared=8)),
            ("parallel", P(heads=5, kv_heads=5, dim=8, vdim=16, scale=0.35, conv=1, window=1000, r_heads=2, r_qk_heads=1, r_dim=40,
                           r_vdim=20, r_conv=2), dense(96)),
            ("parallel", P(heads=3, kv_heads=1, dim=16, vdim=8, scale=0.25, conv=5, window=9, r_heads=5, r_qk_heads=5, r_dim=8,
                           r_vdim=8, r_conv=3, left_scale=2.0, right_scale=0.5), None)])
    if name == "gofezen-tiny-c":     # head sizes the tensor-core attention takes (bfloat16); wide memories
        return gofezen_config(vocab=210, width=64, max_positions=350, embedding_scale=8.0, logit_scale=0.6, layers=[
            ("parallel", P(heads=8, kv_heads=2, dim=64, vdim=32, scale=0.125, conv=4, window=70, r_heads=4, r_qk_heads=2, r_dim=64,
                           r_vdim=32, r_conv=4, left_scale=1.1, right_scale=0.9), E(experts=7, top=2, ff=16, shared=24)),
            ("hgrn2", R(heads=2, dim=70, vdim=16), E(experts=5, top=1, ff=24)),
            ("parallel", P(heads=4, kv_heads=4, dim=32, vdim=64, scale=0.18, conv=2, window=33, r_heads=2, r_qk_heads=2, r_dim=130,
                           r_vdim=24, r_conv=3), dense(80)),
            ("hgrn2", R(heads=4, dim=16, vdim=40), None)])
    return None


def named_config(name: str) -> dict:
    cfg = _kutirax_named(name.lower()) or _bobunex_named(name.lower()) or _dibizen_named(name.lower()) or \
        _gofezen_named(name.lower())
    if cfg is not None:
        return cfg
    try:
        return qwen2_config(**NAMED_SIZES[name.lower()])
    except KeyError:
        known = sorted(NAMED_SIZES) + ["kutirax-tiny-a", "kutirax-tiny-b", "kutirax-tiny-c", "bobunex-tiny-a", "bobunex-tiny-b",
                                       "bobunex-tiny-c", "bobunex-tiny-d", "dibizen-tiny-a", "dibizen-tiny-b", "dibizen-tiny-c",
                                       "gofezen-tiny-a", "gofezen-tiny-b", "gofezen-tiny-c"]
        raise ValueError(f"unknown size name {name!r}; known: {known}") from None
