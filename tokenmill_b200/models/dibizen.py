"""Dibizen as data: config.json -> ``ModelSpec``.

A pre-norm decoder over several residual streams (hyper-connections): every sublayer reads a learned mix of the streams
through a Dynamic Tanh norm and writes its result back into all of them. The stream starts as the embedding row plus a
learned vector per position. Layer by layer, as the file lists them, the mixer is causal grouped-query attention without
a rotation (a query temperature that grows with the position, an output gate per output number, and optionally the keys
and values of an earlier layer instead of its own), linear attention with a constant decay per head, or a selective
state-space mixer; the feed-forward is a mixture of squared-relu experts chosen among groups, with identity outputs, or
absent. The output matrix is a tensor of its own and the logits pass a tanh cap. Tensor names: ``embed``, ``pos``,
``final.norm(.b, .alpha)``, ``head``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc1.*``, ``l<i>.hc2.*``,
``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.dibizen_config import DibizenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture


def dibizen_spec(cfg: DibizenConfig) -> ModelSpec:
    d = cfg.width
    norm = PartSpec("dyt", {"hidden_size": d, "streams": cfg.streams})
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        cache_of = None
        if layer.type == "attention":
            temp = m.get("q_temp")
            mixer = PartSpec("sink_window_attention", {
                "hidden_size": d, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "scale": float(m["scale"]), "position": None, "window": None, "sink": False,
                "qk_norm": False, "head_gate": False, "value_gate": True,
                "q_temp": (float(temp["coef"]), int(temp["every"])) if temp else None,
                "shares_kv": m.get("kv_from") is not None})
            cache_of = m.get("kv_from")
        elif layer.type == "lightning":
            mixer = PartSpec("decay_memory", {"hidden_size": d, "num_heads": m["heads"], "head_dim": m["dim"],
                                              "value_dim": m["vdim"], "decay": [float(a) for a in m["decay"]],
                                              "eps": cfg.eps, "activation": "silu"})
        else:
            mixer = PartSpec("selective_scan", {"hidden_size": d, "inner": m["inner"], "state_size": m["state"],
                                                "dt_rank": m["dt_rank"], "conv_taps": m["conv"]})
        ffn = None
        if layer.mlp is not None:
            r = layer.mlp["router"]
            groups = r.get("groups") or {"count": 1, "keep": 1}
            ffn = PartSpec("routed_choice", {"hidden_size": d, "expert_size": layer.mlp["expert"]["ff"],
                                             "num_experts": r["experts"], "top": r["top"],
                                             "identity": int(r.get("identity") or 0), "groups": groups["count"],
                                             "keep": groups["keep"]})
        layers.append(LayerSpec(prefix=f"l{i}", block="hyper_connections", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm if ffn is not None else None, mixer_name="mix",
                                feed_forward_name="mlp", mixer_norm_name="norm1", feed_forward_norm_name="norm2",
                                block_params={"hidden_size": d, "streams": cfg.streams, "learned": cfg.hyper_connections}))
        order.append(RunEntry(i, cache_of=cache_of))        # (one run per layer: a layer's number is its place in the order)
    return ModelSpec(architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=layers, run_order=order, final_norm=norm, final_norm_prefix="final.norm", lm_head_name="head",
                     max_positions=cfg.max_positions, eos_token_ids=list(cfg.eos_token_ids), position_table_name="pos",
                     streams=cfg.streams, logit_softcap=cfg.logit_softcap)


register_architecture("Dibizen", DibizenConfig.from_dict, dibizen_spec)
