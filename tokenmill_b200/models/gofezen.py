"""Gofezen as data: config.json -> ``ModelSpec``.

A decoder of parallel blocks: one RMS norm per layer, whose output both the mixer and the feed-forward read, and the
stream receives the sum of their results (block ``parallel``). The stream starts as the embedding row times a constant
plus a learned vector per position. Layer by layer, as the file lists them, the mixer is either a pair side by side
(``parallel``: windowed grouped-query attention with biases, a short convolution on q, k and v, a norm per head without
weights, no rotation and talking heads, beside the gated delta rule; their outputs summed with two constants) or a
matrix memory whose forget gate also decides what is written (``hgrn2``). The feed-forward is a dense silu-gated layer, a
mixture of experts with sigmoid scores that multiply the chosen experts' inputs plus a gated shared expert, or absent.
The output matrix is a tensor of its own; the logits are scaled and pass a tanh cap. Tensor names: ``embed``, ``pos``,
``final.norm``, ``head``, and per layer ``l<i>.norm1``, ``l<i>.mix.*`` (``left.*`` / ``right.*`` for a pair), ``l<i>.mlp.*``.
"""

from __future__ import annotations

from ..config.gofezen_config import GofezenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture


def gofezen_spec(cfg: GofezenConfig) -> ModelSpec:
    d = cfg.width
    norm = PartSpec("dyt", {"hidden_size": d, "streams": 1, "kind": "rms", "eps": cfg.eps, "library": "delta"})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "parallel":
            a, r = m["left"], m["right"]
            left = PartSpec("sink_window_attention", {
                "hidden_size": d, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"],
                "value_dim": a["vdim"], "scale": float(a["scale"]), "position": None,
                "window": a["mask"]["size"] if a.get("mask") is not None else None,
                "sink": False, "qk_norm": "head", "head_gate": False, "eps": cfg.eps, "bias": True,
                "conv_taps": a.get("conv") or 0, "talk": True})
            right = PartSpec("gated_delta", {"hidden_size": d, "num_heads": r["heads"], "num_qk_heads": r["kv_heads"],
                                             "head_dim": r["dim"], "value_dim": r["vdim"], "conv_taps": r.get("conv") or 0,
                                             "eps": cfg.eps})
            mixer = PartSpec("pair", {"hidden_size": d, "eps": cfg.eps, "left": left, "right": right, "combine": "weighted",
                                      "left_scale": float(m.get("left_scale", 1.0)),
                                      "right_scale": float(m.get("right_scale", 1.0))})
        else:
            mixer = PartSpec("forget_gate_memory", {"hidden_size": d, "num_heads": m["heads"], "head_dim": m["dim"],
                                                    "value_dim": m["vdim"], "eps": cfg.eps})
        ffn = None
        if layer.mlp is not None and layer.mlp["kind"] == "dense":
            ffn = PartSpec("glu", {"hidden_size": d, "intermediate_size": layer.mlp["ff"], "activation": "silu"})
        elif layer.mlp is not None:
            shared = layer.mlp.get("shared")
            ffn = PartSpec("routed_input_scaled", {"hidden_size": d, "expert_size": layer.mlp["expert"]["ff"],
                                                   "num_experts": layer.mlp["router"]["experts"],
                                                   "top": layer.mlp["router"]["top"],
                                                   "shared_size": shared["ff"] if shared else 0})
        layers.append(LayerSpec(prefix=f"l{i}", block="parallel", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=None, mixer_name="mix", feed_forward_name="mlp", mixer_norm_name="norm1"))
    return ModelSpec(architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=layers, run_order=[RunEntry(i) for i in range(len(layers))], final_norm=norm,
                     final_norm_prefix="final.norm", lm_head_name="head", max_positions=cfg.max_positions,
                     eos_token_ids=list(cfg.eos_token_ids), embedding_scale=cfg.embedding_scale, position_table_name="pos",
                     logit_softcap=cfg.logit_softcap, logit_scale=cfg.logit_scale)


register_architecture("Gofezen", GofezenConfig.from_dict, gofezen_spec)
