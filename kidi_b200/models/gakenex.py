"""Gakenex as a `ModelSpec`.

A decoder-only stack: token embeddings plus a learned vector per position, normalised; layers that run a
differential attention mixer and (where a layer has one) a feed-forward side by side from one norm; a final
norm and a head that shares the embedding table and bounds its logits by a tanh. The norms of the stream are
RMS norms whose weight is stored around zero. A feed-forward is dense (a bounded gate) or routed (many small
SiLU-gated experts, sigmoid scores, the weight on the expert's input).

Tensor names: `embed`, `pos`, `embed.norm`, `final.norm`, and per layer `l<i>.norm1`, `l<i>.mix.*`,
`l<i>.mlp.{gate,up,down}` or `l<i>.mlp.router` with `l<i>.mlp.e<j>.{gate,up,down}`.

This file maps a `GakenexConfig` to parts and their parameters; nothing here computes.
"""
from __future__ import annotations

from ..config.gakenex import DENSE, GakenexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

# Constants the design fixes.
GATE_ALPHA = 1.702        # the dense feed-forward's gate is g * sigmoid(GATE_ALPHA * g)
UP_SHIFT = 1.0            # ... times (u + UP_SHIFT)
POSITIONS = "learned"


def build_spec(config: GakenexConfig) -> ModelSpec:
    hidden, eps = config.width, config.norm_eps
    norm = lambda name, prefix="": PartSpec("rms_norm", {"size": hidden, "eps": eps, "weight_name": name,
                                                         "weight_offset": 1.0}, prefix)
    layers, schedule = [], []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        parts = {
            "input_norm": norm("norm1", prefix),
            "mixer": PartSpec("differential_attention", {
                "hidden_size": hidden, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads, "dim": layer.dim,
                "vdim": layer.vdim, "conv": layer.conv, "diff": layer.diff, "scale": layer.scale, "eps": eps,
                "window": layer.window, "keep_first": layer.keep_first}, prefix + "mix."),
        }
        mlp = layer.mlp
        if mlp is not None and mlp.kind == DENSE:
            parts["feed_forward"] = PartSpec("gated_mlp", {
                "hidden_size": hidden, "intermediate_size": mlp.ff, "activation": "bounded_swish", "limit": mlp.limit,
                "alpha": GATE_ALPHA, "up_shift": UP_SHIFT, "gate_name": "gate", "up_name": "up", "down_name": "down"},
                prefix + "mlp.")
        elif mlp is not None:
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden_size": hidden, "expert_size": mlp.ff, "experts": mlp.experts, "top": mlp.top,
                "score": "sigmoid", "renormalise": False, "weight_on": "input"}, prefix + "mlp.")
        layers.append(LayerSpec(arrangement=PartSpec("parallel"), parts=parts))
        schedule.append(ScheduleEntry(index))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=hidden,
        max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": hidden, "name": "embed"}, ""),
        positions={POSITIONS: PartSpec("learned_positions", {"hidden_size": hidden,
                                                            "max_positions": config.max_positions, "name": "pos"}, "")},
        embedding_norm=norm("embed.norm"),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"hidden_size": hidden, "vocab_size": config.vocab, "name": "head",
                                      "tied_to": "embed", "softcap": config.logit_softcap}, ""),
        eos_token_ids=config.eos_token_ids,
    )


register_architecture("Gakenex", GakenexConfig, build_spec)
