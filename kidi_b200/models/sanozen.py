"""Sanozen as a `ModelSpec`.

A decoder-only stack whose layers are pre-norm blocks (layer norms with weight and bias) around one of two
mixers, attention over a cached latent or an HGRN2 recurrence, and, where a layer has one, a dense feed-forward
with the PolyNorm activation. After its sublayers every layer adds a gated function of the token's own row of a
side table to the stream, and what it hands on is a weighted sum of the embedding output and all layers'
results so far. A latent-attention layer may read the cached rows of an earlier one instead of making its own.

Tensor names: `embed`, `side.embed`, `final.norm(.b)`, `head`, and per layer `l<i>.norm1(.b)`, `l<i>.norm2(.b)`,
`l<i>.mix.*`, `l<i>.mlp.{up,down,act}`, `l<i>.side.{gate,proj,norm}`, `l<i>.dwa`.

This file maps a `SanozenConfig` to parts and their parameters; nothing here computes.
"""
from __future__ import annotations

from ..config.sanozen import LATENT_ATTENTION, SanozenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

SIDE_TABLE = "side"


def rotation_name(base: float, dims: int, width: int) -> str:
    return f"rot_{base!r}_{dims}_{width}"


def build_spec(config: SanozenConfig) -> ModelSpec:
    hidden, eps = config.width, config.norm_eps
    count = len(config.layers)
    positions, layers, schedule = {}, [], []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        norm = lambda name: PartSpec("layer_norm", {"size": hidden, "eps": eps, "weight_name": name,
                                                    "bias_name": name + ".b"}, prefix)
        if layer.type == LATENT_ATTENTION:
            position = rotation_name(layer.rot_base, layer.rot_dims, layer.rot_dim)
            positions.setdefault(position, PartSpec("rotary", {
                "head_dim": layer.rot_dim, "rotary_dim": layer.rot_dims, "theta": layer.rot_base,
                "max_positions": config.max_positions}))
            mixer = PartSpec("latent_attention", {
                "hidden_size": hidden, "num_heads": layer.heads, "dim": layer.dim, "rot_dim": layer.rot_dim,
                "vdim": layer.vdim, "q_rank": layer.q_rank, "kv_rank": layer.kv_rank, "scale": layer.scale,
                "eps": eps, "position": position, "owns_latent": layer.kv_from is None}, prefix + "mix.")
        else:
            mixer = PartSpec("hgrn2", {"hidden_size": hidden, "num_heads": layer.heads, "dim": layer.dim,
                                       "vdim": layer.vdim, "eps": eps}, prefix + "mix.")
        parts = {
            "input_norm": norm("norm1"),
            "mixer": mixer,
            "token_input": PartSpec("gated_token_embedding", {
                "hidden_size": hidden, "dim": config.token_side_dim, "offset": index * config.token_side_dim,
                "table": SIDE_TABLE, "eps": eps}, prefix + "side."),
            "stream_mix": PartSpec("depth_average", {"index": index, "layers": count, "name": "dwa"}, prefix),
        }
        if layer.ff is not None:
            parts["post_norm"] = norm("norm2")
            parts["feed_forward"] = PartSpec("dense_mlp", {
                "hidden_size": hidden, "intermediate_size": layer.ff, "activation": "poly_norm", "eps": eps,
                "up_name": "up", "down_name": "down", "act_name": "act"}, prefix + "mlp.")
        layers.append(LayerSpec(arrangement=PartSpec("pre_norm"), parts=parts))
        schedule.append(ScheduleEntry(index, cache_from=layer.kv_from))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=hidden,
        max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": hidden,
                                               "scale": config.embedding_scale, "name": "embed"}, ""),
        positions=positions,
        shared={SIDE_TABLE: PartSpec("token_table", {"vocab_size": config.vocab,
                                                     "width": count * config.token_side_dim, "name": "side.embed"}, "")},
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("layer_norm", {"size": hidden, "eps": eps, "weight_name": "final.norm",
                                           "bias_name": "final.norm.b"}, ""),
        head=PartSpec("linear_head", {"hidden_size": hidden, "vocab_size": config.vocab, "name": "head"}, ""),
        eos_token_ids=config.eos_token_ids,
    )


register_architecture("Sanozen", SanozenConfig, build_spec)
