"""Typed configuration of Sanozen, read from the model's own config.json keys.

    architecture: "Sanozen"        vocab, width
    embedding: {scale}             norm: {eps}            token_side: {dim}
    layers: [{type, mixer: {...}, mlp: null | {kind: "dense", ff}}, ...]

A layer's `type` is "latent_attention" (mixer: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base,
dims}, optionally kv_from: the index of an earlier latent-attention layer whose cached rows this one reads) or
"hgrn2" (mixer: heads, dim, vdim). `max_positions` is optional (the longest sequence the rotation tables are
built for; default 65,536). Every size is required and positive; a missing or ill-typed key is INVALID_MANIFEST
naming the key.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple

from ..errors import invalid_manifest, unsupported
from .reader import ConfigReader

LATENT_ATTENTION = "latent_attention"
HGRN2 = "hgrn2"
DEFAULT_MAX_POSITIONS = 65536


@dataclasses.dataclass(frozen=True)
class SanozenLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    ff: Optional[int]                # None: the layer has no feed-forward
    # latent attention only
    rot_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    rot_base: float = 0.0
    rot_dims: int = 0
    kv_from: Optional[int] = None

    def to_dict(self) -> dict:
        mixer: dict = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == LATENT_ATTENTION:
            mixer.update(rot_dim=self.rot_dim, q_rank=self.q_rank, kv_rank=self.kv_rank, scale=self.scale,
                         rot={"base": self.rot_base, "dims": self.rot_dims})
            if self.kv_from is not None:
                mixer["kv_from"] = self.kv_from
        return {"type": self.type, "mixer": mixer,
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff is not None else None}


@dataclasses.dataclass(frozen=True)
class SanozenConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    token_side_dim: int
    layers: Tuple[SanozenLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Sanozen"

    @classmethod
    def from_dict(cls, values: Mapping[str, Any]) -> "SanozenConfig":
        reader = ConfigReader(values)
        name = reader.string("architecture", cls.architecture)
        if name != cls.architecture:
            raise invalid_manifest(f"expected architecture '{cls.architecture}', found '{name}'")
        embedding, norm, side = reader.child("embedding"), reader.child("norm"), reader.child("token_side")
        if embedding is None or norm is None or side is None:
            raise invalid_manifest("config.json: 'embedding', 'norm' and 'token_side' must be objects")
        raw_layers = reader.raw("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise invalid_manifest("config.json: 'layers' must be a non-empty list")
        layers = []
        for index, raw in enumerate(raw_layers):
            layer = ConfigReader(raw, f"config.json:layers[{index}]")
            kind = layer.string("type")
            mixer = layer.child("mixer")
            if mixer is None:
                raise invalid_manifest(f"config.json:layers[{index}]: 'mixer' must be an object")
            mlp = layer.child("mlp")
            ff = None
            if mlp is not None:
                if mlp.string("kind") != "dense":
                    raise unsupported(f"layers[{index}]: feed-forward kind '{mlp.string('kind')}' is not supported")
                ff = mlp.integer("ff")
            common = dict(type=kind, heads=mixer.integer("heads"), dim=mixer.integer("dim"),
                          vdim=mixer.integer("vdim"), ff=ff)
            if kind == LATENT_ATTENTION:
                rot = mixer.child("rot")
                if rot is None:
                    raise invalid_manifest(f"config.json:layers[{index}]:mixer: 'rot' must be an object")
                layers.append(SanozenLayer(
                    **common, rot_dim=mixer.integer("rot_dim"), q_rank=mixer.integer("q_rank"),
                    kv_rank=mixer.integer("kv_rank"), scale=mixer.number("scale"), rot_base=rot.number("base"),
                    rot_dims=rot.integer("dims"),
                    kv_from=mixer.integer("kv_from") if mixer.has("kv_from") else None))
            elif kind == HGRN2:
                layers.append(SanozenLayer(**common))
            else:
                raise unsupported(f"layers[{index}]: layer type '{kind}' is not supported")
        eos = reader.raw("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise invalid_manifest("'eos_token_id' must be an integer or a list of integers")
        config = cls(vocab=reader.integer("vocab"), width=reader.integer("width"),
                     embedding_scale=embedding.number("scale"), norm_eps=norm.number("eps"),
                     token_side_dim=side.integer("dim"), layers=tuple(layers),
                     max_positions=reader.integer("max_positions", DEFAULT_MAX_POSITIONS), eos_token_ids=eos_ids)
        config.validate()
        return config

    def validate(self) -> None:
        if min(self.vocab, self.width, self.token_side_dim, self.max_positions) <= 0:
            raise invalid_manifest("invalid Sanozen dimensions: every size must be positive")
        if not self.norm_eps > 0:
            raise invalid_manifest("invalid Sanozen configuration: norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if min(layer.heads, layer.dim, layer.vdim) <= 0 or (layer.ff is not None and layer.ff <= 0):
                raise invalid_manifest(f"{where}: every size must be positive")
            if layer.type != LATENT_ATTENTION:
                continue
            if min(layer.rot_dim, layer.q_rank, layer.kv_rank) <= 0:
                raise invalid_manifest(f"{where}: rot_dim, q_rank and kv_rank must be positive")
            if layer.rot_dims <= 0 or layer.rot_dims % 2 or layer.rot_dims > layer.rot_dim:
                raise invalid_manifest(f"{where}: rot.dims must be even, positive and at most rot_dim")
            if not layer.rot_base > 0:
                raise invalid_manifest(f"{where}: rot.base must be positive")
            if layer.kv_from is not None:
                if not 0 <= layer.kv_from < index:
                    raise invalid_manifest(f"{where}: kv_from must name an earlier layer")
                source = self.layers[layer.kv_from]
                if source.type != LATENT_ATTENTION or source.kv_from is not None:
                    raise invalid_manifest(f"{where}: kv_from must name a latent-attention layer with a latent of its own")
                if (source.kv_rank, source.rot_dim, source.rot_base, source.rot_dims) != \
                        (layer.kv_rank, layer.rot_dim, layer.rot_base, layer.rot_dims):
                    raise invalid_manifest(f"{where}: kv_rank, rot_dim and rotation must equal those of layer {layer.kv_from}")
        if any(token < 0 or token >= self.vocab for token in self.eos_token_ids):
            raise invalid_manifest("eos_token_id lies outside the vocabulary")

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        values = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "token_side": {"dim": self.token_side_dim}, "layers": [layer.to_dict() for layer in self.layers],
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            values["max_positions"] = self.max_positions
        if self.eos_token_ids:
            values["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return values
