"""Typed configuration of Gakenex, read from the model's own config.json keys.

    architecture: "Gakenex"        vocab, width, max_positions, logit_softcap
    norm: {eps}
    layers: [{type: "attention", mixer: {...}, mlp: null | {kind: "dense", ff, limit}
                                                     | {kind: "moe", expert: {ff}, router: {experts, top}}}, ...]

A layer's mixer: heads, kv_heads, dim (the width of a query or key map), vdim, conv (taps of the short
convolution; absent or 0: none), diff, scale, mask: {size, keep_first} (absent: every earlier token is
visible; keep_first absent: 0). `logit_softcap` absent or 0: the logits are not bounded. A missing or
ill-typed key is INVALID_MANIFEST naming the key.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Mapping, Optional, Tuple

from ..errors import invalid_manifest, unsupported
from .reader import ConfigReader

ATTENTION = "attention"
DENSE, ROUTED = "dense", "moe"


@dataclasses.dataclass(frozen=True)
class GakenexFeedForward:
    kind: str
    ff: int                      # dense: the intermediate width; routed: an expert's
    limit: float = 0.0           # dense only
    experts: int = 0             # routed only
    top: int = 0

    def to_dict(self) -> dict:
        if self.kind == DENSE:
            return {"kind": DENSE, "ff": self.ff, "limit": self.limit}
        return {"kind": ROUTED, "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclasses.dataclass(frozen=True)
class GakenexLayer:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    diff: float
    scale: float
    window: Optional[int]
    keep_first: int
    mlp: Optional[GakenexFeedForward]

    def to_dict(self) -> dict:
        mixer: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                       "diff": self.diff, "scale": self.scale}
        if self.conv:
            mixer["conv"] = self.conv
        if self.window is not None:
            mixer["mask"] = {"size": self.window, "keep_first": self.keep_first}
        return {"type": self.type, "mixer": mixer, "mlp": self.mlp.to_dict() if self.mlp is not None else None}


@dataclasses.dataclass(frozen=True)
class GakenexConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_softcap: float
    layers: Tuple[GakenexLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Gakenex"

    @classmethod
    def from_dict(cls, values: Mapping[str, Any]) -> "GakenexConfig":
        reader = ConfigReader(values)
        name = reader.string("architecture", cls.architecture)
        if name != cls.architecture:
            raise invalid_manifest(f"expected architecture '{cls.architecture}', found '{name}'")
        norm = reader.child("norm")
        if norm is None:
            raise invalid_manifest("config.json: 'norm' must be an object")
        raw_layers = reader.raw("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise invalid_manifest("config.json: 'layers' must be a non-empty list")
        layers = []
        for index, raw in enumerate(raw_layers):
            where = f"config.json:layers[{index}]"
            layer = ConfigReader(raw, where)
            kind = layer.string("type")
            if kind != ATTENTION:
                raise unsupported(f"layers[{index}]: layer type '{kind}' is not supported")
            mixer = layer.child("mixer")
            if mixer is None:
                raise invalid_manifest(f"{where}: 'mixer' must be an object")
            mask = mixer.child("mask")
            window = mask.integer("size") if mask is not None and mask.has("size") else None
            keep_first = mask.integer("keep_first", 0) if mask is not None else 0
            mlp = layer.child("mlp")
            feed_forward = None
            if mlp is not None:
                mlp_kind = mlp.string("kind")
                if mlp_kind == DENSE:
                    feed_forward = GakenexFeedForward(DENSE, mlp.integer("ff"), limit=mlp.number("limit"))
                elif mlp_kind == ROUTED:
                    expert, router = mlp.child("expert"), mlp.child("router")
                    if expert is None or router is None:
                        raise invalid_manifest(f"{where}:mlp: 'expert' and 'router' must be objects")
                    feed_forward = GakenexFeedForward(ROUTED, expert.integer("ff"), experts=router.integer("experts"),
                                                      top=router.integer("top"))
                else:
                    raise unsupported(f"layers[{index}]: feed-forward kind '{mlp_kind}' is not supported")
            layers.append(GakenexLayer(
                type=kind, heads=mixer.integer("heads"), kv_heads=mixer.integer("kv_heads"), dim=mixer.integer("dim"),
                vdim=mixer.integer("vdim"), conv=mixer.integer("conv", 0), diff=mixer.number("diff"),
                scale=mixer.number("scale"), window=window, keep_first=keep_first, mlp=feed_forward))
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
                     max_positions=reader.integer("max_positions"), norm_eps=norm.number("eps"),
                     logit_softcap=reader.number("logit_softcap", 0.0), layers=tuple(layers), eos_token_ids=eos_ids)
        config.validate()
        return config

    def validate(self) -> None:
        if min(self.vocab, self.width, self.max_positions) <= 0:
            raise invalid_manifest("invalid Gakenex dimensions: every size must be positive")
        if not self.norm_eps > 0:
            raise invalid_manifest("invalid Gakenex configuration: norm.eps must be positive")
        if self.logit_softcap < 0:
            raise invalid_manifest("invalid Gakenex configuration: logit_softcap cannot be negative")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if min(layer.heads, layer.kv_heads, layer.dim, layer.vdim) <= 0 or layer.conv < 0:
                raise invalid_manifest(f"{where}: every size must be positive")
            if layer.heads % layer.kv_heads:
                raise invalid_manifest(f"{where}: heads must be a multiple of kv_heads")
            if layer.window is not None and layer.window <= 0:
                raise invalid_manifest(f"{where}: mask.size must be positive")
            if layer.keep_first < 0:
                raise invalid_manifest(f"{where}: mask.keep_first cannot be negative")
            mlp = layer.mlp
            if mlp is None:
                continue
            if mlp.ff <= 0:
                raise invalid_manifest(f"{where}: the feed-forward's width must be positive")
            if mlp.kind == DENSE and not mlp.limit > 0:
                raise invalid_manifest(f"{where}: mlp.limit must be positive")
            if mlp.kind == ROUTED and not 0 < mlp.top <= mlp.experts:
                raise invalid_manifest(f"{where}: the router needs 0 < top <= experts")
        if any(token < 0 or token >= self.vocab for token in self.eos_token_ids):
            raise invalid_manifest("eos_token_id lies outside the vocabulary")

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal configuration."""
        values = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                  "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                  "layers": [layer.to_dict() for layer in self.layers]}
        if self.logit_softcap:
            values["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            values["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return values
