"""A per-layer input from the token ids, and the table it reads.

`token_table` (role "shared") is a table [vocab, width] that several layers read columns of; it is built once
per model under a name. `gated_token_embedding` (role "token_input") adds, after a layer's sublayers,

    e = table[token][offset : offset + dim]
    g = gelu_tanh(W_gate x) * e              gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
    y = W_proj g
    x <- x + y / sqrt(mean(y^2) + eps) * w

to the residual stream x (the addition and the norm in 32-bit). Its last kernel can also form the weighted sum of
kept streams of a `stream_mix` part that follows it.

Parameters: hidden_size, dim, offset (first column of the table), table (name of the shared table), eps, and
the tensor names gate, proj, norm under the prefix.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import Part, ResidualStream
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec


@register_part("shared", "token_table")
class TokenTable(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.param("vocab_size"))
        self.width = int(spec.param("width"))
        self.name = spec.param("name", "weight")
        self.init = tuple(spec.param("init", ("normal", 1.0)))
        self.weight: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name, (self.vocab, self.width), init=self.init)]

    def bind(self, tensors) -> None:
        self.weight = tensors[self.name]


@register_part("token_input", "gated_token_embedding")
class GatedTokenEmbedding(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.dim = int(spec.param("dim"))
        self.offset = int(spec.param("offset"))
        self.eps = float(spec.param("eps"))
        self.table = env.shared[spec.param("table")]
        self.names = {key: spec.param(key + "_name", key) for key in ("gate", "proj", "norm")}
        self.gate: Optional[Linear] = None
        self.proj: Optional[Linear] = None
        self.norm: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        n = self.names
        return [ParamSpec(n["gate"], (self.dim, self.hidden), init=("normal", 0.1)),
                ParamSpec(n["proj"], (self.hidden, self.dim), init=("normal", 0.2)),
                ParamSpec(n["norm"], (self.hidden,), init=("one_plus_normal", 0.1))]

    def bind(self, tensors) -> None:
        n = self.names
        self.gate, self.proj = Linear(tensors[n["gate"]]), Linear(tensors[n["proj"]])
        self.norm = tensors[n["norm"]].float().contiguous()

    def forward(self, stream: ResidualStream, ctx, mix=None) -> None:
        """Takes the stream's pending delta, adds this part's contribution and, with `mix`, lets the same
        kernel replace the stream by `mix`'s weighted sum."""
        dtype = self.env.dtype
        x = stream.hidden
        copy = ops.add_cast(x, stream.take_pending(), dtype if dtype != torch.float32 else None)
        gate = self.gate.forward(copy if copy is not None else x)
        y = self.proj.forward(ops.token_gate(gate, self.table.weight, self.offset, ctx.tables.tokens))
        stream.prepared = None
        if mix is not None:
            mix.forward(stream, ctx, addend=(y, self.norm, self.eps))
        else:
            ops.add_normed_mix(x, y, self.norm, self.eps)
