"""HGRN2 as a mixer: a gated linear recurrence with a matrix state per head, whose write strength is the
complement of its forget gate.

Per head, with q = silu(W_q h) [dim], v = W_v h [vdim] and the forget gate f = l + (1 - l) * sigmoid(W_f h + b)
[dim] (l a lower bound per head and channel):

    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T          o_t = S_t^T q_t

(1 - f stands where linear attention has a key; nothing else is scaled). Every head's o_t is RMS-normalised over vdim with
one weight vector shared by the heads; the heads are concatenated and projected by W_o. The state S starts at
zero, is 32-bit, and is kept per cache slot as a `StateRequest`: a sequence's rows of a step run through the
recurrence in order, whatever their number, and leave the state for the next step.

Parameters (`spec.params`): hidden_size, num_heads, dim, vdim, eps, and the tensor names under the prefix: q, f,
f_bias, lower, v, norm, o.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..errors import invalid_argument, unsupported
from ..kernels import ops
from ..kernels import recurrence as recurrence_kernels
from .base import Part, plain_rows
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec

NAMES = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o"}


@register_part("mixer", "hgrn2")
class GatedRecurrence(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.heads = int(spec.param("num_heads"))
        self.dim = int(spec.param("dim"))
        self.vdim = int(spec.param("vdim"))
        self.eps = float(spec.param("eps"))
        if min(self.hidden, self.heads, self.dim, self.vdim) <= 0:
            raise invalid_argument("invalid recurrence dimensions")
        if self.dim > 256:
            raise unsupported(f"a recurrent head of {self.dim} state rows exceeds 256, the most the kernel takes")
        self.names = {key: spec.param(key + "_name", default) for key, default in NAMES.items()}
        self.qfv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.f_bias = self.lower = self.norm = None

    def parameter_specs(self) -> List[ParamSpec]:
        n, width = self.names, self.heads * self.dim
        return [
            # one product for the three projections: [q | f | v]
            ParamSpec("qfv", (2 * width + self.heads * self.vdim, self.hidden), sources=(
                (n["q"], (width, self.hidden)), (n["f"], (width, self.hidden)),
                (n["v"], (self.heads * self.vdim, self.hidden)))),
            ParamSpec(n["f_bias"], (width,), init=("normal", 1.0)),
            ParamSpec(n["lower"], (width,), init=("uniform", 0.9)),
            ParamSpec(n["norm"], (self.vdim,), init=("one_plus_normal", 0.1)),
            ParamSpec(n["o"], (self.hidden, self.heads * self.vdim)),
        ]

    def bind(self, tensors) -> None:
        n = self.names
        self.qfv, self.out = Linear(tensors["qfv"]), Linear(tensors[n["o"]])
        self.f_bias = tensors[n["f_bias"]].float().contiguous()
        self.lower = tensors[n["lower"]].float().contiguous()
        self.norm = tensors[n["norm"]].float().contiguous()

    def cache_requests(self) -> list:
        return [StateRequest((self.heads, self.dim, self.vdim), torch.float32)]

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        if not owns_cache:
            raise invalid_argument("a recurrent layer keeps a state of its own")
        qfv = self.qfv.forward(plain_rows(x))
        read = torch.empty((qfv.shape[0], self.heads * self.vdim), dtype=qfv.dtype, device=qfv.device)
        recurrence_kernels.gated_recurrence(qfv, read, views[0], f_bias=self.f_bias, lower=self.lower,
                                            heads=self.heads, dim=self.dim, vdim=self.vdim, tables=ctx.tables,
                                            seqs=ctx.plan.n_seqs, many_tokens=ctx.plan.max_new >= 64)
        return self.out.forward(ops.rms_rows(read, self.vdim, self.norm, self.eps, out=read))
