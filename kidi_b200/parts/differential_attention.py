"""Differential attention as a mixer: two softmax maps a head over one set of values, and their difference.

With h the mixer's input, H query heads, G key/value heads (query head i reads key/value head i // (H / G)),
d the width of a map and e the width of a value head:

    q = W_q h  [H, 2, d],   k = W_k h  [G, 2, d],   v = W_v h  [G, e]         (no biases)
    q, k, v <- a short causal convolution over time on every channel (`conv` taps; 0: none; 1: a weight a channel)
    q, k    <- per head and map: divided by the root mean square over d, times a weight of d entries
    a_m     = softmax over the visible keys of (q_m . k_m) * scale, times v            m = 1, 2
    o       = a_1 - lambda * a_2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff   (one number a layer)
    o      <- o / sqrt(mean(o^2) + eps) * (1 - diff),  over the head's e values
    y       = W_o (concatenated heads * sigmoid(W_g h))

Key j is visible from position i when j <= i and (i - j < window or j < keep_first); no window: every
earlier key. Positions do not enter the scores.

What a sequence keeps: keys (both maps, normalised) and values for every token (paged: the window is a
mask, not a ring, since the first tokens stay visible), and the last taps - 1 projected rows for the
convolution, as fixed-size state.

Parameters (`spec.params`): hidden_size, num_heads, num_kv_heads, dim, vdim, conv (taps), diff, scale, eps,
window, keep_first, and the tensor names under the prefix (defaults: q, k, v, g, o, q.norm, k.norm, q.conv,
k.conv, v.conv, lq1, lk1, lq2, lk2).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..cache.sequence_cache import KVRequest, StateRequest
from ..errors import invalid_argument, unsupported
from ..kernels import differential
from .base import Part, plain_rows
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec


@register_part("mixer", "differential_attention")
class DifferentialAttention(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.heads = int(spec.param("num_heads"))
        self.kv_heads = int(spec.param("num_kv_heads"))
        self.dim = int(spec.param("dim"))
        self.vdim = int(spec.param("vdim"))
        self.taps = int(spec.param("conv", 0) or 0)
        self.diff = float(spec.param("diff", 0.0))
        self.eps = float(spec.param("eps"))
        scale = spec.param("scale", None)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(self.dim))
        self.window = spec.param("window", None)
        self.keep_first = int(spec.param("keep_first", 0) or 0)
        if min(self.hidden, self.heads, self.kv_heads, self.dim, self.vdim) <= 0 or self.heads % self.kv_heads:
            raise invalid_argument("invalid differential attention dimensions")
        if self.dim > 256 or self.vdim > 256:
            raise unsupported("differential attention takes maps and value heads of at most 256 entries")
        if not 0 <= self.taps <= differential.MAX_TAPS:
            raise unsupported(f"the short convolution takes up to {differential.MAX_TAPS} taps")
        if self.window is not None and int(self.window) <= 0:
            raise invalid_argument("an attention window must be positive")
        if self.keep_first < 0:
            raise invalid_argument("keep_first cannot be negative")
        self.q_width, self.k_width = 2 * self.heads * self.dim, 2 * self.kv_heads * self.dim
        self.v_width, self.o_width = self.kv_heads * self.vdim, self.heads * self.vdim
        self.channels = self.q_width + self.k_width + self.v_width
        self.names = {key: spec.param(key + "_name", default) for key, default in (
            ("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm"),
            ("q_conv", "q.conv"), ("k_conv", "k.conv"), ("v_conv", "v.conv"), ("lq1", "lq1"), ("lk1", "lk1"),
            ("lq2", "lq2"), ("lk2", "lk2"))}
        self.projection: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.conv = self.q_norm = self.k_norm = None
        self.lam = 0.0

    def parameter_specs(self) -> List[ParamSpec]:
        n, hidden = self.names, self.hidden
        specs = [
            ParamSpec("qkvg", (self.channels + self.o_width, hidden), sources=(
                (n["q"], (self.q_width, hidden)), (n["k"], (self.k_width, hidden)), (n["v"], (self.v_width, hidden)),
                (n["g"], (self.o_width, hidden)))),
            ParamSpec(n["o"], (hidden, self.o_width)),
            ParamSpec(n["q_norm"], (self.dim,), init=("one_plus_normal", 0.1)),
            ParamSpec(n["k_norm"], (self.dim,), init=("one_plus_normal", 0.1)),
        ]
        specs += [ParamSpec(n[key], (self.dim,), init=("normal", 0.1)) for key in ("lq1", "lk1", "lq2", "lk2")]
        if self.taps >= 1:
            specs.append(ParamSpec("qkv.conv", (self.channels, self.taps), init=("normal", 0.5), sources=(
                (n["q_conv"], (self.q_width, self.taps)), (n["k_conv"], (self.k_width, self.taps)),
                (n["v_conv"], (self.v_width, self.taps)))))
        return specs

    def bind(self, tensors) -> None:
        n = self.names
        self.projection = Linear(tensors["qkvg"])
        self.out = Linear(tensors[n["o"]])
        # The small vectors are kept in 32-bit: norms, the convolution's sums and lambda are 32-bit arithmetic.
        self.q_norm = tensors[n["q_norm"]].float().contiguous()
        self.k_norm = tensors[n["k_norm"]].float().contiguous()
        self.conv = tensors["qkv.conv"].float().contiguous() if self.taps >= 1 else None
        lq1, lk1, lq2, lk2 = (tensors[n[key]].float() for key in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + self.diff)

    def cache_requests(self) -> list:
        requests = [KVRequest(self.kv_heads, 2 * self.dim, None, self.vdim)]
        if self.taps > 1:
            requests.append(StateRequest((self.taps - 1, self.channels)))
        return requests

    def launch_signature(self, rows: int, longest: int) -> tuple:
        """What a captured decode step freezes of this part's launches: the key splits of the tensor-core kernel."""
        if not differential.tensor_fits(self.env.dtype, self.dim, self.vdim, 64):
            return ()
        return (differential.tensor_splits(rows, self.kv_heads, self._reach(longest), self.env.device),)

    def _reach(self, longest: int) -> int:
        """The most keys a row of a sequence of `longest` tokens reads."""
        if self.window is None:
            return longest
        return min(longest, int(self.window) + self.keep_first + 64)

    def forward(self, x, ctx, views, owns_cache: bool) -> torch.Tensor:
        if not owns_cache:
            raise unsupported("a differential attention layer keeps its own keys, values and convolution state")
        view = views[0]
        state = views[1] if self.taps > 1 else None
        plan = ctx.plan
        geometry = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim)
        projected = self.projection.forward(plain_rows(x))
        rows = projected.shape[0]
        queries = torch.empty((rows, self.q_width), dtype=projected.dtype, device=projected.device)
        differential.prepare(projected, queries, conv=self.conv, state=state, q_norm=self.q_norm, k_norm=self.k_norm,
                             eps=self.eps, tables=ctx.tables, seqs=plan.n_seqs, kv_view=view,
                             one_token=plan.is_decode, **geometry)
        attended = torch.empty((rows, self.o_width), dtype=projected.dtype, device=projected.device)
        differential.attention(ctx, queries, projected[:, self.channels:], attended, scale=self.scale, lam=self.lam,
                               post_scale=1.0 - self.diff, eps=self.eps, window=self.window,
                               keep_first=self.keep_first, kv_view=view, **geometry)
        return self.out.forward(attended)
