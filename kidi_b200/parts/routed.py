"""A feed-forward of many small gated experts, of which each token uses a few.

    z = W_router h                       router logits, 32-bit
    s = sigmoid(z)                       scores; the `top` experts with the largest scores are taken
    w = s of the chosen experts          (divided by their sum when `renormalise` is set)
    y = sum over the chosen experts of expert_e(w_e h)           `weight_on` = "input"
      or sum of w_e expert_e(h)                                   `weight_on` = "output"
    expert(x) = W_down (silu(W_gate x) * (W_up x))

Parameters (`spec.params`): hidden_size, expert_size, experts, top, score ("sigmoid"), renormalise (false),
weight_on ("input"), router_name ("router"), expert_name ("e{index}."), gate_name, up_name, down_name. A file
holds each expert's three matrices under `<prefix><expert_name><gate|up|down>`; they are bound as two stacked
tensors, [experts, 2 * expert_size, hidden] (gate rows, then up rows) and [experts, hidden, expert_size].

Steps of few rows, steps inside a captured decode graph, and every step of the 32-bit engine read the
chosen experts' weights through the choice on the device (no host round trip). Prompts of the bfloat16
engine sort the (row, choice) pairs by expert on the host and gather the scaled rows; every expert's rows are
then padded to one count and run through two batched products of the vendor library, or, where one expert has
far more rows than the others or the widths are no multiples of 8, each expert's rows through the ordinary
products.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..errors import invalid_argument, unsupported
from ..kernels import ops, routed
from .base import Part, plain_rows
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec

# Up to this many (row, choice) pairs a step reads the experts through the choice; above, a bfloat16 prompt
# sorts them by expert.
SLOT_PATH_MAX = 128


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.inter = int(spec.param("expert_size"))
        self.experts = int(spec.param("experts"))
        self.top = int(spec.param("top"))
        self.renormalise = bool(spec.param("renormalise", False))
        self.weight_on_input = spec.param("weight_on", "input") == "input"
        if spec.param("weight_on", "input") not in ("input", "output"):
            raise invalid_argument("routed experts weigh an expert's input or its output")
        if spec.param("score", "sigmoid") != "sigmoid":
            raise unsupported(f"router score '{spec.param('score')}' is not built (sigmoid is)")
        if min(self.hidden, self.inter, self.experts, self.top) <= 0 or self.top > self.experts:
            raise invalid_argument("invalid routed feed-forward dimensions")
        if self.experts > 1024 or self.top > 32:
            raise unsupported("the router takes up to 1,024 experts and 32 choices a token")
        self.router_name = spec.param("router_name", "router")
        self.expert_name = spec.param("expert_name", "e{index}.")
        self.gate_name, self.up_name, self.down_name = (spec.param(key + "_name", key) for key in ("gate", "up", "down"))
        self.router: Optional[torch.Tensor] = None
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        names = [self.expert_name.format(index=index) for index in range(self.experts)]
        both, down = [], []
        for name in names:
            both.append((name + self.gate_name, (self.inter, self.hidden)))
            both.append((name + self.up_name, (self.inter, self.hidden)))
            down.append((name + self.down_name, (self.hidden, self.inter)))
        return [ParamSpec(self.router_name, (self.experts, self.hidden)),
                ParamSpec("experts.gate_up", (self.experts * 2 * self.inter, self.hidden), sources=tuple(both)),
                ParamSpec("experts.down", (self.experts * self.hidden, self.inter), sources=tuple(down))]

    def bind(self, tensors) -> None:
        self.router = tensors[self.router_name]
        self.gate_up = tensors["experts.gate_up"].view(self.experts, 2 * self.inter, self.hidden)
        self.down = tensors["experts.down"].view(self.experts, self.hidden, self.inter)
        self._gate_up = [Linear(self.gate_up[index]) for index in range(self.experts)]
        self._down = [Linear(self.down[index]) for index in range(self.experts)]

    def forward(self, x, ctx) -> torch.Tensor:
        x = plain_rows(x)
        rows = x.shape[0]
        chosen, weight = routed.route(x, self.router, self.top, self.renormalise)
        slots = rows * self.top
        if x.dtype == torch.float32 or self.gate_up.dtype == torch.float32 or ctx.plan.is_decode \
                or slots <= SLOT_PATH_MAX:
            return routed.expert_slots(x, self.gate_up, self.down, chosen, weight, self.weight_on_input)
        # Many rows: (row, choice) pairs in the order of their experts (a stable sort, so a row's place among
        # its expert's rows follows its place in the step), one host round trip for the counts.
        picked = chosen.reshape(-1).cpu().numpy()
        order = np.argsort(picked, kind="stable").astype(np.int32)
        counts = np.bincount(picked, minlength=self.experts)
        place = np.empty(slots, dtype=np.int32)
        most = int(-(-int(counts.max()) // 8) * 8)
        if self.hidden % 8 == 0 and self.inter % 8 == 0 and self.experts * most <= 3 * slots:
            # Every expert's rows padded to one count: two batched products of the vendor library and one gate
            # for all experts (taken unless one expert has far more rows than the others).
            begins = np.concatenate([[0], np.cumsum(counts)[:-1]])
            experts_sorted = picked[order]
            at = (experts_sorted * most + (np.arange(slots) - begins[experts_sorted])).astype(np.int32)
            padded = np.full(self.experts * most, -1, dtype=np.int32)
            padded[at] = order
            place[order] = at
            both_tables = torch.from_numpy(np.concatenate([padded, place])).to(x.device)
            gathered = routed.gather_slots(x, both_tables[:padded.size], weight, self.top, self.weight_on_input)
            both = torch.bmm(gathered.view(self.experts, most, self.hidden), self.gate_up.transpose(1, 2))
            ops.note("library_bmm")
            mid = ops.silu_gate(both.view(self.experts * most, 2 * self.inter))
            result = torch.bmm(mid.view(self.experts, most, self.inter), self.down.transpose(1, 2))
            ops.note("library_bmm")
            return routed.combine_slots(result.view(self.experts * most, self.hidden), both_tables[padded.size:], weight,
                                        rows, self.top, self.weight_on_input)
        place[order] = np.arange(slots, dtype=np.int32)
        both = torch.from_numpy(np.concatenate([order, place])).to(x.device)
        gathered = routed.gather_slots(x, both[:slots], weight, self.top, self.weight_on_input)
        result = torch.empty((slots, self.hidden), dtype=x.dtype, device=x.device)
        begin = 0
        for index, count in enumerate(counts.tolist()):
            if count:
                mid = ops.silu_gate(self._gate_up[index].forward(gathered[begin:begin + count]))
                self._down[index].forward(mid, out=result[begin:begin + count])
                begin += count
        return routed.combine_slots(result, both[slots:], weight, rows, self.top, self.weight_on_input)
