"""Python face of the routed-experts kernels (csrc/routed.cu), compiled when a model with such a
feed-forward first runs."""
from __future__ import annotations

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument
from . import ops
from .ops import _check, c_int, c_void_p, dtype_code

_library = None


def library():
    global _library
    if _library is None:
        lib = load_library("routed")
        lib.kidi_route.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p]
        lib.kidi_expert_slots.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.kidi_gather_slots.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_void_p]
        lib.kidi_combine_slots.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                           c_void_p]
        for name in ("kidi_route", "kidi_expert_slots", "kidi_gather_slots", "kidi_combine_slots"):
            getattr(lib, name).restype = c_int
        _library = lib
    return _library


def route(x: torch.Tensor, router: torch.Tensor, top: int, renormalise: bool):
    """(chosen int32 [rows, top], weight float32 [rows, top]) for rows x [rows, hidden] and a router
    [experts, hidden]: logits in 32-bit, sigmoid scores, the `top` largest (ties: the lower index), their scores as
    weights."""
    ops._need_cuda(x, router)
    if x.dim() != 2 or not x.is_contiguous() or router.dim() != 2 or not router.is_contiguous() \
            or router.shape[1] != x.shape[1]:
        raise invalid_argument("the router takes contiguous rows and a contiguous [experts, hidden] matrix")
    rows, hidden = x.shape
    chosen = torch.empty((rows, top), dtype=torch.int32, device=x.device)
    weight = torch.empty((rows, top), dtype=torch.float32, device=x.device)
    _check(library().kidi_route(x.data_ptr(), dtype_code(x.dtype), router.data_ptr(), dtype_code(router.dtype),
                                chosen.data_ptr(), weight.data_ptr(), rows, hidden, router.shape[0], top,
                                1 if renormalise else 0, ops._stream()), "route")
    return chosen, weight


def expert_slots(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, chosen: torch.Tensor,
                 weight: torch.Tensor, weight_on_input: bool) -> torch.Tensor:
    """Every row through its chosen experts, the experts' weights read through the choice: x [rows, hidden],
    gate_up [experts, 2 * inter, hidden], down [experts, hidden, inter] -> [rows, hidden]."""
    ops._need_cuda(x, gate_up, down, chosen, weight)
    rows, hidden = x.shape
    experts, twice, _ = gate_up.shape
    inter, top = twice // 2, chosen.shape[1]
    if (not x.is_contiguous() or gate_up.shape != (experts, 2 * inter, hidden) or down.shape != (experts, hidden, inter)
            or not gate_up.is_contiguous() or not down.is_contiguous() or gate_up.dtype != down.dtype):
        raise invalid_argument("expert_slots: the experts' weights do not fit the rows")
    mid = torch.empty((rows * top, inter), dtype=x.dtype, device=x.device)
    out = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    _check(library().kidi_expert_slots(x.data_ptr(), dtype_code(x.dtype), gate_up.data_ptr(), down.data_ptr(),
                                       dtype_code(gate_up.dtype), chosen.data_ptr(), weight.data_ptr(), mid.data_ptr(),
                                       out.data_ptr(), rows, top, hidden, inter, 1 if weight_on_input else 0,
                                       ops._stream()), "expert_slots", 2)
    return out


def gather_slots(x: torch.Tensor, order: torch.Tensor, weight: torch.Tensor, top: int, weight_on_input: bool) -> torch.Tensor:
    """Row i of the result is x[order[i] // top] (times weight[order[i]] when the weight is on the input); zeros
    where order[i] is negative."""
    slots, hidden = order.shape[0], x.shape[1]
    out = torch.empty((slots, hidden), dtype=x.dtype, device=x.device)
    _check(library().kidi_gather_slots(x.data_ptr(), dtype_code(x.dtype), order.data_ptr(), weight.data_ptr(),
                                       out.data_ptr(), slots, top, hidden, 1 if weight_on_input else 0, ops._stream()),
           "gather_slots")
    return out


def combine_slots(y: torch.Tensor, place: torch.Tensor, weight: torch.Tensor, rows: int, top: int,
                  weight_on_input: bool) -> torch.Tensor:
    """out[r] = sum over k of y[place[r * top + k]] (times weight[r, k] when the weight is on the output)."""
    hidden = y.shape[1]
    out = torch.empty((rows, hidden), dtype=y.dtype, device=y.device)
    _check(library().kidi_combine_slots(y.data_ptr(), dtype_code(y.dtype), place.data_ptr(), weight.data_ptr(),
                                        out.data_ptr(), rows, top, hidden, 1 if weight_on_input else 0, ops._stream()),
           "combine_slots")
    return out
