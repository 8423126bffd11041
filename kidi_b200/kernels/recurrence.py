"""Python face of the gated linear recurrence kernel (csrc/gated_recurrence.cu), compiled when a model
with such a layer first runs."""
from __future__ import annotations

import ctypes

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument
from . import ops
from .ops import _check, c_int, c_longlong, c_void_p, dtype_code


class RecurrenceArgs(ctypes.Structure):
    _fields_ = [("qfv", c_void_p), ("ld", c_longlong), ("f_bias", c_void_p), ("lower", c_void_p),
                ("state", c_void_p), ("out", c_void_p), ("ldo", c_longlong), ("row_seq", c_void_p),
                ("seq_slot", c_void_p), ("seq_row0", c_void_p), ("seq_len", c_void_p), ("seqs", c_int),
                ("heads", c_int), ("dim", c_int), ("vdim", c_int), ("rows", c_int), ("narrow_blocks", c_int),
                ("gates", c_void_p)]


_library = None


def library():
    global _library
    if _library is None:
        lib = load_library("gated_recurrence")
        lib.kidi_gated_recurrence.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_gated_recurrence.restype = c_int
        _library = lib
    return _library


def gated_recurrence(qfv: torch.Tensor, out: torch.Tensor, state: torch.Tensor, *, f_bias: torch.Tensor,
                     lower: torch.Tensor, heads: int, dim: int, vdim: int, tables, seqs: int,
                     many_tokens: bool = False) -> None:
    """Runs every sequence's rows of the step through the recurrence, from and into `state`
    [slots + 1, heads, dim, vdim] (float32). qfv [rows, 2*heads*dim + heads*vdim] holds the raw projections
    [q | f | v]; out [rows, heads*vdim] gets each head's read-out S^T q, not yet normalised. `many_tokens`: the
    step brings many tokens a sequence (a prompt), so few blocks would run for long: they are made narrower."""
    ops._need_cuda(qfv, out, state, f_bias, lower)
    rows = qfv.shape[0]
    if qfv.shape != (rows, 2 * heads * dim + heads * vdim) or out.shape != (rows, heads * vdim) or out.dtype != qfv.dtype \
            or qfv.stride(1) != 1 or out.stride(1) != 1:
        raise invalid_argument("gated recurrence: projections or output have the wrong shape")
    if state.dtype != torch.float32 or state.shape[1:] != (heads, dim, vdim) or not state.is_contiguous():
        raise invalid_argument("gated recurrence: the state is float32 [slots, heads, dim, vdim]")
    if dim > 256:
        raise invalid_argument("gated recurrence: the kernel takes up to 256 state rows a head")
    for vector, size in ((f_bias, heads * dim), (lower, heads * dim)):
        if vector.dtype != torch.float32 or vector.shape != (size,) or not vector.is_contiguous():
            raise invalid_argument("gated recurrence: bias and lower bound are float32 vectors")
    # many tokens a sequence: the gates of a row are computed once, by a kernel of their own, into scratch memory
    gates = torch.empty((rows, 2 * heads * dim), dtype=torch.float32, device=qfv.device) if many_tokens else None
    args = RecurrenceArgs(qfv.data_ptr(), qfv.stride(0), f_bias.data_ptr(), lower.data_ptr(),
                          state.data_ptr(), out.data_ptr(), out.stride(0), tables.row_seq.data_ptr(),
                          tables.seq_slot.data_ptr(), tables.seq_row0.data_ptr(), tables.seq_len.data_ptr(), seqs,
                          heads, dim, vdim, rows, 1 if many_tokens else 0, gates.data_ptr() if gates is not None else 0)
    _check(library().kidi_gated_recurrence(ctypes.byref(args), dtype_code(qfv.dtype), ops._stream()),
           "gated_recurrence[gates apart]" if gates is not None else "gated_recurrence", 2 if gates is not None else 1)
