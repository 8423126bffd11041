"""Python face of the differential attention kernels (csrc/differential_attention.cu), compiled when a
model with such a layer first runs: the general kernels as one library, the tensor-core kernels once per
pair of widths (the maps' width and the value heads' width)."""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument
from . import ops
from .ops import _check, c_float, c_int, c_longlong, c_void_p, dtype_code

FORCE_GENERAL = os.environ.get("KIDI_B200_GENERIC_ATTENTION", "0") == "1"
MAX_TAPS = 32


class DiffGeometry(ctypes.Structure):
    _fields_ = [("table", c_void_p), ("pages_per_seq", c_int), ("page_shift", c_int), ("heads", c_int),
                ("kv_heads", c_int), ("dim", c_int), ("vdim", c_int)]


class DiffTables(ctypes.Structure):
    _fields_ = [("row_seq", c_void_p), ("row_pos", c_void_p), ("seq_slot", c_void_p), ("seq_start", c_void_p),
                ("seq_len", c_void_p), ("seq_row0", c_void_p)]


class DiffPrepareArgs(ctypes.Structure):
    _fields_ = [("proj", c_void_p), ("ld", c_longlong), ("conv", c_void_p), ("taps", c_int), ("state", c_void_p),
                ("q_norm", c_void_p), ("k_norm", c_void_p), ("q_out", c_void_p), ("k_cache", c_void_p),
                ("v_cache", c_void_p), ("geometry", DiffGeometry), ("tables", DiffTables), ("rows", c_int),
                ("seqs", c_int), ("eps", c_float), ("move_state", c_int)]


class DiffAttentionArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("gate", c_void_p), ("ldg", c_longlong), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("geometry", DiffGeometry), ("tables", DiffTables), ("out", c_void_p), ("rows", c_int), ("seqs", c_int),
                ("max_new", c_int), ("window", c_int), ("keep_first", c_int), ("scale", c_float), ("lambda_", c_float),
                ("post_scale", c_float), ("eps", c_float), ("partial", c_void_p), ("splits", c_int)]


_libraries: Dict[Tuple[int, int], ctypes.CDLL] = {}


def library(dim: int = 0, vdim: int = 0) -> ctypes.CDLL:
    """The kernels; with widths, the library that also holds the tensor-core kernels compiled for them."""
    key = (dim, vdim)
    lib = _libraries.get(key)
    if lib is None:
        if dim:
            lib = load_library(f"differential_attention_d{dim}_v{vdim}", ("differential_attention.cu",),
                               {"KIDI_DIFF_DIM": dim, "KIDI_DIFF_VDIM": vdim})
            lib.kidi_diff_attention_tensor.argtypes = [c_void_p, c_void_p]
            lib.kidi_diff_attention_tensor.restype = c_int
        else:
            lib = load_library("differential_attention")
        lib.kidi_diff_prepare.argtypes = [c_void_p, c_int, c_int, c_void_p]
        lib.kidi_diff_attention_generic.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_diff_prepare.restype = lib.kidi_diff_attention_generic.restype = c_int
        _libraries[key] = lib
    return lib


def tensor_fits(dtype: torch.dtype, dim: int, vdim: int, page_size: int) -> bool:
    """Whether the tensor-core kernels take this layer: bfloat16, widths that are multiples of 16 and at most
    128, 64-token pages."""
    return (not FORCE_GENERAL and dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0
            and 16 <= dim <= 128 and 16 <= vdim <= 128 and page_size == 64)


def _geometry(view, heads: int, kv_heads: int, dim: int, vdim: int) -> DiffGeometry:
    return DiffGeometry(view.table.data_ptr(), view.table.shape[1], view.page_size.bit_length() - 1, heads, kv_heads,
                        dim, vdim)


def _tables(tables) -> DiffTables:
    return DiffTables(tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(),
                      tables.seq_start.data_ptr(), tables.seq_len.data_ptr(), tables.seq_row0.data_ptr())


def prepare(proj: torch.Tensor, q_out: torch.Tensor, *, conv: Optional[torch.Tensor], state: Optional[torch.Tensor],
            q_norm: torch.Tensor, k_norm: torch.Tensor, eps: float, heads: int, kv_heads: int, dim: int, vdim: int,
            tables, seqs: int, kv_view, one_token: bool) -> None:
    """From the projection's rows [rows, >= channels] (query maps, key maps, value heads): the short
    convolution over time (weights `conv` [channels, taps], the sequence's last taps - 1 projected rows in
    `state` [slots + 1, taps - 1, channels], which is moved on), the maps' norms, the query rows into `q_out`
    and the keys and values into the cache at the rows' positions."""
    ops._need_cuda(proj, q_out, conv, state, q_norm, k_norm)
    channels = 2 * (heads + kv_heads) * dim + kv_heads * vdim
    rows = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or proj.shape[1] < channels:
        raise invalid_argument("prepare: the projection's rows are too narrow")
    if q_out.shape != (rows, 2 * heads * dim) or not q_out.is_contiguous() or q_out.dtype != proj.dtype:
        raise invalid_argument("prepare: the query rows have the wrong shape or type")
    taps = 1
    if conv is not None:
        taps = conv.shape[1]
        if conv.shape != (channels, taps) or not conv.is_contiguous() or taps > MAX_TAPS:
            raise invalid_argument(f"prepare: the convolution takes [channels, taps] weights of at most {MAX_TAPS} taps")
        if taps > 1 and (state is None or state.shape[1:] != (taps - 1, channels) or state.dtype != proj.dtype
                         or not state.is_contiguous()):
            raise invalid_argument("prepare: the convolution's state must be [slots + 1, taps - 1, channels]")
        if conv.dtype != q_norm.dtype:
            raise invalid_argument("prepare: convolution and norm weights must have one type")
    if q_norm.shape != (dim,) or k_norm.shape != (dim,) or q_norm.dtype != k_norm.dtype:
        raise invalid_argument("prepare: the maps' norms have `dim` entries and one type")
    if kv_view.keys.dtype != proj.dtype or kv_view.keys.shape[-1] != 2 * dim or kv_view.values.shape[-1] != vdim:
        raise invalid_argument("prepare: the cache does not fit the layer")
    args = DiffPrepareArgs(proj.data_ptr(), proj.stride(0), conv.data_ptr() if conv is not None else 0, taps,
                           state.data_ptr() if state is not None else 0, q_norm.data_ptr(), k_norm.data_ptr(),
                           q_out.data_ptr(), kv_view.keys.data_ptr(), kv_view.values.data_ptr(),
                           _geometry(kv_view, heads, kv_heads, dim, vdim), _tables(tables), rows, seqs, float(eps),
                           1 if one_token else 0)
    launches = 1 if (one_token or taps < 2) else 2
    _check(library().kidi_diff_prepare(ctypes.byref(args), dtype_code(proj.dtype), dtype_code(q_norm.dtype),
                                       ops._stream()), "diff_prepare", launches)


def attention(ctx, q: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, *, heads: int, kv_heads: int,
              dim: int, vdim: int, scale: float, lam: float, post_scale: float, eps: float, window: Optional[int],
              keep_first: int, kv_view, general: bool = False) -> None:
    """Both maps of every head of every row over the cached keys and values (the step's own rows are in the
    cache already), their difference, its norm and the gate: out [rows, heads * vdim]. `gate` is a view
    [rows, heads * vdim] whose rows may be strided."""
    ops._need_cuda(q, gate, out)
    rows = q.shape[0]
    if q.shape != (rows, 2 * heads * dim) or not q.is_contiguous() or out.shape != (rows, heads * vdim) \
            or not out.is_contiguous() or out.dtype != q.dtype:
        raise invalid_argument("differential attention: queries or output have the wrong shape")
    if gate is not None and (gate.shape != out.shape or gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise invalid_argument("differential attention: the gate must match the output")
    plan = ctx.plan
    args = DiffAttentionArgs(q.data_ptr(), gate.data_ptr() if gate is not None else 0,
                             gate.stride(0) if gate is not None else 0, kv_view.keys.data_ptr(),
                             kv_view.values.data_ptr(), _geometry(kv_view, heads, kv_heads, dim, vdim),
                             _tables(ctx.tables), out.data_ptr(), rows, plan.n_seqs, plan.max_new, int(window or 0),
                             int(keep_first), float(scale), float(lam), float(post_scale), float(eps), 0, 1)
    group = heads // kv_heads
    if general or scale <= 0 or not tensor_fits(q.dtype, dim, vdim, kv_view.page_size) \
            or group > (16 if plan.is_decode else 64) \
            or (gate is not None and (gate.stride(0) % 2 or gate.data_ptr() % 4)):
        _check(library().kidi_diff_attention_generic(ctypes.byref(args), dtype_code(q.dtype), ops._stream()),
               "diff_attention")
        return
    reach = plan.max_total if not window else min(plan.max_total, int(window) + int(keep_first) + 64)
    splits = tensor_splits(plan.n_seqs, kv_heads, reach, q.device) if plan.is_decode else 1
    if splits > 1:
        args.partial = ctx.workspace("diff_attention_partial", rows * heads * splits * (2 * vdim + 4)).data_ptr()
        args.splits = splits
    _check(library(dim, vdim).kidi_diff_attention_tensor(ctypes.byref(args), ops._stream()),
           f"diff_attention[tensor{', split' if splits > 1 else ''}]", 2 if splits > 1 else 1)


def tensor_splits(seqs: int, kv_heads: int, reach: int, device: torch.device) -> int:
    """How many blocks share the keys of a (sequence, key/value head) when every sequence brings one token:
    as many as fill three quarters of one round of blocks (two a multiprocessor, by their registers), at most one
    per two pages of 64 keys. Measured on a B200 at 8 sequences x 8 key/value heads x 1,026 tokens: 3 shares 28 us
    a layer, 4 shares 32 us, 6 shares (two rounds) 38 us."""
    from .attention import sm_count
    forced = int(os.environ.get("KIDI_B200_DECODE_SPLITS", "0"))
    pages = max(1, -(-reach // 64))
    if forced:
        return max(1, min(pages, forced))
    items = max(1, seqs * kv_heads)
    wanted = max(1, (3 * sm_count(device)) // (2 * items))
    return max(1, min(wanted, pages // 2, 32))
