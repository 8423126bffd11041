"""Python faces of the latent-attention kernels (csrc/latent_attention.cu).

The library is compiled when a model with such a layer first runs. `prepare` normalises the
latent, rotates the shared key part and the queries' rotated parts and writes the cache row;
`attention` is causal softmax attention of every row of a step over its sequence's cached rows.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument
from . import ops
from .ops import CacheGeometry, _check, c_float, c_int, c_longlong, c_void_p, cache_geometry, dtype_code


class PrepareArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("ldq", c_longlong), ("folded", c_void_p), ("ldf", c_longlong), ("kv", c_void_p),
                ("ldkv", c_longlong), ("kv_norm", c_void_p), ("cos_table", c_void_p), ("sin_table", c_void_p),
                ("row_seq", c_void_p), ("row_pos", c_void_p), ("seq_slot", c_void_p), ("cache", c_void_p),
                ("geometry", CacheGeometry), ("rows", c_int), ("heads", c_int), ("dim", c_int), ("rot_dim", c_int),
                ("rotary_dims", c_int), ("rank", c_int), ("eps", c_float)]


class AttentionArgs(ctypes.Structure):
    _fields_ = [("folded", c_void_p), ("ldf", c_longlong), ("cache", c_void_p), ("geometry", CacheGeometry),
                ("out", c_void_p), ("ldo", c_longlong), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("rows", c_int), ("heads", c_int), ("rank", c_int), ("rot_dim", c_int),
                ("window", c_int), ("scale", c_float)]


_library = None


def library():
    global _library
    if _library is None:
        lib = load_library("latent_attention")
        lib.kidi_latent_prepare.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_latent_attention.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_latent_prepare.restype = lib.kidi_latent_attention.restype = c_int
        _library = lib
    return _library


def prepare(q: torch.Tensor, folded: torch.Tensor, kv: Optional[torch.Tensor], kv_norm: Optional[torch.Tensor], *,
            heads: int, dim: int, rot_dim: int, rank: int, rotary_dims: int, cos: torch.Tensor, sin: torch.Tensor,
            eps: float, tables, kv_view) -> None:
    """q [rows, heads * (dim + rot_dim)]: the rotated part of every head is turned by its row's position and
    written to folded[:, head, rank:] (folded [rows, heads * (rank + rot_dim)]). kv [rows, rank + rot_dim], if
    given: its first `rank` entries, RMS-normalised with `kv_norm`, and its rotated last rot_dim entries become
    the row's cache entry."""
    ops._need_cuda(q, folded, kv, kv_norm, cos, sin)
    rows = q.shape[0]
    if q.shape != (rows, heads * (dim + rot_dim)) or folded.shape != (rows, heads * (rank + rot_dim)) \
            or q.stride(1) != 1 or folded.stride(1) != 1 or folded.dtype != q.dtype:
        raise invalid_argument("latent prepare: queries or folded queries have the wrong shape")
    if cos.dtype != torch.float32 or cos.dim() != 2 or cos.shape[1] != rotary_dims // 2 or sin.shape != cos.shape:
        raise invalid_argument("latent prepare: the rotation tables must be float32 [positions, rotary_dims/2]")
    if kv is not None:
        if kv.shape != (rows, rank + rot_dim) or kv.stride(1) != 1 or kv.dtype != q.dtype:
            raise invalid_argument("latent prepare: the latent rows have the wrong shape")
        if kv_norm is None or kv_norm.dtype != torch.float32 or kv_norm.shape != (rank,) or not kv_norm.is_contiguous():
            raise invalid_argument("latent prepare: the latent's norm weight is a float32 vector of `rank` entries")
        if kv_view is None or kv_view.keys.dtype != q.dtype or kv_view.keys.shape[-1] != rank + rot_dim:
            raise invalid_argument("latent prepare: the cache does not fit the latent rows")
    args = PrepareArgs(
        q.data_ptr(), q.stride(0), folded.data_ptr(), folded.stride(0), kv.data_ptr() if kv is not None else 0,
        kv.stride(0) if kv is not None else 0, kv_norm.data_ptr() if kv is not None else 0, cos.data_ptr(),
        sin.data_ptr(), tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(),
        kv_view.keys.data_ptr() if kv is not None else 0, cache_geometry(kv_view if kv is not None else None, 1,
                                                                         rank + rot_dim),
        rows, heads, dim, rot_dim, rotary_dims, rank, float(eps))
    _check(library().kidi_latent_prepare(ctypes.byref(args), dtype_code(q.dtype), ops._stream()), "latent_prepare")


def attention(folded: torch.Tensor, out: torch.Tensor, *, heads: int, rank: int, rot_dim: int, scale: float,
              window: Optional[int], tables, kv_view) -> None:
    """out[r, head, :rank] = sum_u softmax_u((folded[r, head] . entry_u) * scale) entry_u[:rank] over the cached
    entries u of the row's sequence with u <= the row's position (and u > position - window)."""
    ops._need_cuda(folded, out)
    rows = folded.shape[0]
    if folded.shape != (rows, heads * (rank + rot_dim)) or out.shape != (rows, heads * rank) or out.dtype != folded.dtype \
            or folded.stride(1) != 1 or out.stride(1) != 1:
        raise invalid_argument("latent attention: folded queries or output have the wrong shape")
    if kv_view.keys.dtype != folded.dtype or kv_view.keys.shape[-1] != rank + rot_dim:
        raise invalid_argument("latent attention: the cache does not fit the queries")
    args = AttentionArgs(folded.data_ptr(), folded.stride(0), kv_view.keys.data_ptr(),
                         cache_geometry(kv_view, 1, rank + rot_dim), out.data_ptr(), out.stride(0),
                         tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(), rows, heads,
                         rank, rot_dim, int(window or 0), float(scale))
    _check(library().kidi_latent_attention(ctypes.byref(args), dtype_code(folded.dtype), ops._stream()),
           "latent_attention")
