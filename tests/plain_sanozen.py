"""Sanozen, plainly: whole sequences, no cache, one function per mechanism, float64 or float32 torch on the CPU.

This file shares no code with the package. It takes the config.json dictionary and a dictionary of tensors under
the checkpoint's names, and returns logits [tokens, vocab] (and, if asked, the stream after every layer).

Notation: T tokens, D width, H heads. A linear weight W is stored [out, in]; `lin(W, x)` is x W^T.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch


def lin(weight: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return x @ weight.to(x.dtype).t()


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    centred = x - x.mean(-1, keepdim=True)
    variance = (centred * centred).mean(-1, keepdim=True)
    return centred / torch.sqrt(variance + eps) * weight.to(x.dtype) + bias.to(x.dtype)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotates the first `dims` entries of the last axis of x [T, ..., n]: entries 2i and 2i+1 form a pair that turns
    by the angle position * base^(-2i/dims). Angles are formed in the dtype of x."""
    half = dims // 2
    index = torch.arange(half, dtype=x.dtype)
    frequency = torch.tensor(base, dtype=x.dtype) ** (-2.0 * index / dims)
    angle = positions.to(x.dtype)[:, None] * frequency[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_keys(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping, eps: float,
                positions: torch.Tensor):
    """What a latent-attention layer keeps per token: the normalised latent c [T, kv_rank] and the rotated key part
    shared by all heads [T, rot_dim]."""
    rank, rot_dim = mixer["kv_rank"], mixer["rot_dim"]
    down = lin(w[prefix + "dkv"], h)
    c = rms(down[:, :rank], eps) * w[prefix + "dkv.norm"].to(h.dtype)
    shared = rotate_interleaved(down[:, rank:rank + rot_dim], positions, mixer["rot"]["base"], mixer["rot"]["dims"])
    return c, shared


def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping, eps: float,
                     positions: torch.Tensor, kept) -> torch.Tensor:
    """Causal softmax attention whose keys and values are projections of the latent c; `kept` = (c, shared key part)
    of this layer or of the layer it borrows them from."""
    heads, dim, rot_dim, vdim = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"]
    T = h.shape[0]
    c, shared = kept
    cq = rms(lin(w[prefix + "dq"], h), eps) * w[prefix + "dq.norm"].to(h.dtype)
    q = lin(w[prefix + "uq"], cq).reshape(T, heads, dim + rot_dim)
    q_plain = q[..., :dim]
    q_turned = rotate_interleaved(q[..., dim:], positions, mixer["rot"]["base"], mixer["rot"]["dims"])
    k_plain = lin(w[prefix + "uk"], c).reshape(T, heads, dim)
    value = lin(w[prefix + "uv"], c).reshape(T, heads, vdim)
    scores = torch.einsum("thd,uhd->htu", q_plain, k_plain) + torch.einsum("thd,ud->htu", q_turned, shared)
    scores = scores * mixer["scale"]
    visible = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("htu,uhd->thd", weights, value).reshape(T, heads * vdim)
    return lin(w[prefix + "o"], out)


def hgrn2(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping, eps: float) -> torch.Tensor:
    """A gated linear recurrence per head: S <- diag(f) S + (1 - f) v^T, read out as S^T q."""
    heads, dim, vdim = mixer["heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    q = torch.nn.functional.silu(lin(w[prefix + "q"], h)).reshape(T, heads, dim)
    value = lin(w[prefix + "v"], h).reshape(T, heads, vdim)
    lower = w[prefix + "lower"].to(h.dtype)
    gate = torch.sigmoid(lin(w[prefix + "f"], h) + w[prefix + "f.b"].to(h.dtype))
    forget = (lower + (1.0 - lower) * gate).reshape(T, heads, dim)
    state = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    outs = []
    for t in range(T):
        state = forget[t][:, :, None] * state + (1.0 - forget[t])[:, :, None] * value[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", state, q[t]))
    out = torch.stack(outs)                                         # [T, heads, vdim]
    out = rms(out, eps) * w[prefix + "norm"].to(h.dtype)
    return lin(w[prefix + "o"], out.reshape(T, heads * vdim))


def poly_norm_mlp(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, eps: float) -> torch.Tensor:
    z = lin(w[prefix + "up"], h)
    a, b, c, e = [float(value) for value in w[prefix + "act"].double()]
    act = a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e
    return lin(w[prefix + "down"], act)


def token_side(x: torch.Tensor, tokens: torch.Tensor, w: Mapping[str, torch.Tensor], layer: int, dim: int,
               eps: float) -> torch.Tensor:
    prefix = f"l{layer}.side."
    e = w["side.embed"].to(x.dtype)[tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(lin(w[prefix + "gate"], x)) * e
    y = lin(w[prefix + "proj"], g)
    return x + rms(y, eps) * w[prefix + "norm"].to(x.dtype)


def forward(config: Mapping, w: Mapping[str, torch.Tensor], tokens, dtype=torch.float64,
            layers_out: Optional[List[torch.Tensor]] = None, mixed_out: Optional[List[torch.Tensor]] = None):
    """Logits [T, vocab] of one sequence that starts at position 0."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    eps = float(config["norm"]["eps"])
    side_dim = int(config["token_side"]["dim"])
    x = w["embed"].to(dtype)[tokens] * float(config["embedding"]["scale"])
    history = [x]
    kept: Dict[int, tuple] = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mixer = layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "latent_attention":
            source = mixer.get("kv_from")
            if source is None:
                kept[i] = latent_keys(h, w, p + "mix.", mixer, eps, positions)
                source = i
            x = x + latent_attention(h, w, p + "mix.", mixer, eps, positions, kept[source])
        elif layer["type"] == "hgrn2":
            x = x + hgrn2(h, w, p + "mix.", mixer, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            x = x + poly_norm_mlp(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", eps)
        x = token_side(x, tokens, w, i, side_dim, eps)
        if layers_out is not None:
            layers_out.append(x)
        history.append(x)
        mix = w[p + "dwa"].to(dtype)
        x = sum(mix[j] * history[j] for j in range(i + 2))
        if mixed_out is not None:
            mixed_out.append(x)
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return lin(w["head"], x)
