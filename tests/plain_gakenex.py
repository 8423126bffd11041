"""Gakenex, plainly: whole sequences, no cache, one function per mechanism, float64 or float32 torch on the CPU.

This file shares no code with the package. It takes the config.json dictionary and a dictionary of tensors under
the checkpoint's names, and returns logits [tokens, vocab] (and, if asked, the stream after every layer).

Notation: T tokens, D width, H query heads, G key/value heads, d the width of a query or key map, e the width
of a value head. A linear weight W is stored [out, in]; `lin(W, x)` is x W^T.
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


def one_plus_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The stream's norm: its weight is stored around zero."""
    return rms(x, eps) * (1.0 + weight.to(x.dtype))


def short_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]: y[t] = sum_j taps[:, j] * u[t - K + 1 + j], with zeros before the first token."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + taps[:, j].to(u.dtype)[None, :] * padded[j:j + T]
    return y


def visible(T: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    """[T, T] boolean: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    near = (i - j < size) if size is not None else torch.ones(T, T, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: torch.Tensor) -> torch.Tensor:
    """q [T, d], k [T, d], v [T, e] of one map of one head."""
    scores = (q @ k.t()) * scale
    scores = scores.masked_fill(~mask, float("-inf"))
    return torch.softmax(scores, -1) @ v


def differential_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, e = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    diff = float(mixer.get("diff", 0.0))
    q, k, v = lin(w[prefix + "q"], h), lin(w[prefix + "k"], h), lin(w[prefix + "v"], h)
    if prefix + "q.conv" in w:
        q, k, v = (short_conv(x, w[prefix + name + ".conv"]) for x, name in ((q, "q"), (k, "k"), (v, "v")))
    q = rms(q.reshape(T, H, 2, d), eps) * w[prefix + "q.norm"].to(h.dtype)
    k = rms(k.reshape(T, G, 2, d), eps) * w[prefix + "k.norm"].to(h.dtype)
    v = v.reshape(T, G, e)
    mask_spec = mixer.get("mask") or {}
    mask = visible(T, mask_spec.get("size"), int(mask_spec.get("keep_first", 0)))
    lam = (torch.exp((w[prefix + "lq1"].to(h.dtype) * w[prefix + "lk1"].to(h.dtype)).sum())
           - torch.exp((w[prefix + "lq2"].to(h.dtype) * w[prefix + "lk2"].to(h.dtype)).sum()) + diff)
    heads = []
    for head in range(H):
        g = head // (H // G)
        a1 = softmax_attention(q[:, head, 0], k[:, g, 0], v[:, g], mixer["scale"], mask)
        a2 = softmax_attention(q[:, head, 1], k[:, g, 1], v[:, g], mixer["scale"], mask)
        heads.append(rms(a1 - lam * a2, eps) * (1.0 - diff))
    joined = torch.cat(heads, -1)
    joined = joined * torch.sigmoid(lin(w[prefix + "g"], h))
    return lin(w[prefix + "o"], joined)


def dense_feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mlp: Mapping) -> torch.Tensor:
    limit = float(mlp["limit"])
    g = torch.clamp(lin(w[prefix + "gate"], h), max=limit)
    u = torch.clamp(lin(w[prefix + "up"], h), -limit, limit)
    return lin(w[prefix + "down"], g * torch.sigmoid(1.702 * g) * (u + 1.0))


def routed_feed_forward(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mlp: Mapping) -> torch.Tensor:
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.sigmoid(lin(w[prefix + "router"], h))
    chosen = torch.topk(scores, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for index in chosen[t].tolist():
            x = scores[t, index] * h[t]
            name = f"{prefix}e{index}."
            z = lin(w[name + "gate"], x[None])
            out[t] += lin(w[name + "down"], z * torch.sigmoid(z) * lin(w[name + "up"], x[None]))[0]
    return out


def forward(config: Mapping, w: Mapping[str, torch.Tensor], tokens, dtype=torch.float64,
            streams: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    w = {name: (tensor.to(dtype) if tensor.is_floating_point() else tensor) for name, tensor in w.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][tokens] + w["pos"][:T]
    x = one_plus_norm(x, w["embed.norm"], eps)
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        h = one_plus_norm(x, w[prefix + "norm1"], eps)
        delta = differential_attention(h, w, prefix + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                delta = delta + dense_feed_forward(h, w, prefix + "mlp.", mlp)
            else:
                delta = delta + routed_feed_forward(h, w, prefix + "mlp.", mlp)
        x = x + delta
        if streams is not None:
            streams.append(x.clone())
    logits = lin(w["embed"], one_plus_norm(x, w["final.norm"], eps))
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits
