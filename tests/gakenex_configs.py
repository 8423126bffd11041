"""Small Gakenex configurations and random weights for them, made by the tests themselves.

The configurations differ in every size and constant: one to eight query heads a key/value head, map and value
widths that are equal, smaller and larger than one another, one to four convolution taps, windows shorter and
longer than a cache page with none to seventy kept first tokens (and no window at all), dense, routed and absent
feed-forwards in several orders, one to three experts a token (also all of them). `tensors(config, seed)` draws
every tensor under its checkpoint name.
"""
import torch


def attention(heads, kv_heads, dim, vdim, conv, diff, scale, window=None, keep_first=0, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale}
    if conv:
        mixer["conv"] = conv
    if window is not None:
        mixer["mask"] = {"size": window, "keep_first": keep_first}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def routed(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, positions, eps, softcap, layers):
    config = {"architecture": "Gakenex", "vocab": vocab, "width": width, "max_positions": positions,
              "norm": {"eps": eps}, "layers": layers}
    if softcap:
        config["logit_softcap"] = softcap
    return config


# a dense layer, a routed one without a window (two experts a token), a layer without convolution and feed-forward
SMALL_A = model(97, 64, 512, 1e-5, 20.0, [
    attention(2, 1, 16, 32, 4, 0.5, 0.3, window=40, keep_first=3, mlp=dense(96, 1.5)),
    attention(4, 4, 8, 8, 2, 0.3, 0.4, mlp=routed(6, 2, 24)),
    attention(3, 1, 24, 16, 0, 0.7, 0.25, window=70, keep_first=0),
])

# a routed layer first; widths that are no multiples of 16; a window shorter than a page with kept tokens, and one
# longer than a page that keeps more than a page; every expert taken; no bound on the logits; odd sizes
SMALL_B = model(131, 72, 700, 3e-6, 0.0, [
    attention(6, 2, 12, 20, 3, 0.4, 0.3, window=17, keep_first=5, mlp=routed(5, 1, 20)),
    attention(2, 2, 16, 16, 2, 0.2, 0.35, window=200, keep_first=70, mlp=dense(100, 3.0)),
    attention(1, 1, 40, 24, 1, 0.6, 0.2, window=64, keep_first=1, mlp=routed(3, 3, 16)),     # one tap: a weight a channel
    attention(5, 1, 8, 12, 9, 0.8, 0.5, mlp=dense(64, 0.7)),                                  # nine taps
])

# widths that the tensor-core kernels take: groups of 2, 8, 1 and 3 heads, maps of 32, 64, 128 and 16
WIDE = model(211, 256, 1024, 1e-5, 12.0, [
    attention(4, 2, 32, 64, 3, 0.6, 0.3, window=100, keep_first=2, mlp=routed(8, 2, 64)),
    attention(8, 1, 64, 32, 4, 0.5, 0.2, window=150, keep_first=66, mlp=dense(320, 2.0)),
    attention(2, 2, 128, 128, 2, 0.3, 0.15),
    attention(3, 1, 16, 48, 3, 0.7, 0.4, window=64, keep_first=0, mlp=routed(4, 1, 96)),
])

ALL = {"small_a": SMALL_A, "small_b": SMALL_B, "wide": WIDE}


def tensors(config, seed, logit_scale=5.0, sharp=1.0):
    """Every tensor of a model of `config`, bfloat16, under its checkpoint name. `sharp` multiplies the query
    norms' weights (sharper scores)."""
    generator = torch.Generator().manual_seed(seed)
    width, vocab = config["width"], config["vocab"]

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=generator) * std + mean).to(torch.bfloat16)

    def matrix(out, inner, gain=1.0):
        return normal(out, inner, std=gain / inner ** 0.5)

    out = {"embed": normal(vocab, width, std=0.08), "pos": normal(config["max_positions"], width, std=0.04),
           "embed.norm": normal(width, std=0.2), "final.norm": normal(width, std=0.1 * logit_scale, mean=logit_scale - 1)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        heads, groups, dim, vdim, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv", 0)
        out[p + "norm1"] = normal(width, std=0.2)
        for name, rows in (("q", heads * 2 * dim), ("k", groups * 2 * dim), ("v", groups * vdim)):
            out[p + "mix." + name] = matrix(rows, width, 1.5)
            if taps >= 1:
                out[p + "mix." + name + ".conv"] = normal(rows, taps, std=0.5, mean=0.3)
        out[p + "mix.q.norm"] = normal(dim, std=0.2 * sharp, mean=1.0 * sharp)
        out[p + "mix.k.norm"] = normal(dim, std=0.2, mean=1.0)
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[p + "mix." + name] = normal(dim, std=0.3)
        out[p + "mix.g"] = matrix(heads * vdim, width, 2.0)
        out[p + "mix.o"] = matrix(width, heads * vdim)
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            out[p + "mlp.gate"] = matrix(mlp["ff"], width, 2.0)
            out[p + "mlp.up"] = matrix(mlp["ff"], width, 2.0)
            out[p + "mlp.down"] = matrix(width, mlp["ff"])
        elif mlp:
            out[p + "mlp.router"] = matrix(mlp["router"]["experts"], width, 3.0)
            for e in range(mlp["router"]["experts"]):
                out[p + f"mlp.e{e}.gate"] = matrix(mlp["expert"]["ff"], width, 2.0)
                out[p + f"mlp.e{e}.up"] = matrix(mlp["expert"]["ff"], width, 2.0)
                out[p + f"mlp.e{e}.down"] = matrix(width, mlp["expert"]["ff"], 2.0)
    return out
