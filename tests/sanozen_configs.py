"""Small Sanozen configurations and random weights for them, made by the tests themselves.

The configurations differ in every size and constant: heads from 1 to 5, plain, rotated and value widths that
are all different (and one layer where they are equal), rotations that turn only part of the rotated width,
layers in several orders, borrowed latents from adjacent and from distant layers, with and without
feed-forwards. `tensors(config, seed)` draws every tensor under its checkpoint name.
"""
import torch


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims, ff=None, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale, "rot": {"base": base, "dims": dims}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def recurrent(heads, dim, vdim, ff=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def model(vocab, width, scale, eps, side, layers):
    return {"architecture": "Sanozen", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "token_side": {"dim": side}, "layers": layers}


# attention first, a borrowed latent right behind its source, a recurrence last; only half of the rotated width turns
SMALL_A = model(97, 64, 4.0, 1e-5, 8, [
    latent(2, 16, 16, 24, 24, 40, 0.2, 10000.0, 8, ff=96),
    latent(4, 8, 16, 12, 16, 40, 0.35, 10000.0, 8, kv_from=0),
    recurrent(3, 8, 16, ff=80),
    recurrent(1, 24, 40),
])

# a recurrence first; one head; two latents of different geometry, each borrowed once, one from far back; odd sizes
SMALL_B = model(131, 72, 1.0, 3e-6, 5, [
    recurrent(2, 12, 20),
    latent(1, 24, 8, 40, 20, 56, 0.18, 500.0, 8, ff=100),
    latent(3, 8, 24, 16, 36, 24, 0.25, 1000000.0, 24),
    recurrent(5, 4, 8, ff=64),
    latent(2, 16, 8, 8, 12, 56, 0.3, 500.0, 8, kv_from=1),
    latent(5, 8, 24, 8, 28, 24, 0.22, 1000000.0, 24, ff=72, kv_from=2),
])

# wider: the plain and rotated widths of a head add up to 64 and to 128, the widths of the tcgen05 prompt kernel,
# and to 80 (the mma.sync one), with values narrower than, and as wide as, the keys; sharper scores
WIDE = model(211, 256, 8.0, 1e-5, 16, [
    latent(4, 32, 32, 48, 64, 96, 0.6, 10000.0, 32, ff=320),
    recurrent(2, 64, 64),
    latent(2, 96, 32, 128, 48, 96, 0.5, 10000.0, 32, ff=256, kv_from=0),
    latent(3, 64, 16, 64, 40, 160, 0.7, 300000.0, 16),
    recurrent(4, 32, 48, ff=192),
])

ALL = {"small_a": SMALL_A, "small_b": SMALL_B, "wide": WIDE}


def tensors(config, seed, logit_scale=6.0):
    """Every tensor of a model of `config`, bfloat16, under its checkpoint name."""
    generator = torch.Generator().manual_seed(seed)
    width, vocab, side = config["width"], config["vocab"], config["token_side"]["dim"]
    count = len(config["layers"])

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=generator) * std + mean).to(torch.bfloat16)

    def matrix(out, inner, gain=1.0):
        return normal(out, inner, std=gain / inner ** 0.5)

    out = {"embed": normal(vocab, width, std=0.06), "side.embed": normal(vocab, count * side),
           "final.norm": normal(width, std=0.1 * logit_scale, mean=logit_scale), "final.norm.b": normal(width, std=0.1),
           "head": matrix(vocab, width)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        norms = ["norm1"] + (["norm2"] if layer["mlp"] else [])
        for name in norms:
            out[p + name] = normal(width, std=0.2, mean=1.0)
            out[p + name + ".b"] = normal(width, std=0.1)
        if layer["type"] == "latent_attention":
            heads, dim, rot, vdim = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            out[p + "mix.dq"] = matrix(m["q_rank"], width)
            out[p + "mix.dq.norm"] = normal(m["q_rank"], std=0.2, mean=1.0)
            out[p + "mix.uq"] = matrix(heads * (dim + rot), m["q_rank"], 2.0)
            if "kv_from" not in m:
                out[p + "mix.dkv"] = matrix(m["kv_rank"] + rot, width, 2.0)
                out[p + "mix.dkv.norm"] = normal(m["kv_rank"], std=0.2, mean=1.0)
            out[p + "mix.uk"] = matrix(heads * dim, m["kv_rank"], 2.0)
            out[p + "mix.uv"] = matrix(heads * vdim, m["kv_rank"])
            out[p + "mix.o"] = matrix(width, heads * vdim)
        else:
            heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
            out[p + "mix.q"] = matrix(heads * dim, width)
            out[p + "mix.f"] = matrix(heads * dim, width, 2.0)
            out[p + "mix.f.b"] = normal(heads * dim, std=1.5, mean=1.0)
            out[p + "mix.lower"] = (torch.rand(heads * dim, generator=generator) * 0.9).to(torch.bfloat16)
            out[p + "mix.v"] = matrix(heads * vdim, width)
            out[p + "mix.norm"] = normal(vdim, std=0.2, mean=1.0)
            out[p + "mix.o"] = matrix(width, heads * vdim)
        if layer["mlp"]:
            out[p + "mlp.up"] = matrix(layer["mlp"]["ff"], width)
            out[p + "mlp.down"] = matrix(width, layer["mlp"]["ff"])
            out[p + "mlp.act"] = normal(4, std=0.4, mean=0.4)
        out[p + "side.gate"] = matrix(side, width)
        out[p + "side.proj"] = matrix(width, side)
        out[p + "side.norm"] = normal(width, std=0.2, mean=0.5)
        mix = torch.randn(i + 2, generator=generator) * 0.3
        mix[-1] += 1.0
        out[p + "dwa"] = mix.to(torch.bfloat16)
    return out
