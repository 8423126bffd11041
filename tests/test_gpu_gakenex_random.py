"""Random Gakenex configurations (sizes that are no round numbers, one to eight heads a key/value head, map and value
widths with and without the tensor-core kernels' multiples of 16, none to four taps, windows from 3 to 300 tokens with
none to 90 kept tokens or no window, dense, routed and absent feed-forwards in every order that the draw gives)
through the engine in both precisions against the plain implementation: a prompt in two portions, then eight tokens
decoded one by one. Two of the draws run prompts of more than 1,024 tokens, so that the products of prompts take
their tensor-memory kernel at these sizes and the windows pass over many pages."""
import numpy as np
import pytest
import torch

import gakenex_configs
import plain_gakenex

pytestmark = pytest.mark.gpu

DRAWS = 10


def draw(seed):
    rng = np.random.default_rng(2000 + seed)
    pick = lambda values: int(rng.choice(values))
    width = 8 * pick(range(5, 26)) + pick([0, 0, 4])
    layers = []
    for _ in range(pick([1, 2, 3, 4, 5])):
        groups = pick([1, 1, 2, 3])
        heads = groups * pick([1, 2, 3, 4, 8])
        if rng.random() < 0.5:
            dim, vdim = pick([16, 32, 48, 64]), pick([16, 32, 48, 80, 96])       # widths of the tensor-core kernels
        else:
            dim, vdim = pick([4, 8, 12, 20, 24, 40]), pick([8, 12, 16, 24, 36, 72])
        window = pick([3, 17, 64, 65, 100, 128, 300]) if rng.random() < 0.75 else None
        keep = pick([0, 1, 4, 7, 64, 90]) if window is not None else 0
        kind = rng.random()
        if kind < 0.4:
            mlp = gakenex_configs.dense(pick([40, 72, 100, 136, 256]), float(rng.uniform(0.5, 4.0)))
        elif kind < 0.85:
            experts = pick([2, 3, 5, 8, 12])
            mlp = gakenex_configs.routed(experts, pick([t for t in (1, 2, 3) if t <= experts]), pick([8, 24, 40, 64]))
        else:
            mlp = None
        layers.append(gakenex_configs.attention(heads, groups, dim, vdim, pick([0, 1, 2, 3, 4]), float(rng.uniform(0.1, 0.9)),
                                                float(rng.uniform(0.1, 0.5)), window=window, keep_first=keep, mlp=mlp))
    return gakenex_configs.model(pick(range(61, 400)), width, 1536, float(rng.choice([1e-6, 1e-5, 3e-5])),
                                 float(rng.choice([0.0, 10.0, 25.0])), layers)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(DRAWS))
def test_random_configuration(seed, dtype, record_property):
    from kidi_b200 import Engine, StepBatch
    config = draw(seed)
    tensors = gakenex_configs.tensors(config, 50 + seed)
    length = 1100 if seed in (2, 5) else 60 + 31 * seed
    tokens = np.random.default_rng(seed).integers(0, config["vocab"], size=length + 8).tolist()
    want = plain_gakenex.forward(config, tensors, tokens, dtype=torch.float64)
    engine = Engine.from_config(config, tensors=tensors, dtype=dtype, max_tokens=2048)
    slot = engine.acquire()
    cut = length // 3
    rows = [engine.step(StepBatch([slot], [tokens[:cut]], [list(range(cut))])).double().cpu(),
            engine.step(StepBatch([slot], [tokens[cut:length]], [list(range(length - cut))])).double().cpu()]
    rows += [engine.step(StepBatch([slot], [[token]], None)).double().cpu() for token in tokens[length:]]
    engine.release(slot)
    engine.check_device_errors()
    got = torch.cat(rows)
    assert torch.isfinite(got).all()
    # one row in forty may take another expert in bfloat16 (a router's close call): the bounds hold for the others
    worst_rows = (got - want).abs().max(-1).values / want.abs().max()
    spared = 0 if dtype == "float32" else max(1, got.shape[0] // 40)
    kept = torch.argsort(worst_rows)[:got.shape[0] - spared]
    largest = float(worst_rows[kept].max())
    mean = float((got[kept] - want[kept]).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
    record_property("largest and mean relative difference", (largest, mean))
    assert largest < (1e-4 if dtype == "float32" else 0.4) and mean < (2e-5 if dtype == "float32" else 0.08), \
        (config, largest, mean)
