"""Random Sanozen configurations (sizes that are no round numbers, every layer order that the draw gives, borrowed
latents wherever a layer of equal geometry came before) through the engine in both precisions against the plain
implementation: a whole prompt, then eight tokens decoded one by one. Two of the draws run prompts of more than
1,024 tokens, so that the products of prompts take their tensor-memory kernel at these sizes."""
import numpy as np
import pytest
import torch

import plain_sanozen
import sanozen_configs

pytestmark = pytest.mark.gpu

DRAWS = 8


def draw(seed):
    rng = np.random.default_rng(1000 + seed)
    pick = lambda values: int(rng.choice(values))
    width = 8 * pick(range(5, 26)) + pick([0, 0, 4])
    geometries = [dict(kv_rank=pick([16, 24, 32, 40, 48, 64, 80]), rot_dim=pick([8, 16, 32]), base=float(pick([500, 10000, 1000000])))
                  for _ in range(2)]
    for geometry in geometries:
        geometry["dims"] = pick([d for d in (4, 8, 16, 32) if d <= geometry["rot_dim"]])
    layers, owners = [], {}
    for index in range(pick([2, 3, 4, 5])):
        ff = pick([0, 72, 100, 136, 256])
        if rng.random() < 0.6:
            which = pick([0, 1])
            g = geometries[which]
            source = owners.get(which) if rng.random() < 0.6 else None
            layers.append(sanozen_configs.latent(pick([1, 2, 3, 4, 6]), pick([8, 16, 24, 32, 48]), g["rot_dim"],
                                                 pick([8, 16, 24, 32, 40, 64]), pick([12, 16, 24, 32, 56]), g["kv_rank"],
                                                 float(rng.uniform(0.1, 0.4)), g["base"], g["dims"], ff=ff or None,
                                                 kv_from=source))
            if source is None:
                owners.setdefault(which, index)
        else:
            layers.append(sanozen_configs.recurrent(pick([1, 2, 3, 5]), pick([4, 8, 12, 16, 40, 64]),
                                                    pick([8, 12, 16, 24, 32, 48, 72]), ff=ff or None))
    return sanozen_configs.model(pick(range(61, 400)), width, float(rng.uniform(0.5, 12)), float(rng.choice([1e-6, 1e-5, 3e-5])),
                                 pick([3, 4, 8, 12, 16, 24]), layers)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(DRAWS))
def test_random_configuration(seed, dtype, record_property):
    from kidi_b200 import Engine, StepBatch
    config = draw(seed)
    tensors = sanozen_configs.tensors(config, 50 + seed)
    length = 1100 if seed in (2, 5) else 40 + 23 * seed
    tokens = np.random.default_rng(seed).integers(0, config["vocab"], size=length + 8).tolist()
    want = plain_sanozen.forward(config, tensors, tokens, dtype=torch.float64)
    engine = Engine.from_config(config, tensors=tensors, dtype=dtype, max_tokens=2048)
    slot = engine.acquire()
    rows = [engine.step(StepBatch([slot], [tokens[:length]], [list(range(length))])).double().cpu()]
    rows += [engine.step(StepBatch([slot], [[token]], None)).double().cpu() for token in tokens[length:]]
    engine.release(slot)
    engine.check_device_errors()
    got = torch.cat(rows)
    largest = float((got - want).abs().max() / want.abs().max())
    mean = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
    record_property("largest and mean relative difference", (largest, mean))
    assert largest < (1e-4 if dtype == "float32" else 0.6) and mean < (2e-5 if dtype == "float32" else 0.15), \
        (config, largest, mean)
