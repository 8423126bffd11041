"""Sanozen without a GPU: the typed configuration, the registry, the declared tensors, the run order, random
model folders, and the plain implementation against direct restatements of two of its mechanisms."""
import copy
import json
import math
import os

import pytest
import torch

import plain_sanozen
import sanozen_configs
from kidi_b200.config.sanozen import SanozenConfig
from kidi_b200.engine.model import declared_parameters
from kidi_b200.errors import KidiError
from kidi_b200.registry import registered_architectures, resolve_architecture, spec_from_config


@pytest.mark.parametrize("name", sorted(sanozen_configs.ALL))
def test_configuration_round_trip(name):
    config = sanozen_configs.ALL[name]
    typed = SanozenConfig.from_dict(config)
    assert SanozenConfig.from_dict(typed.to_dict()) == typed
    assert typed.to_dict()["layers"] == config["layers"]
    assert len(typed.layers) == len(config["layers"]) and typed.width == config["width"]
    assert typed.embedding_scale == config["embedding"]["scale"] and typed.norm_eps == config["norm"]["eps"]


def test_registry_chooses_by_the_architecture_key():
    assert "Sanozen" in registered_architectures()
    assert resolve_architecture(sanozen_configs.SMALL_A).name == "Sanozen"
    with pytest.raises(KidiError):
        resolve_architecture({"architecture": "NoSuchDesign"})
    with pytest.raises(KidiError):
        resolve_architecture({"architecture": 3})


def broken(change):
    config = copy.deepcopy(sanozen_configs.SMALL_B)
    change(config)
    return config


@pytest.mark.parametrize("change", [
    lambda c: c.pop("vocab"),
    lambda c: c["norm"].pop("eps"),
    lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][1]["mixer"].__setitem__("heads", 0),
    lambda c: c["layers"][0].__setitem__("type", "convolution"),
    lambda c: c["layers"][1]["mlp"].__setitem__("kind", "routed"),
    lambda c: c["layers"][4]["mixer"].__setitem__("kv_from", 4),          # not an earlier layer
    lambda c: c["layers"][4]["mixer"].__setitem__("kv_from", 0),          # not a latent-attention layer
    lambda c: c["layers"][5]["mixer"].__setitem__("kv_from", 4),          # a layer that borrows itself
    lambda c: c["layers"][4]["mixer"].__setitem__("kv_rank", 48),         # differs from its source
    lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 7),
    lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 26),     # more than rot_dim
    lambda c: c.__setitem__("layers", []),
])
def test_invalid_configurations_are_refused(change):
    with pytest.raises(KidiError):
        SanozenConfig.from_dict(broken(change))


@pytest.mark.parametrize("name", sorted(sanozen_configs.ALL))
def test_declared_tensors_are_the_checkpoint_names(name):
    config = sanozen_configs.ALL[name]
    _, _, spec = spec_from_config(config)
    declared = {}
    for prefix, parameter in declared_parameters(spec):
        for source, shape in (parameter.sources or ((parameter.name, parameter.shape),)):
            declared[prefix + source] = tuple(shape)
    made = {key: tuple(value.shape) for key, value in sanozen_configs.tensors(config, 0).items()}
    assert declared == made


def test_run_order_and_borrowed_caches():
    _, _, spec = spec_from_config(sanozen_configs.SMALL_B)
    assert [entry.layer for entry in spec.schedule] == list(range(6))
    assert [entry.cache_from for entry in spec.schedule] == [None, None, None, None, 1, 2]
    kinds = [layer.parts["mixer"].kind for layer in spec.layers]
    assert kinds == ["hgrn2", "latent_attention", "latent_attention", "hgrn2", "latent_attention", "latent_attention"]
    assert [("feed_forward" in layer.parts) for layer in spec.layers] == [False, True, False, True, False, True]
    assert len(spec.positions) == 2          # two different rotations
    offsets = [layer.parts["token_input"].params["offset"] for layer in spec.layers]
    assert offsets == [5 * i for i in range(6)]


def test_random_model_folder(tmp_path):
    import kidi_b200
    from kidi_b200.weights.safetensors_io import SafetensorsFile
    path = tmp_path / "config.json"
    path.write_text(json.dumps(sanozen_configs.SMALL_A))
    out = tmp_path / "model"
    assert kidi_b200.main(["random-model", "--config", str(path), "--seed", "3", "-o", str(out)]) == 0
    assert kidi_b200.main(["inspect", "-m", str(out)]) == 0
    file = SafetensorsFile(os.path.join(out, "model.safetensors"))
    names = set(file.names())
    assert names == set(sanozen_configs.tensors(sanozen_configs.SMALL_A, 0))
    lower = file.tensor("l2.mix.lower").float()
    assert 0 <= float(lower.min()) and float(lower.max()) < 1
    file.close()


# ------------------------------------------------------------- the plain implementation against restatements
def test_plain_rotation_turns_pairs():
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    positions = torch.tensor([0, 1, 2, 7, 100])
    out = plain_sanozen.rotate_interleaved(x, positions, 1000.0, 8)
    assert torch.equal(out[0], x[0]) and torch.equal(out[..., 8:], x[..., 8:])
    for t, p in enumerate(positions.tolist()):
        for i in range(4):
            angle = p * 1000.0 ** (-2 * i / 8)
            u, v = x[t, 1, 2 * i], x[t, 1, 2 * i + 1]
            assert abs(float(out[t, 1, 2 * i]) - float(u * math.cos(angle) - v * math.sin(angle))) < 1e-12
            assert abs(float(out[t, 1, 2 * i + 1]) - float(v * math.cos(angle) + u * math.sin(angle))) < 1e-12


def test_plain_recurrence_in_closed_form():
    """With a constant forget gate f the state is a geometric sum: S_t = (1 - f) sum_s f^(t-s) v_s."""
    mixer = {"heads": 1, "dim": 3, "vdim": 2}
    T, width = 6, 4
    w = {"q": torch.randn(3, width), "f": torch.zeros(3, width), "f.b": torch.tensor([0.3, -1.0, 2.0]),
         "lower": torch.tensor([0.0, 0.5, 0.2]), "v": torch.randn(2, width), "norm": torch.ones(2),
         "o": torch.eye(2)}
    w = {"m." + key: value.double() for key, value in w.items()}
    h = torch.randn(T, width, dtype=torch.float64)
    got = plain_sanozen.hgrn2(h, w, "m.", mixer, 1e-6)
    lower = w["m.lower"]
    f = lower + (1 - lower) * torch.sigmoid(w["m.f.b"])
    q = torch.nn.functional.silu(h @ w["m.q"].t())
    v = h @ w["m.v"].t()
    for t in range(T):
        state = sum((1 - f)[:, None] * f[:, None] ** (t - s) * v[s][None, :] for s in range(t + 1))
        read = state.t() @ q[t]
        want = read / torch.sqrt((read * read).mean() + 1e-6)
        assert torch.allclose(got[t], want, atol=1e-12)
