"""Gakenex without a GPU: its typed configuration, the registry, the tensors its parts declare, a random model
folder through the command line, and the plain implementation's mechanisms against closed forms."""
import copy
import json

import pytest
import torch

import gakenex_configs
import plain_gakenex


def test_the_configuration_round_trips_and_is_chosen_by_its_name():
    from kidi_b200.config.gakenex import GakenexConfig
    from kidi_b200.registry import registered_architectures, resolve_architecture
    assert "Gakenex" in registered_architectures()
    for config in gakenex_configs.ALL.values():
        assert resolve_architecture(config).config_type is GakenexConfig
        typed = GakenexConfig.from_dict(config)
        assert typed.to_dict() == config
        assert GakenexConfig.from_dict(typed.to_dict()) == typed
    typed = GakenexConfig.from_dict(gakenex_configs.SMALL_B)
    first = typed.layers[0]
    assert (first.heads, first.kv_heads, first.dim, first.vdim, first.conv) == (6, 2, 12, 20, 3)
    assert (first.window, first.keep_first, first.mlp.kind, first.mlp.experts, first.mlp.top) == (17, 5, "moe", 5, 1)
    assert typed.layers[3].window is None and typed.layers[3].mlp.limit == 0.7 and typed.logit_softcap == 0.0


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["layers"][0].update(type="recurrence"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "not supported"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.update(vocab="many"), "vocab"),
])
def test_refused_configurations(change, message):
    from kidi_b200.config.gakenex import GakenexConfig
    from kidi_b200.errors import KidiError
    config = copy.deepcopy(gakenex_configs.SMALL_A)
    change(config)
    with pytest.raises(KidiError) as caught:
        GakenexConfig.from_dict(config)
    assert message in str(caught.value)


def test_declared_tensors_are_the_checkpoint_names():
    from kidi_b200.engine.model import declared_parameters
    from kidi_b200.registry import spec_from_config
    for config in gakenex_configs.ALL.values():
        _, _, spec = spec_from_config(config)
        declared = {}
        for prefix, parameter in declared_parameters(spec):
            if parameter.alias_of is not None:
                assert (prefix + parameter.name, parameter.alias_of) == ("head", "embed")
                continue
            for name, shape in (parameter.sources or ((parameter.name, parameter.shape),)):
                declared[prefix + name] = tuple(shape)
        made = {name: tuple(tensor.shape) for name, tensor in gakenex_configs.tensors(config, 1).items()}
        assert declared == made
    _, _, spec = spec_from_config(gakenex_configs.SMALL_A)
    assert [entry.layer for entry in spec.schedule] == [0, 1, 2] and spec.embedding_norm is not None
    assert "feed_forward" not in spec.layers[2].parts and spec.layers[1].parts["feed_forward"].kind == "routed_experts"


def test_a_random_model_folder_through_the_command_line(tmp_path, capsys):
    import kidi_b200
    from kidi_b200.weights.loader import Checkpoint
    (tmp_path / "config.json").write_text(json.dumps(gakenex_configs.SMALL_A))
    assert kidi_b200.main(["random-model", "--config", str(tmp_path / "config.json"), "-o", str(tmp_path / "model"),
                           "--seed", "3"]) == 0, capsys.readouterr().err
    held = Checkpoint(str(tmp_path / "model"))
    assert held.shape("l1.mlp.e5.down") == (64, 24) and held.shape("l0.mix.q.conv") == (64, 4)
    assert "l2.mix.q.conv" not in held and "head" not in held        # a layer without convolution
    held.close()
    assert kidi_b200.main(["inspect", "-m", str(tmp_path / "model")]) == 0
    assert "Gakenex" in capsys.readouterr().out


def test_the_plain_convolution_and_mask():
    u = torch.arange(12, dtype=torch.float64).reshape(6, 2) + 1
    taps = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 2.0]], dtype=torch.float64)
    y = plain_gakenex.short_conv(u, taps)
    assert y[0].tolist() == [100.0, 4.0]                       # zeros before the first token
    assert y[2].tolist() == [1 * 1 + 10 * 3 + 100 * 5, 2 * 6]
    seen = plain_gakenex.visible(8, 3, 2)
    assert seen[7].tolist() == [True, True, False, False, False, True, True, True]
    assert seen[2].tolist() == [True, True, True, False, False, False, False, False]
    assert plain_gakenex.visible(4, None, 0)[3].all()


def test_the_plain_router_weighs_the_input():
    generator = torch.Generator().manual_seed(2)
    w = {"router": torch.tensor([[5.0, 0.0], [-5.0, 0.0], [0.0, 0.1]], dtype=torch.float64)}
    for e in range(3):
        for name, shape in (("gate", (4, 2)), ("up", (4, 2)), ("down", (2, 4))):
            w[f"e{e}.{name}"] = torch.randn(*shape, generator=generator, dtype=torch.float64)
    h = torch.tensor([[1.0, 0.3]], dtype=torch.float64)
    out = plain_gakenex.routed_feed_forward(h, w, "", {"router": {"experts": 3, "top": 1}})
    score = torch.sigmoid(torch.tensor(5.0, dtype=torch.float64))
    x = score * h
    z = x @ w["e0.gate"].t()
    assert torch.allclose(out, (z * torch.sigmoid(z) * (x @ w["e0.up"].t())) @ w["e0.down"].t())
