"""Sanozen on the GPU against the plain implementation (tests/plain_sanozen.py, float64, whole sequences):
whole prompts, prompts then token-by-token decoding across page borders, portions down to two tokens, batches of
unequal requests against each alone, slots and pages that are used again, a far key that must carry the result,
the recurrence's state over long decoding, and greedy generation through `Engine.generate` and the command line.
Weights and configurations are the tests' own (tests/sanozen_configs.py)."""
import json

import numpy as np
import pytest
import torch

import plain_sanozen
import sanozen_configs

pytestmark = pytest.mark.gpu

# Bounds on a request's logits (the models' logits reach 15 to 30): the largest difference relative to the largest
# logit, and the root mean square of the differences relative to that of the logits. Measured on a B200: 32-bit
# 5e-6 / 2e-6; bfloat16, where six layers of these weights add up rounding, up to 0.10 / 0.025 (the same with
# every product on the 32-bit kernel, so it is the activations' rounding, not a kernel's).
# Sharp scores (the far-key test) amplify the bfloat16 rounding to 0.44 / 0.10. What a fault costs is of order one
# in either precision, and the 32-bit engine runs the same kernels' code with the tight bound.
BOUND = {"float32": 2e-5, "bfloat16": 0.15}
LARGEST = {"float32": 8e-5, "bfloat16": 0.6}
GREEDY = {"float32": 2e-5, "bfloat16": 0.08}      # two logits closer than this (relative to the largest) may swap


def make(name, dtype, seed=1, max_tokens=2048, config=None, tensors=None):
    from kidi_b200 import Engine
    config = config or sanozen_configs.ALL[name]
    tensors = tensors or sanozen_configs.tensors(config, seed)
    engine = Engine.from_config(config, tensors=tensors, dtype=dtype, max_tokens=max_tokens)
    return engine, config, tensors


def prompt(config, length, seed):
    return np.random.default_rng(seed).integers(0, config["vocab"], size=length).tolist()


def plain(config, tensors, tokens):
    return plain_sanozen.forward(config, tensors, tokens, dtype=torch.float64)


def run(engine, slot, tokens, want=None):
    from kidi_b200 import StepBatch
    want = list(range(len(tokens))) if want is None else want
    return engine.step(StepBatch([slot], [list(tokens)], [want])).double().cpu()


def close(got, want, dtype, record=None, what="", slack=1.0):
    scale = float(want.abs().max())
    worst = float((got - want).abs().max()) / scale
    mean = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
    if record is not None:
        record(f"largest and mean relative difference {what}".strip(), (worst, mean))
    assert worst < slack * LARGEST[dtype] and mean < slack * BOUND[dtype], (what, worst, mean, scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(sanozen_configs.ALL))
def test_whole_prompts_and_decoding(name, dtype, record_property):
    """A whole prompt in one step (its first tokens included), then the same request with its last 70 tokens one
    by one (past a page border of the cache), then in portions of 2, 3, 64 and 61 tokens."""
    engine, config, tensors = make(name, dtype)
    tokens = prompt(config, 150, 11)
    want = plain(config, tensors, tokens)
    assert float(want.abs().max()) > 5
    slot = engine.acquire()
    close(run(engine, slot, tokens), want, dtype, record_property, "whole")
    engine.release(slot)
    slot = engine.acquire()
    rows = [run(engine, slot, tokens[:80])] + [run(engine, slot, [token]) for token in tokens[80:]]
    close(torch.cat(rows), want, dtype, record_property, "decoded")
    engine.release(slot)
    slot = engine.acquire()
    rows, at = [], 0
    for size in (2, 3, 64, 61, 2, 1, 17):
        rows.append(run(engine, slot, tokens[at:at + size]))
        at += size
    assert at == len(tokens)
    close(torch.cat(rows), want, dtype, record_property, "portions")
    engine.release(slot)
    engine.cache.check()
    engine.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small_b", "wide"])
def test_batches_of_unequal_requests(name, dtype, record_property):
    """Requests of 1, 70 and 131 tokens start together and are decoded together; the shortest ends first. Every
    request's logits equal those it gets alone; slots and pages that were given back are used again."""
    from kidi_b200 import StepBatch
    engine, config, tensors = make(name, dtype, seed=2, max_tokens=1024)
    # a request that ran before leaves state, keys and pages behind
    slot = engine.acquire()
    run(engine, slot, prompt(config, 200, 3))
    engine.release(slot)
    requests = [prompt(config, n, 20 + n) for n in (9, 78, 139)]
    starts = [1, 70, 131]
    steps = [8, 8, 8]
    want = [plain(config, tensors, tokens) for tokens in requests]
    slots = [engine.acquire() for _ in requests]
    got = [[] for _ in requests]
    logits = engine.step(StepBatch(slots, [r[:s] for r, s in zip(requests, starts)],
                                   [list(range(s)) for s in starts])).double().cpu()
    at = 0
    for i, s in enumerate(starts):
        got[i].append(logits[at:at + s])
        at += s
    live = [0, 1, 2]
    for step in range(8):
        logits = engine.step(StepBatch([slots[i] for i in live], [[requests[i][starts[i] + step]] for i in live],
                                       [[0] for _ in live])).double().cpu()
        for row, i in enumerate(live):
            got[i].append(logits[row:row + 1])
        if step == 3:                       # one request leaves, and a new one takes its slot at once
            engine.release(slots[0])
            live = [1, 2]
            other = engine.acquire()
            assert other == slots[0]
            fresh = prompt(config, 66, 77)
            close(run(engine, other, fresh), plain(config, tensors, fresh), dtype, None, "a reused slot")
            engine.release(other)
    for i in range(3):
        found = torch.cat(got[i])
        close(found, want[i][:found.shape[0]], dtype, record_property, f"request {i} in a batch")
    engine.cache.check()


def test_batches_do_not_change_32_bit_logits():
    """In 32-bit a request's logits are the same bits alone and in a batch, whole and decoded in steps of one."""
    from kidi_b200 import StepBatch
    engine, config, tensors = make("small_a", "float32", seed=4)
    a, b = prompt(config, 90, 1), prompt(config, 33, 2)
    sa, sb = engine.acquire(), engine.acquire()
    both = engine.step(StepBatch([sa, sb], [a, b], [list(range(90)), list(range(33))])).cpu()
    engine.release(sa), engine.release(sb)
    slot = engine.acquire()
    alone = run(engine, slot, a).float()
    engine.release(slot)
    assert torch.equal(both[:90].double(), alone.double())


@pytest.mark.parametrize("rot_dim,rank", [(8, 32), (16, 48)])     # the second: widths the tensor-core kernels take
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_carries_the_result(dtype, rot_dim, rank, record_property):
    """One latent-attention layer whose query and key maps are made so that the last token's score against one key
    far back (past several pages) stands out by a wide margin: the result then is that key's value, and a key one
    place off would show. The same holds when the last token is decoded alone."""
    config = sanozen_configs.model(64, 64, 1.0, 1e-5, 4, [
        sanozen_configs.latent(2, 16, rot_dim, 16, 16, rank, 1.0, 10000.0, 8, ff=64)])
    tensors = sanozen_configs.tensors(config, 5)
    tensors["l0.mix.uq"] = (tensors["l0.mix.uq"].float() * 4).to(torch.bfloat16)      # sharp scores
    tensors["l0.mix.uk"] = (tensors["l0.mix.uk"].float() * 4).to(torch.bfloat16)
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    for length, seed in ((200, 1), (321, 2), (449, 3)):
        tokens = prompt(config, length, seed)
        want = plain(config, tensors, tokens)
        slot = engine.acquire()
        whole = run(engine, slot, tokens)
        engine.release(slot)
        close(whole, want, dtype, record_property, f"whole {length}", slack=2.0)    # sharp scores amplify rounding
        slot = engine.acquire()
        run(engine, slot, tokens[:-1], want=[])
        last = run(engine, slot, tokens[-1:])
        engine.release(slot)
        close(last, want[-1:], dtype, record_property, f"decoded {length}", slack=2.0)
    # the scores are sharp indeed: the plain model's largest attention weight of the last rows is near one
    h = plain_sanozen.layer_norm(tensors["embed"].double()[tokens], tensors["l0.norm1"], tensors["l0.norm1.b"], 1e-5)
    mixer = config["layers"][0]["mixer"]
    positions = torch.arange(len(tokens))
    c, shared = plain_sanozen.latent_keys(h, {k: v.double() for k, v in tensors.items()}, "l0.mix.", mixer, 1e-5, positions)
    cq = plain_sanozen.rms(plain_sanozen.lin(tensors["l0.mix.dq"].double(), h), 1e-5) * tensors["l0.mix.dq.norm"].double()
    q = plain_sanozen.lin(tensors["l0.mix.uq"].double(), cq).reshape(len(tokens), 2, 16 + rot_dim)
    k = plain_sanozen.lin(tensors["l0.mix.uk"].double(), c).reshape(len(tokens), 2, 16)
    q_turned = plain_sanozen.rotate_interleaved(q[..., 16:], positions, 10000.0, 8)
    scores = torch.einsum("hd,uhd->hu", q[-1, :, :16], k) + torch.einsum("hd,ud->hu", q_turned[-1], shared)
    weights = torch.softmax(scores, -1)
    assert float(weights.max(-1).values.min()) > 0.5 and int(weights.argmax(-1).min()) < len(tokens) - 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_recurrence_keeps_its_state_over_long_decoding(dtype, record_property):
    """A model of recurrent layers only, with forget gates near one (a long memory): 300 tokens decoded one by one
    after a prompt of three still see what the first tokens wrote."""
    config = sanozen_configs.model(50, 48, 2.0, 1e-5, 4, [
        sanozen_configs.recurrent(2, 16, 24, ff=64), sanozen_configs.recurrent(3, 8, 8)])
    tensors = sanozen_configs.tensors(config, 6)
    for layer in ("l0", "l1"):
        tensors[layer + ".mix.f.b"] = (tensors[layer + ".mix.f.b"].float() + 6).to(torch.bfloat16)
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    tokens = prompt(config, 303, 9)
    want = plain(config, tensors, tokens)
    changed = plain(config, tensors, [(tokens[0] + 1) % 50] + tokens[1:])
    assert float((want[-1] - changed[-1]).abs().max()) > 10 * LARGEST["float32"] * float(want.abs().max())   # a long memory
    slot = engine.acquire()
    rows = [run(engine, slot, tokens[:3])] + [run(engine, slot, [token]) for token in tokens[3:]]
    engine.release(slot)
    close(torch.cat(rows), want, dtype, record_property, "long decoding")
    # a slot that is handed out again starts from a zero state
    slot = engine.acquire()
    close(run(engine, slot, tokens[:40]), want[:40], dtype, None, "after reuse")
    engine.release(slot)


def teacher_forced(config, tensors, request, tokens, bound):
    logits = plain(config, tensors, list(request) + list(tokens))[len(request) - 1:-1].numpy()
    close_calls = 0
    for place, token in enumerate(tokens):
        row = logits[place]
        best, second = np.sort(row)[-1], np.sort(row)[-2]
        margin = bound * float(np.abs(row).max())
        if best - second >= margin:
            assert token == int(np.argmax(row)), (request, tokens, place)
        else:
            close_calls += 1
            assert row[token] >= best - margin
    return close_calls


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("use_graph", [True, False])
def test_greedy_generation_through_the_engine(dtype, use_graph):
    """`Engine.generate`: batches of unequal prompts, decode steps replayed as a captured graph (with padding rows:
    three live sequences in four rows), slots reused by the next batch."""
    engine, config, tensors = make("small_b", dtype, seed=7, max_tokens=1024)
    requests = [prompt(config, n, 40 + n) for n in (5, 1, 70, 12, 33)]
    found = engine.generate(requests, max_new_tokens=12, ignore_eos=True, max_active=3, use_graph=use_graph)
    close_calls = sum(teacher_forced(config, tensors, r, t, GREEDY[dtype]) for r, t in zip(requests, found))
    assert all(len(tokens) == 12 for tokens in found) and close_calls <= 20
    again = engine.generate(requests[:2], max_new_tokens=12, ignore_eos=True, use_graph=use_graph)
    if dtype == "float32":
        assert again == found[:2]
    engine.cache.check()
    assert not engine.cache.slots.held
    engine.check_device_errors()


def test_the_command_line_generates(tmp_path, capsys):
    import kidi_b200
    from kidi_b200.weights.safetensors_io import write_safetensors
    config = sanozen_configs.SMALL_A
    tensors = sanozen_configs.tensors(config, 8)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(str(folder / "model.safetensors"), tensors, metadata={"format": "pt"})
    requests = [prompt(config, n, n) for n in (4, 19)]
    (tmp_path / "in.jsonl").write_text("".join(json.dumps({"token_ids": r, "id": str(i)}) + "\n"
                                              for i, r in enumerate(requests)))
    code = kidi_b200.main(["generate", "-m", str(folder), "-i", str(tmp_path / "in.jsonl"), "-o",
                           str(tmp_path / "out.jsonl"), "--max-new-tokens", "6", "--ignore-eos", "--precision", "fp32"])
    assert code == 0, capsys.readouterr().err
    records = [json.loads(line) for line in (tmp_path / "out.jsonl").read_text().splitlines()]
    assert len(records) == 2
    for record in records:
        request = requests[int(record["id"])]
        assert teacher_forced(config, tensors, request, record["token_ids"], LARGEST["float32"]) == 0


def test_which_kernels_run(record_property):
    """bfloat16 prompts from position 0 take the unfolded form (keys and values per head through the tensor-core
    prompt kernels: tcgen05 where a head's plain and rotated widths add up to 64 or 128); decoding, later portions
    and the 32-bit engine take the folded form over the cached latents. Both forms agree within rounding."""
    from kidi_b200 import StepBatch
    from kidi_b200.kernels import ops
    engine, config, tensors = make("wide", "bfloat16", seed=3)
    tokens = prompt(config, 200, 5)
    slot = engine.acquire()
    with ops.record_launches() as names:
        whole = run(engine, slot, tokens)
    engine.release(slot)
    assert names.count("latent_pack") == 3 and names.count("latent_gather") == 1 and "latent_attention" not in names
    assert names.count("attention_prefill_tcgen05") == 2 and names.count("attention_prefill[mma.sync]") == 1
    assert names.count("gated_recurrence[gates apart]") == 2 and names.count("add_layernorm") == 5 + 3 + 1
    slot = engine.acquire()
    run(engine, slot, tokens[:1], want=[])
    with ops.record_launches() as names:
        rest = run(engine, slot, tokens[1:])          # continues a cached sequence: the folded form
    with ops.record_launches() as decode_names:
        engine.step(StepBatch([slot], [[7]], None))
    engine.release(slot)
    folded = [name for name in names if name.startswith("latent_attention[mma.sync")]
    assert len(folded) == 3 and "latent_pack" not in names and "latent_attention" not in names
    assert len([name for name in decode_names if name.startswith("latent_attention[mma.sync")]) == 3
    assert decode_names.count("gated_recurrence") == 2
    difference = float((rest - whole[1:]).pow(2).mean().sqrt() / whole.pow(2).mean().sqrt())
    record_property("folded against unfolded, mean relative difference", difference)
    assert difference < 0.05
    engine32, _, _ = make("wide", "float32", seed=3)
    slot = engine32.acquire()
    with ops.record_launches() as names:
        run(engine32, slot, tokens)
    assert names.count("latent_attention") == 3 and "latent_pack" not in names and "library_mm" not in names
    assert not any("tcgen05" in name or "skinny" in name for name in names)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_heads_and_wide_states(dtype, record_property):
    """Twenty heads (two tiles of sixteen for the tensor-core folded kernel, the second partly filled) over a cached
    latent, and recurrent heads of 160 state rows (more than a warp's slice of 16 rows at 8 warps) by 40 columns
    (no multiple of a block's 32 or 16)."""
    config = sanozen_configs.model(80, 96, 2.0, 1e-5, 8, [
        sanozen_configs.latent(20, 16, 16, 8, 24, 32, 0.3, 20000.0, 16, ff=128),
        sanozen_configs.recurrent(2, 160, 40),
        sanozen_configs.latent(20, 16, 16, 24, 24, 32, 0.3, 20000.0, 16, kv_from=0)])
    tensors = sanozen_configs.tensors(config, 12)
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    tokens = prompt(config, 140, 13)
    want = plain(config, tensors, tokens)
    slot = engine.acquire()
    rows = [run(engine, slot, tokens[:70])] + [run(engine, slot, tokens[70:75])] + \
           [run(engine, slot, [token]) for token in tokens[75:]]
    engine.release(slot)
    close(torch.cat(rows), want, dtype, record_property, "many heads")
