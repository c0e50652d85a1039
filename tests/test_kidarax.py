"""The Kidarax decoder in the engine against the plain float64 statement of it (``plain_kidarax``).

Small configurations of the tests' own, random weights shaped so that faults show (peaked attention, sinks of the
scores' size, slow decays, norms with slopes and shifts of their own, routers whose scores spread), and every way of
cutting and batching. The same tests run on a CPU with the plain PyTorch statements of the kernels (host logic: pages,
slots, state, the caches of a layer that runs several times) and, marked ``gpu``, with the compiled kernels in float32
and bfloat16. The kernels' new options are also compared one by one with their plain statements.
"""

import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_kidarax as plain
import traces

from tiny_kidarax import (ATT, ATT_FULL, ATT_ODD, CONFIGS, LAT, LAT_ODD, LAT_OPEN, LAT_WIDE, LENGTHS, PAGE, RET, RET_ODD, RET_WIDE,
                          TOL, att, dense, lat, make_folder, model, moe, plant, plant_latent, prompts, ret)

ROOT = Path(__file__).resolve().parent.parent
# A routing margin (the gap between two logits, which are a few units large) below this may fall the other way: in
# bfloat16 through the rounding of the router's input and of the layers before it, in float32 through the order of sums.
CLOSE_CALL = {"float32": 1e-3, "bfloat16": 0.2}


def runner_for(folder, dtype, device, page, max_tokens, ops=None, max_requests=4, context=None, **kw):
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner

    cfg = EngineConfig(dtype=dtype, device=device, page_size=page, max_tokens=max_tokens, max_requests=max_requests,
                       context=context or max_tokens, cuda_graphs=False, **kw)
    return ModelRunner(folder, cfg, ops=ops)


def oracle(config, w, tokens):
    """(logits [T, vocab], margin [T]): the least routing margin of a position over all routed layer runs; where it is
    a close call, the engine may decide the other way (and every later position may feel it through the mixers)."""
    margins = []
    logits = plain.forward(tokens, w, config, margins=margins).numpy()
    least = np.full(len(tokens), np.inf)
    for per_layer in margins:
        least = np.minimum(least, np.asarray(per_layer))
    return logits, least


def compare(got, want, dtype, what):
    for rid, (logits, least) in want.items():
        rows = np.nonzero(least >= CLOSE_CALL[dtype])[0]
        if dtype != "float32":
            error = np.abs(got[rid] - logits).max(axis=-1) / np.abs(logits).max()
            assert np.median(error) <= 0.5 * TOL[dtype], f"{what}: request {rid}: median error {np.median(error):.3g}"
            if len(rows) == 0:
                continue
        bad = traces.first_bad(got[rid][rows], logits[rows], TOL[dtype])
        assert bad is None, (f"{what}: request {rid} first differs at position {rows[bad]} "
                             f"{traces.worst(got[rid][rows], logits[rows])}")


def run_modes(key, dtype, device, ops, tmp_path, modes):
    config = CONFIGS[key]
    folder, w = make_folder(config, seed=31, folder=tmp_path / key)
    reqs = {f"r{i}": p for i, p in enumerate(prompts(config["vocab"], LENGTHS[key], seed=6))}
    want = {rid: oracle(config, w, toks) for rid, toks in reqs.items()}
    page = PAGE[key]
    longest = -(-max(len(t) for t in reqs.values()) // page) * page
    for mode in modes:
        if mode == "mixed":
            steps, peak = traces.mixed(reqs, {rid: max(1, len(t) - 9) for rid, t in reqs.items()}, seed=3, live=3, page=page)
            runner = runner_for(folder, dtype, device, page, peak, ops, max_requests=3, context=longest)
        else:
            steps = getattr(traces, mode)(reqs)
            runner = runner_for(folder, dtype, device, page, longest, ops, max_requests=2)
        got = traces.replay(runner, steps)
        assert not runner.cache.live() and runner.cache.min_free_pages() == runner.cache.num_pages
        compare(got, want, dtype, f"{key}/{dtype}/{mode}")


MODES = ["whole", "tail_decoded", "portions", "mixed"]


@pytest.mark.parametrize("key", list(CONFIGS))
def test_every_way_of_cutting_on_the_plain_operations(key, tmp_path):
    from akas_b200.ops import reference

    run_modes(key, "float32", "cpu", reference, tmp_path, MODES)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(CONFIGS))
def test_every_way_of_cutting_on_the_kernels(key, dtype, tmp_path):
    run_modes(key, dtype, "cuda:0", None, tmp_path, MODES)


def test_config_round_trip_registry_and_inventory(tmp_path):
    from akas_b200.config import ConfigError, KidaraxConfig, config_from_dict, load_config
    from akas_b200.engine.runner import kernel_kinds
    from akas_b200.ops import reference
    from akas_b200.weights.loader import WeightError

    config = config_from_dict(CONFIGS["mix"])
    assert isinstance(config, KidaraxConfig) and config_from_dict(config.to_dict()) == config
    assert config_from_dict(json.loads(json.dumps(config.to_dict()))) == config
    spec = config.model_spec()
    assert [l.mixer.kind for l in spec.layers] == ["decayed_linear_attention", "latent_attention", "attention",
                                                    "decayed_linear_attention", "latent_attention", "attention"]
    # layers 1..3 three times in a row, each run with a cache of its own; the embedding again before passes two and three
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4, 5]
    assert [i for i, e in enumerate(spec.schedule) if e.add_embedding] == [4, 7] and all(e.cache is None for e in spec.schedule)
    assert all(l.arrangement == "sandwich" and l.mixer_post_norm.kind == "dynamic_tanh" for l in spec.layers)
    first, second, third = spec.layers[0], spec.layers[1], spec.layers[2]
    assert first.mixer.decay == (0.9, 0.97, 0.995) and first.mixer.activation is None and not first.mixer.norm_weight
    assert not first.mixer.whole_norm and first.mixer.gate_activation == "silu" and first.mixer.q_scale == 0.25
    assert (first.ffn.scoring, first.ffn.weight_on, first.ffn.renormalize, first.ffn.correction) == ("sigmoid", "input", False, False)
    assert first.ffn.top == 2 and first.ffn.num_experts == 6 and first.ffn.shared_size == 40 and first.ffn.shared_gate
    assert second.mixer.q_rank is None and second.mixer.gate == "head" and second.mixer.sink == "learned" and second.mixer.window is None
    assert second.mixer.position.blend == (6.0, 16.0, 8.0, 0.5) and second.mixer.position.amplitude == pytest.approx(0.1 * math.log(6.0) + 1.0)
    assert second.ffn.kind == "mlp" and second.ffn.activation == "relu2" and second.ffn.intermediate_size == 48
    assert third.mixer.bias and third.mixer.gate == "channel" and not third.mixer.sink and third.mixer.position.linear_factor == 4.0
    assert third.ffn.shared_size is None and spec.layers[3].ffn is None and spec.layers[3].ffn_post_norm is None
    assert spec.head_name is None and spec.logit_scale == 0.7 and spec.final_norm.kind == "dynamic_tanh"
    assert set(kernel_kinds(spec)) == {"attention_general", "latent", "rope", "recurrent", "moe"}
    assert config_from_dict(CONFIGS["alone"]).loop is None and len(config_from_dict(CONFIGS["ragged"]).model_spec().schedule) == 3
    folder, _ = make_folder(CONFIGS["odd"], seed=1, folder=tmp_path / "m")
    assert load_config(folder) == config_from_dict(CONFIGS["odd"])
    for change, message in ((lambda c: c["layers"][2]["mixer"].update(kv_heads=2), "kv_heads"),
                            (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
                            (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 0.5, 1.5, 0.5, 0.5]), "decay"),
                            (lambda c: c["layers"][0]["mixer"].update(rot_dim=8), "must equal rot_dim"),
                            (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=5), "rot.dims"),
                            (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
                            (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
                            (lambda c: c["loop"].update(stop=7), "loop"),
                            (lambda c: c["loop"].update(times=0), "times"),
                            (lambda c: c["layers"][0].update(type="convolution"), "type")):
        broken = json.loads(json.dumps(CONFIGS["odd"]))
        change(broken)
        with pytest.raises(ConfigError, match=message):
            config_from_dict(broken)
    # a checkpoint without a norm's slope, or with a tensor the design does not have, is refused
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(folder / "model.safetensors"))
    assert "l1.mix.norm" not in tensors and "head" not in tensors and tensors["l0.norm1b.alpha"].shape == ()
    assert tensors["l0.mlp.shared.sg"].shape == (1, 52) and tensors["l0.mix.g"].shape == (3, 52) and tensors["l2.mix.g"].shape == (84, 52)
    del tensors["l0.norm2b.alpha"]
    tensors["l1.mix.norm"] = torch.ones(10, dtype=torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match="l0.norm2b.alpha") as caught:
        runner_for(folder, "float32", "cpu", 8, 64, reference)
    assert "l1.mix.norm" in str(caught.value)


# --------------------------------------------------------------------------- each mechanism alone


def one_mechanism(config, tmp_path, seed=5, length=40, **kw):
    """The engine on the plain operations against the oracle for a small model that isolates a mechanism."""
    from akas_b200.ops import reference

    folder, w = make_folder(config, seed=seed, folder=tmp_path / "one", **kw)
    toks = prompts(config["vocab"], [length], seed=seed)[0]
    runner = runner_for(folder, "float32", "cpu", 8, -(-length // 8) * 8, reference)
    got = traces.replay(runner, traces.portions({"a": toks}, sizes=(9, 1, 2, 17)))["a"]
    want = plain.forward(toks, w, config).numpy()
    assert traces.first_bad(got, want, TOL["float32"]) is None, traces.worst(got, want)
    return w, toks, want


def test_norms_on_both_sides_of_a_sublayer():
    """The norm behind a sublayer reads the sublayer's result, not the stream, and its shift reaches the stream even
    where the sublayer returns nothing; the kernel-level statement against the oracle's."""
    from akas_b200.ops import reference

    g = torch.Generator().manual_seed(3)
    x, y = torch.randn(7, 20, generator=g), torch.randn(7, 20, generator=g) * 3
    w = {"n": torch.randn(20, generator=g).double(), "n.alpha": torch.tensor(0.7).double(), "n.b": torch.randn(20, generator=g).double()}
    got = reference.dynamic_tanh(y, w["n.alpha"].float(), w["n"].float(), w["n.b"].float(), torch.float32, residual=x.clone())
    assert np.abs(got.double() - (x.double() + plain.dyt(y.double(), w, "n"))).max() < 1e-6
    zero = reference.dynamic_tanh(torch.zeros(7, 20), w["n.alpha"].float(), w["n"].float(), w["n.b"].float(), torch.float32, residual=x.clone())
    assert np.abs(zero.double() - (x.double() + w["n.b"])).max() < 1e-6


def test_rotary_rates_linear_and_blended():
    """The rates the engine's rotation is built with against the oracle's, for a plain, an evenly stretched and a
    blended rotation (edges inside the pairs, outside them, and a blend that leaves every pair alone)."""
    from akas_b200.config.kidarax import _rope
    from akas_b200.parts.base import Runtime
    from akas_b200.parts.rope import Rope

    rt = Runtime(torch.float32, torch.device("cpu"), None)
    cases = [
        (dict(base=10000.0, dims=16), False),
        (dict(base=10000.0, dims=16, scaling=dict(factor=4.0)), False),
        (dict(base=300.0, dims=16, scaling=dict(factor=6.0, original=48, fast=8.0, slow=0.5)), True),
        (dict(base=400000.0, dims=32, scaling=dict(factor=4.0, original=1024, fast=16.0, slow=2.0)), True),
        (dict(base=50.0, dims=6, scaling=dict(factor=3.0, original=4000, fast=2.0, slow=1.0)), True),   # every pair slowed or nearly
        (dict(base=1e6, dims=8, scaling=dict(factor=5.0, original=2, fast=64.0, slow=32.0)), True),     # lo = hi = 0: a step at pair 0
    ]
    for rot, blended in cases:
        rope = Rope(_rope(rot["dims"], rot, rot["dims"], blended), rt)
        want, amp = plain.rates(rot)
        assert np.allclose(rope.inv_freq.numpy(), np.asarray(want), rtol=1e-12, atol=0.0), rot
        assert rope.amplitude == pytest.approx(amp, rel=1e-12)
    slowed = plain.rates(cases[2][0])[0]
    bare = plain.rates(dict(base=300.0, dims=16))[0]
    assert slowed[0] == bare[0] and slowed[7] == pytest.approx(bare[7] / 6.0) and bare[2] / 6.0 < slowed[2] < bare[2]


@pytest.mark.parametrize("mixer", [RET, RET_WIDE, RET_ODD])
def test_retention_alone(mixer, tmp_path):
    from akas_b200.ops import reference

    config = model(48, 60, [ret(mixer, None)])
    w, toks, _ = one_mechanism(config, tmp_path, length=50)
    # the state that 50 tokens leave in the request's slot is the oracle's last S (kept transposed, keys not yet scaled)
    folder = tmp_path / "one"
    runner = runner_for(folder, "float32", "cpu", 8, 56, reference)
    from akas_b200.engine.batch import StepEntry

    runner.step([StepEntry("a", toks[:31], ())])
    runner.step([StepEntry("a", toks[31:], ())])
    states = []
    x = w["embed"][torch.as_tensor(toks)]
    plain.retention(plain.dyt(x, w, "l0.norm1"), w, "l0.mix.", mixer, config["norm"]["eps"], trace=states)
    held = runner.cache.views[0].state[runner.cache.slot("a")].double()  # [heads, vdim, dim]
    want = states[0].transpose(1, 2) * mixer["dim"] ** 0.5
    assert np.abs(held - want).max() <= 1e-4 * max(1.0, float(want.abs().max()))


def test_attention_alone(tmp_path):
    for mixer in (ATT, ATT_FULL, ATT_ODD):
        one_mechanism(model(48, 60, [att(mixer, None)]), tmp_path / str(mixer["dim"]))


@pytest.mark.parametrize("mixer", [LAT, LAT_ODD, LAT_OPEN, LAT_WIDE])
def test_latent_attention_alone(mixer, tmp_path):
    config = model(48, 60, [lat(mixer, None)])
    w, toks, want = one_mechanism(config, tmp_path)
    # the sink takes weight: without it the logits differ
    w2 = dict(w)
    w2["l0.mix.sink"] = w["l0.mix.sink"] - 30.0
    assert np.abs(plain.forward(toks, w2, config).numpy() - want).max() > 1e-3 * np.abs(want).max()


def test_feed_forwards_alone(tmp_path):
    """Dense; routed with one and with several experts a token, with and without the expert that every token passes;
    as many experts a token as there are; and what each rule changes, on the oracle."""
    for i, mlp in enumerate((dense(40), moe(16, 5, 1), moe(24, 6, 2, shared=40), moe(8, 3, 3, shared=8), moe(12, 1, 1))):
        config = model(48, 60, [ret(RET, mlp)])
        found, toks, want = one_mechanism(config, tmp_path / str(i))
        if i == 3:
            w = found  # three experts of eight and a shared one of eight
    h = torch.randn(9, 48, dtype=torch.float64)
    mlp = moe(8, 3, 2, shared=8)
    wf = {k[len("l0.mlp."):]: v for k, v in w.items() if k.startswith("l0.mlp.")}
    out = plain.feed_forward(h, wf, "", mlp)
    chosen, weights = plain.route(h, wf, "", mlp["router"])
    assert ((weights > 0) & (weights < 1)).all() and not np.allclose(weights.sum(-1).numpy(), 1.0)  # scores as they are
    by_output = torch.zeros_like(h)
    for t in range(9):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            by_output[t] += g * plain.expert(h[t], wf, f"e{e}.")
    by_output += torch.sigmoid(h @ wf["shared.sg"].T) * plain.expert(h, wf, "shared.")
    assert (out - by_output).abs().max() > 1e-4  # the weight on the input is not the weight on the result


def test_the_loop_and_the_embedding_that_returns(tmp_path):
    """A loop of one pass is no loop; with more passes every pass has a cache of its own and the embedding's output
    comes back in front of each but the first."""
    layers = [ret(RET, dense(24)), att(ATT, None), lat(LAT, moe(16, 4, 1, shared=8))]
    once = model(48, 60, layers, loop=(0, 3, 1))
    w, toks, want = one_mechanism(once, tmp_path / "once")
    assert np.array_equal(plain.forward(toks, w, model(48, 60, layers)).numpy(), want)
    twice = model(48, 60, layers, loop=(1, 3, 2))
    _, _, want2 = one_mechanism(twice, tmp_path / "twice")
    assert plain.run_order(twice) == [(0, False), (1, False), (2, False), (1, True), (2, False)]
    # without the embedding's return the logits differ: the oracle's own statement, with the embedding zeroed for the sum
    trace = []
    plain.forward(toks, w, twice, trace)
    assert len(trace) == 5 and np.abs(want2 - want).max() > 1e-3


# --------------------------------------------------------------------------- what a position sees


def seen_case(device, dtype, ops, tmp_path, decode, kind):
    """One layer: the logits at position i change with the token at position j iff j <= i: keys far back, at page
    borders, the first tokens, next to the query, the query itself; later tokens never; with the query in a prompt's
    portion or decoded alone."""
    from akas_b200.engine.batch import StepEntry

    i = 290
    if kind == "attention":
        config = model(48, 120, [att(ATT, None)])
        folder, _ = make_folder(config, seed=44, folder=tmp_path / "edge", sharp=False)
        w = plant(folder, config, key_token=119, query_token=118)  # token 119 at position j is felt by token 118 at position i
    else:
        config = model(48, 120, [lat(LAT, None)])
        folder, _ = make_folder(config, seed=44, folder=tmp_path / "edge", sharp=False)
        w = plant_latent(folder, config, key_token=119, query_token=118)
    cases = [(0, True), (1, True), (7, True), (8, True), (63, True), (64, True), (255, True), (256, True), (i - 1, True),
             (i, True), (i + 1, False), (299, False)]
    base = prompts(118, [300], seed=9)[0]
    base[i] = 118

    def logits_at_i(tokens):
        runner = runner_for(folder, dtype, device, 8, 320, ops)
        if decode:
            runner.step([StepEntry("a", tokens[:i], ())])
            out = runner.step([StepEntry("a", tokens[i:i + 1], (0,))])
        else:
            runner.step([StepEntry("a", tokens[:277], ())])
            out = runner.step([StepEntry("a", tokens[277:], (i - 277,))])
        return out.float().cpu().numpy()[0][:118]  # (the two planted tokens' own logits are large: the head is the embedding)

    ref = logits_at_i(base)
    for j, seen in cases:
        changed = list(base)
        changed[j] = 119 if j != i else 7
        got = logits_at_i(changed)
        diff = np.abs(got - ref).max()
        if seen:
            assert diff > 5e-3 * np.abs(ref).max(), f"position {i} does not see {j}"
        else:
            assert diff == 0.0, f"position {i} sees {j} (difference {diff})"
        if dtype == "float32" and seen:
            want = plain.forward(changed[: i + 1], w, config)[i].numpy()[:118]
            assert np.abs(got - want).max() <= TOL[dtype] * np.abs(want).max()


KINDS = ["attention", "latent attention"]


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("decode", [False, True])
def test_what_a_position_sees_on_the_plain_operations(decode, kind, tmp_path):
    from akas_b200.ops import reference

    seen_case("cpu", "float32", reference, tmp_path, decode, kind)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_what_a_position_sees_on_the_kernels(decode, dtype, kind, tmp_path):
    seen_case("cuda:0", dtype, None, tmp_path, decode, kind)


def far_key_case(device, dtype, ops, tmp_path):
    """One key far back among hundreds is made to stand out: the last position's attention must find it through
    scattered pages, in a portion and decoded alone, in both passes of a looped layer (each has its own pages)."""
    from akas_b200.engine.batch import StepEntry

    config = model(48, 120, [att(ATT, None)], loop=(0, 1, 2))
    folder, _ = make_folder(config, seed=47, folder=tmp_path / "far", sharp=False)
    w = plant(folder, config, key_token=119, query_token=118, strength=1.1, loud=4.0)
    toks = prompts(118, [500], seed=2)[0]
    toks[3], toks[-1] = 119, 118  # the key appears once, far back; the query is the last token
    want = plain.forward(toks, w, config)[-1].numpy()
    without = list(toks)
    without[3] = 5
    felt = np.abs(plain.forward(without, w, config)[-1].numpy() - want).max()
    assert felt > 0.05 * np.abs(want).max(), "the far key does not stand out"
    for cuts in ([500], [499, 1], [130, 70, 2, 290, 8]):
        runner = runner_for(folder, dtype, device, 16, 576, ops, context=512)
        runner.admit("other")  # the request's pages are not the pool's first
        runner.cache.reserve("other", 40)
        at = 0
        for c in cuts:
            out = runner.step([StepEntry("a", toks[at:at + c], (c - 1,) if at + c == 500 else ())])
            at += c
        got = out.float().cpu().numpy()[0]
        assert np.abs(got - want).max() <= TOL[dtype] * np.abs(want).max(), cuts


def test_a_far_key_is_found_on_the_plain_operations(tmp_path):
    from akas_b200.ops import reference

    far_key_case("cpu", "float32", reference, tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_is_found_on_the_kernels(dtype, tmp_path):
    far_key_case("cuda:0", dtype, None, tmp_path)


def far_token_case(device, dtype, ops, tmp_path):
    """Retention keeps what a token left for as long as the head's decay allows: with a decay of one the first token is
    felt 400 tokens on, with a decay of zero only the token itself is; through portions and single tokens alike."""
    from akas_b200.engine.batch import StepEntry

    toks = prompts(60, [400], seed=4)[0]
    other = [(toks[0] + 1) % 60] + toks[1:]
    for decay, felt in ((1.0, True), (0.0, False)):
        mixer = dict(heads=2, dim=16, vdim=16, decay=[decay, decay])
        config = model(48, 60, [ret(mixer, None)])
        folder, w = make_folder(config, seed=9, folder=tmp_path / str(decay))
        want = plain.forward(toks, w, config)[-1].numpy()
        moved = np.abs(plain.forward(other, w, config)[-1].numpy() - want).max()
        assert (moved > 1e-5 * np.abs(want).max()) if felt else moved == 0.0
        for cuts in ([400], [399, 1], [130, 70, 2, 190, 1, 1, 1, 1, 1, 1, 1, 1]):
            runner = runner_for(folder, dtype, device, 16, 448, ops)
            at = 0
            for c in cuts:
                out = runner.step([StepEntry("a", toks[at:at + c], (c - 1,) if at + c == 400 else ())])
                at += c
            got = out.float().cpu().numpy()[0]
            assert np.abs(got - want).max() <= TOL[dtype] * np.abs(want).max(), (decay, cuts)


def test_a_far_token_is_felt_through_the_state_on_the_plain_operations(tmp_path):
    from akas_b200.ops import reference

    far_token_case("cpu", "float32", reference, tmp_path)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_token_is_felt_through_the_state_on_the_kernels(dtype, tmp_path):
    far_token_case("cuda:0", dtype, None, tmp_path)


def test_freed_pages_and_slots_are_used_again_and_not_read(tmp_path):
    """Two requests one after the other in a pool of one slot and just enough pages: the second gets the first one's
    pages and its state slot (in every pass of the loop) and must compute as if it were alone."""
    from akas_b200.engine.batch import StepEntry
    from akas_b200.ops import reference

    config = CONFIGS["odd"]
    folder, w = make_folder(config, seed=12, folder=tmp_path / "m")
    a, b = prompts(config["vocab"], [30, 26], seed=5)
    runner = runner_for(folder, "float32", "cpu", 8, 32, reference, max_requests=1)
    runner.step([StepEntry("a", a, ())])
    runner.release("a")
    got = runner.step([StepEntry("b", b[:11], ()),])
    got = runner.step([StepEntry("b", b[11:], tuple(range(15)))]).numpy()
    want = plain.forward(b, w, config).numpy()[11:]
    assert traces.first_bad(got, want, TOL["float32"]) is None, traces.worst(got, want)


def test_a_batch_of_unequal_requests_equals_each_alone(tmp_path):
    """A request's logits beside three others of other lengths, and alone."""
    from akas_b200.engine.batch import StepEntry
    from akas_b200.ops import reference

    config = CONFIGS["mix"]
    folder, _ = make_folder(config, seed=14, folder=tmp_path / "m")
    ps = prompts(config["vocab"], [1, 37, 2, 80], seed=5)
    runner = runner_for(folder, "float32", "cpu", 8, 256, reference)
    together = runner.step([StepEntry(i, p, (len(p) - 1,)) for i, p in enumerate(ps)]).numpy()
    for i, p in enumerate(ps):
        alone = runner_for(folder, "float32", "cpu", 8, 256, reference).step([StepEntry("x", p, (len(p) - 1,))]).numpy()
        assert np.abs(alone[0] - together[i]).max() <= 1e-5 * np.abs(alone).max()


# --------------------------------------------------------------------------- generation


def _greedy(config, w, prompt, count):
    toks = list(prompt)
    for _ in range(count):
        toks.append(int(plain.forward(toks, w, config)[-1].argmax()))
    return toks[len(prompt):]


def generation_case(device, dtype, ops, tmp_path, graphs):
    from akas_b200 import Engine, EngineConfig

    config = CONFIGS["mix"]
    folder, w = make_folder(config, seed=61, folder=tmp_path / "gen")
    ps = prompts(config["vocab"], [1, 9, 40, 23, 3], seed=8)
    cfg = EngineConfig(dtype=dtype, device=device, page_size=8, max_requests=3, context=128, max_tokens=1024, prefill_chunk=13,
                       prefill_requests=2, cuda_graphs=graphs)
    with Engine(str(folder), config=cfg, ops=ops) as engine:
        results = engine.generate(ps, max_tokens=10)
    for prompt, result in zip(ps, results):
        assert result["generated_tokens"] == _greedy(config, w, prompt, 10)


def test_greedy_generation_through_the_scheduler_on_the_plain_operations(tmp_path):
    from akas_b200.ops import reference

    generation_case("cpu", "float32", reference, tmp_path, False)


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler_on_the_kernels(graphs, tmp_path):
    generation_case("cuda:0", "float32", None, tmp_path, graphs)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, tmp_path):
    """200 decoded tokens for three requests of different lengths through captured graphs, against one whole pass of
    the plain model."""
    from akas_b200 import Engine, EngineConfig, StepEntry

    config = CONFIGS["mix"]
    folder, w = make_folder(config, seed=71, folder=tmp_path / "long")
    ps = prompts(config["vocab"], [5, 70, 33], seed=3)
    feed = prompts(config["vocab"], [200, 200, 200], seed=4)
    cfg = EngineConfig(dtype=dtype, device="cuda:0", page_size=8, max_requests=4, context=512, max_tokens=2048)
    with Engine(str(folder), config=cfg) as engine:
        runner = engine.runner
        runner.step([StepEntry(i, p, ()) for i, p in enumerate(ps)])
        rows = [[] for _ in ps]
        for t in range(200):
            logits = runner.step([StepEntry(i, (feed[i][t],), (0,)) for i in range(3)]).float().cpu().numpy()
            for i in range(3):
                rows[i].append(logits[i])
        assert 4 in runner._graphs
    want = {}
    for i, p in enumerate(ps):
        logits, least = oracle(config, w, p + feed[i])
        want[i] = (logits[len(p):], least[len(p):])
    compare({i: np.stack(r) for i, r in enumerate(rows)}, want, dtype, f"long decoding/{dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(dtype, tmp_path):
    """bin/trace_run as a user calls it, on a Kidarax folder: steps on standard input, logits as files."""
    config = CONFIGS["alone"]
    folder, w = make_folder(config, seed=27, folder=tmp_path / "m")
    reqs = {f"q{i}": p for i, p in enumerate(prompts(config["vocab"], [50, 3, 71, 20, 130], seed=7))}
    steps, peak = traces.mixed(reqs, {rid: max(1, len(t) - 5) for rid, t in reqs.items()}, seed=1, live=4, page=64)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(peak)],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    want = {rid: oracle(config, w, t) for rid, t in reqs.items()}
    at = {rid: 0 for rid in reqs}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if not wanted:
            continue
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(wanted, config["vocab"])
        row = 0
        for e in s["entries"]:
            for k in e["want"]:
                logits, least = want[e["id"]]
                p = at[e["id"]] + k
                if least[p] >= CLOSE_CALL[dtype]:
                    assert np.abs(data[row] - logits[p]).max() <= TOL[dtype] * np.abs(logits).max(), (s["step"], e["id"], k)
                row += 1
            at[e["id"]] += len(e["tokens"])


# --------------------------------------------------------------------------- the kernels' new options one by one


def _close(got, want, tol, what):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / max(1e-30, float(want.abs().max())))
    assert err <= tol, f"{what}: {err:.3g}"


@pytest.mark.gpu
@pytest.mark.parametrize("n,c", [(9, 20), (300, 52), (7, 50), (1, 1), (33, 1024)])
def test_dynamic_tanh_that_adds_and_activation_kernels(n, c):
    from akas_b200.ops import cuda, reference

    cuda.require(["elementwise"])
    g = torch.Generator().manual_seed(n * 1000 + c)
    y, x = (torch.randn(n, c, generator=g) * 3).cuda(), torch.randn(n, c, generator=g).cuda()
    alpha = torch.tensor(0.6).cuda()
    w, b = torch.randn(c, generator=g).cuda(), torch.randn(c, generator=g).cuda()
    kept = x.clone()
    out = cuda.dynamic_tanh(y, alpha, w, b, torch.float32, residual=x)
    assert out is x
    _close(out, reference.dynamic_tanh(y, alpha, w, b, torch.float32, residual=kept.clone()), 1e-6, "dynamic tanh into the stream")
    for kind in ("relu2", "gelu_tanh", "silu"):
        for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 8e-3)):
            wide = (torch.randn(n, c + 5, generator=g) * 2).cuda()
            for z in (wide[:, :c], wide[:, :c].to(torch.bfloat16)):
                _close(cuda.activation(z, kind, dtype), reference.activation(z, kind, dtype), tol, f"{kind} {dtype}")
    assert float(cuda.activation(torch.tensor([[-2.0, 0.0, 3.0]]).cuda(), "relu2", torch.float32).cpu().sub(torch.tensor([[0.0, 0.0, 9.0]])).abs().max()) == 0.0


@pytest.mark.gpu
def test_rotary_tables_with_an_amplitude():
    from akas_b200.ops import cuda, reference

    cuda.require(["rope"])
    positions = torch.tensor([0, 1, 17, 4095, 100000], dtype=torch.int32).cuda()
    rates = torch.tensor(plain.rates(dict(base=300.0, dims=16, scaling=dict(factor=6.0, original=48, fast=8.0, slow=0.5)))[0], dtype=torch.float64).cuda()
    for amp in (1.0, 1.1791759469228055):
        got = cuda.rope_tables(positions, rates, amp) if amp != 1.0 else cuda.rope_tables(positions, rates)
        want = reference.rope_tables(positions, rates, amp)
        _close(got[0], want[0], 2e-7, "cos"), _close(got[1], want[1], 2e-7, "sin")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim", [(3, 24), (2, 8), (5, 10), (4, 32), (2, 1100)])
def test_gated_norm_without_a_weight(heads, vdim, dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["recurrent"])
    g = torch.Generator().manual_seed(heads * 100 + vdim)
    o = (torch.randn(37, heads * vdim, generator=g) * 5).cuda()
    gate = torch.randn(37, heads * vdim + 8, generator=g).to(dtype).cuda()[:, : heads * vdim]
    got = cuda.gated_rmsnorm(o, None, 1e-5, gate, heads, vdim, dtype, gate_activation="silu")
    want = reference.gated_rmsnorm(o, None, 1e-5, gate, heads, vdim, dtype, gate_activation="silu")
    _close(got, want, 1e-5 if dtype == torch.float32 else 8e-3, "norm without a weight")
    ones = cuda.gated_rmsnorm(o, torch.ones(vdim).cuda(), 1e-5, gate, heads, vdim, dtype, gate_activation="silu")
    assert torch.equal(ones, got)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page", [(6, 2, 24, 16, 8), (4, 4, 16, 24, 16), (3, 1, 20, 28, 4), (8, 4, 64, 32, 64),
                                                         (4, 1, 64, 64, 64)])
def test_a_gate_per_channel_in_the_general_attention(heads, kv_heads, dim, vdim, page, dtype):
    """Prompt portions, single tokens with their keys in parts, and both beside each other, against the plain statement."""
    from akas_b200.ops import cuda, reference

    cuda.require(["attention_general"] + (["attention_general_tc"] if dtype == torch.bfloat16 else []))
    g = torch.Generator().manual_seed(heads * 10 + dim)
    lengths = [1, 1, 70, 2, 33]           # the tokens each request brings
    before = [140, 7, 0, 61, 20]          # and what its cache holds already
    pages_each = [-(-(a + b) // page) for a, b in zip(before, lengths)]
    table = torch.full((len(lengths), max(pages_each)), -1, dtype=torch.int32)
    order = torch.randperm(sum(pages_each), generator=g).tolist()
    at = 0
    for r, count in enumerate(pages_each):
        table[r, :count] = torch.tensor(order[at:at + count], dtype=torch.int32)
        at += count
    k_pool = torch.randn(sum(pages_each), kv_heads, page, dim, generator=g).to(dtype).cuda()
    v_pool = torch.randn(sum(pages_each), kv_heads, page, vdim, generator=g).to(dtype).cuda()
    seq = torch.tensor([r for r, c in enumerate(lengths) for _ in range(c)], dtype=torch.int32).cuda()
    pos = torch.tensor([b + i for b, c in zip(before, lengths) for i in range(c)], dtype=torch.int32).cuda()
    n = sum(lengths)
    q = (torch.randn(n, heads * dim, generator=g) * 1.5).to(dtype).cuda()
    gate = torch.randn(n, heads * vdim + 16, generator=g).to(dtype).cuda()[:, 16:]

    class Ctx:
        query_lens = tuple(lengths)
        cu_seqlens = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32).cuda()
        max_context = 256
        decode_only = False

    args = (q, k_pool, v_pool, table.cuda(), seq, pos, 0.2, None, 0, None, None, None, False, gate, page)
    want = reference.attention_general(*args, gate_channels=True)
    got = cuda.attention_general(*args, Ctx, gate_channels=True)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    _close(got, want, tol, "a gate per channel")
    plainly = cuda.attention_general(*args, None, gate_channels=True)  # the kernel for any sizes
    _close(plainly, want, tol, "a gate per channel, plain kernel")
    per_head = reference.attention_general(*args[:13], gate[:, :heads].contiguous(), page)
    assert (per_head.double() - want.double()).abs().max() > 1e-2
    if dtype == torch.bfloat16:
        # the gate's logits as a float32 product leaves them (rows that are parts of wider rows), per channel and per head
        wide = torch.zeros(n, heads * vdim + 12, device="cuda")
        wide[:, 4 : 4 + heads * vdim] = gate.float()
        for ctx in (Ctx, None):
            _close(cuda.attention_general(*args[:13], wide[:, 4 : 4 + heads * vdim], page, ctx, gate_channels=True), want, tol, "float32 logits")
            _close(cuda.attention_general(*args[:13], wide[:, 4 : 4 + heads], page, ctx), per_head, tol, "float32 logits, a gate per head")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,c,f,extra", [(6, 2, 80, 24, 1), (5, 1, 48, 16, 0), (3, 3, 52, 20, 1), (16, 1, 160, 72, 1),
                                                   (64, 6, 1104, 24, 2), (1, 1, 24, 8, 1)])
def test_sigmoid_routing_weighted_inputs_and_a_shared_expert(experts, top, c, f, extra, dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["moe"] + (["moe_grouped"] if dtype == torch.bfloat16 else []))
    g = torch.Generator().manual_seed(experts * 100 + c)
    n = 45
    h = torch.randn(n, c + 8, generator=g).to(dtype).cuda()[:, :c]
    w_router = (torch.randn(experts + extra, c, generator=g) * (3.0 / c ** 0.5)).cuda()
    want = reference.moe_route(h, w_router, None, 1, 1, top, scoring="sigmoid", renormalize=False, extra=extra)
    got = cuda.moe_route(h, w_router, None, 1, 1, top, scoring="sigmoid", renormalize=False, extra=extra)
    assert len(got) == (3 if extra else 2)
    same = (got[0] == want[0]).all(dim=1)  # a choice may differ where two scores are within rounding of each other
    assert same.float().mean() > 0.9
    _close(got[1][same], want[1][same], 1e-4, "weights")
    if extra:
        assert got[2].shape == (n, extra)
        _close(got[2], want[2], 1e-4, "the further rows' sigmoids")
    scores = torch.sigmoid(h.float() @ w_router[:experts].T)
    _close(want[1], torch.gather(scores, 1, want[0].long()), 1e-5, "the weights are the scores as they are")
    # renormalised sigmoid scores, for a design that wants them
    renorm = cuda.moe_route(h, w_router, None, 1, 1, top, scoring="sigmoid", renormalize=True, extra=extra)
    _close(renorm[1][same], (want[1] / want[1].sum(-1, keepdim=True))[same], 1e-4, "renormalised")
    chosen, weights = want[0], want[1]
    w_gate_up = (torch.randn(experts, 2 * f, c, generator=g) * c ** -0.5).to(dtype).cuda()
    w_down = (torch.randn(experts, c, f, generator=g) * f ** -0.5).to(dtype).cuda()
    shared = torch.randn(n, c, generator=g).cuda()
    gate = want[2][:, :1] if extra else None
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for rows in (n, 5):  # 45 tokens: the grouped product in bfloat16 where it takes the sizes; 5: token by token
        sl = slice(0, rows)
        sh = (shared[sl].contiguous(), None if gate is None else gate[sl])
        ref = reference.moe_experts(h[sl], w_gate_up, w_down, chosen[sl], weights[sl], weight_input=True, shared=sh)
        out = cuda.moe_experts(h[sl], w_gate_up, w_down, chosen[sl], weights[sl], weight_input=True, shared=sh)
        _close(out, ref, tol, f"weighted inputs and a shared expert, {rows} tokens")
        bare = cuda.moe_experts(h[sl], w_gate_up, w_down, chosen[sl], weights[sl], weight_input=True)
        _close(bare, reference.moe_experts(h[sl], w_gate_up, w_down, chosen[sl], weights[sl], weight_input=True), tol, "weighted inputs")
    # the statement itself: expert(w h), token by token in float64
    t = 3
    direct = torch.zeros(c, dtype=torch.float64)
    for e, wgt in zip(chosen[t].tolist(), weights[t].double().cpu()):
        x = wgt * h[t].double().cpu()
        gu = w_gate_up[e].double().cpu() @ x
        direct += w_down[e].double().cpu() @ (gu[:f] * torch.sigmoid(gu[:f]) * gu[f:])
    _close(bare[t], direct, 5e-5 if dtype == torch.float32 else 3e-2, "expert(w h)")
    if dtype == torch.bfloat16:
        assert cuda.moe_grouped_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_cached_row_without_a_query_latent(dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["latent", "rope"])
    g = torch.Generator().manual_seed(5)
    kv_rank, rot, page, n = 32, 8, 8, 21
    proj = torch.randn(n, kv_rank + rot + 4, generator=g).cuda()
    kw = torch.randn(kv_rank, generator=g).cuda()
    seq, pos = torch.zeros(n, dtype=torch.int32).cuda(), torch.arange(n, dtype=torch.int32).cuda()
    table = torch.tensor([[2, 0, 1]], dtype=torch.int32).cuda()
    cos, sin = reference.rope_tables(pos, torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=torch.float64).cuda(), 1.2)
    pools = [torch.zeros(3, 1, page, kv_rank + rot, dtype=dtype).cuda() for _ in range(2)]
    for ops, pool in zip((reference, cuda), pools):
        out = ops.latent_norm_store(proj, 0, kv_rank, rot, None, kw, 1e-5, cos, sin, False, pool, table, seq, pos, page)
        assert out.shape == (n, 0)
    _close(pools[1], pools[0], 1e-6 if dtype == torch.float32 else 8e-3, "the cached rows")


@pytest.mark.gpu
@pytest.mark.parametrize("activation", ["relu2", "gelu_tanh", "silu"])
@pytest.mark.parametrize("n,k,o", [(3, 64, 48), (16, 192, 320), (9, 2048, 48), (1, 128, 1008), (40, 264, 528), (128, 2048, 320),
                                   (300, 200, 264), (700, 512, 1536), (20, 100, 40), (33, 64, 20)])
def test_products_with_an_activation_in_the_read_out(n, k, o, activation):
    """The three product kernels' bfloat16 read-out with an activation on the float32 sums, and the fused norm in
    front of it for few tokens, against the product in float32 followed by the activation's own kernel's statement."""
    from akas_b200.ops import cuda, reference

    cuda.require(cuda.libraries_for(torch.bfloat16, ()))
    g = torch.Generator().manual_seed(n * 7 + o)
    x = torch.randn(n, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(o, k, generator=g) * k ** -0.5).to(torch.bfloat16).cuda()
    want = reference.activation(reference.linear(x, w, out_dtype=torch.float32), activation, torch.bfloat16)
    got = cuda.linear_activated(x, w, activation)
    if got is None:  # sizes that no fused read-out takes: the part's other way
        assert k % 8 or o % 8
        got = cuda.activation(cuda.linear(x, w, out_dtype=torch.float32), activation, torch.bfloat16)
    _close(got, want, 1.2e-2, f"{activation} in the read-out")
    for status in (cuda.skinny_status, cuda.gemm_rows_status, cuda.gemm_pair_status):
        assert status() == 0
    if n <= 16 and k % 64 == 0:
        h = (torch.randn(n + 2, k, generator=g) * 2).cuda()
        rows = torch.arange(n, dtype=torch.int32).cuda() + 1
        alpha = torch.tensor(0.8).cuda()
        nw, nb = torch.randn(k, generator=g).cuda(), torch.randn(k, generator=g).cuda() * 0.2
        fused = cuda.dyt_linear_activated(h, alpha, nw, nb, w, activation, rows)
        assert fused is not None
        normed = reference.dynamic_tanh(h, alpha, nw, nb, torch.bfloat16, rows)
        _close(fused, reference.activation(reference.linear(normed, w, out_dtype=torch.float32), activation, torch.bfloat16), 1.5e-2,
               "norm, product and activation")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_widths_of_a_real_model(dtype, tmp_path):
    """Widths at which every product, both attentions, the chunked recurrence and the grouped experts run on their
    tensor-core kernels (a width of 1,024, heads of 64 and 128, sixteen experts of 512), a prompt of 700 tokens in one
    step, in portions beside another request, and its last tokens decoded: against the plain model."""
    from akas_b200.engine.batch import StepEntry

    retention = dict(heads=8, dim=64, vdim=128, decay=[1.0 - 2.0 ** -(4 + i) for i in range(8)])
    attention = dict(heads=16, kv_heads=4, dim=64, vdim=64, scale=0.125, rot=dict(base=500000.0, dims=64, scaling=dict(factor=8.0)))
    latent = dict(heads=8, dim=64, rot_dim=64, vdim=64, kv_rank=64, scale=0.11,
                  rot=dict(base=1000000.0, dims=64, scaling=dict(factor=4.0, original=256, fast=16.0, slow=2.0)))
    # (only the last layer routes: a choice that falls the other way then moves its own position and no later one)
    config = model(1024, 2048, [ret(retention, dense(4096)), att(attention, dense(1024)), lat(latent, dense(2048)),
                                ret(retention, moe(512, 16, 3, shared=1024))], loop=(1, 3, 2), eps=1e-6, logit_scale=1024 ** -0.5)
    # (a deviation of 0.02: with the tiny configurations' 0.08 every product of 1,024 terms saturates the norm behind it,
    # and float32's own rounding is then magnified four thousand times on the way to the logits)
    folder, w = make_folder(config, seed=5, folder=tmp_path / "m", std=0.02)
    toks, other = prompts(config["vocab"], [700, 150], seed=3)
    logits, least = oracle(config, w, toks)
    held = least >= {"float32": 1e-3, "bfloat16": 0.05}[dtype]  # (logits of about one unit: bfloat16 moves them by a hundredth)
    rows = list(range(0, 700, 37)) + list(range(690, 700))
    tol = TOL[dtype]

    def check(got, at, what):
        keep = [i for i, p in enumerate(at) if held[p]]
        assert len(keep) > len(at) // 2
        err = np.abs(got[keep] - logits[np.asarray(at)[keep]]).max() / np.abs(logits).max()
        assert err <= tol, f"{what}: {err:.3g}"

    runner = runner_for(folder, dtype, "cuda:0", 64, 1024, None, max_requests=2, context=768)
    check(runner.step([StepEntry("a", toks, tuple(rows))]).float().cpu().numpy(), rows, "one step")
    runner.release("a")
    at, got, places = 0, [], []
    for k, (count, beside) in enumerate(((300, 100), (2, 0), (130, 50), (258, 0))):
        entries = [StepEntry("a", toks[at:at + count], tuple(range(count)))]
        if beside:
            entries.append(StepEntry("b", other[:beside] if k == 0 else other[100:150], ()))
        got.append(runner.step(entries).float().cpu().numpy())
        places += list(range(at, at + count))
        at += count
    for p in range(at, 700):
        got.append(runner.step([StepEntry("b", (5,), ()), StepEntry("a", toks[p:p + 1], (0,))]).float().cpu().numpy())
        places.append(p)
    check(np.concatenate(got), places, "portions beside another request, then single tokens")
