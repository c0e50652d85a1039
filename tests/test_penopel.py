"""The Penopel decoder in the engine against the plain float64 statement of it (``plain_penopel``).

Small configurations of the tests' own, random weights shaped so that faults show (peaked attention, sinks of the
scores' size, norms with slopes and shifts of their own, biases that are not small), and every way of cutting and
batching. The same tests run on a CPU with the plain PyTorch statements of the kernels (host logic: pages, windows,
a cache read by several layers) and, marked ``gpu``, with the compiled kernels in float32 and bfloat16. The kernels
are also compared one by one with their plain statements, and those with the oracle's functions.
"""

import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_penopel as plain
import traces

from tiny_penopel import (ATT, ATT_FULL, ATT_ODD, CONFIGS, LAT, LAT_ODD, LAT_OPEN, LAT_SELF, LAT_WIDE, LENGTHS, PAGE, SLOWED,
                          TOL, att, lat, make_folder, model, plant, plant_latent, prompts)

ROOT = Path(__file__).resolve().parent.parent


def runner_for(folder, dtype, device, page, max_tokens, ops=None, max_requests=4, context=None, **kw):
    from akas_b200.config import EngineConfig
    from akas_b200.engine.runner import ModelRunner

    cfg = EngineConfig(dtype=dtype, device=device, page_size=page, max_tokens=max_tokens, max_requests=max_requests,
                       context=context or max_tokens, cuda_graphs=False, **kw)
    return ModelRunner(folder, cfg, ops=ops)


def compare(got, want, dtype, what):
    for rid, logits in want.items():
        bad = traces.first_bad(got[rid], logits, TOL[dtype])
        assert bad is None, f"{what}: request {rid} first differs at position {bad} {traces.worst(got[rid], logits)}"


def run_modes(key, dtype, device, ops, tmp_path, modes):
    config = CONFIGS[key]
    folder, w = make_folder(config, seed=31, folder=tmp_path / key)
    reqs = {f"r{i}": p for i, p in enumerate(prompts(config["vocab"], LENGTHS[key], seed=6))}
    want = {rid: plain.forward(toks, w, config).numpy() for rid, toks in reqs.items()}
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
    from akas_b200.config import ConfigError, PenopelConfig, config_from_dict, load_config
    from akas_b200.engine.runner import kernel_kinds
    from akas_b200.ops import reference
    from akas_b200.weights.loader import WeightError

    config = config_from_dict(CONFIGS["mix"])
    assert isinstance(config, PenopelConfig) and config_from_dict(config.to_dict()) == config
    assert config_from_dict(json.loads(json.dumps(config.to_dict()))) == config
    spec = config.model_spec()
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["latent_attention", "attention", "latent_attention", "attention", "attention", "attention", "latent_attention"]
    assert [e.cache for e in spec.schedule] == [None, None, None, 1, None, 1, None]
    assert spec.layers[2].ffn is None and spec.layers[0].ffn.intermediate_size == 48 and spec.layers[0].ffn.bias
    assert spec.layers[1].mixer.own_kv and not spec.layers[3].mixer.own_kv and spec.layers[1].mixer.sink is True
    assert spec.layers[1].mixer.position.scaling == (8.0, 2.0, 6.0, 64.0) and not spec.layers[1].mixer.position.interleaved
    assert spec.layers[0].mixer.window == 11 and spec.layers[6].mixer.window is None and spec.layers[6].mixer.position is None
    assert spec.layers[0].mixer.position.interleaved and spec.layers[0].mixer.sink == "learned"
    assert spec.embedding_multiplier == 3.0 and spec.logit_softcap == 12.0 and spec.final_norm.kind == "dynamic_tanh"
    assert set(kernel_kinds(spec)) == {"attention_general", "latent", "rope"}
    folder, _ = make_folder(CONFIGS["odd"], seed=1, folder=tmp_path / "m")
    assert load_config(folder) == config_from_dict(CONFIGS["odd"])
    for change, message in ((lambda c: c["layers"][1]["mixer"].update(kv_heads=2), "kv_heads"),
                            (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
                            (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
                            (lambda c: c["layers"][3]["mixer"].update(vdim=12), "vdim differs"),
                            (lambda c: c["layers"][0]["mixer"].update(rot_dim=8), "must equal rot_dim"),
                            (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
                            (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
                            (lambda c: c["layers"][0].update(type="convolution"), "type")):
        broken = json.loads(json.dumps(CONFIGS["odd"]))
        change(broken)
        with pytest.raises(ConfigError, match=message):
            config_from_dict(broken)
    # a checkpoint without a norm's slope, or with keys for a layer that reads another's, is refused
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(folder / "model.safetensors"))
    assert "l3.mix.k" not in tensors and "l3.mix.v.b" not in tensors and tensors["l0.norm1.alpha"].shape == ()
    del tensors["l0.norm2.alpha"]
    tensors["l3.mix.k"] = tensors["l1.mix.k"].clone()
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError, match="l0.norm2.alpha") as caught:
        runner_for(folder, "float32", "cpu", 8, 64, reference)
    assert "l3.mix.k" in str(caught.value)


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


def test_dynamic_tanh_alone():
    from akas_b200.ops import reference

    g = torch.Generator().manual_seed(2)
    x = torch.randn(9, 20, generator=g) * 4.0
    w = {"n": torch.randn(20, generator=g).double(), "n.b": torch.randn(20, generator=g).double(), "n.alpha": torch.tensor(0.37).double()}
    want = plain.dyt(x.double(), w, "n")
    got = reference.dynamic_tanh(x, w["n.alpha"].float(), w["n"].float(), w["n.b"].float(), torch.float32)
    assert torch.allclose(got.double(), want, atol=1e-6)
    rows = torch.tensor([7, 0, 7], dtype=torch.int32)
    assert torch.equal(reference.dynamic_tanh(x, w["n.alpha"].float(), w["n"].float(), w["n.b"].float(), torch.float32, rows), got[rows.long()])
    # no statistics: a row's result does not depend on its other channels, and large inputs saturate at +-w + b
    big = plain.dyt(torch.full((1, 20), 1e4, dtype=torch.float64), w, "n")
    assert torch.allclose(big[0], w["n"] + w["n.b"])


def test_slowed_long_waves():
    """The three regimes of the rotation's rates against the oracle's, and by hand at the two borders."""
    from akas_b200.config.specs import RopeSpec
    from akas_b200.parts.base import Runtime
    from akas_b200.parts.rope import Rope

    for base, dims, scaling in ((10000.0, 16, SLOWED), (300.0, 16, SLOWED), (1e6, 32, dict(factor=4.0, low=1.0, high=4.0, original=48)),
                                (50.0, 4, None)):
        rot = dict(base=base, dims=dims)
        packed = None
        if scaling is not None:
            rot["scaling"] = scaling
            packed = (scaling["factor"], scaling["low"], scaling["high"], scaling["original"])
        rope = Rope(RopeSpec(dims + 8, base, dims, scaling=packed), Runtime(torch.float32, torch.device("cpu"), None))
        want = torch.tensor(plain.frequencies(rot), dtype=torch.float64)
        assert torch.allclose(rope.inv_freq, want, rtol=1e-12)
        plainly = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        if scaling is not None:
            wave = 2 * math.pi / plainly
            short, long = wave < scaling["original"] / scaling["high"], wave > scaling["original"] / scaling["low"]
            assert torch.equal(want[short], plainly[short]) and torch.allclose(want[long], plainly[long] / scaling["factor"])
            between = ~short & ~long
            assert ((want[between] < plainly[between]) & (want[between] > plainly[between] / scaling["factor"])).all()
    assert short.any() and long.any() and between.any()


def test_biased_attention_with_a_unit_sink_alone(tmp_path):
    config = model(48, 70, [att(ATT, None)])
    w, toks, want = one_mechanism(config, tmp_path)
    # the biases matter, and so does the one in the denominator
    for name in ("l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b"):
        assert np.abs(plain.forward(toks, dict(w, **{name: w[name] * 0}), config).numpy() - want).max() > 1e-3 * np.abs(want).max()
    h = torch.randn(7, 48, dtype=torch.float64)
    y = plain.attention(h, w, "l0.mix.", ATT)
    # row 0 sees one key at position 0, where nothing turns: its output is v times e / (1 + e)
    q = (h[0] @ w["l0.mix.q"].T + w["l0.mix.q.b"]).reshape(ATT["heads"], ATT["dim"])
    k = (h[0] @ w["l0.mix.k"].T + w["l0.mix.k.b"]).reshape(ATT["kv_heads"], ATT["dim"])
    v = (h[0] @ w["l0.mix.v"].T + w["l0.mix.v.b"]).reshape(ATT["kv_heads"], ATT["vdim"])
    group = ATT["heads"] // ATT["kv_heads"]
    heads = []
    for a in range(ATT["heads"]):
        e = torch.exp((q[a] @ k[a // group]) * ATT["scale"])
        heads.append(v[a // group] * e / (1.0 + e))
    assert torch.allclose(torch.cat(heads) @ w["l0.mix.o"].T, y[0], atol=1e-10)
    # the rotation turns pairs (i, i + dims / 2) of the first dims channels and nothing else
    x = torch.randn(3, 2, ATT["dim"], dtype=torch.float64)
    r = plain.rotate(x, ATT["rot"], interleaved=False)
    assert torch.equal(r[0], x[0]) and torch.equal(r[:, :, ATT["rot"]["dims"]:], x[:, :, ATT["rot"]["dims"]:])
    f = plain.frequencies(ATT["rot"])
    half = ATT["rot"]["dims"] // 2
    assert torch.allclose(r[2, 1, 3], x[2, 1, 3] * math.cos(2 * f[3]) - x[2, 1, 3 + half] * math.sin(2 * f[3]))


def test_a_layer_that_reads_another_layers_cache(tmp_path):
    """Two layers read layer 0's keys and values; the oracle's shared keys are the owner's after ITS rotation."""
    config = model(48, 70, [att(ATT_ODD, 16), att(ATT_ODD, None, kv_from=0), att(ATT_ODD, 24, kv_from=0)])
    w, toks, want = one_mechanism(config, tmp_path)
    assert "l1.mix.k" not in w and "l2.mix.v" not in w and "l1.mix.q.b" in w
    # with keys of its own instead (a copy of the owner's matrices) the reader would compute something else
    own = json.loads(json.dumps(config))
    del own["layers"][1]["mixer"]["kv_from"]
    w2 = dict(w, **{f"l1.mix.{n}": w[f"l0.mix.{n}"] for n in ("k", "k.b", "v", "v.b")})
    assert np.abs(plain.forward(toks, w2, own).numpy() - want).max() > 1e-3 * np.abs(want).max()


@pytest.mark.parametrize("mixer", [LAT, LAT_ODD, LAT_SELF, LAT_OPEN, LAT_WIDE])
def test_latent_attention_alone(mixer, tmp_path):
    config = model(48, 70, [lat(mixer, None)])
    w, toks, want = one_mechanism(config, tmp_path, length=90 if mixer is LAT_WIDE else 40)
    p = "l0.mix."
    # the sink, the gate and the shared rotated key part matter
    assert np.abs(plain.forward(toks, dict(w, **{p + "sink": w[p + "sink"] - 60.0}), config).numpy() - want).max() > 1e-3 * np.abs(want).max()
    assert np.abs(plain.forward(toks, dict(w, **{p + "g": w[p + "g"] * 0}), config).numpy() - want).max() > 1e-3 * np.abs(want).max()
    # row 0 sees itself only: per head v_0 times e / (e + exp(sink)), times the gate
    h = torch.randn(6, 48, dtype=torch.float64)
    y = plain.latent_attention(h, w, p, mixer, 1e-5)
    H, D, R, V, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    cq = plain.rms(h[0] @ w[p + "dq"].T, 1e-5) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(H, D + R)
    down = h[0] @ w[p + "dkv"].T
    c = plain.rms(down[:rank], 1e-5) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).reshape(H, D)
    v = (c @ w[p + "uv"].T).reshape(H, V)
    heads = []
    for a in range(H):
        e = torch.exp((q[a, :D] @ k[a] + q[a, D:] @ down[rank:]) * mixer["scale"])
        heads.append(v[a] * e / (e + torch.exp(w[p + "sink"][a])))
    gate = torch.sigmoid(h[0] @ w[p + "g"].T)
    assert torch.allclose((torch.cat(heads) * gate) @ w[p + "o"].T, y[0], atol=1e-10)
    if mixer.get("mask") is not None and mixer["mask"]["size"] < 6:
        # rows beyond the window do not depend on the first row
        h2 = h.clone()
        h2[0] += 1.0
        y2 = plain.latent_attention(h2, w, p, mixer, 1e-5)
        size = mixer["mask"]["size"]
        assert torch.equal(y2[size:], y[size:]) and (size == 1 or not torch.equal(y2[size - 1], y[size - 1]))


def test_gated_feed_forward_alone(tmp_path):
    from akas_b200.ops import reference

    g = torch.Generator().manual_seed(4)
    gu = torch.randn(5, 2 * 12 + 3, generator=g) * 2.0
    bias = torch.randn(24, generator=g)
    got = reference.gated_activation(gu, 12, bias, "gelu_tanh", torch.float32)
    z, u = (gu[:, :12] + bias[:12]).double(), (gu[:, 12:24] + bias[12:]).double()
    assert torch.allclose(got.double(), plain.gelu_tanh(z) * u, atol=1e-6)
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12
    res = torch.zeros(5, 7)
    reference.gated_activation(gu, 12, None, "gelu_tanh", torch.float32, residual=res, residual_bias=torch.arange(7.0))
    assert torch.equal(res, torch.arange(7.0).expand(5, 7))
    config = model(40, 70, [att(ATT_FULL, 28)])
    w, toks, want = one_mechanism(config, tmp_path)
    for name in ("l0.mlp.gate.b", "l0.mlp.up.b", "l0.mlp.down.b"):
        assert np.abs(plain.forward(toks, dict(w, **{name: w[name] * 0}), config).numpy() - want).max() > 1e-3 * np.abs(want).max()


# --------------------------------------------------------------------------- what a position sees


def seen_case(device, dtype, ops, tmp_path, decode, kind):
    """One layer: the logits at position i change with the token at position j iff i sees j: every j <= i for the
    causal layer (keys far back, at page borders, the first tokens, next to the query); 0 <= i - j < window for the
    windowed one (just inside and just outside the window, which starts inside a page); with the query in a prompt's
    portion or decoded alone."""
    from akas_b200.engine.batch import StepEntry

    i = 290
    if kind == "attention":
        config = model(48, 120, [att(ATT, None)])
        folder, _ = make_folder(config, seed=44, folder=tmp_path / "edge", sharp=False)
        w = plant(folder, config, key_token=119, query_token=118)  # token 119 at position j is felt by token 118 at position i
        cases = [(0, True), (1, True), (7, True), (8, True), (63, True), (64, True), (255, True), (256, True), (i - 1, True),
                 (i, True), (i + 1, False), (299, False)]
    else:
        window = 70 if kind == "window above a page" else 11
        mixer = dict(LAT, mask=dict(size=window))
        config = model(48, 120, [lat(mixer, None)])
        folder, _ = make_folder(config, seed=44, folder=tmp_path / "edge", sharp=False)
        w = plant_latent(folder, config, key_token=119, query_token=118)
        first = i - window + 1  # the first position that i sees
        cases = [(0, False), (1, False), (first - 9, False), (first - 2, False), (first - 1, False), (first, True), (first + 1, True),
                 (i - 1, True), (i, True), (i + 1, False)]
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
        return out.float().cpu().numpy()[0]

    ref = logits_at_i(base)
    for j, seen in cases:
        changed = list(base)
        changed[j] = 119 if j != i else 7
        got = logits_at_i(changed)
        diff = np.abs(got - ref).max()
        if seen:
            # (the latent layer's values are small beside the residual stream: a key that takes all the weight moves less)
            assert diff > (2e-2 if kind == "attention" else 5e-3) * np.abs(ref).max(), f"position {i} does not see {j}"
        else:
            assert diff == 0.0, f"position {i} sees {j} (difference {diff})"
        if dtype == "float32" and seen:
            want = plain.forward(changed[: i + 1], w, config)[i].numpy()
            assert np.abs(got - want).max() <= TOL[dtype] * np.abs(want).max()


KINDS = ["attention", "window below a page", "window above a page"]


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
    """One key far back among hundreds is made to stand out (its key and the last token's queries are long along a
    channel that the rotation leaves alone): the last position's attention must find it through scattered pages, in
    a portion and decoded alone, in the layer that owns the cache and in the layer that only reads it."""
    from akas_b200.engine.batch import StepEntry

    config = model(48, 120, [att(ATT, None), att(ATT, None, kv_from=0)])
    folder, _ = make_folder(config, seed=47, folder=tmp_path / "far", sharp=False)
    w = plant(folder, config, key_token=119, query_token=118, strength=1.1, loud=4.0)
    toks = prompts(118, [500], seed=2)[0]
    toks[3], toks[-1] = 119, 118  # the key appears once, far back; the query is the last token
    want = plain.forward(toks, w, config)[-1].numpy()
    without = list(toks)
    without[3] = 5
    felt = np.abs(plain.forward(without, w, config)[-1].numpy() - want).max()
    assert felt > 0.05 * np.abs(want).max(), "the far key does not stand out"
    # the reader alone feels it too: with the owner's queries blind to the channel the difference stays
    blind = dict(w)
    blind["l0.mix.q"] = w["l0.mix.q"].clone()
    blind["l0.mix.q"][ATT["dim"] - 1 :: ATT["dim"]] = 0.0
    assert np.abs(plain.forward(without, blind, config)[-1].numpy() - plain.forward(toks, blind, config)[-1].numpy()).max() > 0.02 * np.abs(want).max()
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


def test_freed_pages_are_used_again_and_not_read(tmp_path):
    """Two requests one after the other in a pool of one slot and just enough pages: the second gets the first one's
    pages (also those a window gave back early) and must compute as if it were alone."""
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
    """Bit for bit on the plain operations: a request's logits beside three others of other lengths, and alone."""
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
    cfg = EngineConfig(dtype=dtype, device=device, page_size=8, max_requests=3, context=128, max_tokens=512, prefill_chunk=13,
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
    """200 decoded tokens for three requests of different lengths through captured graphs (every window passes over
    decoded tokens, pages behind it are given back on the way), against one whole pass of the plain model."""
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
    want = {i: plain.forward(p + feed[i], w, config).numpy()[len(p):] for i, p in enumerate(ps)}
    compare({i: np.stack(r) for i, r in enumerate(rows)}, want, dtype, f"long decoding/{dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(dtype, tmp_path):
    """bin/trace_run as a user calls it, on a Penopel folder: steps on standard input, logits as files."""
    config = CONFIGS["latent"]
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
    want = {rid: plain.forward(t, w, config).numpy() for rid, t in reqs.items()}
    at = {rid: 0 for rid in reqs}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if not wanted:
            continue
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(wanted, config["vocab"])
        row = 0
        for e in s["entries"]:
            for k in e["want"]:
                ref = want[e["id"]][at[e["id"]] + k]
                assert np.abs(data[row] - ref).max() <= TOL[dtype] * np.abs(want[e["id"]]).max(), (s["step"], e["id"], k)
                row += 1
            at[e["id"]] += len(e["tokens"])


# --------------------------------------------------------------------------- the kernels one by one


def _batch(lengths, device):
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=device)
    seq = torch.repeat_interleave(torch.arange(len(lengths)), torch.tensor(lengths)).to(torch.int32).to(device)
    return cu, seq


def _close(got, want, tol, what):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= tol, f"{what}: {err:.3g} > {tol}"


@pytest.mark.gpu
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,c", [(9, 20), (300, 52), (7, 50), (1, 1), (33, 1024)])
def test_dynamic_tanh_kernel(n, c, out_dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["elementwise"])
    g = torch.Generator().manual_seed(n + c)
    x = (torch.randn(n, c, generator=g) * 3.0).cuda()
    alpha, w, b = torch.tensor(0.7).cuda(), torch.randn(c, generator=g).cuda(), torch.randn(c, generator=g).cuda()
    tol = 1e-6 if out_dtype == torch.float32 else 5e-3
    _close(cuda.dynamic_tanh(x, alpha, w, b, out_dtype), reference.dynamic_tanh(x, alpha, w, b, out_dtype), tol, "all rows")
    rows = torch.tensor([n - 1, 0, n // 2], dtype=torch.int32).cuda()
    got = cuda.dynamic_tanh(x, alpha, w, b, out_dtype, rows)
    assert got.shape == (3, c)
    _close(got, reference.dynamic_tanh(x, alpha, w, b, out_dtype, rows), tol, "gathered rows")


@pytest.mark.gpu
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,f,pad", [(5, 12, 3), (130, 320, 0), (2, 1100, 16), (40, 7, 2)])
def test_gated_activation_kernel(n, f, pad, out_dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["elementwise"])
    g = torch.Generator().manual_seed(n + f)
    wide = (torch.randn(n, 2 * f + pad, generator=g) * 2.0).cuda()
    bias = torch.randn(2 * f, generator=g).cuda()
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    for activation in ("gelu_tanh", "silu"):
        for b in (bias, None):
            _close(cuda.gated_activation(wide, f, b, activation, out_dtype), reference.gated_activation(wide, f, b, activation, out_dtype),
                   tol, f"{activation} bias {b is not None}")
    res = torch.randn(n, 11, generator=g).cuda()
    want = res + torch.arange(11.0).cuda()
    cuda.gated_activation(wide, f, bias, "gelu_tanh", out_dtype, residual=res, residual_bias=torch.arange(11.0).cuda())
    _close(res, want, 1e-7, "the bias the next product's sum starts from")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_rank,kv_rank,rot,interleaved,page", [(40, 32, 8, True, 8), (28, 18, 6, True, 16), (16, 24, 0, False, 64),
                                                                (96, 200, 64, False, 32), (300, 512, 64, True, 64)])
def test_latent_norm_store_kernel(q_rank, kv_rank, rot, interleaved, page, dtype):
    from akas_b200.ops import cuda, reference

    cuda.require(["latent", "rope"])
    g = torch.Generator().manual_seed(q_rank + kv_rank)
    starts, lengths = [150, 0, 77, 301], [1, 45, 30, 1]
    blocks = -(-400 // page)
    table = torch.randperm(4 * blocks, generator=g).to(torch.int32).view(4, blocks).cuda()
    n = sum(lengths)
    _, seq = _batch(lengths, "cuda")
    pos = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lengths)]).to(torch.int32).cuda()
    proj = (torch.randn(n, q_rank + kv_rank + rot + 24, generator=g) * 3.0).cuda()
    qw, kw = (1.0 + 0.3 * torch.randn(q_rank, generator=g)).cuda(), (1.0 + 0.3 * torch.randn(kv_rank, generator=g)).cuda()
    cos = sin = None
    if rot:
        inv_freq = (torch.tensor(300.0, dtype=torch.float64) ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).cuda()
        cos, sin = cuda.rope_tables(pos, inv_freq)
    fresh = torch.randn(4 * blocks, 1, page, kv_rank + rot, generator=g).to(dtype).cuda()
    pools = [fresh.clone(), fresh.clone(), fresh.clone()]
    out = [ops.latent_norm_store(proj, q_rank, kv_rank, rot, qw, kw, 1e-5, cos, sin, interleaved, pool, table, seq, pos, page)
           for ops, pool in zip((reference, cuda), pools)]
    tol = 2e-6 if dtype == torch.float32 else 5e-3
    _close(out[1], out[0], tol, "query latent")
    _close(pools[1], pools[0], tol, "pages")
    assert not torch.equal(pools[1], fresh)
    same = cuda.latent_norm_store(proj, q_rank, kv_rank, rot, qw, kw, 1e-5, cos, sin, interleaved, pools[2], table, seq, pos, page, write=False)
    assert torch.equal(pools[2], fresh) and torch.equal(same, out[1])
    # against the oracle: row 1 of the step is position 0 of its request, where nothing turns
    row = proj[1].double().cpu()
    c = plain.rms(row[q_rank : q_rank + kv_rank], 1e-5) * kw.double().cpu()
    stored = pools[0][table[1, 0].item(), 0, 0].double().cpu()
    _close(stored, torch.cat([c, row[q_rank + kv_rank : q_rank + kv_rank + rot]]), tol, "the cache row against the oracle")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,o,k,t,n", [(4, 32, 24, 8, 37), (20, 48, 8, 16, 37), (3, 18, 20, 6, 37), (5, 24, 16, 0, 37),
                                           (2, 300, 72, 0, 37), (3, 40, 520, 4, 37), (16, 64, 512, 0, 37), (1, 7, 5, 2, 37),
                                           (6, 96, 64, 32, 150), (6, 64, 96, 0, 21), (3, 32, 16, 8, 64), (2, 512, 128, 64, 200),
                                           (40, 48, 160, 0, 2100), (5, 16, 32, 6, 70)])
def test_head_linear_kernel(heads, o, k, t, n, dtype):
    """Sizes for the plain kernel and (inner and outer sizes that are multiples of 16, in bfloat16) for the one on the
    tensor cores: a part of a tile, several tiles, more tiles than a block's share."""
    from akas_b200.ops import cuda, reference

    cuda.require(["latent", "rope"])
    g = torch.Generator().manual_seed(heads + o + k)
    wide = torch.randn(n, heads * (k + t) + 8, generator=g).to(dtype).cuda()
    x = wide[:, : heads * (k + t)]
    w = (torch.randn(heads, o, k, generator=g) / k ** 0.5).to(dtype).cuda()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    _close(cuda.head_linear(x, w, heads), reference.head_linear(x, w, heads), tol, "plain")
    gates = torch.randn(n, heads * o + 4, generator=g).cuda()
    for gate in (gates[:, : heads * o], gates[:, : heads * o].to(dtype).contiguous()):
        _close(cuda.head_linear(x, w, heads, gate=gate), reference.head_linear(x, w, heads, gate=gate), tol, "gated")
    if t:
        pos = torch.arange(100, 100 + n, dtype=torch.int32).cuda()
        inv_freq = (torch.tensor(50.0, dtype=torch.float64) ** (-2.0 * torch.arange(t // 2, dtype=torch.float64) / t)).cuda()
        cos, sin = cuda.rope_tables(pos, inv_freq)
        for interleaved in (False, True):
            got = cuda.head_linear(x, w, heads, cos=cos, sin=sin, interleaved=interleaved)
            _close(got, reference.head_linear(x, w, heads, cos=cos, sin=sin, interleaved=interleaved), tol, f"tails turned {interleaved}")
        # the tail against the oracle's rotation
        tails = x.double().cpu().reshape(n, heads, k + t)[:, :, k:]
        want = plain.rotate(tails, dict(base=50.0, dims=t), interleaved=True, first_position=100)
        _close(got.reshape(n, heads, o + t)[:, :, o:], want, tol, "tails against the oracle")
    # a token's result does not depend on its place in the batch or on the batch
    alone = cuda.head_linear(x[20:21], w, heads)
    assert torch.equal(alone[0], cuda.head_linear(x, w, heads)[20])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot,page", [(6, 2, 24, 16, 16, 8), (4, 4, 16, 24, 16, 16), (3, 1, 20, 28, 6, 4),
                                                             (8, 2, 128, 64, 64, 64)])
def test_biased_projections_kernels(heads, kv_heads, dim, vdim, rot, page, dtype):
    """qk_norm_store fed with a float32 product and biases, writing pages of the compute dtype; with nothing to write,
    only the queries are read (the keys' and values' pointers may be anything); then attention with a unit sink."""
    from types import SimpleNamespace

    from akas_b200.ops import cuda, reference

    cuda.require(["attention_general", "rope"])
    g = torch.Generator().manual_seed(heads + dim)
    starts, lengths = [150, 0, 77, 301], [1, 45, 30, 1]
    blocks = -(-400 // page)
    table = torch.randperm(4 * blocks, generator=g).to(torch.int32).view(4, blocks).cuda()
    k_pool = torch.randn(4 * blocks, kv_heads, page, dim, generator=g).to(dtype).cuda()
    v_pool = torch.randn(4 * blocks, kv_heads, page, vdim, generator=g).to(dtype).cuda()
    n = sum(lengths)
    cu, seq = _batch(lengths, "cuda")
    pos = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lengths)]).to(torch.int32).cuda()
    nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
    proj = torch.randn(n, nq + nk + nv + 16, generator=g).cuda()
    bias = torch.randn(nq + nk + nv, generator=g).cuda()
    q, k, v = proj[:, :nq], proj[:, nq : nq + nk], proj[:, nq + nk : nq + nk + nv]
    biases = dict(q_bias=bias[:nq], k_bias=bias[nq : nq + nk], v_bias=bias[nq + nk :])
    inv_freq = (torch.tensor(10000.0, dtype=torch.float64) ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).cuda()
    cos, sin = cuda.rope_tables(pos, inv_freq)
    pools = [(k_pool.clone(), v_pool.clone()) for _ in range(2)]
    qn = [ops.qk_norm_store(q, k, v, heads, kv_heads, dim, vdim, None, None, 0.0, kp, vp, table, seq, pos, page, cos=cos, sin=sin,
                            interleaved=False, **biases) for ops, (kp, vp) in zip((reference, cuda), pools)]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert qn[1].dtype == dtype
    _close(qn[1], qn[0], tol, "rotated q")
    _close(pools[1][0], pools[0][0], tol, "k pages")
    _close(pools[1][1], pools[0][1], tol, "v pages")
    want_q = plain.rotate((q + bias[:nq])[1:46].double().cpu().reshape(45, heads, dim), dict(base=10000.0, dims=rot), interleaved=False)
    _close(qn[0][1:46], want_q.reshape(45, -1), tol, "bias and rotation against the oracle")
    page_of = table[1, 44 // page].item()
    _close(pools[1][1][page_of, :, 44 % page].reshape(-1), (v + bias[nq + nk :])[45], tol, "biased values in the pages")
    kept = (pools[1][0].clone(), pools[1][1].clone())
    reader = cuda.qk_norm_store(q, q, q, heads, kv_heads, dim, vdim, None, None, 0.0, *pools[1], table, seq, pos, page, write=False,
                                cos=cos, sin=sin, interleaved=False, q_bias=bias[:nq])
    assert torch.equal(reader, qn[1]) and torch.equal(pools[1][0], kept[0]) and torch.equal(pools[1][1], kept[1])
    ctx = SimpleNamespace(query_lens=tuple(lengths), decode_only=False, cu_seqlens=cu, max_context=400)
    want = reference.attention_general(qn[0], *pools[0], table, seq, pos, 0.2, None, 0, 0.0, None, None, True, None, page)
    none = reference.attention_general(qn[0], *pools[0], table, seq, pos, 0.2, None, 0, 0.0, None, None, False, None, page)
    assert (want - none).abs().max() > 0.02, "the one in the denominator does not matter"
    for layout in (None, ctx):
        got = cuda.attention_general(qn[0], *pools[0], table, seq, pos, 0.2, None, 0, 0.0, None, None, True, None, page, layout)
        _close(got, want, 2e-5 if dtype == torch.float32 else 1.5e-2, f"attention with a unit sink {layout is None}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,width,vdim,window,page", [(4, 40, 32, 11, 8), (20, 64, 48, 70, 64), (3, 24, 18, 5, 16), (5, 24, 24, None, 32),
                                                         (16, 128, 96, 100, 64), (70, 16, 8, 33, 64), (8, 576, 512, 128, 64)])
def test_attention_over_rows_that_hold_key_and_value(heads, width, vdim, window, page, dtype):
    """One key/value head whose rows are key and, by their first channels, value, shared by all query heads; windows
    that start inside pages; learned sinks; prompt portions beside decoded tokens, and a step of single tokens with
    keys in parts."""
    from types import SimpleNamespace

    from akas_b200.ops import cuda, reference

    cuda.require(["attention_general"])
    g = torch.Generator().manual_seed(heads + width)
    starts, lengths = [150, 0, 77, 301], [1, 45, 30, 1]
    blocks = -(-400 // page)
    table = torch.randperm(4 * blocks, generator=g).to(torch.int32).view(4, blocks).cuda()
    pool = torch.randn(4 * blocks, 1, page, width, generator=g).to(dtype).cuda()
    n = sum(lengths)
    cu, seq = _batch(lengths, "cuda")
    pos = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lengths)]).to(torch.int32).cuda()
    q = (torch.randn(n, heads * width, generator=g) * (2.0 / width ** 0.5)).to(dtype).cuda()
    sinks = (torch.randn(heads, generator=g) * 2.0).cuda()
    args = (0.9, window, 0, None, None, None, False, None, page)
    want = reference.attention_general(q, pool, pool, table, seq, pos, *args, sinks=sinks, values_in_keys=vdim)
    assert want.shape == (n, heads * vdim)
    # the plain statement against attention over a separate copy of the values
    copy = pool[..., :vdim].contiguous()
    assert torch.equal(reference.attention_general(q, pool, copy, table, seq, pos, *args, sinks=sinks), want)
    ctx = SimpleNamespace(query_lens=tuple(lengths), decode_only=False, cu_seqlens=cu, max_context=400)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for layout in (None, ctx):
        got = cuda.attention_general(q, pool, pool, table, seq, pos, *args, layout, sinks=sinks, values_in_keys=vdim)
        _close(got, want, tol, f"rows as keys and values {layout is None}")
    singles = [399, 130, 64, 257]
    pos1 = torch.tensor(singles, dtype=torch.int32).cuda()
    cu1, seq1 = _batch([1, 1, 1, 1], "cuda")
    q1 = q[:4].contiguous()
    want1 = reference.attention_general(q1, pool, pool, table, seq1, pos1, *args, sinks=sinks, values_in_keys=vdim)
    for most in (0, 400):
        ctx1 = SimpleNamespace(query_lens=(1, 1, 1, 1), decode_only=True, cu_seqlens=cu1, max_context=most)
        got1 = cuda.attention_general(q1, pool, pool, table, seq1, pos1, *args, ctx1, sinks=sinks, values_in_keys=vdim)
        _close(got1, want1, tol, f"single tokens, keys in parts: {most > 0}")


def _plain_gated(x, w2, f, bias, activation):
    gu = x.double() @ w2.double().T
    g, u = gu[:, :f], gu[:, f : 2 * f]
    if bias is not None:
        g, u = g + bias[:f].double(), u + bias[f:].double()
    act = g * torch.sigmoid(g) if activation == "silu" else 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    return act * u


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,k,o", [(3, 64, 48), (16, 192, 320), (9, 2048, 48), (1, 128, 1008), (40, 264, 528), (128, 2048, 320),
                                   (17, 64, 16), (300, 96, 208), (2048, 256, 512), (333, 520, 1168), (5, 100, 36), (60, 52, 20)])
def test_products_with_biases_and_a_gated_read_out(n, k, o, dtype):
    """x . w^T + b rounded once, added into a float32 stream, and act(g + b_g) * (u + b_u) from the stacked gate and up
    matrices, at sizes for each product kernel (few tokens, up to 128, more) and sizes that none of them takes."""
    from akas_b200.ops import cuda

    cuda.require()
    g = torch.Generator().manual_seed(n + k + o)
    x = torch.randn(n, k, generator=g).to(dtype).cuda()
    w = (torch.randn(o, k, generator=g) * 0.05).to(dtype).cuda()
    b = torch.randn(o, generator=g).cuda()
    tol = 3e-6 * max(1.0, (k / 64) ** 0.5) if dtype == torch.float32 else 1e-2
    want = x.double() @ w.double().T + b.double()
    got = cuda.linear(x, w, bias=b)
    assert got.dtype == dtype
    _close(got, want, tol, "bias, rounded once")
    _close(cuda.linear(x, w, out_dtype=torch.float32, bias=b), want, tol, "bias, float32 out")
    h = (torch.randn(n, o, generator=g) * 2.0).cuda()
    h0 = h.clone()
    assert cuda.linear(x, w, residual=h, bias=b) is h
    _close(h, h0.double() + want, tol, "bias and product into the stream")
    if o % 2 == 0:
        f = o // 2
        for activation in ("gelu_tanh", "silu"):
            for bias in (b, None):
                got = cuda.linear_gated(x, w, f, bias, activation)
                assert got.shape == (n, f) and got.dtype == dtype
                _close(got, _plain_gated(x, w, f, bias, activation), tol, f"gated {activation} bias {bias is not None}")
    padded = torch.cat([w, torch.zeros(16, k, dtype=dtype, device="cuda")])  # rows of padding below the two matrices
    if o % 2 == 0:
        _close(cuda.linear_gated(x, padded, o // 2, b, "gelu_tanh"), _plain_gated(x, w, o // 2, b, "gelu_tanh"), tol, "padded")
    assert cuda.skinny_status() == 0 and cuda.gemm_rows_status() == 0 and cuda.gemm_pair_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,o", [(1, 64, 48), (8, 192, 320), (9, 2048, 48), (16, 1024, 1008), (5, 128, 16), (3, 100, 40), (20, 64, 32)])
def test_a_norm_without_sums_in_front_of_a_product(m, k, o):
    """tanh(alpha x) * w + b of gathered float32 rows as the way into a product of few tokens, with the plain, the
    float32 and the gated read-out; sizes the kernel does not take are refused with None."""
    from akas_b200.ops import cuda

    cuda.require()
    g = torch.Generator().manual_seed(m + k + o)
    h = (torch.randn(m + 3, k, generator=g) * 3.0).cuda()
    alpha = torch.tensor(0.6).cuda()
    nw, nb = torch.randn(k, generator=g).cuda(), (torch.randn(k, generator=g) * 0.3).cuda()
    w = (torch.randn(o, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    bias = torch.randn(o, generator=g).cuda()
    rows = torch.randperm(m + 3, generator=g)[:m].to(torch.int32).cuda()
    for r in (None, rows):
        src = h[:m] if r is None else h[r.long()]
        normed = (torch.tanh(alpha.double() * src.double()) * nw.double() + nb.double()).to(torch.bfloat16)
        want = normed.double() @ w.double().T
        got = cuda.dyt_linear(h[:m].contiguous() if r is None else h, alpha, nw, nb, w, None, r)
        if k % 64 or m > 16:
            assert got is None
            return
        assert got.dtype == torch.bfloat16
        _close(got, want, 1e-2, "rounded out")
        got = cuda.dyt_linear(h[:m].contiguous() if r is None else h, alpha, nw, nb, w, torch.float32, r)
        assert got.dtype == torch.float32
        _close(got, want, 2e-3, "float32 out")
        for activation in ("gelu_tanh", "silu"):
            for b in (bias, None):
                got = cuda.dyt_linear(h[:m].contiguous() if r is None else h, alpha, nw, nb, w, None, r, gated=(o // 2, b, activation))
                _close(got, _plain_gated(normed, w, o // 2, b, activation), 1e-2, f"gated {activation} bias {b is not None}")
    assert cuda.skinny_status() == 0
