"""Tiny Penopel configurations of the tests' own, and a folder of random weights shaped so that faults show.

Sizes differ from layer to layer and between the configurations: value heads smaller and larger than the keys',
query heads over 1, 2 or as many key/value heads, rotations of a whole head, of a part and of nothing, with and
without slowed long waves; latents narrower and wider than a head, windows of one token, below a page, above a page
and none, more heads than a block of the general kernel takes at once, rows that the tensor-core kernels take and
that they do not, layers without a feed-forward, layers that read another layer's cache (one cache read by two),
widths that are no multiple of 8.
"""

import json
from pathlib import Path

import torch

SLOWED = dict(factor=8.0, low=2.0, high=6.0, original=64)  # waves of 10.7 to 32 positions are blended, longer ones slowed

ATT = dict(heads=6, kv_heads=2, dim=24, vdim=16, scale=0.31, rot=dict(base=10000.0, dims=16, scaling=SLOWED))
ATT_FULL = dict(heads=4, kv_heads=4, dim=16, vdim=24, scale=0.4, rot=dict(base=500.0, dims=16))
ATT_ODD = dict(heads=3, kv_heads=1, dim=20, vdim=28, scale=0.27, rot=dict(base=1000000.0, dims=6))
ATT_BARE = dict(heads=36, kv_heads=2, dim=8, vdim=8, scale=0.5, rot=dict(base=100.0, dims=0))

LAT = dict(heads=4, dim=24, rot_dim=8, vdim=16, q_rank=40, kv_rank=32, scale=0.3, mask=dict(size=11),
           rot=dict(base=10000.0, dims=8))
LAT_WIDE = dict(heads=20, dim=8, rot_dim=16, vdim=12, q_rank=24, kv_rank=48, scale=0.45, mask=dict(size=70),
                rot=dict(base=300.0, dims=16, scaling=SLOWED))
LAT_ODD = dict(heads=3, dim=20, rot_dim=6, vdim=12, q_rank=28, kv_rank=18, scale=0.27, mask=dict(size=5),
               rot=dict(base=1000000.0, dims=6))
LAT_SELF = dict(heads=2, dim=12, rot_dim=4, vdim=20, q_rank=10, kv_rank=14, scale=0.5, mask=dict(size=1),
                rot=dict(base=50.0, dims=4))
ATT_BIG = dict(heads=4, kv_heads=1, dim=128, vdim=128, scale=0.09, rot=dict(base=500000.0, dims=128))
ATT_MID = dict(heads=8, kv_heads=4, dim=64, vdim=32, scale=0.125, rot=dict(base=10000.0, dims=32, scaling=SLOWED))
LAT_ROW64 = dict(heads=12, dim=48, rot_dim=16, vdim=16, q_rank=128, kv_rank=48, scale=0.15, mask=dict(size=64),
                 rot=dict(base=1000000.0, dims=16))
LAT_ROW320 = dict(heads=2, dim=128, rot_dim=64, vdim=128, q_rank=32, kv_rank=256, scale=0.07, mask=dict(size=33),
                  rot=dict(base=100.0, dims=64))
LAT_OPEN = dict(heads=5, dim=16, rot_dim=0, vdim=8, q_rank=16, kv_rank=24, scale=0.35, rot=dict(base=10.0, dims=0))  # no mask, no rotation


def layer(kind, mixer, ff, **more):
    return dict(type=kind, mixer=dict(mixer, **more), mlp=None if ff is None else dict(kind="dense", ff=ff))


def att(mixer, ff, **more):
    return layer("attention", mixer, ff, **more)


def lat(mixer, ff):
    return layer("latent_attention", mixer, ff)


def model(width, vocab, layers, eps=1e-5, scale=3.0, cap=12.0):
    out = dict(architecture="Penopel", width=width, vocab=vocab, norm=dict(eps=eps), embedding=dict(scale=scale), layers=layers)
    if cap is not None:
        out["logit_softcap"] = cap
    return out


CONFIGS = {
    "mix": model(80, 200, [
        lat(LAT, 48),
        att(ATT, 56),
        lat(LAT_WIDE, None),
        att(ATT, 40, kv_from=1),
        att(ATT_FULL, 24),
        att(ATT, None, kv_from=1),
        lat(LAT_OPEN, 32),
    ]),
    "odd": model(52, 90, [lat(LAT_ODD, 20), att(ATT_ODD, 36), lat(LAT_SELF, None), att(ATT_ODD, 12, kv_from=1)], eps=1e-6, scale=1.7,
                 cap=None),
    # sizes that are multiples of nothing much: rows of 50 and 77
    "ragged": model(50, 77, [att(ATT_BARE, 10), lat(LAT_ODD, 14), att(ATT_BARE, None, kv_from=0)], eps=1e-3, scale=-2.2, cap=5.0),
    "latent": model(48, 120, [lat(LAT, None), lat(LAT_WIDE, 24)], scale=4.0),
    # sizes that the tensor-core kernels take (heads of 128 and 64 with values of 128 and 32, cached rows of 64) beside a
    # cached row of 320 numbers that they do not; windows of a page, of half a page and none
    "mid": model(128, 300, [att(ATT_BIG, 192), lat(LAT_ROW64, 192), lat(LAT_ROW320, 192), att(ATT_MID, 192)], eps=1e-6, scale=11.3,
                 cap=None),
}
PAGE = {"mix": 8, "odd": 16, "ragged": 32, "latent": 64, "mid": 64}
LENGTHS = {"mix": [1, 45, 2, 97, 33, 130, 64], "odd": [70, 3, 41, 100], "ragged": [75, 2, 140], "latent": [90, 1, 150],
           "mid": [200, 129, 64]}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}  # largest |difference| over largest |reference logit|


def make_folder(config, seed, folder, sharp=True):
    """A model folder with random weights. ``sharp``: queries and keys large enough for peaked scores; always: sinks of
    both signs and of the scores' size, norms with slopes of their own, shifts and biases that are not small."""
    from safetensors.torch import save_file

    from akas_b200.config import config_from_dict
    from akas_b200.weights import random_tensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config_from_dict(config), seed=seed, std=0.08, dtype="float32")
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(tensors):
        if sharp and name.endswith(("mix.q", "mix.k", "mix.uq", "mix.uk")):
            tensors[name] = tensors[name] * 2.5
        if name.endswith("mix.dkv"):
            tensors[name] = tensors[name] * 4.0  # the shared rotated key part is not normed: as large as the normed latent
        if name.endswith("mix.sink"):
            tensors[name] = torch.randn(tensors[name].shape, generator=g) * 2.0
        if name.endswith(".alpha"):
            tensors[name] = 0.3 + torch.rand(tensors[name].shape, generator=g)
        if name.endswith(".b"):
            tensors[name] = torch.randn(tensors[name].shape, generator=g) * 0.3
    tensors = {k: v.to(torch.bfloat16).contiguous() for k, v in tensors.items()}  # stored as a checkpoint stores them
    save_file(tensors, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(config))
    return folder, {k: v.to(torch.float64) for k, v in tensors.items()}


def _signs(c):
    u, u2 = torch.ones(c), torch.ones(c)
    u[1::2] = -1.0
    u2[2::4] = u2[3::4] = -1.0
    return u, u2


def plant(folder, config, key_token, query_token, strength=0.7, loud=1.0):
    """Rewrites a folder whose layer 0 is an attention layer so that ``query_token``'s queries and ``key_token``'s
    keys are long along one channel that the rotation leaves alone: wherever the two stand, the query's score for that
    key is far above the others', so the key is felt among hundreds. The two tokens' embeddings are two orthogonal
    vectors of +-1 (the norm keeps their signs); the channel's row of every query head (of EVERY attention layer, also
    of those that read layer 0's cache) points along the query token's, of every key head along the key token's.
    ``loud``: the value matrices times this, so that what the key brings is large beside the residual stream."""
    from safetensors.torch import load_file, save_file

    m = config["layers"][0]["mixer"]
    channel = m["dim"] - 1
    assert config["layers"][0]["type"] == "attention" and m["rot"]["dims"] <= channel
    tensors = load_file(str(Path(folder) / "model.safetensors"))
    c = config["width"]
    assert c % 4 == 0
    u, u2 = _signs(c)
    tensors["embed"][key_token] = u.to(torch.bfloat16)
    tensors["embed"][query_token] = u2.to(torch.bfloat16)
    for i, entry in enumerate(config["layers"]):
        if entry["type"] != "attention":
            continue
        for a in range(m["heads"]):
            tensors[f"l{i}.mix.q"][a * m["dim"] + channel] = (strength * u2 / c ** 0.5).to(torch.bfloat16)
        if entry["mixer"].get("kv_from") is None:
            for a in range(m["kv_heads"]):
                tensors[f"l{i}.mix.k"][a * m["dim"] + channel] = (strength * u / c ** 0.5).to(torch.bfloat16)
            tensors[f"l{i}.mix.v"] = (tensors[f"l{i}.mix.v"].float() * loud).to(torch.bfloat16)
    save_file(tensors, str(Path(folder) / "model.safetensors"))
    return {k: v.to(torch.float64) for k, v in tensors.items()}


def plant_latent(folder, config, key_token, query_token, strength=3.0):
    """The same for a folder whose layer 0 is a latent attention layer, through the latents: the key token's latent is
    long along its channel 0 (the down projection's row 0 points along the key token's embedding; after the norm that
    channel holds nearly all of the latent), every head's plain key channel 0 reads latent channel 0, and likewise the
    query latent's channel 0, the query token and every head's plain query channel 0."""
    from safetensors.torch import load_file, save_file

    m = config["layers"][0]["mixer"]
    assert config["layers"][0]["type"] == "latent_attention"
    tensors = load_file(str(Path(folder) / "model.safetensors"))
    c = config["width"]
    assert c % 4 == 0
    u, u2 = _signs(c)
    tensors["embed"][key_token] = u.to(torch.bfloat16)
    tensors["embed"][query_token] = u2.to(torch.bfloat16)
    tensors["l0.mix.dkv"][0] = (strength * u / c ** 0.5).to(torch.bfloat16)
    tensors["l0.mix.dq"][0] = (strength * u2 / c ** 0.5).to(torch.bfloat16)
    for a in range(m["heads"]):
        tensors["l0.mix.uk"][a * m["dim"], 0] = 1.0
        tensors["l0.mix.uq"][a * (m["dim"] + m["rot_dim"]), 0] = 1.0
    save_file(tensors, str(Path(folder) / "model.safetensors"))
    return {k: v.to(torch.float64) for k, v in tensors.items()}


def prompts(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
