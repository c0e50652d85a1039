"""Tiny Kidarax configurations of the tests' own, and a folder of random weights shaped so that faults show.

Sizes differ from layer to layer and between the configurations: retention heads whose keys are narrower and wider
than their values, decays from 0 to 1 and the same for all heads; query heads over 1, 2 or as many key/value heads,
value heads smaller and larger than the keys', rotations of a whole head, of a part and of nothing, with and without
a scaling; latents narrower and wider than a head, rotated parts of other sizes than the plain part, blends whose
edges lie inside and outside the pairs; dense and routed feed-forwards and none, one and several experts a token,
with and without the expert that every token passes, of another size than the routed ones; loops over one layer, over
all layers, over none, once and three times; widths that are no multiple of 8.
"""

import json
from pathlib import Path

import torch

RET = dict(heads=3, dim=16, vdim=24, decay=[0.9, 0.97, 0.995])
RET_WIDE = dict(heads=2, dim=40, vdim=8, decay=[1.0, 0.5])
RET_ODD = dict(heads=5, dim=6, vdim=10, decay=[0.0, 0.99, 0.999, 0.9, 0.8])
RET_MID = dict(heads=4, dim=64, vdim=32, decay=[0.98, 0.99, 0.995, 0.999])

ATT = dict(heads=6, kv_heads=2, dim=24, vdim=16, scale=0.31, rot=dict(base=10000.0, dims=16, scaling=dict(factor=4.0)))
ATT_FULL = dict(heads=4, kv_heads=4, dim=16, vdim=24, scale=0.4, rot=dict(base=500.0, dims=16))
ATT_ODD = dict(heads=3, kv_heads=1, dim=20, vdim=28, scale=0.27, rot=dict(base=1000000.0, dims=6, scaling=dict(factor=1.5)))
ATT_BARE = dict(heads=12, kv_heads=2, dim=8, vdim=8, scale=0.5, rot=dict(base=100.0, dims=0))
ATT_MID = dict(heads=8, kv_heads=4, dim=64, vdim=32, scale=0.125, rot=dict(base=10000.0, dims=32, scaling=dict(factor=8.0)))

BLEND = dict(factor=6.0, original=48, fast=8.0, slow=0.5)  # the blend's edges lie inside the pairs of a part of 16 at base 300
LAT = dict(heads=4, dim=24, rot_dim=8, vdim=16, kv_rank=32, scale=0.3, rot=dict(base=10000.0, dims=8, scaling=dict(BLEND, original=16)))
LAT_WIDE = dict(heads=20, dim=8, rot_dim=16, vdim=12, kv_rank=48, scale=0.45, rot=dict(base=300.0, dims=16, scaling=BLEND))
LAT_ODD = dict(heads=3, dim=20, rot_dim=6, vdim=12, kv_rank=18, scale=0.27, rot=dict(base=1000000.0, dims=6))
LAT_OPEN = dict(heads=5, dim=16, rot_dim=0, vdim=8, kv_rank=24, scale=0.35, rot=dict(base=10.0, dims=0))  # no rotation
LAT_ROW64 = dict(heads=12, dim=48, rot_dim=16, vdim=16, kv_rank=48, scale=0.15,
                 rot=dict(base=1000000.0, dims=16, scaling=dict(factor=16.0, original=64, fast=32.0, slow=1.0)))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, shared=None):
    out = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared is not None:
        out["shared"] = dict(ff=shared)
    return out


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=dict(mixer), mlp=mlp)


def ret(mixer, mlp):
    return layer("retention", mixer, mlp)


def att(mixer, mlp):
    return layer("attention", mixer, mlp)


def lat(mixer, mlp):
    return layer("latent_attention", mixer, mlp)


def model(width, vocab, layers, loop=None, eps=1e-5, logit_scale=0.7):
    out = dict(architecture="Kidarax", width=width, vocab=vocab, norm=dict(eps=eps), layers=layers, logit_scale=logit_scale)
    if loop is not None:
        out["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return out


CONFIGS = {
    "mix": model(80, 200, [
        ret(RET, moe(24, 6, 2, shared=40)),
        lat(LAT, dense(48)),
        att(ATT, moe(16, 5, 1)),
        ret(RET_WIDE, None),
        lat(LAT_WIDE, moe(32, 3, 3, shared=8)),
        att(ATT_FULL, dense(24)),
    ], loop=(1, 4, 3)),
    "odd": model(52, 90, [lat(LAT_ODD, moe(20, 4, 2, shared=12)), ret(RET_ODD, dense(36)), att(ATT_ODD, None), lat(LAT_OPEN, moe(12, 7, 1))],
                 loop=(0, 4, 2), eps=1e-6, logit_scale=1.3),
    # sizes that are multiples of nothing much: rows of 50 and 77; a loop over nothing
    "ragged": model(50, 77, [att(ATT_BARE, moe(10, 3, 2, shared=6)), ret(RET_ODD, None), lat(LAT_ODD, dense(14))], loop=(1, 1, 4), eps=1e-3,
                    logit_scale=-2.2),
    "alone": model(48, 120, [ret(RET, dense(24)), lat(LAT, moe(24, 4, 1, shared=24))]),  # no loop at all
    # sizes that the tensor-core kernels take, with a looped last layer
    "mid": model(128, 300, [ret(RET_MID, dense(192)), att(ATT_MID, moe(64, 8, 2, shared=64)), lat(LAT_ROW64, moe(128, 4, 1, shared=192))],
                 loop=(2, 3, 2), eps=1e-6, logit_scale=0.5),
}
PAGE = {"mix": 8, "odd": 16, "ragged": 32, "alone": 64, "mid": 64}
LENGTHS = {"mix": [1, 45, 2, 97, 33, 130, 64], "odd": [70, 3, 41, 100], "ragged": [75, 2, 140], "alone": [90, 1, 150],
           "mid": [200, 129, 64]}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}  # largest |difference| over largest |reference logit|


def make_folder(config, seed, folder, sharp=True, std=0.08):
    """A model folder with random weights of deviation ``std`` (a wide model wants a smaller one, or every product
    saturates the norm behind it). ``sharp``: queries and keys large enough for peaked scores; always: sinks of both
    signs and of the scores' size, norms with slopes of their own, shifts and biases that are not small, routers whose
    scores spread over (0, 1)."""
    from safetensors.torch import save_file

    from akas_b200.config import config_from_dict
    from akas_b200.weights import random_tensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config_from_dict(config), seed=seed, std=std, dtype="float32")
    g = torch.Generator().manual_seed(seed + 1)
    kinds = {f"l{i}.": entry["type"] for i, entry in enumerate(config["layers"])}
    for name in list(tensors):
        kind = kinds.get(name.split("mix.")[0]) if "mix." in name else None
        if sharp and kind != "retention" and name.endswith(("mix.q", "mix.k", "mix.uk")):
            tensors[name] = tensors[name] * 2.5
        if name.endswith("mix.dkv"):
            tensors[name] = tensors[name] * 4.0  # the shared rotated key part is not normed: as large as the normed latent
        if name.endswith("mix.sink"):
            tensors[name] = torch.randn(tensors[name].shape, generator=g) * 2.0
        if name.endswith(("mlp.router", "shared.sg")):
            tensors[name] = tensors[name] * (0.48 / std) * min(1.0, (64.0 / config["width"]) ** 0.5)  # logits of a few units at any width
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


def _rewrite(folder, change):
    from safetensors.torch import load_file, save_file

    tensors = load_file(str(Path(folder) / "model.safetensors"))
    change(tensors)
    save_file(tensors, str(Path(folder) / "model.safetensors"))
    return {k: v.to(torch.float64) for k, v in tensors.items()}


def plant(folder, config, key_token, query_token, strength=0.7, loud=1.0):
    """Rewrites a folder whose layer 0 is an attention layer so that ``query_token``'s queries and ``key_token``'s keys
    are long along one channel that the rotation leaves alone: wherever the two stand, the query's score for that key
    is far above the others', so the key is felt among hundreds. The two tokens' embeddings are two orthogonal vectors
    of +-1 (the norm keeps their signs); the channel's row of every query head points along the query token's, of
    every key head along the key token's. ``loud``: the value matrix times this."""
    m = config["layers"][0]["mixer"]
    channel = m["dim"] - 1
    assert config["layers"][0]["type"] == "attention" and m["rot"]["dims"] <= channel
    c = config["width"]
    u, u2 = _signs(c)

    def change(t):
        t["embed"][key_token] = u.to(torch.bfloat16)
        t["embed"][query_token] = u2.to(torch.bfloat16)
        for a in range(m["heads"]):
            t["l0.mix.q"][a * m["dim"] + channel] = (strength * u2 / c ** 0.5).to(torch.bfloat16)
        for a in range(m["kv_heads"]):
            t["l0.mix.k"][a * m["dim"] + channel] = (strength * u / c ** 0.5).to(torch.bfloat16)
        t["l0.mix.v"] = (t["l0.mix.v"].float() * loud).to(torch.bfloat16)
        t["l0.mix.g"] = (t["l0.mix.g"].float() * 0.1).to(torch.bfloat16)  # gates near a half: what attention finds gets through

    return _rewrite(folder, change)


def plant_latent(folder, config, key_token, query_token, strength=3.0):
    """The same for a folder whose layer 0 is a latent attention layer, through the latent: the key token's latent is
    long along its channel 0 (the down projection's row 0 points along the key token's embedding; after the norm that
    channel holds nearly all of the latent), every head's plain key channel 0 reads latent channel 0, and every head's
    plain query channel 0 points along the query token's embedding."""
    m = config["layers"][0]["mixer"]
    assert config["layers"][0]["type"] == "latent_attention"
    c = config["width"]
    u, u2 = _signs(c)

    def change(t):
        t["embed"][key_token] = u.to(torch.bfloat16)
        t["embed"][query_token] = u2.to(torch.bfloat16)
        t["l0.mix.dkv"][0] = (strength * u / c ** 0.5).to(torch.bfloat16)
        for a in range(m["heads"]):
            t["l0.mix.uk"][a * m["dim"], 0] = 1.0
            t["l0.mix.q"][a * (m["dim"] + m["rot_dim"])] = (strength * u2 / c ** 0.5).to(torch.bfloat16)
        t["l0.mix.g"] = (t["l0.mix.g"].float() * 0.1).to(torch.bfloat16)

    return _rewrite(folder, change)


def prompts(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
