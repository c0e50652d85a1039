"""A plain, slow statement of the Penopel decoder: the tests' oracle.

One function per mechanism, in float64 torch on the CPU, query by query. It shares no code with the engine: weights
come as a dict of tensors under the checkpoint's names, sizes and constants from the configuration dict.

Notation: x is the residual stream [T, C] of ONE sequence whose first token has position 0, h its normed copy;
W y means ``y @ W.T`` for a stored [out, in] matrix.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def dyt(x, w, name):
    """The norm without statistics: tanh(alpha x) * weight + shift, alpha one learned number."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def rms(y, eps):
    """y over the root of (the mean of its squares plus eps), along the last axis."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def frequencies(rot):
    """One turning rate per rotated pair: base^(-2i / dims), then, where ``scaling`` is given, long waves slowed:
    a wave shorter than original / high keeps its rate, one longer than original / low turns ``factor`` times
    slower, and between the two the rate is blended by where original / wavelength lies between low and high."""
    dims = rot["dims"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        if sc is not None:
            wave = 2.0 * math.pi / f
            if wave > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wave >= sc["original"] / sc["high"]:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate(y, rot, interleaved, first_position=0):
    """Rotary positions on the first rot.dims channels of every head of y [T, heads, D]; the other channels pass.
    Pair i is (channel i, channel i + dims / 2), or, ``interleaved``, (channel 2i, channel 2i + 1)."""
    T = y.shape[0]
    dims = rot["dims"]
    out = y.clone()
    pos = torch.arange(first_position, first_position + T, dtype=F)
    for i, f in enumerate(frequencies(rot)):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + dims // 2)
        ang = pos * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = y[:, :, a], y[:, :, b]
        out[:, :, a] = u * c - v * s
        out[:, :, b] = v * c + u * s
    return out


def keys_and_values(h, w, p, m):
    """What an attention layer with projections of its own leaves for itself and for the layers that read it: keys
    after the rotation [T, G, D], values [T, G, V]."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, D)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, V)
    return rotate(k, m["rot"], interleaved=False), v


def attention(h, w, p, m, kv=None):
    """Causal grouped-query attention with biased projections, rotate-half rotary on the first rot.dims channels, and
    a softmax whose denominator holds one more term exp(0) that has no value. ``kv``: another layer's rotated keys
    and its values, for a layer that has none of its own."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, D), m["rot"], interleaved=False)
    k, v = kv if kv is not None else keys_and_values(h, w, p, m)
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        for a in range(H):
            g = a // (H // G)
            e = torch.exp((k[: i + 1, g] @ q[i, a]) * m["scale"])
            out[i, a] = (e / (1.0 + e.sum())) @ v[: i + 1, g]
    return out.reshape(T, H * V) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Attention whose queries, keys and values come out of low-rank latents. Per head the query is [dim plain
    channels, rot_dim rotated]; the plain keys and the values are two projections of the normed latent c, and one
    rotated key part (rows kv_rank.. of the down projection, not normed) serves all heads. Position i sees j with
    0 <= i - j < mask.size; the denominator holds exp(sink_h) too; the heads' outputs pass sigmoid(W_g h)."""
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = dict(m["rot"], dims=R)
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[:, :, :D], rotate(q[:, :, D:], rot, interleaved=True)
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate(down[:, rank:].reshape(T, 1, R), rot, interleaved=True)[:, 0]
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    size = m["mask"]["size"] if m.get("mask") is not None else T + 1  # no mask: every earlier position
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        lo = max(0, i - size + 1)
        for a in range(H):
            s = (k_plain[lo : i + 1, a] @ q_plain[i, a] + k_rot[lo : i + 1] @ q_rot[i, a]) * m["scale"]
            e = torch.exp(s)
            out[i, a] = (e / (e.sum() + torch.exp(w[p + "sink"][a]))) @ v[lo : i + 1, a]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * V) * gate) @ w[p + "o"].T


def feed_forward(h, w, p):
    """W_down (gelu(W_gate h + b) * (W_up h + b)) + b."""
    act = gelu_tanh(h @ w[p + "gate"].T + w[p + "gate.b"]) * (h @ w[p + "up"].T + w[p + "up.b"])
    return act @ w[p + "down"].T + w[p + "down.b"]


def forward(tokens, w, cfg, trace=None):
    """Logits [T, vocab] of one sequence; ``trace``, a list, receives the residual stream after every layer."""
    w = {k: v.to(F) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    left = {}  # layer -> (rotated keys, values) of the attention layers that project their own
    for i, entry in enumerate(cfg["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        h = dyt(x, w, p + "norm1")
        if entry["type"] == "attention":
            if m.get("kv_from") is not None:
                x = x + attention(h, w, p + "mix.", m, kv=left[m["kv_from"]])
            else:
                left[i] = keys_and_values(h, w, p + "mix.", m)
                x = x + attention(h, w, p + "mix.", m, kv=left[i])
        else:
            x = x + latent_attention(h, w, p + "mix.", m, eps)
        if entry.get("mlp") is not None:
            x = x + feed_forward(dyt(x, w, p + "norm2"), w, p + "mlp.")
        if trace is not None:
            trace.append(x.clone())
    logits = dyt(x, w, "final.norm") @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
