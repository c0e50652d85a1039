"""A plain, slow statement of the Kidarax decoder: the tests' oracle.

One function per mechanism, in float64 torch on the CPU. It shares no code with the engine: weights come as a dict
of tensors under the checkpoint's names, sizes and constants from the configuration dict.

Notation: x is the residual stream [T, C] of ONE sequence whose first token has position 0, h a normed copy of it;
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


def silu(z):
    return z * torch.sigmoid(z)


def rates(rot):
    """One turning rate per rotated pair and the factor on both tables.

    Pair i turns at base^(-2i / dims). ``scaling`` with only a factor divides every rate by it. ``scaling`` with
    ``original`` as well blends: with d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    r_i rate / factor + (1 - r_i) rate, and cosine and sine are both multiplied by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], float(rot["base"])
    out = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc is None:
        return out, 1.0
    factor = float(sc["factor"])
    if "original" not in sc:
        return [f / factor for f in out], 1.0

    def d(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo, hi = max(math.floor(d(sc["fast"])), 0), min(math.ceil(d(sc["slow"])), dims - 1)
    blended = []
    for i, f in enumerate(out):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        blended.append(f / factor * r + f * (1.0 - r))
    return blended, 0.1 * math.log(factor) + 1.0


def rotate(y, rot, first_position=0):
    """Rotary positions on the first rot.dims channels of every head of y [T, heads, D]; the other channels pass.
    Pair i is (channel i, channel i + dims / 2)."""
    T = y.shape[0]
    dims = rot["dims"]
    out = y.clone()
    pos = torch.arange(first_position, first_position + T, dtype=F)
    freq, amp = rates(rot)
    for i, f in enumerate(freq):
        a, b = i, i + dims // 2
        ang = pos * f
        c, s = amp * torch.cos(ang)[:, None], amp * torch.sin(ang)[:, None]
        u, v = y[:, :, a], y[:, :, b]
        out[:, :, a] = u * c - v * s
        out[:, :, b] = v * c + u * s
    return out


def retention(h, w, p, m, eps, trace=None):
    """Linear attention with one constant decay per head and no softmax: S_t = a S_(t-1) + (k_t / sqrt(dim)) v_t^T,
    o_t = S_t^T q_t; every head's o over its root mean square (no weight), the heads side by side times
    silu(W_g h), then W_o. ``trace`` receives the last state [heads, dim, vdim]."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, H, D) * D ** -0.5
    v = (h @ w[p + "v"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F)
    S = torch.zeros(H, D, V, dtype=F)
    decay = torch.tensor([float(a) for a in m["decay"]], dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    if trace is not None:
        trace.append(S)
    o = rms(out, eps).reshape(T, H * V) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def attention(h, w, p, m):
    """Causal grouped-query softmax attention with biased projections, rotary positions on the first rot.dims
    channels of a head, the score scale of the configuration, and the heads' outputs times sigmoid(W_g h), channel
    by channel."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, D), m["rot"])
    k = rotate((h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, D), m["rot"])
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, V)
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        for a in range(H):
            g = a // (H // G)
            s = (k[: i + 1, g] @ q[i, a]) * m["scale"]
            out[i, a] = torch.softmax(s, dim=0) @ v[: i + 1, g]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * V) * gate) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values come out of one low-rank latent. Per head the query is [dim plain channels,
    rot_dim rotated]; the plain keys and the values are two projections of the normed latent c, and one rotated key
    part (rows kv_rank.. of the down projection, not normed) serves all heads. Causal; the softmax's denominator
    holds exp(sink_h) too; head a's output is multiplied by sigmoid(W_g h)_a, one number a head."""
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = dict(m["rot"], dims=R)
    q = (h @ w[p + "q"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[:, :, :D], rotate(q[:, :, D:], rot)
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate(down[:, rank:].reshape(T, 1, R), rot)[:, 0]
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        for a in range(H):
            s = (k_plain[: i + 1, a] @ q_plain[i, a] + k_rot[: i + 1] @ q_rot[i, a]) * m["scale"]
            e = torch.exp(s - s.max())
            out[i, a] = (e / (e.sum() + torch.exp(w[p + "sink"][a] - s.max()))) @ v[: i + 1, a]
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, H]
    return (out * gate[:, :, None]).reshape(T, H * V) @ w[p + "o"].T


def expert(h, w, p):
    """W_down (silu(W_gate h) * (W_up h))."""
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, r, margins=None):
    """The chosen experts [T, top] and their weights: the largest of sigmoid(W_router h), as they are. ``margins``, a
    list, receives per token the gap between the last logit that was chosen and the first that was not."""
    z = h @ w[p + "router"].T
    s = torch.sigmoid(z)
    weights, chosen = torch.topk(s, r["top"], dim=-1)
    if margins is not None:
        ordered = torch.sort(z, dim=-1, descending=True).values
        margins.append((ordered[:, r["top"] - 1] - ordered[:, r["top"]]).tolist() if r["top"] < s.shape[1] else [1.0] * h.shape[0])
    return chosen, weights


def feed_forward(h, w, p, mlp, margins=None):
    """``dense``: W_down relu(W_up h)^2. ``moe``: every token's chosen experts run on the token's row times the
    expert's weight, and their results are summed; an expert that every token passes is added, times
    sigmoid(W_sg h), one number a token."""
    if mlp["kind"] == "dense":
        return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T
    chosen, weights = route(h, w, p, mlp["router"], margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            out[t] += expert(g * h[t], w, f"{p}e{e}.")
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.")
    return out


def run_order(cfg):
    """(layer, whether the embedding's output is added in front of it) for every layer run: the layers
    loop.start .. loop.stop - 1 run loop.times times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if loop is None:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for turn in range(loop["times"]):
        order += [(i, turn > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(tokens, w, cfg, trace=None, margins=None):
    """Logits [T, vocab] of one sequence; ``trace``, a list, receives the residual stream after every layer run;
    ``margins``, a list, one list per routed layer run of the tokens' routing margins (see ``route``)."""
    w = {k: v.to(F) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    first = w["embed"][torch.as_tensor(tokens)]
    x = first
    for i, again in run_order(cfg):
        entry = cfg["layers"][i]
        p, m = f"l{i}.", entry["mixer"]
        if again:
            x = x + first
        h = dyt(x, w, p + "norm1")
        if entry["type"] == "retention":
            y = retention(h, w, p + "mix.", m, eps)
        elif entry["type"] == "attention":
            y = attention(h, w, p + "mix.", m)
        else:
            y = latent_attention(h, w, p + "mix.", m, eps)
        x = x + dyt(y, w, p + "norm1b")
        if entry.get("mlp") is not None:
            x = x + dyt(feed_forward(dyt(x, w, p + "norm2"), w, p + "mlp.", entry["mlp"], margins), w, p + "norm2b")
        if trace is not None:
            trace.append(x.clone())
    return dyt(x, w, "final.norm") @ w["embed"].T * cfg.get("logit_scale", 1.0)
