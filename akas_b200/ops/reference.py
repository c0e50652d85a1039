"""Plain PyTorch statements of every kernel, with the kernels' own signatures.

Each function here says, in a few tensor expressions, what the CUDA kernel of
the same name in ``akas_b200.ops.cuda`` computes: same arguments, same layouts
of pages, block tables and state slots, same in-place effects. The kernel tests
compare each kernel with its neighbour here, and the step function's host logic
(batches, pages, slots) can be exercised on a CPU by handing this module to the
runner as ``ops``. The engine never picks it by itself: without the compiled
kernels it fails.

Layouts. Pages: ``[num_pages, kv_heads, page_size, head_dim]``. Block table:
int32 ``[requests, max_blocks]``, ``-1`` where a request holds no page. Flat
batch: ``seq_of_token[N]`` names each token's request (row of the block table and
of ``slots``; ``-1`` marks padding that must touch nothing), ``positions[N]`` its
absolute position, ``cu_seqlens[R + 1]`` the extent of each request's tokens.
"""

from __future__ import annotations

import torch

name = "reference"


def embedding(token_ids, table):
    return table[token_ids.long()].to(torch.float32)


def rmsnorm(x, weight, eps, zero_centered, out_dtype, rows=None):
    if rows is not None:
        x = x[rows.long()]
    xf = x.to(torch.float32)
    w = weight.to(torch.float32)
    if zero_centered:
        w = w + 1.0
    y = xf * torch.rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps) * w
    return y.to(out_dtype)


def linear(x, w, out_dtype=None, residual=None, bias=None):
    """x [N, K] times w [O, K] transposed, float32 accumulation, plus ``bias`` (float32 [O]) where one is given, before
    the one rounding; ``residual`` (float32) is added to in place."""
    y = x.to(torch.float32) @ w.to(torch.float32).T
    if bias is not None:
        y = y + bias
    if residual is not None:
        residual += y
        return residual
    return y.to(out_dtype or x.dtype)


def swiglu(gate_up):
    f = gate_up.shape[-1] // 2
    g = gate_up[:, :f].to(torch.float32)
    u = gate_up[:, f:].to(torch.float32)
    return (g / (1 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear_swiglu(x, w_gate_up):
    return swiglu(linear(x, w_gate_up))


def norm_linear(h, norm_weight, eps, zero_centered, w, out_dtype=None, rows=None, swiglu_out=False):
    x = rmsnorm(h, norm_weight, eps, zero_centered, w.dtype, rows)
    return linear_swiglu(x, w) if swiglu_out else linear(x, w, out_dtype=out_dtype)


def short_conv(bcx, taps, bias, state, cu_seqlens, seq_of_token, slots, decode_only=False, write=True):
    n, c3 = bcx.shape
    c = c3 // 3
    l = taps.shape[1]
    bf = bcx.to(torch.float32)
    u = bf[:, :c] * bf[:, 2 * c :]
    gate = bf[:, c : 2 * c]
    out = torch.zeros((n, c), dtype=torch.float32, device=bcx.device)
    cu = cu_seqlens.tolist()
    for r, slot in enumerate(slots.tolist()):
        a, b = cu[r], cu[r + 1]
        if slot < 0 or b <= a:
            continue
        hist = torch.cat((state[slot], u[a:b]), dim=0)  # [L-1 + n_r, C], oldest first
        acc = torch.zeros((b - a, c), dtype=torch.float32, device=bcx.device)
        for j in range(l):
            acc = acc + hist[j : j + b - a] * taps[:, j]
        if bias is not None:
            acc = acc + bias
        out[a:b] = gate[a:b] * acc
        if write:
            state[slot] = hist[-(l - 1) :]
    return out.to(bcx.dtype)


def add_bias(x, bias, out_dtype=None):
    """x float32 [N, C] plus bias [C], rounded once to ``out_dtype``; in place when that is float32."""
    if out_dtype in (None, torch.float32):
        return x.add_(bias)
    return (x + bias).to(out_dtype)


def scale_cap(x, scale=1.0, cap=0.0):
    """In place on float32 x: times ``scale``, then ``cap * tanh(x / cap)`` where ``cap`` > 0."""
    x.mul_(scale)
    if cap > 0:
        x.copy_(cap * torch.tanh(x / cap))
    return x


def rope_tables(positions, inv_freq, amplitude=1.0):
    """cos and sin of position x rate, both times ``amplitude``, float32 [N, pairs]."""
    ang = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    return (amplitude * torch.cos(ang)).to(torch.float32), (amplitude * torch.sin(ang)).to(torch.float32)


def _page_addresses(block_table, seq_of_token, positions, page_size):
    live = seq_of_token >= 0
    seq = seq_of_token.clamp(min=0).long()
    pos = positions.long()
    page = block_table[seq, pos // page_size].long()
    return live, page, pos % page_size


def kv_store(k, v, k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    """k, v: [N, kv_heads * head_dim] -> pages at each live token's (page, offset)."""
    kh, d = k_pool.shape[1], k_pool.shape[3]
    live, page, off = _page_addresses(block_table, seq_of_token, positions, page_size)
    k_pool[page[live], :, off[live]] = k.reshape(-1, kh, d)[live].to(k_pool.dtype)
    v_pool[page[live], :, off[live]] = v.reshape(-1, kh, d)[live].to(v_pool.dtype)


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, zero_centered, cos, sin,
                       k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    """Per-head RMSNorm of q and k, rotation of both, k (in place in ``qkv``) and v into the pages; returns q."""
    n = qkv.shape[0]
    d = head_dim
    q = qkv[:, : heads * d].reshape(n, heads, d).to(torch.float32)
    k = qkv[:, heads * d : (heads + kv_heads) * d].reshape(n, kv_heads, d).to(torch.float32).clone()  # written back below
    if q_weight is not None:
        q = rmsnorm(q, q_weight, eps, zero_centered, torch.float32)
        k = rmsnorm(k, k_weight, eps, zero_centered, torch.float32)
    if cos is not None:
        half = cos.shape[1]

        def rotate(x):
            left, right, rest = x[..., :half], x[..., half : 2 * half], x[..., 2 * half :]
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.cat((left * c - right * s, left * s + right * c, rest), dim=-1)

        q, k = rotate(q), rotate(k)
    qkv[:, heads * d : (heads + kv_heads) * d] = k.reshape(n, kv_heads * d).to(qkv.dtype)
    if k_pool is not None:
        kv_store(qkv[:, heads * d : (heads + kv_heads) * d], qkv[:, (heads + kv_heads) * d :], k_pool, v_pool,
                 block_table, seq_of_token, positions, page_size)
    return q.reshape(n, heads * d).to(qkv.dtype)


def paged_attention(q, k_pool, v_pool, block_table, seq_of_token, positions, scale, window, page_size, ctx=None):
    n = q.shape[0]
    kh, d = k_pool.shape[1], k_pool.shape[3]
    heads = q.shape[1] // d
    group = heads // kh
    out = torch.zeros((n, heads * d), dtype=torch.float32, device=q.device)
    seqs, poss = seq_of_token.tolist(), positions.tolist()
    for t in range(n):
        r, p = seqs[t], poss[t]
        if r < 0:
            continue
        first = 0 if window is None else max(0, p - window + 1)
        idx = torch.arange(first, p + 1, device=q.device)
        pages = block_table[r, idx // page_size].long()
        offs = idx % page_size
        keys = k_pool[pages, :, offs].to(torch.float32)  # [S, kh, d]
        vals = v_pool[pages, :, offs].to(torch.float32)
        qt = q[t].reshape(kh, group, d).to(torch.float32)
        scores = torch.einsum("kgd,skd->kgs", qt, keys) * scale
        prob = torch.softmax(scores, dim=-1)
        out[t] = torch.einsum("kgs,skd->kgd", prob, vals).reshape(heads * d)
    return out.to(q.dtype)


def argmax(logits):
    """Greedy token per row; ties go to the lowest index."""
    top = logits.max(dim=-1, keepdim=True).values
    v = logits.shape[-1]
    idx = torch.arange(v, device=logits.device).expand_as(logits)
    return torch.where(logits == top, idx, v).min(dim=-1).values.to(torch.int32)


def sample(logits, temperature, top_k, top_p, uniform):
    """Per row with temperature T: T <= 0 is the argmax. Else w_i = exp((x_i - max x) / T); tokens are ranked by
    logit, larger first, equal logits by id, lower first (the order of the reference's rank loop,
    src/akas/ops/vocabulary/kernel.py:586-622). Token i is kept iff its rank is below top_k (top_k <= 0 or >= V:
    no limit) and the kept tokens ranked before it hold at most top_p of the kept mass (top_p >= 1: no limit);
    the result is the first kept i, in index order, whose running kept mass exceeds uniform * (kept mass)."""
    out = argmax(logits).clone()
    m, v = logits.shape
    for r in range(m):
        t = float(temperature[r])
        if t <= 0:
            continue
        x = logits[r].to(torch.float32)
        w = torch.exp((x - x.max()) * torch.tensor(1.0 / t, dtype=torch.float32, device=x.device)).double()
        order = torch.sort(x, descending=True, stable=True).indices  # equal logits: the lower id first
        rank = torch.empty(v, dtype=torch.long, device=x.device)
        rank[order] = torch.arange(v, device=x.device)
        keep = torch.ones(v, dtype=torch.bool, device=x.device)
        k = int(top_k[r])
        if 0 < k < v:
            keep &= rank < k
        p = float(top_p[r])
        if p < 1.0:
            kept_w = torch.where(keep, w, torch.zeros_like(w))
            before = torch.cumsum(kept_w[order], 0) - kept_w[order]  # kept mass ranked before each token
            keep &= before[rank] <= p * kept_w.sum()
        kept_w = torch.where(keep, w, torch.zeros_like(w))
        run = torch.cumsum(kept_w, 0)
        hit = torch.nonzero(keep & (run > float(uniform[r]) * run[-1]))
        out[r] = int(hit[0]) if len(hit) else int(torch.nonzero(keep)[-1])
    return out


def adjust_logits(logits, softcap, penalty, history):
    """The stages before top-k of the reference's sampler (src/akas/ops/vocabulary/kernel.py:556-577), in place:
    x = c tanh(x / c) where the row's softcap c > 0; then every token of the row's history (-1: none), once, becomes
    x / q if x > 0 else x * q where the row's penalty q != 1."""
    for r in range(logits.shape[0]):
        c, q = float(softcap[r]), float(penalty[r])
        if c > 0:
            logits[r] = c * torch.tanh(logits[r] / c)
        if q != 1.0:
            tokens = torch.unique(history[r][history[r] >= 0]).long()
            x = logits[r, tokens]
            logits[r, tokens] = torch.where(x > 0, x / q, x * q)
    return logits


def take_tokens(token_ids, source, previous):
    live = source >= 0
    token_ids[live] = previous[source[live].long()]


def zero_rows(state, slot):
    state[:, slot].zero_()


# --------------------------------------------------------------------------- learned positions, PolyNorm


def add_rows(h, table, index):
    """h[n] += table[index[n]] in place (h float32)."""
    h += table[index.long()].to(torch.float32)
    return h


def polynorm(z, coeffs, eps, out_dtype):
    """a N(z) + b N(z^2) + c N(z^3) + e per row, N(x) = x / sqrt(mean(x^2) + eps); coeffs = (a, b, c, e), float32."""
    zf = z.to(torch.float64)
    c = coeffs.to(torch.float64)

    def unit(x):
        return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)

    return (c[0] * unit(zf) + c[1] * unit(zf * zf) + c[2] * unit(zf ** 3) + c[3]).to(out_dtype)


# --------------------------------------------------------------------------- recurrent mixers
#
# State layouts. A request's state row lives at ``state[slot]``; ``slots[r]`` is the slot of the step's request r
# (-1: padding, touch nothing) and ``cu_seqlens`` gives the extent of its tokens. A matrix state is a head's S
# transposed, ``[slots, heads, value_dim, key_dim]`` float32 (the kernels' threads own runs of key channels); a
# convolution's state ``[slots, taps - 1, channels]`` float32, oldest
# row first. Both may be views into a wider row per slot (only the slot stride is free).


def decay_gates(low, w_up, bias, tau):
    """sigmoid(low . w_up + bias)^(1 / tau) in float32: [N, O] for low [N, R] (any float dtype), w_up [R, O] (the up
    matrix of a low-rank pair, transposed)."""
    z = low.to(torch.float64) @ w_up.to(torch.float64) + bias.to(torch.float64)
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau).to(torch.float32)


def _requests(cu_seqlens, slots):
    cu = cu_seqlens.tolist()
    for r, slot in enumerate(slots.tolist()):
        if slot >= 0 and cu[r + 1] > cu[r]:
            yield slot, cu[r], cu[r + 1]


def gla_scan(q, k, v, alpha, state, cu_seqlens, slots, heads, dim, vdim, q_scale, write=True):
    """Per request and head, token by token: S <- diag(alpha_t) S + k_t v_t^T; o_t = S^T (q_scale q_t).
    q, k, alpha [N, heads * dim], v [N, heads * vdim] -> o float32 [N, heads * vdim]."""
    n = q.shape[0]
    o = torch.zeros((n, heads, vdim), dtype=torch.float32, device=q.device)
    qf = q.to(torch.float64).reshape(n, heads, dim) * q_scale
    kf = k.to(torch.float64).reshape(n, heads, dim)
    vf = v.to(torch.float64).reshape(n, heads, vdim)
    af = alpha.to(torch.float64).reshape(n, heads, dim)
    for slot, a, b in _requests(cu_seqlens, slots):
        s = state[slot].to(torch.float64)
        for t in range(a, b):
            s = af[t][:, None, :] * s + vf[t][:, :, None] * kf[t][:, None, :]
            o[t] = torch.einsum("hvd,hd->hv", s, qf[t]).to(torch.float32)
        if write:
            state[slot] = s.to(torch.float32)
    return o.reshape(n, heads * vdim)


def decay_scan(q, k, v, decay, state, cu_seqlens, slots, heads, dim, vdim, q_scale, activation=None, write=True, longest=None):
    """Per request and head, token by token: S <- decay_h S + k_t v_t^T; o_t = S^T (q_scale q_t) with one constant
    decay per head (float32 [heads]); ``activation="silu"``: q, k and v pass silu first.
    q, k [N, heads * dim], v [N, heads * vdim] -> o float32 [N, heads * vdim]; state [slots, heads, vdim, dim]."""
    n = q.shape[0]
    o = torch.zeros((n, heads, vdim), dtype=torch.float32, device=q.device)
    qf, kf, vf = (t.to(torch.float64) for t in (q, k, v))
    if activation == "silu":
        qf, kf, vf = (t * torch.sigmoid(t) for t in (qf, kf, vf))
    qf = qf.reshape(n, heads, dim) * q_scale
    kf = kf.reshape(n, heads, dim)
    vf = vf.reshape(n, heads, vdim)
    df = decay.to(torch.float64).reshape(heads, 1, 1)
    for slot, a, b in _requests(cu_seqlens, slots):
        s = state[slot].to(torch.float64)
        for t in range(a, b):
            s = df * s + vf[t][:, :, None] * kf[t][:, None, :]
            o[t] = torch.einsum("hvd,hd->hv", s, qf[t]).to(torch.float32)
        if write:
            state[slot] = s.to(torch.float32)
    return o.reshape(n, heads * vdim)


def causal_conv_silu(x, taps, state, cu_seqlens, seq_of_token, slots, write=True):
    """silu of a causal depthwise convolution over each request's tokens: y_t = silu(sum_j taps[:, j] x_(t - L + 1 + j)),
    inputs before the step's first token from ``state`` (zero at a request's start). x [N, C] -> float32 [N, C]."""
    n, c = x.shape
    l = taps.shape[1]
    xf = x.to(torch.float32)
    out = torch.zeros((n, c), dtype=torch.float32, device=x.device)
    for slot, a, b in _requests(cu_seqlens, slots):
        hist = torch.cat((state[slot], xf[a:b]), dim=0)
        acc = torch.zeros((b - a, c), dtype=torch.float32, device=x.device)
        for j in range(l):
            acc = acc + hist[j : j + b - a] * taps[:, j]
        out[a:b] = acc * torch.sigmoid(acc)
        if write and l > 1:
            state[slot] = hist[-(l - 1):]
    return out


def delta_prep(y, kv_heads, dim, q_scale, unit_eps, b, a, a_log, dt_bias):
    """What the delta rule needs besides its convolved inputs. In place on float32 y [N, >= 2 kv_heads dim]: each
    head of q (the first kv_heads * dim columns) and of k (the next) becomes x / sqrt(sum x^2 + unit_eps), q times
    q_scale too. Returns (beta, g), float32 [N, H]: beta = sigmoid(b), g = exp(-exp(a_log) * softplus(a + dt_bias))."""
    n = y.shape[0]
    qk = y[:, : 2 * kv_heads * dim].reshape(n, 2 * kv_heads, dim).to(torch.float64)
    qk = qk / torch.sqrt((qk * qk).sum(dim=-1, keepdim=True) + unit_eps)
    qk[:, :kv_heads] *= q_scale
    y[:, : 2 * kv_heads * dim] = qk.reshape(n, -1).to(torch.float32)
    beta = torch.sigmoid(b.to(torch.float64)).to(torch.float32)
    g = torch.exp(-torch.exp(a_log.to(torch.float64)) * torch.nn.functional.softplus(a.to(torch.float64) + dt_bias.to(torch.float64)))
    return beta, g.to(torch.float32)


def delta_scan(q, k, v, beta, g, state, cu_seqlens, slots, heads, kv_heads, dim, vdim, write=True):
    """Per request and head, token by token: S <- g_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t.
    q, k [N, kv_heads * dim] (head h reads q/k head h // (heads / kv_heads)), v [N, heads * vdim] -> o float32."""
    n = q.shape[0]
    rep = heads // kv_heads
    o = torch.zeros((n, heads, vdim), dtype=torch.float32, device=q.device)
    qf = q.to(torch.float64).reshape(n, kv_heads, dim).repeat_interleave(rep, dim=1)
    kf = k.to(torch.float64).reshape(n, kv_heads, dim).repeat_interleave(rep, dim=1)
    vf = v.to(torch.float64).reshape(n, heads, vdim)
    bf, gf = beta.to(torch.float64), g.to(torch.float64)
    for slot, a, b in _requests(cu_seqlens, slots):
        s = state[slot].to(torch.float64)
        for t in range(a, b):
            s = gf[t][:, None, None] * s
            u = bf[t][:, None] * (vf[t] - torch.einsum("hvd,hd->hv", s, kf[t]))
            s = s + u[:, :, None] * kf[t][:, None, :]
            o[t] = torch.einsum("hvd,hd->hv", s, qf[t]).to(torch.float32)
        if write:
            state[slot] = s.to(torch.float32)
    return o.reshape(n, heads * vdim)


def gated_rmsnorm(o, weight, eps, gate, heads, vdim, out_dtype, gate_activation="silu", out=None, out_scale=1.0):
    """Each head of o [N, heads * vdim] over its root mean square (eps under the root), times weight [vdim] (None: ones), times
    silu(gate) [N, heads * vdim] (or, ``gate_activation="sigmoid"``, sigmoid(gate)), times ``out_scale``; written into
    ``out`` (a view [N, heads * vdim] whose rows may be parts of wider rows) where that is given. A norm over all
    heads together is the call with heads = 1."""
    n = o.shape[0]
    of = o.to(torch.float64).reshape(n, heads, vdim)
    of = of / torch.sqrt((of * of).mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        of = of * weight.to(torch.float64)
    gf = gate.to(torch.float64)
    act = torch.sigmoid(gf) if gate_activation == "sigmoid" else gf * torch.sigmoid(gf)
    y = of.reshape(n, heads * vdim) * act * out_scale
    if out is not None:
        out.copy_(y.to(out.dtype))
        return out
    return y.to(out_dtype)


# --------------------------------------------------------------------------- general attention


def qk_norm_store(q, k, v, heads, kv_heads, dim, vdim, q_weight, k_weight, eps, k_pool, v_pool, block_table,
                  seq_of_token, positions, page_size, write=True, cos=None, sin=None, interleaved=False,
                  q_bias=None, k_bias=None, v_bias=None):
    """First, where biases (float32 [heads * dim], [kv_heads * dim], [kv_heads * vdim]) are given, q, k and v plus
    their biases (q, k and v may then be float32 results of a product, rounded here for the first time). Then
    per-head RMSNorm (plain weight; None: no norm) of q [N, heads * dim] and k [N, kv_heads * dim], then, where
    ``cos`` and ``sin`` (float32 [N, rot / 2]) are given, the rotation of the first ``rot`` channels of every head of
    q and k: channel 2i with 2i + 1 (``interleaved``) or i with i + rot / 2. k and the untouched v [N, kv_heads * vdim]
    go into the pages (k pages [.., kv_heads, page, dim], v pages [.., kv_heads, page, vdim]); returns q, contiguous,
    in the pools' dtype."""
    n = q.shape[0]
    qf = q.to(torch.float32)
    if q_bias is not None:
        qf = qf + q_bias
    qf = qf.reshape(n, heads, dim)
    if write:
        kf, vf = k.to(torch.float32), v.to(torch.float32)
        if k_bias is not None:
            kf = kf + k_bias
        if v_bias is not None:
            vf = vf + v_bias
        kf = kf.reshape(n, kv_heads, dim)
    else:
        kf = torch.zeros((n, kv_heads, dim), dtype=torch.float32, device=q.device)  # nothing of k and v is read
    if q_weight is not None:
        qf = rmsnorm(qf, q_weight, eps, False, torch.float32)
        kf = rmsnorm(kf, k_weight, eps, False, torch.float32)
    if cos is not None:
        half = cos.shape[1]
        c, sn = cos[:, None, :].to(torch.float32), sin[:, None, :].to(torch.float32)

        def turn(x):
            x = x.clone()
            a = x[..., 0 : 2 * half : 2] if interleaved else x[..., :half]
            b = x[..., 1 : 2 * half : 2] if interleaved else x[..., half : 2 * half]
            ra, rb = a * c - b * sn, b * c + a * sn
            if interleaved:
                x[..., 0 : 2 * half : 2], x[..., 1 : 2 * half : 2] = ra, rb
            else:
                x[..., :half], x[..., half : 2 * half] = ra, rb
            return x

        qf, kf = turn(qf), turn(kf)
    if write:
        live, page, off = _page_addresses(block_table, seq_of_token, positions, page_size)
        k_pool[page[live], :, off[live]] = kf[live].to(k_pool.dtype)
        v_pool[page[live], :, off[live]] = vf.reshape(n, kv_heads, vdim)[live].to(v_pool.dtype)
    return qf.reshape(n, heads * dim).to(k_pool.dtype).contiguous()


def attention_general(q, k_pool, v_pool, block_table, seq_of_token, positions, scale, window, keep_first, softcap,
                      r1, r2, sink, gate, page_size, ctx=None, sinks=None, out=None, out_scale=1.0, values_in_keys=0,
                      gate_channels=False):
    """``values_in_keys`` = V > 0: a key's row holds its value too, as its first V channels (``v_pool`` is not read).
    ``gate_channels``: ``gate`` is [N, heads * vdim], one logit per channel of the output, not one per head.
    Attention of every token over the keys of its request that it sees: j <= i and (no window, or i - j < window,
    or j < keep_first). score = q . k * scale; with softcap, cap * tanh(score / cap); with r1 and r2 (float32
    [heads]), minus r1_h * ln(1 + r2_h * (i - j)); softmax over the keys, with ``sink`` one more term exp(0) in the
    denominator, or with ``sinks`` (float32 [heads]) the term exp(sinks_h); the head's output times
    sigmoid(gate[n, h]) where ``gate`` [N, heads] is given, times ``out_scale``.
    q [N, heads * dim] -> [N, heads * vdim] in q's dtype, written into ``out`` (rows may be parts of wider rows) where given."""
    n = q.shape[0]
    if values_in_keys:
        v_pool = k_pool[..., :values_in_keys]
    kh, d, vd = k_pool.shape[1], k_pool.shape[3], v_pool.shape[3]
    heads = q.shape[1] // d
    group = heads // kh
    given = out
    out = torch.zeros((n, heads, vd), dtype=torch.float64, device=q.device)
    seqs, poss = seq_of_token.tolist(), positions.tolist()
    for t in range(n):
        r, p = seqs[t], poss[t]
        if r < 0:
            continue
        idx = torch.arange(0, p + 1, device=q.device)
        if window:
            idx = idx[(p - idx < window) | (idx < keep_first)]
        pages = block_table[r, idx // page_size].long()
        offs = idx % page_size
        keys = k_pool[pages, :, offs].to(torch.float64)  # [S, kh, d]
        vals = v_pool[pages, :, offs].to(torch.float64)
        qt = q[t].reshape(kh, group, d).to(torch.float64)
        s = torch.einsum("kgd,skd->kgs", qt, keys) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if r1 is not None:
            dist = (p - idx).to(torch.float64)
            s = s - r1.to(torch.float64).reshape(kh, group, 1) * torch.log1p(r2.to(torch.float64).reshape(kh, group, 1) * dist)
        top = s.max(dim=-1, keepdim=True).values
        level = None
        if sinks is not None:
            level = sinks.to(torch.float64).reshape(kh, group, 1)
        elif sink:
            level = torch.zeros((kh, group, 1), dtype=torch.float64, device=q.device)
        if level is not None:
            top = torch.maximum(top, level)
        e = torch.exp(s - top)
        denom = e.sum(dim=-1, keepdim=True) + (torch.exp(level - top) if level is not None else 0.0)
        out[t] = torch.einsum("kgs,skd->kgd", e / denom, vals).reshape(heads, vd)
    if gate is not None and gate_channels:
        out = out * torch.sigmoid(gate.to(torch.float64)).reshape(n, heads, vd)
    elif gate is not None:
        out = out * torch.sigmoid(gate.to(torch.float64))[:, :, None]
    result = (out * out_scale).reshape(n, heads * vd)
    if given is not None:
        given.copy_(result.to(given.dtype))
        return given
    return result.to(q.dtype)


# --------------------------------------------------------------------------- latent attention, norms without sums


def dynamic_tanh(x, alpha, weight, shift, out_dtype, rows=None, residual=None):
    """tanh(alpha * x) * weight + shift per element of float32 x [N, C] (alpha a float32 tensor of one number, weight
    and shift float32 [C]); ``rows``: int32 indices of the rows to norm and return. With ``residual`` (float32 [N, C])
    the result is added to it in place and it is returned."""
    if rows is not None:
        x = x[rows.long()]
    y = torch.tanh(alpha.to(torch.float32) * x.to(torch.float32)) * weight + shift
    if residual is not None:
        residual += y
        return residual
    return y.to(out_dtype)


def _activation(z, kind):
    if kind == "gelu_tanh":
        return 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z * z * z)))
    if kind == "silu":
        return z * torch.sigmoid(z)
    if kind == "relu2":
        return torch.relu(z) ** 2
    raise ValueError(f"unknown activation {kind!r}")


def activation(z, kind, out_dtype):
    """act(z) element by element in float32, rounded once to ``out_dtype``; "relu2" is the square of max(z, 0)."""
    return _activation(z.to(torch.float32), kind).to(out_dtype)


def gated_activation(gate_up, width, bias, activation, out_dtype, residual=None, residual_bias=None):
    """act(g + b_g) * (u + b_u) for float32 gate_up [N, >= 2 width] whose first ``width`` columns are g and whose next
    are u; bias float32 [2 width] (b_g then b_u) or None -> [N, width] in ``out_dtype``, rounded once. With
    ``residual`` (float32 [N, C]), ``residual_bias`` [C] is added to it in place."""
    if residual is not None:
        residual.add_(residual_bias)
    g, u = gate_up[:, :width].to(torch.float32), gate_up[:, width : 2 * width].to(torch.float32)
    if bias is not None:
        g, u = g + bias[:width], u + bias[width:]
    return (_activation(g, activation) * u).to(out_dtype)


def linear_gated(x, w_gate_up, width, bias, activation):
    """act(g + b_g) * (u + b_u) for [g | u | ...] = x . w^T with w the stacked gate and up matrices (``width`` = F rows
    each, then rows of padding, if any) -> [N, F] in x's dtype."""
    return gated_activation(linear(x, w_gate_up, out_dtype=torch.float32), width, bias, activation, x.dtype)


def latent_norm_store(proj, q_rank, kv_rank, rot, q_weight, kv_weight, eps, cos, sin, interleaved, pool, block_table,
                      seq_of_token, positions, page_size, write=True):
    """From a row of proj [N, >= q_rank + kv_rank + rot] (float32): its first q_rank columns over their root mean
    square (eps under the root) times q_weight -> returned [N, q_rank] in the pool's dtype. The next kv_rank columns
    over THEIR root mean square times kv_weight, then the last rot columns rotated as a whole (cos, sin float32
    [N, rot / 2]; pairs (2i, 2i + 1) when ``interleaved``, else (i, i + rot / 2); no tables: as they are) -> the
    token's row [kv_rank + rot] of ``pool`` [pages, 1, page, kv_rank + rot]."""
    n = proj.shape[0]
    pf = proj.to(torch.float32)
    if q_rank:
        out = rmsnorm(pf[:, :q_rank], q_weight, eps, False, pool.dtype)
    else:  # no query latent: only the cached row is made
        out = torch.empty((n, 0), dtype=pool.dtype, device=proj.device)
    if write:
        c = rmsnorm(pf[:, q_rank : q_rank + kv_rank], kv_weight, eps, False, torch.float32)
        tail = pf[:, q_rank + kv_rank : q_rank + kv_rank + rot]
        if cos is not None and rot:
            tail = _turn(tail.reshape(n, 1, rot), cos, sin, interleaved).reshape(n, rot)
        live, page, off = _page_addresses(block_table, seq_of_token, positions, page_size)
        pool[page[live], 0, off[live]] = torch.cat((c, tail), dim=1)[live].to(pool.dtype)
    return out.contiguous()


def _turn(x, cos, sin, interleaved):
    """The first 2 * cos.shape[1] channels of every head of float32 x [N, heads, D] rotated by the token's angles."""
    half = cos.shape[1]
    c, sn = cos[:, None, :].to(torch.float32), sin[:, None, :].to(torch.float32)
    x = x.clone()
    a = x[..., 0 : 2 * half : 2] if interleaved else x[..., :half]
    b = x[..., 1 : 2 * half : 2] if interleaved else x[..., half : 2 * half]
    ra, rb = a * c - b * sn, b * c + a * sn
    if interleaved:
        x[..., 0 : 2 * half : 2], x[..., 1 : 2 * half : 2] = ra, rb
    else:
        x[..., :half], x[..., half : 2 * half] = ra, rb
    return x


def head_linear(x, w, heads, gate=None, cos=None, sin=None, interleaved=False):
    """A product per head: for w [heads, O, K] and x [N, heads * (K + T)] (head h's K channels, then T more),
    out[n, h, :O] = w[h] x[n, h, :K], float32 accumulation, and out[n, h, O:] = the head's T further channels, rotated
    as a whole where ``cos`` and ``sin`` (float32 [N, T / 2]) are given. ``gate`` [N, heads * O] (any float dtype, rows
    may be parts of wider rows): the products times sigmoid(gate). -> [N, heads * (O + T)] in x's dtype."""
    n = x.shape[0]
    h, o, k = w.shape
    t = x.shape[1] // heads - k
    xf = x.to(torch.float32).reshape(n, heads, k + t)
    y = torch.einsum("nhk,hok->nho", xf[:, :, :k], w.to(torch.float32))
    if gate is not None:
        y = y * torch.sigmoid(gate.to(torch.float32).reshape(n, heads, o))
    if t:
        tail = xf[:, :, k:]
        if cos is not None:
            tail = _turn(tail, cos, sin, interleaved)
        y = torch.cat((y, tail), dim=2)
    return y.reshape(n, heads * (o + t)).to(x.dtype)


# --------------------------------------------------------------------------- routed experts, parallel blocks


def moe_route(h, w_router, correction, groups, keep, top, scoring="softmax", renormalize=True, extra=0):
    """For every row of h [N, C]: scores = softmax(h . w_router^T) over the R router outputs (float32 w_router
    [R, C]); choice scores = scores + correction [R]; the outputs form ``groups`` equal groups of neighbours whose
    score is their largest choice score, and only outputs of the ``keep`` best groups can be chosen; the ``top``
    largest choice scores win (ties: the lower index). Returns (chosen int32 [N, top], weights float32 [N, top]): the
    chosen outputs in the order of their choice scores and their plain scores over their sum (+ 1e-20).
    ``scoring="sigmoid"``: a score is the sigmoid of its logit (without a correction the choice goes by the logits, which
    order the same way); ``correction`` None: none; ``renormalize`` False: the
    weights are the chosen scores as they are. ``extra`` = X > 0: w_router has X more rows [R + X, C] that take no part
    in the choice; the sigmoids of their logits are returned as a third result, float32 [N, X]."""
    n = h.shape[0]
    r = w_router.shape[0] - extra
    z = h.to(torch.float32) @ w_router.to(torch.float32).T
    s = torch.softmax(z[:, :r], dim=-1) if scoring == "softmax" else torch.sigmoid(z[:, :r])
    if correction is not None:
        pick = s + correction.to(torch.float32)
    else:  # the logits order as their scores do, and still compare where two sigmoids round to one
        pick = z[:, :r].clone() if scoring == "sigmoid" else s
    if groups > 1 and keep < groups:
        best = pick.reshape(n, groups, r // groups).max(dim=-1).values
        order = torch.argsort(best, dim=-1, descending=True, stable=True)
        stays = torch.zeros((n, groups), dtype=torch.bool, device=h.device)
        stays.scatter_(1, order[:, :keep], True)
        pick = pick.masked_fill(~stays.repeat_interleave(r // groups, dim=1), float("-inf"))
    chosen = torch.argsort(pick, dim=-1, descending=True, stable=True)[:, :top]
    w = torch.gather(s, 1, chosen)
    if renormalize:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    if extra:
        return chosen.to(torch.int32), w, torch.sigmoid(z[:, r:]).contiguous()
    return chosen.to(torch.int32), w


def moe_experts(h, w_gate_up, w_down, chosen, weights, update=None, weight_input=False, shared=None):
    """``weight_input``: the weight multiplies the expert's input, out[n] = sum_k expert(weights[n, k] h[n]) (computed
    as silu(w g) * (w u) on the float32 sums g, u of the unweighted row). ``shared`` = (y float32 [N, C], gate float32
    [N, 1] or None): y, times its gate, is added to the sum. With ``update`` = (x, a, scale_a, scale_b, mult): x += mult * (scale_a * a + scale_b * out) in place, returns x. Else
    out[n] = sum_k weights[n, k] * expert_(chosen[n, k])(h[n]) in float32 [N, C]. Expert e < E computes
    w_down[e] (silu(gate) * up) with [gate; up] = w_gate_up[e] h (w_gate_up [E, 2 F, C], w_down [E, C, F]; the hidden
    activations are rounded to h's dtype, as the kernels round them); an expert number from E on returns h itself."""
    n, c = h.shape
    e_count, f2, _ = w_gate_up.shape
    out = torch.zeros((n, c), dtype=torch.float32, device=h.device)
    hf = h.to(torch.float32)
    for k in range(chosen.shape[1]):
        for e in torch.unique(chosen[:, k]).tolist():
            rows = (chosen[:, k] == e).nonzero().flatten()
            g = weights[rows, k][:, None]
            if e >= e_count:
                out[rows] += g * hf[rows]
                continue
            gu = hf[rows] @ w_gate_up[e].to(torch.float32).T
            if weight_input:
                gu, g = gu * g, 1.0
            act = (torch.nn.functional.silu(gu[:, : f2 // 2]) * gu[:, f2 // 2 :]).to(h.dtype).to(torch.float32)
            out[rows] += g * (act @ w_down[e].to(torch.float32).T)
    if shared is not None:
        y, gate = shared
        out += y if gate is None else gate.reshape(n, 1) * y
    if update is not None:
        x, a, scale_a, scale_b, mult = update
        return scaled_add(x, a, scale_a, out, scale_b, mult)
    return out


def scaled_add(x, a, scale_a, b, scale_b, mult):
    """x += mult * (scale_a * a + scale_b * b) in place on float32 x [N, C]; the scales are float32 [C] (None: ones),
    b may be None."""
    total = a if scale_a is None else a * scale_a
    if b is not None:
        total = total + (b if scale_b is None else b * scale_b)
    x += mult * total
    return x
