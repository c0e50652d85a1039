"""Throughput measurement: prefill and decode tokens a second, with the bytes and flops behind them.

The protocol is kreasof-ai/akas's ``native-token-step-v2`` (src/akas/benchmarking/runner.py:72-105,
src/akas/benchmarking/workload.py:29-38): seeded synthetic prompt ids, a device synchronize at both
boundaries, load and warm-up excluded; prefill includes the head and the first predicted token; decode
counts the steps after it; ``prefill tok/s = sum of prompt lengths / seconds`` and ``decode tok/s =
batch x steps / seconds``. Times here are CUDA-event times on the launching stream.
"""

from __future__ import annotations

import statistics
from typing import Dict, List, Sequence

import numpy as np
import torch

from .engine.batch import StepEntry
from .engine.runner import ModelRunner


def synthetic_prompts(batch: int, prefix: int, vocab: int, seed: int = 17) -> List[List[int]]:
    """src/akas/benchmarking/workload.py:29-38: one generator per (batch, prefix) cell."""
    rng = np.random.default_rng(seed + batch * 4099 + prefix)
    return rng.integers(0, vocab, (batch, prefix)).tolist()


def matrix_params(runner: ModelRunner) -> Dict[str, int]:
    """Parameters of the matrix products a token passes through (per layer run, head apart). Of a routed feed-forward's
    stacked experts [experts, rows, columns] a token passes through ``top`` (less the share of identity experts)."""
    layers = 0
    for entry in runner.model.schedule:
        block = runner.model.blocks[entry.layer]
        for part in (block.mixer, block.ffn):
            if part is None:
                continue
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.dim() == 2 and value.dtype == runner.dtype:
                    layers += value.numel()
                elif isinstance(value, torch.Tensor) and value.dim() == 3 and value.dtype == runner.dtype:
                    s = part.spec
                    if not hasattr(s, "top"):  # a matrix per head: a token passes through all of them
                        layers += value.numel()
                        continue
                    real = s.top * s.num_experts / (s.num_experts + s.num_identity)
                    layers += int(value[0].numel() * real)
    return dict(layers=layers, head=runner.model.head.numel())


def _mixer_specs(spec):
    """The specs of the mixers a layer's mixer is made of (itself, unless it holds several side by side)."""
    if getattr(spec, "kind", "") == "parallel_mixer":
        return [branch for _, branch, _ in spec.branches]
    return [spec]


def prefill_flops(runner: ModelRunner, tokens: int, start: int = 0) -> float:
    """Matrix products of ``tokens`` prompt tokens, causal attention over them, and one row of the head."""
    p = matrix_params(runner)
    flops = 2.0 * tokens * p["layers"] + 2.0 * p["head"]
    for entry in runner.model.schedule:
      for spec in _mixer_specs(runner.model.blocks[entry.layer].mixer.spec):
        kind = getattr(spec, "kind", "")
        if kind == "attention":
            # q.k and p.v over the keys the i-th token sees (all start + i of them, or a window's worth): 2 flops per
            # (query, key, head, channel) for each of the two products
            if spec.window:
                pairs = sum(min(start + i + 1, spec.window + getattr(spec, "keep_first", 0)) for i in range(tokens))
            else:
                pairs = tokens * start + tokens * (tokens + 1) / 2
            flops += 2.0 * pairs * spec.num_heads * (spec.head_dim + getattr(spec, "value_dim", spec.head_dim))
        elif kind == "latent_attention":
            # as computed: every head's query against the cached rows [latent, rotated part], weights times the latent
            pairs = sum(min(start + i + 1, spec.window) for i in range(tokens)) if spec.window else tokens * start + tokens * (tokens + 1) / 2
            flops += 2.0 * pairs * spec.num_heads * (2 * spec.kv_rank + spec.rope_dim)
        elif kind in ("gated_linear_attention", "gated_delta", "decayed_linear_attention"):
            # the matrix state: decay and rank-one update, read-out (and the delta rule's read before the update)
            per = 6.0 if kind == "gated_delta" else 4.0
            flops += per * tokens * spec.num_heads * spec.key_dim * spec.value_dim
    return flops


def decode_bytes(runner: ModelRunner, contexts: Sequence[int]) -> float:
    """Bytes one decode step has to read: every weight it uses once, the keys and values of the live
    requests, and their fixed-size state (read and written)."""
    elem = 2 if runner.dtype == torch.bfloat16 else 4
    total = float(runner.weight_bytes)
    if runner.model.head is not runner.model.embedding:
        total -= runner.model.embedding.numel() * elem  # an untied embedding is only gathered from
    views = []
    for view in runner.cache.views:
        views.extend(view if isinstance(view, tuple) else [view])
    for view in views:
        spec = getattr(view, "spec", None)
        if spec is None:
            continue
        if hasattr(spec, "num_kv_heads") or hasattr(spec, "width"):
            if hasattr(spec, "width"):  # one row per token that is key and value of every head
                per_token = spec.width * elem
            else:
                per_token = spec.num_kv_heads * (spec.head_dim + (getattr(spec, "v_head_dim", None) or spec.head_dim)) * elem
            for c in contexts:
                total += per_token * (min(c, spec.window + getattr(spec, "keep_first", 0)) if spec.window else c)
        else:
            total += 2 * len(contexts) * int(np.prod(spec.shape)) * 4
    return total


def _event_ms(fn) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def fill_requests(runner: ModelRunner, prompts: Sequence[Sequence[int]], chunk: int = 2048, ids=None):
    """Admits one request per prompt and runs the prompts through in portions; returns the request ids."""
    ids = list(ids) if ids is not None else [f"bench-{i}" for i in range(len(prompts))]
    budget = max(chunk, 8192)
    at = {rid: 0 for rid in ids}
    while any(at[rid] < len(p) for rid, p in zip(ids, prompts)):
        entries, used = [], 0
        for rid, p in zip(ids, prompts):
            if at[rid] >= len(p) or used >= budget:
                continue
            k = min(chunk, len(p) - at[rid], budget - used)
            entries.append(StepEntry(rid, p[at[rid]:at[rid] + k], ()))
            at[rid] += k
            used += k
        runner.step(entries)
    return ids


def measure_prefill(runner: ModelRunner, prompt: Sequence[int], repeats: int = 7, warmup: int = 3) -> float:
    """Median milliseconds to run one whole prompt and produce its first token (head and argmax included). The warm-up
    runs also let the step function capture the prompt's shape (it does when a shape comes a third time), so the timed
    runs are replays, as in serving where portions of one size keep coming."""
    times = []
    for i in range(warmup + repeats):
        def run():
            logits = runner.step([StepEntry("prefill", prompt, (len(prompt) - 1,))])
            runner.ops.argmax(logits)
        ms = _event_ms(run)
        runner.release("prefill")
        if i >= warmup:
            times.append(ms)
    return statistics.median(times)


def measure_decode(runner: ModelRunner, batch: int, prefix: int, steps: int, warmup: int, seed: int = 17,
                   chunk: int = 2048, repeats: int = 5) -> Dict[str, float]:
    """Milliseconds per decode step at ``batch`` requests whose prompts of ``prefix`` tokens are cached.

    Each timed step feeds one given (synthetic) token per request and includes the head and the argmax;
    nothing is read back inside the timed region. A region is exactly ``steps`` steps between two synchronisations,
    timed with CUDA events; it is run up to ``repeats`` times, one after the other (the requests keep decoding, as far
    as the context allows), and the median region is reported: a single short region right after a synchronisation
    also holds the host's preparation of its first step and whatever the clocks do on their way up. The entries of
    every step are built beforehand.
    """
    vocab = runner.vocab_size
    prompts = synthetic_prompts(batch, prefix, vocab, seed)
    ids = fill_requests(runner, prompts, chunk)
    room = runner.config.context - prefix - warmup - 1
    repeats = max(1, min(repeats, room // max(steps, 1)))
    total = warmup + repeats * steps
    feed = np.random.default_rng(seed + 1).integers(0, vocab, (total, batch)).tolist()
    entries = [[StepEntry(rid, (feed[i][j],), (0,)) for j, rid in enumerate(ids)] for i in range(total)]

    def run(first, count):
        for i in range(first, first + count):
            runner.ops.argmax(runner.step(entries[i]))

    run(0, warmup)
    regions, launches = [], 0
    for r in range(repeats):
        before = runner.ops.launch_count
        regions.append(_event_ms(lambda: run(warmup + r * steps, steps)))
        launches = runner.ops.launch_count - before
    ms = statistics.median(regions)
    at = sorted(range(repeats), key=lambda r: regions[r])[repeats // 2]  # the region whose time is reported
    contexts = [prefix + warmup + at * steps + steps // 2] * batch
    for rid in ids:
        runner.release(rid)
    return dict(ms_per_step=ms / steps, tokens_per_s=batch * steps / (ms / 1e3), bytes=decode_bytes(runner, contexts),
                launches=launches, regions_ms=[round(x, 4) for x in regions])


def case_lengths(batch: int, prompt: int, mixed: bool) -> List[int]:
    """Prompt length per slot: all ``prompt``, or staggered as the reference staggers them
    (src/akas/benchmarking/cases.py:30-35)."""
    return [max(1, prompt - i % min(prompt, 7)) if mixed else prompt for i in range(batch)]


def run_matrix(model_dir, config, batches=(1, 8), prompts=(2048,), generated=128, repeats=5, warmup=1, seed=17,
               prefill_chunk=None, depths=(0,), mixed=False) -> dict:
    """The reference's pp/tg matrix (src/akas/benchmarking/cases.py:8-61): for every (batch, prompt length, depth)
    the median prefill and decode tokens a second over ``repeats`` repetitions after ``warmup``. ``depth``: tokens
    already in the cache of every request before its measured prompt; ``mixed``: prompt lengths staggered over the
    slots."""
    from dataclasses import replace

    if any(d < 0 for d in depths) or generated < 1 or min(batches) < 1 or min(prompts) < 1:
        raise ValueError("positive batch/prompt/generation and nonnegative depth required")
    longest = max(depths) + max(prompts) + generated
    need = max(batches) * (longest + 64)
    config = replace(config, max_requests=max(config.max_requests, max(batches)),
                     context=max(config.context, longest + 1), max_tokens=None)
    if config.pool_tokens < need:
        config = replace(config, max_tokens=need)
    runner = ModelRunner(model_dir, config)
    chunk = prefill_chunk or config.prefill_chunk
    rows = []
    for batch in batches:
        for prefix in prompts:
            for depth in depths:
                lengths = case_lengths(batch, prefix, mixed)
                pp, tg = [], []
                for rep in range(warmup + repeats):
                    data = [p[:n] for p, n in zip(synthetic_prompts(batch, prefix, runner.vocab_size, seed), lengths)]
                    ids = [f"m{j}" for j in range(batch)]
                    if depth:
                        fill_requests(runner, synthetic_prompts(batch, depth, runner.vocab_size, seed + 1), chunk, ids)

                    def prefill():
                        fill_requests(runner, [p[:-1] for p in data], chunk, ids)
                        logits = runner.step([StepEntry(rid, (p[-1],), (0,)) for rid, p in zip(ids, data)])
                        return runner.ops.argmax(logits)

                    holder = {}
                    pp_ms = _event_ms(lambda: holder.setdefault("t", prefill()))
                    tokens = holder["t"]

                    def decode():
                        # every step feeds the tokens that the step before picked; they stay on the device (an entry
                        # names its place among them), as in the engine's own loop, so nothing waits for the host
                        t = tokens
                        entries = [StepEntry(rid, (0,), (0,), source=j) for j, rid in enumerate(ids)]
                        for _ in range(generated - 1):
                            t = runner.ops.argmax(runner.step(entries, previous=t))

                    tg_ms = _event_ms(decode)
                    for rid in ids:
                        runner.release(rid)
                    if rep >= warmup:
                        pp.append(sum(lengths) / (pp_ms / 1e3))
                        if generated > 1:
                            tg.append(batch * (generated - 1) / (tg_ms / 1e3))
                rows.append(dict(batch=batch, prompt=prefix, generated=generated, depth=depth, mixed=mixed,
                                 prefill_tokens_per_s=statistics.median(pp),
                                 decode_tokens_per_s=statistics.median(tg) if tg else None))
    return dict(protocol="native-token-step-v2", dtype=config.dtype, seed=seed, repeats=repeats, warmup=warmup,
                prefill_chunk=chunk, rows=rows)


def compare_reports(report: dict, baseline: dict, max_regression: float = 0.1) -> List[dict]:
    """Every measured case against the same case of an earlier report, as the reference's bench gate does
    (src/akas/cli.py:527, 666-680): raises if the baseline lacks a case, returns the changes, and marks a case whose
    prefill or decode rate fell by more than ``max_regression`` of the baseline's."""
    if not 0 <= max_regression < 1:
        raise ValueError("invalid regression setting")
    key = lambda row: (row["batch"], row["prompt"], row.get("generated"), row.get("depth", 0), row.get("mixed", False))
    before = {key(row): row for row in baseline.get("rows", [])}
    changes = []
    for row in report["rows"]:
        old = before.get(key(row))
        if old is None:
            raise ValueError("baseline must cover every measured case")
        change = dict(batch=row["batch"], prompt=row["prompt"], depth=row.get("depth", 0), mixed=row.get("mixed", False))
        for name in ("prefill_tokens_per_s", "decode_tokens_per_s"):
            if row.get(name) and old.get(name):
                change[name + "_ratio"] = row[name] / old[name]
        change["regressed"] = any(v < 1 - max_regression for k, v in change.items() if k.endswith("_ratio"))
        changes.append(change)
    return changes


# --------------------------------------------------------------------------- single kernels


def _time_kernel(fn, iters: int, flush_bytes: int = 256 << 20) -> float:
    """Median milliseconds of ``fn()``; a buffer larger than L2 is rewritten before every timed call."""
    flush = torch.empty(flush_bytes, dtype=torch.uint8, device="cuda")
    times = []
    for i in range(iters + 3):
        flush.fill_(i & 1)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def bench_linear(m: int, o: int, k: int, mode: str, iters: int = 20) -> dict:
    """One matrix product of the bfloat16 path, cold L2: mode is bf16 | f32 | acc | swiglu | norm | norm_swiglu."""
    from .ops import cuda as ops

    ops.require(ops.libraries_for(torch.bfloat16))
    g = torch.Generator(device="cuda").manual_seed(0)
    w = (torch.randn((o, k), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.bfloat16)
    h = torch.randn((m, k), device="cuda", generator=g)
    nw = torch.ones(k, device="cuda")
    res = torch.zeros((m, o), device="cuda")
    fn = {
        "bf16": lambda: ops.linear(x, w),
        "f32": lambda: ops.linear(x, w, out_dtype=torch.float32),
        "acc": lambda: ops.linear(x, w, residual=res),
        "swiglu": lambda: ops.linear_swiglu(x, w),
        "norm": lambda: ops.norm_linear(h, nw, 1e-5, False, w),
        "norm_swiglu": lambda: ops.norm_linear(h, nw, 1e-5, False, w, None, None, True),
    }[mode]
    ms = _time_kernel(fn, iters)
    nbytes = w.numel() * 2
    return dict(kernel="linear", mode=mode, m=m, o=o, k=k, ms=round(ms, 5), weight_gb_s=round(nbytes / ms / 1e6, 1),
                tflops=round(2.0 * m * o * k / ms / 1e9, 2))


def bench_experts(tokens: int, c: int, f: int, experts: int = 14, identity: int = 2, top: int = 4, groups: int = 4, keep: int = 2,
                  iters: int = 20) -> dict:
    """The routed feed-forward's kernels one by one, cold L2, bfloat16: router, sorting the pairs by expert, the grouped
    gate/up and down products, the weighted gather; beside them the dense SwiGLU feed-forward (gate/up with its
    activation, then down) of a width that costs a token as many multiply-adds as its real experts do."""
    from .ops import cuda as ops

    ops.require(ops.libraries_for(torch.bfloat16, ("moe",)))
    g = torch.Generator(device="cuda").manual_seed(0)
    outputs = experts + identity
    h = torch.randn((tokens, c), device="cuda", generator=g).to(torch.bfloat16)
    w_router = torch.randn((outputs, c), device="cuda", generator=g) * (2.0 / c ** 0.5)
    correction = torch.randn(outputs, device="cuda", generator=g) * 0.1
    w_gate_up = (torch.randn((experts, 2 * f, c), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w_down = (torch.randn((experts, c, f), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    chosen, weights = ops.moe_route(h, w_router, correction, groups, keep, top)
    real = int((chosen < experts).sum())
    rows = {"tokens": tokens, "width": c, "expert_width": f, "experts": experts, "identity": identity, "top": top,
            "real_pairs": real}
    rows["route_ms"] = round(_time_kernel(lambda: ops.moe_route(h, w_router, correction, groups, keep, top), iters), 5)
    whole = _time_kernel(lambda: ops.moe_experts(h, w_gate_up, w_down, chosen, weights), iters)
    rows["experts_ms"] = round(whole, 5)
    flops = 2.0 * real * 3 * c * f
    rows["experts_tflops"] = round(flops / whole / 1e9, 1)
    if tokens * top > ops._MOE_SIMPLE_PAIRS and ops.moe_kernels == "auto":
        cap = int(ops._fn("moe_grouped", "akas_moe_grouped_rows")(tokens * top, experts))
        row_of_pair = torch.empty(tokens * top, dtype=torch.int32, device="cuda")
        tile_expert = torch.empty(cap // 128, dtype=torch.int32, device="cuda")
        plan = torch.empty(4, dtype=torch.int32, device="cuda")
        srt = torch.empty((cap, c), dtype=torch.bfloat16, device="cuda")
        act = torch.zeros((cap, f), dtype=torch.bfloat16, device="cuda")
        y = torch.empty((cap, c), dtype=torch.float32, device="cuda")
        out = torch.empty((tokens, c), dtype=torch.float32, device="cuda")
        st = ops._stream
        p = lambda t: t.data_ptr()
        sort = lambda: ops._fn("moe_grouped", "akas_moe_sort")(p(h), c, p(chosen), p(row_of_pair), p(tile_expert), p(plan), p(srt),
                                                              tokens, top, c, experts, st())
        gemm = ops._fn("moe_grouped", "akas_moe_grouped_gemm")
        up = lambda: gemm(p(srt), p(w_gate_up), p(act), p(tile_expert), p(plan), cap, experts, 2 * f, c, 2, st())
        down = lambda: gemm(p(act), p(w_down), p(y), p(tile_expert), p(plan), cap, experts, c, f, 1, st())
        comb = lambda: ops._fn("moe_grouped", "akas_moe_combine")(p(h), c, p(y), p(row_of_pair), p(weights), p(out), tokens, top, c, None, None, None, None, 0.0, st())
        sort()
        for name, fn, work in (("sort_ms", sort, 0.0), ("gate_up_ms", up, 2.0 * real * 2 * c * f), ("down_ms", down, 2.0 * real * c * f),
                               ("combine_ms", comb, 0.0)):
            ms = _time_kernel(fn, iters)
            rows[name] = round(ms, 5)
            if work:
                rows[name.replace("_ms", "_tflops")] = round(work / ms / 1e9, 1)
        rows["grouped_status"] = ops.moe_grouped_status()
    # the dense feed-forward of equal work per token: width = (real pairs per token) * f
    dense = max(256, int(round(real / tokens * f / 256)) * 256)
    w13 = (torch.randn((2 * dense, c), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn((c, dense), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    res = torch.zeros((tokens, c), device="cuda")
    mid = ops.linear_swiglu(h, w13)
    for name, fn, work in (("dense_gate_up_ms", lambda: ops.linear_swiglu(h, w13), 2.0 * tokens * 2 * c * dense),
                           ("dense_down_ms", lambda: ops.linear(mid, w2, residual=res), 2.0 * tokens * c * dense)):
        ms = _time_kernel(fn, iters)
        rows[name] = round(ms, 5)
        rows[name.replace("_ms", "_tflops")] = round(work / ms / 1e9, 1)
    rows["dense_width"] = dense
    return rows


def bench_attention(kind: str, batch: int, context: int, heads: int = 32, kv_heads: int = 8, dim: int = 64,
                    page: int = 64, iters: int = 20) -> dict:
    """Paged attention of the bfloat16 path, cold L2. ``decode``: ``batch`` requests of ``context`` cached tokens,
    one query token each. ``prompt``: ``batch`` requests whose whole ``context`` tokens are queries."""
    from types import SimpleNamespace

    from .ops import cuda as ops

    ops.require(ops.libraries_for(torch.bfloat16))
    g = torch.Generator(device="cuda").manual_seed(0)
    blocks = -(-context // page)
    pages = batch * blocks
    k = torch.randn((pages, kv_heads, page, dim), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((pages, kv_heads, page, dim), device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).view(batch, blocks)
    if kind == "decode":
        n = batch
        seq = torch.arange(batch, dtype=torch.int32, device="cuda")
        pos = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
        ctx = SimpleNamespace(decode_only=True, max_context=context, query_lens=(1,) * batch, cu_seqlens=None, memo={})
        flops = 4.0 * batch * context * heads * dim
    else:
        n = batch * context
        seq = torch.arange(batch, dtype=torch.int32, device="cuda").repeat_interleave(context)
        pos = torch.arange(context, dtype=torch.int32, device="cuda").repeat(batch)
        cu = torch.arange(0, n + 1, context, dtype=torch.int32, device="cuda")
        ctx = SimpleNamespace(decode_only=False, max_context=context, query_lens=(context,) * batch, cu_seqlens=cu, memo={})
        flops = 4.0 * batch * context * (context + 1) / 2 * heads * dim
    q = torch.randn((n, heads * dim), device="cuda", generator=g).to(torch.bfloat16)
    ms = _time_kernel(lambda: ops.paged_attention(q, k, v, table, seq, pos, dim ** -0.5, None, page, ctx), iters)
    kv_bytes = 2.0 * batch * context * kv_heads * dim * 2
    return dict(kernel="attention", kind=kind, batch=batch, context=context, heads=heads, kv_heads=kv_heads, head_dim=dim,
                ms=round(ms, 5), kv_gb_s=round(kv_bytes / ms / 1e6, 1), tflops=round(flops / ms / 1e9, 2))


SHAPES = {
    # the dense LFM2 sizes named by the benchmark configurations (config.json keys; everything else at its default)
    "350m": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=6656),
    "700m": dict(hidden_size=1536, num_attention_heads=24, num_key_value_heads=8, intermediate_size=10240),
    "1.2b": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288),
}


def shape_config(name: str) -> dict:
    base = dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", num_hidden_layers=16,
                full_attn_idxs=[2, 5, 8, 10, 12, 14], vocab_size=65536, rope_theta=1000000.0, norm_eps=1e-5,
                conv_L_cache=3, conv_bias=False, block_auto_adjust_ff_dim=True, block_multiple_of=256,
                block_ffn_dim_multiplier=1.0, tie_embedding=True, max_position_embeddings=128000)
    base.update(SHAPES[name])
    return base


# Gigusun at LFM2's layer sizes: the same width, vocabulary and number of layers, mixers and feed-forwards with as many
# parameters as LFM2's (a short-convolution layer holds 4 C^2 of them, so does a matrix-state mixer with H D = C / 2 and
# H V = C; PolyNorm's two matrices at the width that gives SwiGLU's three), attention in every third layer.
def gigusun_shape_config(name: str) -> dict:
    lfm2 = config_from_shape(name)
    c, ff3 = lfm2.hidden_size, lfm2.feed_forward_size
    heads = c // 128
    ff = -(-(3 * ff3 // 2) // 256) * 256
    attention = dict(heads=lfm2.num_attention_heads, kv_heads=lfm2.num_key_value_heads, dim=lfm2.head_dim, vdim=lfm2.head_dim,
                     scale=lfm2.head_dim ** -0.5, softcap=30.0, mask=dict(size=1024, keep_first=4))
    gla = dict(heads=heads, dim=64, vdim=128, tau=16.0, rank=64)
    delta = dict(heads=heads, kv_heads=heads // 2, dim=128, vdim=128, conv=4)
    kinds = {"attention": attention, "gla": gla, "delta": delta}
    order = ["gla", "delta", "attention"] * 5 + ["gla"]
    return dict(architecture="Gigusun", width=c, vocab=lfm2.vocab_size, max_positions=8192, norm=dict(eps=1e-5),
                layers=[dict(type=k, mixer=kinds[k], mlp=dict(ff=ff, kind="dense")) for k in order])


# Girelix at LFM2's layer sizes: the same width, vocabulary and number of layers. Every layer holds sink attention (half
# as many query channels as the width, a quarter as many key/value heads as LFM2), linear attention with a constant
# decay (C / 4 key channels, C / 2 value channels) and 14 experts + 2 identities in 4 groups of which 2 stay, 4 per
# token, each a quarter as wide as LFM2's feed-forward: a token passes through about as many feed-forward parameters
# as in LFM2, the model holds 3.5 times as many.
def girelix_shape_config(name: str) -> dict:
    lfm2 = config_from_shape(name)
    c, ff3 = lfm2.hidden_size, lfm2.feed_forward_size
    left = dict(heads=c // 128, kv_heads=max(1, lfm2.num_key_value_heads // 4), dim=64, vdim=64, scale=0.125,
                rot=dict(base=1000000.0, dims=64))
    heads = c // 256
    right = dict(heads=heads, dim=64, vdim=128, decay=[1.0 - 2.0 ** -(3 + 5 * i / max(1, heads - 1)) for i in range(heads)])
    mlp = dict(kind="moe", expert=dict(ff=ff3 // 4), router=dict(experts=14, identity=2, top=4, groups=dict(count=4, keep=2)))
    entry = dict(type="parallel", mixer=dict(left=left, right=right, left_scale=1.0, right_scale=1.0), mlp=mlp)
    return dict(architecture="Girelix", width=c, vocab=lfm2.vocab_size, norm=dict(eps=1e-5), residual_mult=0.5,
                layers=[entry] * len(lfm2.layer_kinds))


# Penopel at LFM2's layer sizes: the same width, vocabulary and number of layers, a gated feed-forward of LFM2's width in
# every layer. Of every four layers two are latent attention (a head per 128 channels of the width, 64 plain and 32
# rotated channels a head, a key/value latent of 96, so a cached row of 128 numbers; a window of 1,024), one is
# attention with LFM2's head counts, and one reads that layer's cache with queries of its own.
def penopel_shape_config(name: str) -> dict:
    lfm2 = config_from_shape(name)
    c, ff3 = lfm2.hidden_size, lfm2.feed_forward_size
    rot = dict(base=500000.0, dims=lfm2.head_dim, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192))
    attention = dict(heads=lfm2.num_attention_heads, kv_heads=lfm2.num_key_value_heads, dim=lfm2.head_dim, vdim=lfm2.head_dim,
                     scale=lfm2.head_dim ** -0.5, rot=rot)
    latent = dict(heads=c // 128, dim=64, rot_dim=32, vdim=64, q_rank=3 * c // 8, kv_rank=96, scale=96 ** -0.5,
                  mask=dict(size=1024), rot=dict(base=1000000.0, dims=32))
    mlp = dict(kind="dense", ff=ff3)
    layers = []
    for i in range(len(lfm2.layer_kinds)):
        if i % 4 == 1:
            layers.append(dict(type="attention", mixer=attention, mlp=mlp))
        elif i % 4 == 3:
            layers.append(dict(type="attention", mixer=dict(attention, kv_from=i - 2), mlp=mlp))
        else:
            layers.append(dict(type="latent_attention", mixer=latent, mlp=mlp))
    return dict(architecture="Penopel", width=c, vocab=lfm2.vocab_size, norm=dict(eps=1e-5), embedding=dict(scale=float(c) ** 0.5),
                logit_softcap=30.0, layers=layers)


# Kidarax at LFM2's layer sizes: the same width and vocabulary; fourteen layers of which two run twice (a loop), so sixteen
# layer runs like LFM2's. The mixers take turns: retention (a head per 128 channels of the width, keys of 64 and values
# of 128), latent attention (a head per 128 channels, 64 plain and 32 rotated channels, a latent of 96: a cached row of
# 128 numbers) and biased attention with LFM2's head counts and a gate per channel. Feed-forwards take turns too: a dense
# one without a gate, as wide as LFM2's gated one (four times the model's width at the 1.2b sizes), and sixteen experts of
# a quarter of that width of which a token passes three, beside one more that every token passes.
def kidarax_shape_config(name: str) -> dict:
    lfm2 = config_from_shape(name)
    c, ff3 = lfm2.hidden_size, lfm2.feed_forward_size
    heads = c // 128
    retention = dict(heads=heads, dim=64, vdim=128, decay=[1.0 - 2.0 ** -(4 + 6 * i / max(1, heads - 1)) for i in range(heads)])
    attention = dict(heads=lfm2.num_attention_heads, kv_heads=lfm2.num_key_value_heads, dim=lfm2.head_dim, vdim=lfm2.head_dim,
                     scale=lfm2.head_dim ** -0.5, rot=dict(base=500000.0, dims=lfm2.head_dim, scaling=dict(factor=8.0)))
    latent = dict(heads=heads, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=96 ** -0.5,
                  rot=dict(base=1000000.0, dims=32, scaling=dict(factor=8.0, original=4096, fast=32.0, slow=1.0)))
    dense = dict(kind="dense", ff=ff3)
    moe = dict(kind="moe", expert=dict(ff=ff3 // 4), router=dict(experts=16, top=3), shared=dict(ff=ff3 // 4))
    mixers = (("retention", retention), ("latent_attention", latent), ("attention", attention))
    runs = len(lfm2.layer_kinds)
    layers = [dict(type=mixers[i % 3][0], mixer=mixers[i % 3][1], mlp=moe if i % 2 else dense) for i in range(runs - 2)]
    return dict(architecture="Kidarax", width=c, vocab=lfm2.vocab_size, norm=dict(eps=1e-5), logit_scale=float(c) ** -0.5,
                loop=dict(start=runs // 2 - 2, stop=runs // 2, times=2), layers=layers)


def config_from_shape(name: str):
    from .config import config_from_dict

    return config_from_dict(shape_config(name))


def compare_designs(shape: str = "1.2b", prompt: int = 2048, batches=(8, 64), steps: int = 64, warmup: int = 4,
                    designs=("lfm2", "gigusun")) -> List[dict]:
    """The named designs at equal layer sizes, random weights, bfloat16: milliseconds and tokens a second of a
    ``prompt``-token prefill and of decode steps at each batch size (captured graphs), and the device time of every
    kind of operation in an eager prefill and an eager decode step at the first batch size (CUDA events around each
    call). One row per design."""
    import tempfile

    from .config import EngineConfig, config_from_dict
    from .ops import cuda as cuda_ops
    from .ops.timed import TimedOps
    from .weights import write_random_model

    import sys

    def say(what):
        print(f"[compare] {what}", file=sys.stderr, flush=True)

    rows = []
    shapes = {"lfm2": shape_config, "gigusun": gigusun_shape_config, "girelix": girelix_shape_config,
              "penopel": penopel_shape_config, "kidarax": kidarax_shape_config}
    for design, data in ((name, shapes[name](shape)) for name in designs):
        say(f"{design} {shape}: writing random weights")
        model_config = config_from_dict(data)
        with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
            write_random_model(folder, model_config, seed=0, dtype="bfloat16")
            context = prompt + 1024
            options = dict(dtype="bfloat16", max_requests=max(batches), context=context, max_tokens=max(batches) * context,
                           page_size=64, prefill_chunk=prompt, prefill_token_budget=max(8192, prompt))
            runner = ModelRunner(folder, EngineConfig(**options))
            vocab = runner.vocab_size
            text = synthetic_prompts(1, prompt, vocab)[0]
            say(f"{design}: prefill of {prompt} tokens")
            pre_ms = measure_prefill(runner, text, repeats=5, warmup=3)
            row = dict(design=design, shape=shape, parameters=sum(matrix_params(runner).values()),
                       prefill=dict(tokens=prompt, ms=round(pre_ms, 3), tokens_per_s=round(prompt / pre_ms * 1e3, 1),
                                    tflops=round(prefill_flops(runner, prompt) / pre_ms / 1e9, 1)), decode={})
            for batch in batches:
                say(f"{design}: decode at {batch} requests")
                run = measure_decode(runner, batch, prompt, steps, warmup, repeats=3)
                row["decode"][str(batch)] = dict(ms_per_step=round(run["ms_per_step"], 4), tokens_per_s=round(run["tokens_per_s"], 1),
                                                 gb_per_s=round(run["bytes"] / run["ms_per_step"] / 1e6, 1),
                                                 kernels=runner.kernels_per_decode_step.get(runner.decode_capacity(batch), 0))
            del runner
            torch.cuda.empty_cache()
            say(f"{design}: time per operation")
            timed = TimedOps(cuda_ops)
            eager = ModelRunner(folder, EngineConfig(**dict(options, cuda_graphs=False)), ops=timed)
            for _ in range(2):
                eager.step([StepEntry("p", text, (prompt - 1,))])
                eager.release("p")
            timed.clear()
            eager.step([StepEntry("p", text, (prompt - 1,))])
            row["prefill_ops"] = [dict(op=r["op"], calls=r["calls"], ms=round(r["ms"], 4)) for r in timed.table()]
            eager.release("p")
            batch = batches[0]
            ids = fill_requests(eager, synthetic_prompts(batch, prompt, vocab), prompt)
            step = [StepEntry(rid, (1,), (0,)) for rid in ids]
            for _ in range(3):
                eager.step(step)
            timed.clear()
            eager.step(step)
            row["decode_ops"] = [dict(op=r["op"], calls=r["calls"], ms=round(r["ms"], 4)) for r in timed.table()]
            del eager
            torch.cuda.empty_cache()
        rows.append(row)
    return rows


def _random_engine(shape: str, **options):
    import tempfile

    from . import Engine, EngineConfig
    from .config import config_from_dict
    from .weights import write_random_model

    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        return Engine(folder, config=EngineConfig(dtype="bfloat16", **options))


def bench_serving(shape: str = "350m", requests: int = 256, shortest: int = 128, longest: int = 2048, generated: int = 128,
                  chunk: int = 512, seed: int = 17) -> dict:
    """Many requests at once through the engine: random prompt lengths, prompts cut into portions of ``chunk``
    that share steps with decoding requests. Wall time from the first submit to the last token."""
    import time

    rng = np.random.default_rng(seed)
    lengths = rng.integers(shortest, longest + 1, requests).tolist()
    vocab = shape_config(shape)["vocab_size"]
    prompts = [rng.integers(0, vocab, n).tolist() for n in lengths]
    pool = sum(-(-(n + generated) // 64) * 64 for n in lengths)
    engine = _random_engine(shape, max_requests=requests, context=longest + generated + 64, max_tokens=pool + 64 * requests,
                            prefill_chunk=chunk, prefill_requests=32, prefill_token_budget=8192)
    with engine:
        engine.warm_up()  # the decode graphs of every batch size
        engine.generate(prompts[:4], max_tokens=8)  # kernels and library handles of the prompt path
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        results = engine.generate(prompts, max_tokens=generated)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        stats = dict(engine.stats)
    out = sum(len(r["generated_tokens"]) for r in results)
    return dict(bench="serving", shape=shape, requests=requests, prompt_tokens=sum(lengths), generated_tokens=out,
                seconds=round(seconds, 3), output_tokens_per_s=round(out / seconds, 1),
                total_tokens_per_s=round((out + sum(lengths)) / seconds, 1), steps=stats["steps"],
                steps_ahead=stats["steps_ahead"], preemptions=stats["preemptions"], max_active=stats["max_active"])


def bench_long_context(shape: str = "700m", requests: int = 8, prompt: int = 30000, generated: int = 256,
                       chunk: int = 2048, seed: int = 17) -> dict:
    """A few very long prompts, then decoding: the paged cache and the split-key decode attention under load."""
    vocab = shape_config(shape)["vocab_size"]
    context = -(-(prompt + generated + 64) // 64) * 64
    engine = _random_engine(shape, max_requests=requests, context=context, max_tokens=requests * context,
                            prefill_chunk=chunk, prefill_token_budget=8192)
    runner = engine.runner
    prompts = synthetic_prompts(requests, prompt, vocab, seed)
    pre = []
    for rep in range(2):
        ids = [f"w{rep}-{i}" for i in range(requests)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for rid, tokens in zip(ids, prompts):
            for at in range(0, prompt, chunk):
                part = tokens[at:at + chunk]
                runner.step([StepEntry(rid, part, (len(part) - 1,) if at + chunk >= prompt else ())])
        stop.record()
        torch.cuda.synchronize()
        pre.append(start.elapsed_time(stop))
        if rep == 0:
            for rid in ids:
                runner.release(rid)
    feed = np.random.default_rng(seed + 1).integers(0, vocab, (generated + 8, requests)).tolist()

    def step(i):
        logits = runner.step([StepEntry(rid, (feed[i][j],), (0,)) for j, rid in enumerate(ids)])
        return runner.ops.argmax(logits)

    for i in range(8):
        step(i)
    ms = _event_ms(lambda: [step(8 + i) for i in range(generated)])
    contexts = [prompt + 8 + generated // 2] * requests
    nbytes = decode_bytes(runner, contexts)
    engine.close()
    return dict(bench="long_context", shape=shape, requests=requests, prompt=prompt, generated=generated,
                prefill_tokens_per_s=round(requests * prompt / (pre[-1] / 1e3), 1), prefill_ms=round(pre[-1], 1),
                decode_ms_per_step=round(ms / generated, 4), decode_tokens_per_s=round(requests * generated / (ms / 1e3), 1),
                decode_gb_per_step=round(nbytes / 1e9, 3), decode_gb_s=round(nbytes / (ms / generated / 1e3) / 1e9, 1))


def bench_ops(shape: str = "1.2b", prompt: int = 2048, batch: int = 8, steps: int = 16) -> dict:
    """Where the device time of one prompt of ``prompt`` tokens and of ``steps`` decode steps of ``batch`` requests
    goes, by operation (CUDA events around every call of the step function's operations; no captured graphs)."""
    import tempfile

    from .config import EngineConfig, config_from_dict
    from .ops import cuda as cuda_ops
    from .ops.timed import TimedOps
    from .weights import write_random_model

    cuda_ops.require(cuda_ops.libraries_for(torch.bfloat16))
    timed = TimedOps(cuda_ops)
    config = EngineConfig(dtype="bfloat16", max_requests=batch, context=prompt + steps + 64, cuda_graphs=False)
    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        runner = ModelRunner(folder, config, ops=timed)
    prompts = synthetic_prompts(batch, prompt, runner.vocab_size)
    ids = [f"o{j}" for j in range(batch)]
    fill_requests(runner, [p[:-1] for p in prompts[1:]], config.prefill_chunk, ids[1:])  # the others, and a warm-up
    timed.clear()
    runner.step([StepEntry(ids[0], prompts[0][:-1], ())])
    prefill = timed.table()
    tokens = [p[-1] for p in prompts]
    runner.step([StepEntry(rid, (t,), (0,)) for rid, t in zip(ids, tokens)])  # first decode step: set-up costs
    timed.clear()
    for _ in range(steps):
        logits = runner.step([StepEntry(rid, (t,), (0,)) for rid, t in zip(ids, tokens)])
        tokens = timed.argmax(logits).tolist()
    decode = timed.table()
    for row in decode:
        row["ms"] /= steps
    round_rows = lambda rows: [dict(op=r["op"], calls=r["calls"], ms=round(r["ms"], 4), share=round(r["share"], 3)) for r in rows]
    return dict(bench="ops", shape=shape, prompt=prompt, batch=batch, prefill=round_rows(prefill),
                decode_per_step=round_rows(decode))


def bench_ops_mixed(shape: str = "350m", portion: int = 512, decoding: int = 255, shortest: int = 128,
                    longest: int = 2176, steps: int = 4) -> dict:
    """Where the device time of a MIXED step goes, by operation: a prompt portion of ``portion`` tokens (of a request
    that already holds as many) beside ``decoding`` requests with contexts spread evenly from ``shortest`` to
    ``longest``, one decoded token each. Measured for both ways of running the decoded tokens' attention: "split"
    (they go to the split-key decode kernel, the portion to the prompt kernel) and "tiles" (every token is a query
    tile of the prompt kernel). CUDA events around every call of the step function's operations; no captured graphs."""
    import tempfile

    from .config import EngineConfig, config_from_dict
    from .ops import cuda as cuda_ops
    from .ops.timed import TimedOps
    from .weights import write_random_model

    cuda_ops.require(cuda_ops.libraries_for(torch.bfloat16))
    timed = TimedOps(cuda_ops)
    lengths = [shortest + (longest - shortest) * j // max(decoding - 1, 1) for j in range(decoding)]
    context = max(longest, 2 * portion) + steps * (portion + 1) + 64
    pool = sum(-(-(n + steps + 64) // 64) * 64 for n in lengths) + context + 64
    config = EngineConfig(dtype="bfloat16", max_requests=decoding + 1, context=context, max_tokens=pool, cuda_graphs=False)
    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        runner = ModelRunner(folder, config, ops=timed)
    rng = np.random.default_rng(7)
    ids = [f"d{j}" for j in range(decoding)]
    fill_requests(runner, [rng.integers(0, runner.vocab_size, n).tolist() for n in lengths], config.prefill_chunk, ids)
    runner.step([StepEntry("p", rng.integers(0, runner.vocab_size, portion).tolist(), ())])
    report = dict(bench="ops-mixed", shape=shape, portion=portion, decoding=decoding, contexts=[shortest, longest])
    before = cuda_ops.mixed_attention
    try:
        for policy in ("split", "tiles"):
            cuda_ops.mixed_attention = policy
            for step in range(steps + 1):
                if step == 1:
                    timed.clear()  # the first step of a policy pays for set-up
                entries = [StepEntry(rid, (int(rng.integers(0, runner.vocab_size)),), (0,)) for rid in ids]
                entries.append(StepEntry("p", rng.integers(0, runner.vocab_size, portion).tolist(), ()))
                runner.step(entries)
            rows = timed.table()
            total = sum(r["ms"] for r in rows) / steps
            report[policy] = dict(ms_per_step=round(total, 4), tokens_per_step=decoding + portion,
                                  ops=[dict(op=r["op"], calls=r["calls"] // steps, ms=round(r["ms"] / steps, 4),
                                            share=round(r["share"], 3)) for r in rows])
            for rid in ["p"]:  # the portioned request starts over, so that both policies see the same lengths
                runner.release(rid)
            runner.step([StepEntry("p", rng.integers(0, runner.vocab_size, portion).tolist(), ())])
    finally:
        cuda_ops.mixed_attention = before
    return report


def bench_timeline(shape: str = "1.2b", batch: int = 8, prompt: int = 2048, context: int = 4096) -> dict:
    """The kernels of ONE captured decode step of ``batch`` requests as the GPU ran them (torch's profiler around a
    graph replay): per kernel name the number of launches, the summed duration, and the time the step advanced while
    it ran, i.e. from the end of the kernels before it to its own end: kernels of the decode path are launched ahead
    of their predecessor's end and wait inside, so durations overlap and their sum exceeds the step."""
    import tempfile

    from torch.profiler import ProfilerActivity, profile

    from .config import EngineConfig, config_from_dict
    from .weights import write_random_model

    config = EngineConfig(dtype="bfloat16", max_requests=max(batch, 1), context=context, max_tokens=batch * context,
                          cuda_graphs=True)
    with tempfile.TemporaryDirectory(prefix="akas-bench-") as folder:
        write_random_model(folder, config_from_dict(shape_config(shape)), seed=0, dtype="bfloat16")
        runner = ModelRunner(folder, config)
    ids = fill_requests(runner, synthetic_prompts(batch, prompt, runner.vocab_size))

    def decode(steps):
        for i in range(steps):
            runner.ops.argmax(runner.step([StepEntry(rid, (5 + i,), (0,)) for rid in ids]))

    decode(5)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        decode(2)
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type.name == "CUDA" and "Memcpy" not in e.name and "Memset" not in e.name),
                    key=lambda e: e.time_range.start)
    first = max(i for i, e in enumerate(events) if "embedding" in e.name)  # the second step
    events = events[first:]
    start = done = events[0].time_range.start
    table: Dict[str, list] = {}
    for e in events:
        name = e.name.replace("(anonymous namespace)::", "")
        name = (name[5:] if name.startswith("void ") else name).split("(")[0].strip()
        row = table.setdefault(name, [0, 0.0, 0.0])
        row[0] += 1
        row[1] += e.time_range.end - e.time_range.start
        row[2] += max(0.0, e.time_range.end - max(done, e.time_range.start))
        done = max(done, e.time_range.end)
    rows = [dict(kernel=k, launches=v[0], duration_us=round(v[1], 1), advanced_us=round(v[2], 1))
            for k, v in sorted(table.items(), key=lambda kv: -kv[1][2])]
    return dict(bench="timeline", shape=shape, batch=batch, prompt=prompt, step_us=round(done - start, 1),
                kernels_per_step=len(events), kernels=rows)


def _main():
    import argparse
    import json

    ap = argparse.ArgumentParser(description="single kernels of the bfloat16 path (cold L2, CUDA events), and two whole-engine runs")
    sub = ap.add_subparsers(dest="what", required=True)
    lin = sub.add_parser("linear", help="y = x . w^T with one of the epilogues")
    lin.add_argument("--m", type=int, nargs="+", default=[8])
    lin.add_argument("--o", type=int, default=2048)
    lin.add_argument("--k", type=int, default=2048)
    lin.add_argument("--mode", default="bf16", choices=("bf16", "f32", "acc", "swiglu", "norm", "norm_swiglu"))
    lin.add_argument("--iters", type=int, default=20)
    att = sub.add_parser("attention", help="paged attention over the cache")
    att.add_argument("--kind", default="decode", choices=("decode", "prompt"))
    att.add_argument("--batch", type=int, nargs="+", default=[8])
    att.add_argument("--context", type=int, default=2048)
    att.add_argument("--heads", type=int, default=32)
    att.add_argument("--kv-heads", type=int, default=8)
    att.add_argument("--head-dim", type=int, default=64)
    att.add_argument("--iters", type=int, default=20)
    exp = sub.add_parser("experts", help="the routed feed-forward's kernels beside a dense feed-forward of equal work")
    exp.add_argument("--tokens", type=int, nargs="+", default=[2048])
    exp.add_argument("--width", type=int, default=2048)
    exp.add_argument("--expert-width", type=int, default=2048)
    exp.add_argument("--experts", type=int, default=14)
    exp.add_argument("--identity", type=int, default=2)
    exp.add_argument("--top", type=int, default=4)
    exp.add_argument("--iters", type=int, default=20)
    srv = sub.add_parser("serving", help="many requests through the engine, prompt portions mixed with decoding")
    srv.add_argument("--shape", default="350m", choices=sorted(SHAPES))
    srv.add_argument("--requests", type=int, default=256)
    srv.add_argument("--generated", type=int, default=128)
    srv.add_argument("--chunk", type=int, default=512)
    lng = sub.add_parser("long-context", help="a few very long prompts, then decoding")
    lng.add_argument("--shape", default="700m", choices=sorted(SHAPES))
    lng.add_argument("--requests", type=int, default=8)
    lng.add_argument("--prompt", type=int, default=30000)
    lng.add_argument("--generated", type=int, default=256)
    tml = sub.add_parser("timeline", help="the kernels of one captured decode step as the GPU ran them")
    tml.add_argument("--shape", default="1.2b", choices=sorted(SHAPES))
    tml.add_argument("--batch", type=int, default=8)
    tml.add_argument("--prompt", type=int, default=2048)
    per = sub.add_parser("ops", help="device time of a prompt and of decode steps, by operation")
    per.add_argument("--shape", default="1.2b", choices=sorted(SHAPES))
    per.add_argument("--prompt", type=int, default=2048)
    per.add_argument("--batch", type=int, default=8)
    per.add_argument("--steps", type=int, default=16)
    per.add_argument("--mixed", type=int, nargs=2, metavar=("PORTION", "DECODING"), default=None,
                     help="a mixed step instead: a prompt portion of PORTION tokens beside DECODING decoding requests")
    args = ap.parse_args()
    if args.what == "timeline":
        print(json.dumps(bench_timeline(args.shape, args.batch, args.prompt), indent=1))
        return
    if args.what == "ops" and args.mixed:
        print(json.dumps(bench_ops_mixed(args.shape, args.mixed[0], args.mixed[1], steps=min(args.steps, 8)), indent=1))
        return
    if args.what == "ops":
        print(json.dumps(bench_ops(args.shape, args.prompt, args.batch, args.steps), indent=1))
        return
    if args.what == "serving":
        print(json.dumps(bench_serving(args.shape, args.requests, generated=args.generated, chunk=args.chunk)))
        return
    if args.what == "long-context":
        print(json.dumps(bench_long_context(args.shape, args.requests, args.prompt, args.generated)))
        return
    if args.what == "experts":
        for n in args.tokens:
            print(json.dumps(bench_experts(n, args.width, args.expert_width, args.experts, args.identity, args.top, iters=args.iters)))
        return
    if args.what == "attention":
        for b in args.batch:
            print(json.dumps(bench_attention(args.kind, b, args.context, args.heads, args.kv_heads, args.head_dim,
                                             iters=args.iters)))
        return
    for m in args.m:
        print(json.dumps(bench_linear(m, args.o, args.k, args.mode, args.iters)))


if __name__ == "__main__":
    _main()
