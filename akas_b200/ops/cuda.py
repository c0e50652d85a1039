"""The compiled sm_100a kernels behind the signatures that the parts call.

Every function takes torch CUDA tensors, allocates its output with torch, and
launches the kernel of ``akas_b200/csrc`` on torch's current stream through the
library's C entry point. ``akas_b200.ops.reference`` states the same functions in
plain PyTorch. A missing compiler, a failed build or a launch error raises; there
is no other path.
"""

from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Iterable, Optional

import torch

from . import build

name = "cuda-sm100a"

_F32, _BF16 = 0, 1
_CODE = {torch.float32: _F32, torch.bfloat16: _BF16}
_WORKSPACE_BYTES = 64 << 20
_workspaces = {}
launch_count = 0  # kernels launched through this module since import (library products count as one)

_SIGNATURES = {
    "elementwise": {
        "akas_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
        "akas_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_take_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "akas_zero_row": [c_void_p, c_longlong, c_int, c_int, c_longlong, c_void_p],
        "akas_add_bias": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_scale_cap": [c_void_p, c_float, c_float, c_longlong, c_void_p],
        "akas_add_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_polynorm": [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_scaled_add": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p],
        "akas_dynamic_tanh": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_activation": [c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_gated_activation": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_int, c_void_p],
    },
    "latent": {
        "akas_latent_norm_store": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                   c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                   c_void_p],
        "akas_head_linear": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
    "moe": {
        "akas_moe_route": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "akas_moe_gate_up": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_void_p, c_void_p],
        "akas_moe_down": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_longlong,
                          c_void_p],
    },
    "recurrent": {
        "akas_decay_gates": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "akas_gla_scan": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "akas_delta_scan": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                            c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "akas_causal_conv_silu": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "akas_delta_prep": [c_void_p, c_longlong, c_int, c_int, c_float, c_float, c_void_p, c_longlong, c_void_p, c_longlong,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_gated_rmsnorm": [c_void_p, c_void_p, c_float, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_float, c_longlong, c_void_p],
        "akas_decay_chunk_scratch": [c_int, c_int, c_int, c_int, c_int],
        "akas_decay_scan_chunked": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                    c_int, c_void_p],
        "akas_decay_scan": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                            c_void_p],
    },
    "attention_general": {
        "akas_qk_norm_store": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_float,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p],
        "akas_attention_general": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int,
                                   c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_int, c_void_p, c_float, c_longlong, c_longlong, c_int, c_int, c_void_p],
    },
    "attention_general_tc": {
        "akas_attention_general_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float,
                                      c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_longlong, c_void_p, c_int,
                                      c_longlong, c_int, c_int, c_void_p],
        "akas_attention_general_tc_takes": [c_int, c_int],
    },
    "moe_grouped": {
        "akas_moe_grouped_rows": [c_int, c_int],
        "akas_moe_grouped_takes": [c_int, c_int, c_int],
        "akas_moe_sort": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                          c_void_p, c_void_p],
        "akas_moe_grouped_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "akas_moe_combine": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_longlong, c_void_p],
        "akas_moe_grouped_status": [],
    },
    "conv": {
        "akas_short_conv": [c_void_p] * 8 + [c_int] * 6 + [c_void_p],
        "akas_short_conv_decode": [c_void_p] * 7 + [c_int] * 5 + [c_void_p],
    },
    "rope": {
        "akas_rope_tables": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
        "akas_qk_norm_rope_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int,
                                    c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_void_p],
        "akas_kv_store": [c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
    "attention": {
        "akas_paged_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "akas_paged_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p],
    },
    "attention_prefill": {
        "akas_prefill_attention_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
    "attention_prefill_tc": {
        "akas_prefill_attention_tc": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "akas_prefill_attention_tc_status": [],
    },
    "attention_decode": {
        "akas_decode_attention_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p],
        "akas_decode_attention_bf16_paged": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int,
                                             c_int, c_int, c_void_p],
        "akas_decode_attention_from_qkv": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int,
                                           c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p],
        "akas_decode_attention_items": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int,
                                        c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_void_p],
        "akas_decode_attention_items_places": [c_int, c_int],
        "akas_decode_attention_status": [],
    },
    "gemm_tcgen05": {
        "akas_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_gemm_tcgen05_status": [],
    },
    "gemm_pair": {
        "akas_gemm_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_gemm_pair_bias": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
        "akas_gemm_pair_status": [],
    },
    "gemm_rows": {
        "akas_gemm_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "akas_gemm_rows_bias": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
        "akas_gemm_rows_takes": [c_int, c_int, c_int, c_int],
        "akas_gemm_rows_status": [],
    },
    "gemm_stream": {
        "akas_stream_gemm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_int, c_void_p],
        "akas_stream_gemm_takes": [c_int, c_int, c_int, c_int, c_int],
        "akas_stream_gemm_status": [],
    },
    "skinny_gemm": {
        "akas_skinny_gemm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_int, c_int, c_void_p],
        "akas_skinny_gemm_conv": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "akas_skinny_gemm_more": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_int, c_int, c_void_p, c_int, c_void_p],
        "akas_skinny_gemm_status": [],
    },
    "decode_chain": {
        "akas_chain_set_scratch": [c_void_p],
        "akas_chain_scratch_words": [],
        "akas_chain_begin": [],
        "akas_chain_count": [],
        "akas_chain_takes": [c_int] * 5,
        "akas_chain_gemm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int],
        "akas_chain_conv": [c_void_p] * 7 + [c_int] * 4,
        "akas_chain_embed": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int],
        "akas_chain_run": [c_void_p],
        "akas_chain_status": [],
    },
    "sgemm": {
        "akas_sgemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "gemm_bf16": {
        "akas_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong,
                           c_void_p],
    },
    "sampling": {
        "akas_argmax": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "akas_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "akas_adjust_logits": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
}

_RESTYPES = {"akas_decay_chunk_scratch": c_longlong}  # everything else returns an int (an error code or a small answer)
_functions = {}


def libraries_for(dtype: torch.dtype, parts: Iterable[str] = ("attention", "short_conv")) -> list:
    """The kernel files a model of this compute dtype needs under the switches as they stand: what a first call
    compiles. ``parts``: the kinds of kernels its mixers asked for (``Part.kernels``); the default is LFM2's. A file
    that only a switch's other value needs (the library arm of the products, the tcgen05 decode products, the decode
    chain) is built when that value is first used."""
    names = ["elementwise", "sampling"]
    for kind in parts:
        for name in _PART_FILES[kind](dtype):
            if name not in names:
                names.append(name)
    if dtype == torch.float32:
        return names + ["sgemm"]
    names += ["gemm_tcgen05", "gemm_pair", "gemm_rows", "skinny_gemm"]
    if products == "library":
        names.append("gemm_bf16")
    if decode_products == "stream":
        names.append("gemm_stream")
    if decode_chain == "1":
        names.append("decode_chain")
    return names


_PART_FILES = {
    "attention": lambda dtype: ["rope", "attention"] + (["attention_prefill", "attention_prefill_tc", "attention_decode"]
                                                        if dtype == torch.bfloat16 else []),
    "short_conv": lambda dtype: ["conv"],
    "attention_general": lambda dtype: ["attention_general"] + (["attention_general_tc"] if dtype == torch.bfloat16 else []),
    "recurrent": lambda dtype: ["recurrent"],
    "moe": lambda dtype: ["moe"] + (["moe_grouped"] if dtype == torch.bfloat16 else []),
    "rope": lambda dtype: ["rope"],
    "latent": lambda dtype: ["latent"],
}


def require(names: Optional[Iterable[str]] = None) -> None:
    """Builds (if need be) and loads the named kernel files, or all of them; raises if that fails."""
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: akas_b200's kernels run on an NVIDIA B200 (sm_100a) only")
    names = list(names) if names is not None else list(_SIGNATURES)
    build.ensure_built(names)
    for n in names:
        _bind(n)
    if "decode_chain" in names:
        _chain_barrier_word(torch.device("cuda", torch.cuda.current_device()))


def _bind(lib_name: str) -> None:
    lib = build.library(lib_name)
    for fn_name, argtypes in _SIGNATURES[lib_name].items():
        if fn_name not in _functions:
            fn = getattr(lib, fn_name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(fn_name, c_int)
            _functions[fn_name] = fn


def _fn(lib_name: str, fn_name: str):
    fn = _functions.get(fn_name)
    if fn is None:
        _bind(lib_name)
        fn = _functions[fn_name]
    return fn


def _check(err: int, what: str, kernels: int = 1) -> None:
    global launch_count
    launch_count += kernels
    if err:
        if err >= 2000:
            detail = f"cuBLASLt found no algorithm (status {err - 2000})"
        elif err >= 1000:
            detail = f"cuBLAS status {err - 1000}"
        else:
            detail = f"CUDA error {err}"
        raise RuntimeError(f"{what} failed: {detail}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The handle of torch's current stream on the current device (every launch goes there)."""
    if _raw_stream is not None:  # the same value as below without building a Stream object per launch
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _code(t: torch.Tensor) -> int:
    try:
        return _CODE[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _dense(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    return t


# --------------------------------------------------------------------------- chained decode steps
#
# A decode step is a chain of small operations: products for a handful of tokens, the short convolution, the
# embedding look-up. Between ``chain_begin`` and ``chain_end`` (the decoder brackets a decode step with them) the
# functions below that can join a chain do not launch: they allocate their output, add themselves to a program, and
# return; the program runs as ONE persistent launch (csrc/decode_chain.cu) when an operation comes that cannot join
# (every other function of this module flushes first), when it is full, or at ``chain_end``. A part that touches
# tensors by other means than this module's functions must not run inside a chain: the decoder flushes before any
# block whose parts do not declare ``chain_safe``. Chains are off unless AKAS_B200_DECODE_CHAIN=1: measured on the
# 1.2B shape at 8 tokens a chained step takes 1.03 ms against 0.89 ms for one launch per operation (a meeting of the
# whole grid inside a kernel costs what a kernel boundary with a programmatic dependent launch costs, and one block
# per SM keeps fewer bytes in flight than two); both are tested.
decode_chain = os.environ.get("AKAS_B200_DECODE_CHAIN", "0")
if decode_chain not in ("0", "1"):
    raise ValueError(f"AKAS_B200_DECODE_CHAIN must be 0 or 1, got {decode_chain!r}")
_CHAIN_ROWS = 16
_chain_open = False
_chain_keep = []  # tensors of the program under construction, kept alive until it has been launched
_chain_words = {}
_chain_answers = {}


def _chain_barrier_word(device):
    """The words of device memory that the blocks of a chain meet on and count tiles in (zeroed once; the kernel
    leaves them as it found them)."""
    word = _chain_words.get(device)
    if word is None:
        count = int(_fn("decode_chain", "akas_chain_scratch_words")())
        word = _chain_words[device] = torch.zeros(count, dtype=torch.int32, device=device)
        _check(_fn("decode_chain", "akas_chain_set_scratch")(_ptr(word)), "chain scratch", kernels=0)
    return word


def chain_begin(num_tokens: int) -> bool:
    """Opens a chain for a decode step of ``num_tokens`` tokens; False if chains are off or the step is too large."""
    global _chain_open
    device = torch.device("cuda", torch.cuda.current_device())
    if decode_chain != "1" or num_tokens > _CHAIN_ROWS or _chain_open or device not in _chain_words:
        return False  # (no barrier word: the chain's library was not asked for, as for a float32 model)
    _fn("decode_chain", "akas_chain_begin")()
    _chain_open = True
    return True


def chain_flush() -> None:
    """Launches what the chain holds so far; the chain stays open."""
    if _chain_open and _fn("decode_chain", "akas_chain_count")():
        err = _fn("decode_chain", "akas_chain_run")(_stream())
        _chain_keep.clear()
        _check(err, "decode chain")


def chain_end() -> None:
    global _chain_open
    try:
        chain_flush()
    finally:
        _chain_open = False
        _chain_keep.clear()


def chain_status() -> int:
    """0 unless a bounded wait inside the chain kernel has run out on this device. Synchronises."""
    return int(_fn("decode_chain", "akas_chain_status")())


def _chain_takes(m: int, o: int, k: int, in_mode: int, mode: int) -> bool:
    if not _chain_open or m > _CHAIN_ROWS:
        return False
    key = (m > 8, o % 2, k, in_mode, mode)
    answer = _chain_answers.get(key)
    if answer is None:
        answer = _chain_answers[key] = bool(_fn("decode_chain", "akas_chain_takes")(m, o, k, in_mode, mode))
    return answer


_CHAIN_OPS = int(os.environ.get("AKAS_B200_CHAIN_OPS", "24"))  # the most operations of one launch


def _chain_add(fn_name: str, keep, *args) -> None:
    """Adds an operation to the open chain (launching the chain first when it is full)."""
    fn = _fn("decode_chain", fn_name)
    if _fn("decode_chain", "akas_chain_count")() >= _CHAIN_OPS:
        chain_flush()
    err = fn(*args)
    if err == 1:  # the program is full
        chain_flush()
        err = fn(*args)
    if err:
        raise RuntimeError(f"{fn_name} failed: error {err}")
    _chain_keep.extend(keep)


def _flushes(fn):
    """An operation that cannot join a chain: whatever the chain holds runs first."""
    @functools.wraps(fn)
    def flushed(*args, **kwargs):
        if _chain_open:
            chain_flush()
        return fn(*args, **kwargs)
    return flushed


# --------------------------------------------------------------------------- elementwise


def embedding(token_ids, table):
    n, c = token_ids.numel(), table.shape[1]
    out = torch.empty((n, c), dtype=torch.float32, device=table.device)
    if _chain_open and n <= _CHAIN_ROWS:
        _chain_add("akas_chain_embed", (token_ids, table, out), _ptr(token_ids), _ptr(_dense(table, "table")), _ptr(out), n, c,
                   _code(table))
        return out
    _check(_fn("elementwise", "akas_embedding")(_ptr(token_ids), _ptr(_dense(table, "table")), _ptr(out), n, c,
                                               _code(table), _stream()), "embedding")
    return out


@_flushes
def take_tokens(token_ids, source, previous):
    """token_ids[i] = previous[source[i]] where source[i] >= 0 (all int32, in place)."""
    _check(_fn("elementwise", "akas_take_tokens")(_ptr(token_ids), _ptr(source), _ptr(previous), previous.numel(),
                                                 token_ids.numel(), _stream()), "take_tokens")


@_flushes
def rmsnorm(x, weight, eps, zero_centered, out_dtype, rows=None):
    c = x.shape[-1]
    _dense(x, "x")
    lead = x.shape[:-1]
    m = rows.numel() if rows is not None else x.numel() // c
    out_shape = (m, c) if rows is not None else (*lead, c)
    out = torch.empty(out_shape, dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "akas_rmsnorm")(_ptr(x), _ptr(weight), _ptr(out), _ptr(rows), m, c, float(eps),
                                             int(bool(zero_centered)), _code(x), _CODE[out_dtype], _stream()),
           "rmsnorm")
    return out


@_flushes
def swiglu(gate_up):
    n, f2 = gate_up.shape
    out = torch.empty((n, f2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(_fn("elementwise", "akas_swiglu")(_ptr(_dense(gate_up, "gate_up")), _ptr(out), n, f2 // 2, _code(gate_up),
                                            _stream()), "swiglu")
    return out


@_flushes
def add_bias(x, bias, out_dtype=None):
    """x [N, C] float32 plus bias [C] float32, rounded once to ``out_dtype``; in place when that is float32."""
    n, c = x.shape
    if x.dtype != torch.float32 or bias.dtype != torch.float32 or bias.numel() != c:
        raise ValueError("add_bias takes float32 x [N, C] and a float32 bias [C]")
    target = out_dtype or torch.float32
    out = x if target == torch.float32 else torch.empty((n, c), dtype=target, device=x.device)
    _check(_fn("elementwise", "akas_add_bias")(_ptr(_dense(x, "x")), _ptr(bias), _ptr(out), n, c, _CODE[target], _stream()),
           "add_bias")
    return out


@_flushes
def scale_cap(x, scale=1.0, cap=0.0):
    """In place on float32 x: times ``scale``, then ``cap * tanh(x / cap)`` where ``cap`` > 0."""
    if x.dtype != torch.float32:
        raise TypeError("scale_cap takes float32")
    _check(_fn("elementwise", "akas_scale_cap")(_ptr(_dense(x, "x")), float(scale), float(cap), x.numel(), _stream()),
           "scale_cap")
    return x


@_flushes
def zero_rows(state, slot):
    """state[:, slot] = 0 for a contiguous tensor [layers, slots, ...]."""
    row = state[0, 0].numel()
    if state.dtype != torch.float32 or not state.is_contiguous():
        state[:, slot].zero_()
        return
    _check(_fn("elementwise", "akas_zero_row")(_ptr(state), row, int(slot), state.shape[0], state[0].numel(), _stream()),
           "zero_rows")


# --------------------------------------------------------------------------- matrix products


def _workspace(device):
    ws = _workspaces.get(device)
    if ws is None:
        ws = _workspaces[device] = torch.empty(_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    return ws


def linear(x, w, out_dtype=None, residual=None, bias=None):
    """x [N, K] times w [O, K] transposed. With ``residual`` (float32 [N, O]) the product is added into it. ``bias``
    (float32 [O]) rides in the read-out of a product that is added into the residual; elsewhere it is added by a
    kernel of its own, before the one rounding."""
    if bias is not None:
        return _linear_bias(x, w, out_dtype, residual, bias)
    n, k = x.shape
    o = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"linear: x has {k} columns, w has {w.shape[1]}")
    _dense(x, "x")
    _dense(w, "w")
    if x.dtype != w.dtype:
        raise TypeError(f"linear: x is {x.dtype}, w is {w.dtype}")
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (n, o) or not residual.is_contiguous():
            raise ValueError("linear: residual must be contiguous float32 [N, O]")
    if x.dtype == torch.float32:
        if _chain_open:
            chain_flush()
        out = residual if residual is not None else torch.empty((n, o), dtype=torch.float32, device=x.device)
        _check(_fn("sgemm", "akas_sgemm")(_ptr(x), _ptr(w), _ptr(out), _ptr(residual), n, o, k, _stream()), "sgemm")
        if residual is None and out_dtype not in (None, torch.float32):
            out = out.to(out_dtype)
        return out
    if x.dtype != torch.bfloat16:
        raise TypeError(f"linear takes float32 or bfloat16, got {x.dtype}")
    if k % 8 and _pad_inner:
        # The tensor-core kernels take inner sizes that are multiples of 8 (16 bytes of bfloat16): both operands get
        # columns of zeros up to the next one. The weights are padded once and kept.
        x, w = _padded_inner(x, False), _padded_inner(w, True)
        k = x.shape[1]
    target = out_dtype or torch.bfloat16
    mode = _OUT_ACC if residual is not None else _OUT_F32 if target == torch.float32 else _OUT_BF16
    if _chain_takes(n, o, k, 0, mode):
        out = residual if residual is not None else torch.empty((n, o), dtype=target, device=x.device)
        _chain_add("akas_chain_gemm", (x, w, out), _ptr(x), None, None, 0.0, 0, _ptr(w), _ptr(out), n, o, k, 0, mode)
        return out
    if _chain_open:
        chain_flush()
    if _stream_takes(n, o, k, False, mode):
        # few tokens: the weights are streamed once through the tensor cores
        out = residual if residual is not None else torch.empty((n, o), dtype=target, device=x.device)
        _stream_product(x, None, None, 0.0, False, False, w, out, n, o, k, mode)
        return out
    if _skinny_fits(n, k):
        out = residual if residual is not None else torch.empty((n, o), dtype=target, device=x.device)
        _skinny(x, None, None, 0.0, False, w, out, n, o, k, 0, mode)
        return out
    if k % 8:
        raise ValueError(f"bfloat16 matrix products need an inner size that is a multiple of 8, got {k}")
    route = _product_route(k, o, mode)
    if route == "paired":
        return paired_product(x, w, out_dtype=target, residual=residual)
    if route == "block":
        return block_product(x, w, out_dtype=target, residual=residual)
    if residual is not None:
        out, out_f32, acc = residual, 1, 1
    else:
        out = torch.empty((n, o), dtype=target, device=x.device)
        out_f32, acc = int(target == torch.float32), 0
    ws = _workspace(x.device)
    _check(_fn("gemm_bf16", "akas_gemm_bf16")(_ptr(x), _ptr(w), _ptr(out), n, o, k, out_f32, acc, _ptr(ws),
                                             ws.numel(), _stream()), f"bfloat16 product [{n}x{k}] x [{o}x{k}]^T")
    return out


def _biased_route(x, w, n, o, k, gated: bool):
    """Which kernel with a biased read-out takes a bfloat16 product of these sizes: "skinny", "rows", "paired" or None."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or _chain_open or decode_products != "skinny" or products == "library":
        return None
    if _skinny_fits(n, k):
        return "skinny"
    if k % 8 or (gated and o % 16) or (not gated and o % 4):
        return None
    if _rows_takes(n, o, k, 2 if gated else 1):
        return "rows"
    return "paired" if n > _SKINNY_ROWS else None


def _linear_bias(x, w, out_dtype, residual, bias):
    n, k = x.shape
    o = w.shape[0]
    if bias.dtype != torch.float32 or bias.numel() != o or not bias.is_contiguous():
        raise ValueError("linear: bias must be a dense float32 vector with one number per output channel")
    route = _biased_route(_dense(x, "x"), _dense(w, "w"), n, o, k, False) if residual is not None and w.shape[1] == k else None
    if route is None:
        if residual is not None:
            return linear(x, w, residual=add_bias(residual, bias))
        return add_bias(linear(x, w, out_dtype=torch.float32), bias, out_dtype or x.dtype)
    if residual.dtype != torch.float32 or residual.shape != (n, o) or not residual.is_contiguous():
        raise ValueError("linear: residual must be contiguous float32 [N, O]")
    if route == "skinny":
        _check(_fn("skinny_gemm", "akas_skinny_gemm_more")(_ptr(x), None, None, None, None, _ptr(w), _ptr(residual), n, o, k, 0,
                                                          _OUT_ACC, _ptr(bias), 0, _stream()), "skinny product with a bias")
    else:
        name = "gemm_rows" if route == "rows" else "gemm_pair"
        _check(_fn(name, f"akas_{name}_bias")(_ptr(x), _ptr(w), _ptr(residual), n, o, k, 1, _ptr(bias), 0, _stream()),
               f"{name} product with a bias")
    return residual


def linear_gated(x, w_gate_up, width, bias, activation):
    """act(g + b_g) * (u + b_u) for [g | u] = x . w^T with w the stacked gate and up matrices (``width`` = F rows each,
    then rows of padding, if any), bias float32 [2F] or None, activation "silu" or "gelu_tanh": [N, F] in x's dtype. In bfloat16 the activation rides in the
    product's read-out (the [N, 2F] intermediate is never written); elsewhere the product leaves float32 and
    ``gated_activation`` follows."""
    n, k = x.shape
    f2 = w_gate_up.shape[0]
    if activation not in _ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}")
    if f2 < 2 * width or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != 2 * width or not bias.is_contiguous())):
        raise ValueError("linear_gated takes the stacked gate and up matrices and a dense float32 bias [2F]")
    # (rows of padding below the two matrices: the read-out pairs row f with row F + f of exactly 2F rows)
    route = _biased_route(_dense(x, "x"), _dense(w_gate_up, "w"), n, f2, k, True) if w_gate_up.shape[1] == k and f2 == 2 * width else None
    if route is None:
        if _chain_open:
            chain_flush()
        return gated_activation(linear(x, w_gate_up, out_dtype=torch.float32), width, bias, activation, x.dtype)
    out = torch.empty((n, f2 // 2), dtype=torch.bfloat16, device=x.device)
    act = _READOUT_ACTIVATIONS[activation]
    if route == "skinny":
        _check(_fn("skinny_gemm", "akas_skinny_gemm_more")(_ptr(x), None, None, None, None, _ptr(w_gate_up), _ptr(out), n, f2, k, 0,
                                                          _OUT_SWIGLU, _ptr(bias), act, _stream()), "skinny gated product")
    else:
        name = "gemm_rows" if route == "rows" else "gemm_pair"
        _check(_fn(name, f"akas_{name}_bias")(_ptr(x), _ptr(w_gate_up), _ptr(out), n, f2, k, 2, _ptr(bias), act, _stream()),
               f"{name} gated product")
    return out


_READOUT_PLAIN = {"gelu_tanh": 1, "relu2": 2, "silu": 3}  # the bfloat16 read-outs' activations without a gate (0: none)


def linear_activated(x, w, activation):
    """act(x . w^T) in x's dtype, for an activation without a gate ("relu2", "gelu_tanh", "silu"). In bfloat16 the
    activation rides in the product's read-out on the float32 sums; None where no kernel with that read-out takes the
    sizes (the caller then runs the product in float32 and ``activation``)."""
    n, k = x.shape
    o = w.shape[0]
    if activation not in _READOUT_PLAIN:
        raise ValueError(f"unknown activation {activation!r}")
    if (w.shape[1] != k or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or _chain_open or decode_products != "skinny"
            or products == "library"):
        return None
    _dense(x, "x"), _dense(w, "w")
    if _skinny_fits(n, k):
        route = "skinny"
    elif k % 8 or o % 8:
        return None
    elif _rows_takes(n, o, k, 0):
        route = "rows"
    elif n > _SKINNY_ROWS:
        route = "paired"
    else:
        return None
    out = torch.empty((n, o), dtype=torch.bfloat16, device=x.device)
    act = _READOUT_PLAIN[activation]
    if route == "skinny":
        _check(_fn("skinny_gemm", "akas_skinny_gemm_more")(_ptr(x), None, None, None, None, _ptr(w), _ptr(out), n, o, k, 0,
                                                          _OUT_BF16, None, act, _stream()), "skinny product with an activation")
    else:
        name = "gemm_rows" if route == "rows" else "gemm_pair"
        _check(_fn(name, f"akas_{name}_bias")(_ptr(x), _ptr(w), _ptr(out), n, o, k, 0, None, act, _stream()),
               f"{name} product with an activation")
    return out


def dyt_linear_activated(h, alpha, weight, shift, w, activation, rows=None):
    """act(linear(dynamic_tanh(h[rows]), w)) for few tokens: the norm on the product's way in, the activation in its
    read-out. None where the fused kernel does not take the sizes or the dtype."""
    m = rows.numel() if rows is not None else h.shape[0]
    k, o = h.shape[1], w.shape[0]
    if activation not in _READOUT_PLAIN:
        raise ValueError(f"unknown activation {activation!r}")
    if (w.dtype != torch.bfloat16 or h.dtype != torch.float32 or not h.is_contiguous() or w.shape[1] != k or _chain_open
            or decode_products != "skinny" or not _skinny_fits(m, k) or alpha.dtype != torch.float32):
        return None
    out = torch.empty((m, o), dtype=torch.bfloat16, device=h.device)
    _check(_fn("skinny_gemm", "akas_skinny_gemm_more")(_ptr(h), _ptr(rows), _ptr(weight), _ptr(shift), _ptr(alpha), _ptr(_dense(w, "w")),
                                                      _ptr(out), m, o, k, 2, _OUT_BF16, None, _READOUT_PLAIN[activation], _stream()),
           "skinny product behind a norm without sums, with an activation")
    return out


def dyt_linear(h, alpha, weight, shift, w, out_dtype=None, rows=None, gated=None):
    """linear(dynamic_tanh(h[rows]), w) for few tokens, the norm computed on the product's way in; with ``gated`` =
    (width, bias or None, activation) through the gated read-out as ``linear_gated``. None where the fused kernel does not take
    the sizes or the dtype (the caller then runs the norm by itself)."""
    m = rows.numel() if rows is not None else h.shape[0]
    k, o = h.shape[1], w.shape[0]
    if (w.dtype != torch.bfloat16 or h.dtype != torch.float32 or not h.is_contiguous() or w.shape[1] != k or _chain_open
            or decode_products != "skinny" or not _skinny_fits(m, k) or alpha.dtype != torch.float32):
        return None
    bias, act, mode = None, 0, _OUT_F32 if out_dtype == torch.float32 else _OUT_BF16
    if gated is not None:
        width, bias, activation = gated
        if o != 2 * width or activation not in _ACTIVATIONS or (bias is not None and (bias.dtype != torch.float32 or bias.numel() != o)):
            return None
        act, mode = _READOUT_ACTIVATIONS[activation], _OUT_SWIGLU
    elif out_dtype not in (None, torch.bfloat16, torch.float32):
        return None
    out = torch.empty((m, o // 2 if gated is not None else o), dtype=torch.float32 if mode == _OUT_F32 else torch.bfloat16,
                      device=h.device)
    _check(_fn("skinny_gemm", "akas_skinny_gemm_more")(_ptr(h), _ptr(rows), _ptr(weight), _ptr(shift), _ptr(alpha), _ptr(_dense(w, "w")),
                                                      _ptr(out), m, o, k, 2, mode, _ptr(bias), act, _stream()),
           "skinny product behind a norm without sums")
    return out


_pad_inner = True  # False: an inner size that is no multiple of 8 is refused, as the kernels themselves refuse it
_padded_weights = {}


def _padded_inner(t, keep: bool):
    """``t`` [rows, K] with zero columns up to the next multiple of 8; for weights (``keep``) made once per tensor."""
    key = (t.data_ptr(), tuple(t.shape), t.device)
    if keep and key in _padded_weights:
        return _padded_weights[key][1]
    out = torch.nn.functional.pad(t, (0, -t.shape[1] % 8)).contiguous()
    if keep:
        _padded_weights[key] = (t, out)  # the original is held too, so that its address is not handed out again
    return out


def _skinny_fits(m: int, k: int) -> bool:
    """Whether the skinny kernel takes this product: few tokens, an inner size that is a multiple of 64 (its TMA
    boxes), and activations that fit in shared memory beside the ring of weight chunks."""
    tokens = 8 if m <= 8 else 16
    return decode_products == "skinny" and m <= _SKINNY_ROWS and k % 64 == 0 and 1024 + 8 * 8192 + tokens * 512 + tokens * (k + 32) * 2 <= 226 * 1024


_SKINNY_ROWS = 16
# Which kernels run the products of more than 16 tokens (prompt portions, mixed steps, large decode batches). "own"
# (default; "auto" and "tcgen05" mean the same): the hand-written tcgen05 kernels everywhere: the kernel for pairs of
# SMs (gemm_pair.cu, TMA-written read-outs) for every product whose output rows TMA can write, the one-block kernel
# (gemm_tcgen05.cu, masked read-outs) for the rest. "library": cuBLASLt everywhere, with SwiGLU as a kernel of its
# own: the arm that the hand-written kernels are measured against.
products = os.environ.get("AKAS_B200_PRODUCTS", "own")
if products not in ("own", "auto", "tcgen05", "library"):
    raise ValueError(f"AKAS_B200_PRODUCTS must be own or library, got {products!r}")


def _product_route(k: int, o: int, mode: int) -> str:
    """Which kernel runs a product of more than 16 tokens with inner size k and o output channels (for SwiGLU the
    stacked 2F): "paired", "block", "library", or (SwiGLU only) "unfused"."""
    if products == "library":
        return "library"
    if mode == _OUT_SWIGLU:
        return "paired" if o % 16 == 0 else "unfused"  # unfused: the plain product, then the SwiGLU kernel
    pitch_ok = o % 8 == 0 if mode == _OUT_BF16 else o % 4 == 0
    return "paired" if pitch_ok else "block"


_sms = 0


def _sm_count() -> int:
    global _sms
    if not _sms:
        _sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sms


@_flushes
def block_product(x, w, swiglu_out: bool = False, out_dtype=None, residual=None):
    """The same products on the one-block tcgen05 kernel (gemm_tcgen05.cu), whose masked read-outs take any width:
    the route of sizes whose rows TMA cannot write (a pitch that is no multiple of 16 bytes). A float32 result is
    summed into zeros."""
    n, k = x.shape
    o = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k or k % 8:
        raise ValueError("block_product takes bfloat16 [N, K] and [O, K] with K a multiple of 8")
    kernels = 1
    if swiglu_out:
        if o % 16:
            raise ValueError("block_product: the stacked gate and up matrices need a height that is a multiple of 16")
        out, epilogue = torch.empty((n, o // 2), dtype=torch.bfloat16, device=x.device), 2
    elif residual is not None:
        out, epilogue = residual, 1
    elif out_dtype == torch.float32:
        out, epilogue, kernels = torch.zeros((n, o), dtype=torch.float32, device=x.device), 1, 2
    else:
        out, epilogue = torch.empty((n, o), dtype=torch.bfloat16, device=x.device), 0
    _check(_fn("gemm_tcgen05", "akas_gemm_tcgen05")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                                   _stream()), f"tcgen05 product [{n}x{k}] x [{o}x{k}]^T", kernels=kernels)
    return out


def _tma_product(name, x, w, swiglu_out, out_dtype, residual):
    """The checks and the output of a product whose read-out TMA writes: (out, epilogue code)."""
    n, k = x.shape
    o = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k or k % 8:
        raise ValueError(f"{name} takes bfloat16 [N, K] and [O, K] with K a multiple of 8")
    if swiglu_out:
        if o % 16:
            raise ValueError(f"{name}: the stacked gate and up matrices need a height that is a multiple of 16")
        return torch.empty((n, o // 2), dtype=torch.bfloat16, device=x.device), 2
    if residual is not None:
        if residual.dtype != torch.float32 or residual.shape != (n, o) or not residual.is_contiguous() or o % 4:
            raise ValueError(f"{name}: residual must be contiguous float32 [N, O] with O a multiple of 4")
        return residual, 1
    if out_dtype == torch.float32:
        if o % 4:
            raise ValueError(f"{name}: a float32 result needs a width that is a multiple of 4")
        return torch.empty((n, o), dtype=torch.float32, device=x.device), 3
    if o % 8:
        raise ValueError(f"{name}: a bfloat16 result needs a width that is a multiple of 8")
    return torch.empty((n, o), dtype=torch.bfloat16, device=x.device), 0


# Products of 17 to 128 tokens (decode steps of many requests, short portions) stream the weights through every SM
# (gemm_rows.cu); AKAS_B200_ROWS_PRODUCTS=0 gives them to the kernel for pairs of SMs like longer portions.
_ROWS_MAX = 128
rows_products = os.environ.get("AKAS_B200_ROWS_PRODUCTS", "1") != "0"
_rows_answers = {}


def _rows_takes(n: int, o: int, k: int, epilogue: int) -> bool:
    if not rows_products or n > _ROWS_MAX:
        return False
    key = (torch.cuda.current_device(), n, o, k, epilogue)
    answer = _rows_answers.get(key)
    if answer is None:
        answer = _rows_answers[key] = bool(_fn("gemm_rows", "akas_gemm_rows_takes")(n, o, k, epilogue))
    return answer


@_flushes
def rows_product(x, w, swiglu_out: bool = False, out_dtype=None, residual=None):
    """x [N, K] times w [O, K] transposed for at most 128 tokens: the weights streamed once through all SMs, the
    read-outs of ``paired_product``."""
    n, k = x.shape
    o = w.shape[0]
    out, epilogue = _tma_product("rows_product", x, w, swiglu_out, out_dtype, residual)
    if not _rows_takes(n, o, k, epilogue):
        raise ValueError(f"rows_product does not take [{n}x{k}] x [{o}x{k}]^T (at most {_ROWS_MAX} tokens)")
    _check(_fn("gemm_rows", "akas_gemm_rows")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                             _stream()), f"streamed tcgen05 product [{n}x{k}] x [{o}x{k}]^T")
    return out


def gemm_rows_status() -> int:
    """0 unless a bounded wait inside the kernel of ``rows_product`` has run out on this device. Synchronises."""
    return int(_fn("gemm_rows", "akas_gemm_rows_status")())


@_flushes
def paired_product(x, w, swiglu_out: bool = False, out_dtype=None, residual=None, few_rows=True):
    """x [N, K] times w [O, K] transposed on pairs of SMs. bfloat16 out by default; float32 out with ``out_dtype``;
    added into ``residual`` (float32 [N, O]) when that is given; with ``swiglu_out`` w is the stacked [2F, K] gate and
    up matrices and the result is swiglu of the product, bfloat16 [N, F]. Up to 128 tokens go to ``rows_product``
    unless ``few_rows`` is False."""
    n, k = x.shape
    o = w.shape[0]
    out, epilogue = _tma_product("paired_product", x, w, swiglu_out, out_dtype, residual)
    if few_rows and _rows_takes(n, o, k, epilogue):
        _check(_fn("gemm_rows", "akas_gemm_rows")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                                 _stream()), f"streamed tcgen05 product [{n}x{k}] x [{o}x{k}]^T")
        return out
    _check(_fn("gemm_pair", "akas_gemm_pair")(_ptr(_dense(x, "x")), _ptr(_dense(w, "w")), _ptr(out), n, o, k, epilogue,
                                             _stream()), f"paired tcgen05 product [{n}x{k}] x [{o}x{k}]^T")
    return out


def gemm_pair_status() -> int:
    """0 unless a bounded wait inside the paired-SM product kernel has run out on this device. Synchronises."""
    return int(_fn("gemm_pair", "akas_gemm_pair_status")())


def gemm_tcgen05_status() -> int:
    """0 unless a bounded wait inside the tcgen05 product kernel has run out on this device. Synchronises."""
    return int(_fn("gemm_tcgen05", "akas_gemm_tcgen05_status")())


_OUT_BF16, _OUT_F32, _OUT_ACC, _OUT_SWIGLU = 0, 1, 2, 3


# Which kernel runs the products of decode steps (few tokens): "skinny", the mma.sync kernel, for up to 16 tokens;
# "stream", the tcgen05 kernel that streams the weights through the tensor cores (K split over a thread-block
# cluster where output channels are few), for up to _STREAM_ROWS tokens. Measured on the 1.2B shape at 8 tokens
# the skinny kernel is the faster one (1.01 ms a step against 1.35 ms), so it is the default; both are tested.
decode_products = os.environ.get("AKAS_B200_DECODE_PRODUCTS", "skinny")
if decode_products not in ("stream", "skinny"):
    raise ValueError(f"AKAS_B200_DECODE_PRODUCTS must be stream or skinny, got {decode_products!r}")
_STREAM_ROWS = 128
_stream_answers = {}


def _stream_takes(m: int, o: int, k: int, in_norm: bool, mode: int) -> bool:
    if decode_products != "stream" or m > _STREAM_ROWS or k % 8:
        return False
    key = (m, o, k, in_norm, mode)
    answer = _stream_answers.get(key)
    if answer is None:
        answer = _stream_answers[key] = bool(_fn("gemm_stream", "akas_stream_gemm_takes")(m, o, k, int(in_norm), mode))
    return answer


def _stream_product(x, rows, norm_w, eps, zero_centered, in_norm, w, out, m, o, k, mode):
    _check(_fn("gemm_stream", "akas_stream_gemm")(_ptr(x), _ptr(rows), _ptr(norm_w), float(eps), int(bool(zero_centered)),
                                                 int(in_norm), _ptr(w), _ptr(out), m, o, k, mode, _stream()),
           f"streamed product [{m}x{k}] x [{o}x{k}]^T")


def stream_status() -> int:
    """0 unless a bounded wait inside the streamed product kernel has run out on this device (then its results
    since are not valid). Synchronises with the device."""
    return int(_fn("gemm_stream", "akas_stream_gemm_status")())


def _skinny(x, rows, norm_w, eps, zero_centered, w, out, m, o, k, in_mode, out_mode):
    _check(_fn("skinny_gemm", "akas_skinny_gemm")(_ptr(x), _ptr(rows), _ptr(norm_w), float(eps), int(bool(zero_centered)),
                                                 _ptr(w), _ptr(out), m, o, k, in_mode, out_mode, _stream()),
           f"skinny product [{m}x{k}] x [{o}x{k}]^T")


def skinny_status() -> int:
    """0 unless a bounded wait inside the skinny product kernel has run out on this device (then its results
    since are not valid). Synchronises with the device."""
    return int(_fn("skinny_gemm", "akas_skinny_gemm_status")())


def linear_swiglu(x, w_gate_up):
    """swiglu(x . w^T) with w the stacked [2F, K] gate and up matrices: [N, F] in x's dtype."""
    n, k = x.shape
    f2 = w_gate_up.shape[0]
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and f2 % 2 == 0 and _chain_takes(n, f2, k, 0, _OUT_SWIGLU):
        out = torch.empty((n, f2 // 2), dtype=torch.bfloat16, device=x.device)
        _chain_add("akas_chain_gemm", (x, w_gate_up, out), _ptr(_dense(x, "x")), None, None, 0.0, 0,
                   _ptr(_dense(w_gate_up, "w")), _ptr(out), n, f2, k, 0, _OUT_SWIGLU)
        return out
    if _chain_open:
        chain_flush()
    if x.dtype == torch.bfloat16 and f2 % 2 == 0 and _stream_takes(n, f2, k, False, _OUT_SWIGLU):
        out = torch.empty((n, f2 // 2), dtype=torch.bfloat16, device=x.device)
        _stream_product(_dense(x, "x"), None, None, 0.0, False, False, _dense(w_gate_up, "w"), out, n, f2, k, _OUT_SWIGLU)
        return out
    if x.dtype == torch.bfloat16 and f2 % 2 == 0 and _skinny_fits(n, k):
        out = torch.empty((n, f2 // 2), dtype=torch.bfloat16, device=x.device)
        _skinny(_dense(x, "x"), None, None, 0.0, False, _dense(w_gate_up, "w"), out, n, f2, k, 0, _OUT_SWIGLU)
        return out
    if x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and k % 8 == 0 and \
            _product_route(k, f2, _OUT_SWIGLU) == "paired":
        # SwiGLU in the read-out of the product: the [N, 2F] intermediate is never written
        return paired_product(x, w_gate_up, swiglu_out=True)
    return swiglu(linear(x, w_gate_up))


def norm_linear(h, norm_weight, eps, zero_centered, w, out_dtype=None, rows=None, swiglu_out=False):
    """linear(rmsnorm(h[rows]), w), optionally through swiglu: the norm rides in the product for few tokens."""
    m = rows.numel() if rows is not None else h.shape[0]
    k, o = h.shape[1], w.shape[0]
    target = torch.bfloat16 if swiglu_out else (out_dtype or torch.bfloat16)
    mode = _OUT_SWIGLU if swiglu_out else _OUT_F32 if target == torch.float32 else _OUT_BF16
    fusable = w.dtype == torch.bfloat16 and h.dtype == torch.float32 and h.is_contiguous() and (not swiglu_out or o % 2 == 0)
    if fusable and _chain_takes(m, o, k, 1, mode):
        out = torch.empty((m, o // 2 if swiglu_out else o), dtype=target, device=h.device)
        _chain_add("akas_chain_gemm", (h, rows, norm_weight, w, out), _ptr(h), _ptr(rows), _ptr(norm_weight), float(eps),
                   int(bool(zero_centered)), _ptr(_dense(w, "w")), _ptr(out), m, o, k, 1, mode)
        return out
    if _chain_open:
        chain_flush()
    if fusable and _stream_takes(m, o, k, True, mode):
        out = torch.empty((m, o // 2 if swiglu_out else o), dtype=target, device=h.device)
        _stream_product(h, rows, norm_weight, eps, zero_centered, True, _dense(w, "w"), out, m, o, k, mode)
        return out
    if fusable and _skinny_fits(m, k):
        out = torch.empty((m, o // 2 if swiglu_out else o), dtype=target, device=h.device)
        _skinny(h, rows, norm_weight, eps, zero_centered, _dense(w, "w"), out, m, o, k, 1, mode)
        return out
    x = rmsnorm(h, norm_weight, eps, zero_centered, w.dtype, rows)
    return linear_swiglu(x, w) if swiglu_out else linear(x, w, out_dtype=out_dtype)


# A decode step's in projection and gated short convolution as one kernel (csrc/skinny_gemm.cu, read-out "conv"):
# AKAS_B200_FUSED_CONV=0 runs them as the product and the convolution kernel.
fused_conv = os.environ.get("AKAS_B200_FUSED_CONV", "1") != "0"


def norm_linear_short_conv(h, norm_weight, eps, zero_centered, w_in, taps, bias, state, seq_of_token, slots, write=True):
    """``short_conv(norm_linear(h, ...), ...)`` for a decode step (every token the single token of its request) in one
    launch, or None where the fused kernel does not take the sizes (the caller then runs the two by themselves)."""
    m, k = h.shape
    c3 = w_in.shape[0]
    c, l = c3 // 3, taps.shape[1]
    if not fused_conv or _chain_open or w_in.dtype != torch.bfloat16 or h.dtype != torch.float32 or not h.is_contiguous() \
            or c3 % 3 or c % 8 or not 2 <= l <= 16 or not _skinny_fits(m, k) or state.dtype != torch.float32:
        return None
    out = torch.empty((m, c), dtype=torch.bfloat16, device=h.device)
    _check(_fn("skinny_gemm", "akas_skinny_gemm_conv")(
        _ptr(h), None, _ptr(norm_weight), float(eps), int(bool(zero_centered)), _ptr(_dense(w_in, "w")), _ptr(out), m, c, k, 1,
        _ptr(taps), _ptr(bias), _ptr(state), _ptr(seq_of_token), _ptr(slots), l, int(bool(write)), _stream()),
        f"fused in projection and short convolution [{m}x{k}] x [{c3}x{k}]^T")
    return out


# --------------------------------------------------------------------------- mixers


def short_conv(bcx, taps, bias, state, cu_seqlens, seq_of_token, slots, decode_only=False, write=True):
    """The gated short convolution over the flat batch; ``write=False`` reads the state and leaves it as it is."""
    n, c3 = bcx.shape
    c, l = c3 // 3, taps.shape[1]
    out = torch.empty((n, c), dtype=bcx.dtype, device=bcx.device)
    if decode_only and _chain_open and n <= _CHAIN_ROWS and bcx.dtype == torch.bfloat16:
        _chain_add("akas_chain_conv", (bcx, taps, bias, state, seq_of_token, slots, out), _ptr(_dense(bcx, "bcx")), _ptr(taps),
                   _ptr(bias), _ptr(state), _ptr(seq_of_token), _ptr(slots), _ptr(out), n, c, l, int(bool(write)))
        return out
    if _chain_open:
        chain_flush()
    if decode_only:
        _check(_fn("conv", "akas_short_conv_decode")(_ptr(_dense(bcx, "bcx")), _ptr(taps), _ptr(bias), _ptr(state),
                                                    _ptr(seq_of_token), _ptr(slots), _ptr(out), n, c, l, _code(bcx),
                                                    int(bool(write)), _stream()), "short_conv_decode")
        return out
    _check(_fn("conv", "akas_short_conv")(_ptr(_dense(bcx, "bcx")), _ptr(taps), _ptr(bias), _ptr(state),
                                         _ptr(cu_seqlens), _ptr(seq_of_token), _ptr(slots), _ptr(out), n,
                                         slots.numel(), c, l, _code(bcx), int(bool(write)), _stream()), "short_conv",
           kernels=2 if write else 1)
    return out


def rope_tables(positions, inv_freq, amplitude=1.0):
    n, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _check(_fn("rope", "akas_rope_tables")(_ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), n, half, float(amplitude),
                                          _stream()), "rope_tables")
    return cos, sin


@_flushes
def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, zero_centered, cos, sin,
                       k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    n = qkv.shape[0]
    _dense(qkv, "qkv")
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise ValueError("qkv width does not match (heads + 2 kv_heads) * head_dim")
    q = torch.empty((n, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    rotary = 2 * cos.shape[1] if cos is not None else 0
    _check(_fn("rope", "akas_qk_norm_rope_store")(
        _ptr(qkv), _ptr(q), _ptr(q_weight), _ptr(k_weight), float(eps), int(bool(zero_centered)), _ptr(cos), _ptr(sin),
        rotary, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), page_size, n, heads, kv_heads, head_dim, _code(qkv), _stream()), "qk_norm_rope_store")
    return q


@_flushes
def kv_store(k, v, k_pool, v_pool, block_table, seq_of_token, positions, page_size):
    n = k.shape[0]
    kh, d = k_pool.shape[1], k_pool.shape[3]
    if k.stride(1) != 1 or v.stride(1) != 1:
        raise ValueError("kv_store: k and v must have unit inner stride")
    _check(_fn("rope", "akas_kv_store")(_ptr(k), _ptr(v), k.stride(0), v.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                       block_table.shape[1], _ptr(seq_of_token), _ptr(positions), page_size, n, kh, d,
                                       _code(k_pool), _stream()), "kv_store")


# Which kernel runs attention over prompt portions in bfloat16: "mma" (the mma.sync kernel, 64-query tiles),
# "tcgen05" (the tensor-memory kernel, 128-query tiles, where it takes the sizes: head size 64, page size a multiple
# of 64) or "auto": the tensor-memory kernel when the step's requests mostly bring more than 64 tokens. Measured on
# the 1.2B shape: 222 against 182 TFLOP/s at 2,048 tokens, 392 against 220 at 8,192 (mma.sync peaks at 550 here).
prompt_attention = os.environ.get("AKAS_B200_PROMPT_ATTENTION", "auto")
if prompt_attention not in ("auto", "tcgen05", "mma"):
    raise ValueError(f"AKAS_B200_PROMPT_ATTENTION must be auto, tcgen05 or mma, got {prompt_attention!r}")


# How the decoded tokens of a step that also holds prompt portions are attended: "split" (default), by the split-key
# decode kernel, or "tiles", inside the prompt kernels as query tiles with one live row each.
mixed_attention = os.environ.get("AKAS_B200_MIXED_ATTENTION", "split")
if mixed_attention not in ("split", "tiles"):
    raise ValueError(f"AKAS_B200_MIXED_ATTENTION must be split or tiles, got {mixed_attention!r}")


def decode_attention_status() -> int:
    """0 unless a bounded wait inside the TMA-fed decode-attention kernel has run out on this device."""
    return int(_fn("attention_decode", "akas_decode_attention_status")())


def prefill_attention_tc_status() -> int:
    """0 unless a bounded wait inside the tcgen05 prompt-attention kernel has run out on this device."""
    return int(_fn("attention_prefill_tc", "akas_prefill_attention_tc_status")())


_DECODE_BLOCKS = int(os.environ.get("AKAS_B200_DECODE_BLOCKS", "300"))
_DECODE_SPLITS = int(os.environ.get("AKAS_B200_DECODE_SPLITS", "0"))  # a number of key parts for every step, for measurements


def decode_splits(num_tokens: int, kv_heads: int, head_tiles: int, max_context: int) -> int:
    """How many parts the keys of a decoding request are cut into, from sizes known on the host: enough blocks for
    two per SM (measured on a B200 at 2,048 to 4,096 keys: a block's fixed cost, its query load, barriers and the
    partial result it writes for the merge, outweighs a fuller GPU beyond that; 8 requests of 8 KV heads run fastest
    in 4 to 5 parts, 0.861 ms a step against 0.888 ms in 16), two parts even where the requests alone give that many
    (64 requests: 44.8k tokens/s in 2 parts, 43.4k in 1, 44.4k in 4), and at least four 64-key tiles per part."""
    blocks = max(1, num_tokens * kv_heads * head_tiles)
    want = _DECODE_SPLITS or max(-(-_DECODE_BLOCKS // blocks), 2)
    most = max(1, -(-max_context // 256))
    return max(1, min(want, most, 64))


_decode_cluster_merge = os.environ.get("AKAS_B200_DECODE_CLUSTER_MERGE", "1") != "0"


def _merges_in_cluster(blocks: int, splits: int, head_dim: int, page_size: int) -> bool:
    """Whether the decode attention kernel merges its key parts itself (they form a thread-block cluster: the TMA-fed
    kernel, 2 to 8 parts, up to four blocks per SM in all) instead of leaving them to a second kernel; the rule of
    csrc/attention_decode.cu::launch_tma."""
    return (_decode_cluster_merge and 2 <= splits <= 8 and head_dim == 64 and page_size % 64 == 0
            and blocks * splits <= 4 * _sm_count())


# Decode attention by blocks that walk the step's items instead of a block per item: "auto" (where a block per item
# would come to more blocks than the GPU holds at once: alone and with a cold L2, 64 requests of 2,048 keys take 50 us
# against 58 us), "0" never, "1" wherever the kernel takes the sizes.
decode_items = os.environ.get("AKAS_B200_DECODE_ITEMS", "auto")
if decode_items not in ("auto", "0", "1"):
    raise ValueError(f"AKAS_B200_DECODE_ITEMS must be auto, 0 or 1, got {decode_items!r}")
_items_places_cache = {}


def _items_places(heads: int, kv_heads: int) -> int:
    key = (torch.cuda.current_device(), heads // kv_heads)
    if key not in _items_places_cache:
        _items_places_cache[key] = int(_fn("attention_decode", "akas_decode_attention_items_places")(heads, kv_heads))
    return _items_places_cache[key]


def decode_plan(num_tokens: int, heads: int, kv_heads: int, head_dim: int, page_size: int, keys: int, dtype):
    """(key parts, whether the blocks walk the items) for a decode step's attention, from sizes known on the host."""
    head_tiles = -(-(heads // kv_heads) // 16)
    splits = decode_splits(num_tokens, kv_heads, head_tiles, keys)
    if dtype != torch.bfloat16 or head_dim != 64 or page_size % 64 or decode_items == "0":
        return splits, False
    blocks = num_tokens * kv_heads * head_tiles
    if splits > 8 and keys <= 4096 and _merges_in_cluster(blocks, 8, head_dim, page_size):
        # up to 8 tiles a part: 8 parts that meet inside their cluster, rather than more parts and a kernel that merges
        # them (one request of 2,048 keys: 1,495 against 1,478 tokens/s)
        splits = 8
    if decode_items == "auto" and not 3 * _sm_count() < blocks * splits <= 8 * _sm_count():
        # up to three blocks per SM all run at once; far more than the GPU holds are spread well by the hardware as they
        # come (128 requests of 8,192 keys: 40.1k tokens/s with a block per item, 37.7k with blocks that walk them,
        # whose items are dealt out beforehand); in between, the last round would run part empty (32 requests: 24.5k
        # against 25.9k, at 8,192 keys 18.3k against 20.4k)
        return splits, False
    # (the same parts: measured at 64 requests of 2,048 keys, 48.1k tokens/s in 2 parts, 47.3k in 3, 46.4k in 6 and
    # 44.3k in 11 against 47.2k with a block per item: what an item costs beside its tiles is not hidden by the ring)
    return splits, _items_places(heads, kv_heads) > 0


def _decode_attention(q, n, out, k_pool, v_pool, block_table, seq_of_token, positions, scale, win, page_size, keys):
    """Split-key attention of the first ``n`` tokens of q, each the single token of its request, into out[:n]."""
    kh, d = k_pool.shape[1], k_pool.shape[3]
    heads = q.shape[1] // d
    group = heads // kh
    if q.dtype == torch.bfloat16 and d in (16, 32, 64, 128):
        # tensor-core kernel: the query heads of a group are the rows of one tile
        splits, walks = decode_plan(n, heads, kh, d, page_size, keys, q.dtype)
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((n, heads, splits, d), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=q.device)
        if walks:
            err = _fn("attention_decode", "akas_decode_attention_items")(
                _ptr(q), None, None, None, 0.0, 0, None, None, 0, 0, _ptr(k_pool), _ptr(v_pool), k_pool.shape[0],
                _ptr(block_table), block_table.shape[1], _ptr(seq_of_token), _ptr(positions), _ptr(out), _ptr(part_o),
                _ptr(part_ml), float(scale), win, page_size, n, heads, kh, d, splits, _stream())
            if err != 3999:
                _check(err, "decode_attention (items)", kernels=2 if splits > 1 else 1)
                return
            splits = decode_splits(n, kh, -(-group // 16), keys)  # (pointers that the kernel does not take)
            if splits > 1:
                part_o = torch.empty((n, heads, splits, d), dtype=torch.float32, device=q.device)
                part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=q.device)
        _check(_fn("attention_decode", "akas_decode_attention_bf16_paged")(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
            _ptr(positions), _ptr(out), _ptr(part_o), _ptr(part_ml), float(scale), win, page_size, n, heads, kh, d,
            splits, _stream()), "decode_attention", kernels=2 if splits > 1 and not _merges_in_cluster(n * kh * -(-group // 16), splits, d, page_size) else 1)
        return
    gt = 8 if group >= 8 else 4 if group > 2 else group
    splits = decode_splits(n, kh, -(-group // gt), keys)
    part_o = torch.empty((n, heads, splits, d), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=q.device)
    _check(_fn("attention", "akas_paged_attention_decode")(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), _ptr(out), _ptr(part_o), _ptr(part_ml), float(scale), win, page_size, n, heads, kh, d,
        splits, _code(q), _stream()), "paged_attention_decode", kernels=2)


# Whether a decode step's attention layers run as one kernel from the qkv product on (norm and rotation of q and k, the
# write into the pages and attention; measured on the 1.2B shape: 6 launches fewer a step).
fused_qkv_attention = os.environ.get("AKAS_B200_FUSED_QKV_ATTENTION", "1") != "0"


@_flushes
def qkv_decode_attention(qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, zero_centered, cos, sin, k_pool, v_pool,
                         block_table, seq_of_token, positions, scale, window, page_size, ctx, write=True):
    """``paged_attention(qk_norm_rope_store(qkv, ...), ...)`` for a decode step (every token the single token of its
    request) in one launch, or None where the fused kernel does not take the sizes or the dtype (the caller then runs
    the two by themselves). With ``write=False`` the pages are read as they are and nothing is written."""
    if not fused_qkv_attention or qkv.dtype != torch.bfloat16 or head_dim != 64 or page_size % 64 or k_pool.dtype != torch.bfloat16:
        return None
    n = qkv.shape[0]
    _dense(qkv, "qkv")
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise ValueError("qkv width does not match (heads + 2 kv_heads) * head_dim")
    rotary = 2 * cos.shape[1] if cos is not None else 0
    if rotary % 16:
        return None
    win = int(window) if window else 0
    group = heads // kv_heads
    splits, walks = decode_plan(n, heads, kv_heads, head_dim, page_size, win if win else ctx.max_context, qkv.dtype)
    merged = splits == 1 or (not walks and _merges_in_cluster(n * kv_heads * -(-group // 16), splits, head_dim, page_size))
    out = torch.empty((n, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n, heads, splits, head_dim), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n, heads, splits, 2), dtype=torch.float32, device=qkv.device)
    prep = (_ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), int(bool(zero_centered)), _ptr(cos), _ptr(sin), rotary,
            int(bool(write)), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table), block_table.shape[1],
            _ptr(seq_of_token), _ptr(positions), _ptr(out), _ptr(part_o), _ptr(part_ml), float(scale), win, page_size, n,
            heads, kv_heads, head_dim, splits, _stream())
    if walks:
        err = _fn("attention_decode", "akas_decode_attention_items")(None, *prep)
    else:
        err = _fn("attention_decode", "akas_decode_attention_from_qkv")(*prep)
    if err == 3999:
        return None
    _check(err, "decode attention from qkv", kernels=1 if merged else 2)
    return out


def _leading_single_tokens(ctx) -> int:
    """How many requests at the front of the step bring exactly one token (the scheduler puts decoding requests first)."""
    lens = getattr(ctx, "query_lens", ()) if ctx is not None else ()
    count = 0
    while count < len(lens) and lens[count] == 1:
        count += 1
    return count


@_flushes
def paged_attention(q, k_pool, v_pool, block_table, seq_of_token, positions, scale, window, page_size, ctx=None):
    n = q.shape[0]
    kh, d = k_pool.shape[1], k_pool.shape[3]
    heads = q.shape[1] // d
    _dense(q, "q")
    out = torch.empty_like(q)
    win = int(window) if window else 0
    if ctx is not None and ctx.decode_only:
        _decode_attention(q, n, out, k_pool, v_pool, block_table, seq_of_token, positions, scale, win, page_size,
                          win if win else ctx.max_context)
        return out
    tensor_cores = q.dtype == torch.bfloat16 and d in (16, 32, 64, 128)
    # A step that mixes portions of prompts with decoded tokens: the single tokens at its front go to the split-key
    # kernel (one block per request, key/value head and part of the keys) instead of a 64-query tile each of which one
    # row is alive; the prompt kernels then start at the first request that brings more. Two launches, one output.
    first = _leading_single_tokens(ctx) if tensor_cores and mixed_attention == "split" else 0
    lens = ctx.query_lens[first:] if first else (getattr(ctx, "query_lens", ()) if ctx is not None else ())
    if first:
        _decode_attention(q, first, out, k_pool, v_pool, block_table, seq_of_token, positions, scale, win, page_size,
                          win if win else ctx.max_context)
        if not lens:
            return out
    tiles, wide = sum(-(-c // 64) for c in lens), sum(-(-c // 128) for c in lens)
    requests = len(lens) if first else (ctx.cu_seqlens.numel() - 1 if tiles else 0)
    # the prompt kernels find their tiles from cu_seqlens and address block tables by request: both start at `first`
    cu = ctx.cu_seqlens[first:] if tiles else None
    table = block_table[first:] if first else block_table
    # A 128-query tile of the tensor-memory kernel costs about what a 64-query tile of the mma.sync kernel costs
    # (measured: 1.8 times the throughput): it pays when requests bring more than 64 tokens, not for single tokens.
    tensor_memory = prompt_attention == "tcgen05" or (prompt_attention == "auto" and 0 < wide and wide <= 0.9 * tiles)
    if q.dtype == torch.bfloat16 and tensor_memory and d == 64 and page_size % 64 == 0 and 0 < tiles <= 65535:
        # prompt portions, head size 64, pages of whole half tiles: 128-query tiles on tcgen05
        err = _fn("attention_prefill_tc", "akas_prefill_attention_tc")(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0] * k_pool.shape[1] * k_pool.shape[2], _ptr(table),
            block_table.shape[1], _ptr(cu), _ptr(positions), _ptr(out), float(scale), win, page_size, tiles, n,
            heads, kh, d, requests, _stream())
        if err != 3999:
            _check(err, "prefill_attention_tc")
            return out
    if tensor_cores and 0 < tiles <= 65535:
        # prompt portions (and whatever decodes beside them): 64-query tiles on the tensor cores
        _check(_fn("attention_prefill", "akas_prefill_attention_bf16")(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table), block_table.shape[1], _ptr(cu),
            _ptr(positions), _ptr(out), float(scale), win, page_size, tiles, heads, kh, d, requests,
            _stream()), "prefill_attention")
        return out
    _check(_fn("attention", "akas_paged_attention")(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), _ptr(out), float(scale), win, page_size, n, heads, kh, d, _code(q), _stream()),
        "paged_attention")
    return out


# --------------------------------------------------------------------------- learned positions, PolyNorm


@_flushes
def add_rows(h, table, index):
    """h[n] += table[index[n]] in place on float32 h [N, C]."""
    n, c = h.shape
    if h.dtype != torch.float32 or table.shape[1] != c:
        raise ValueError("add_rows takes float32 h [N, C] and a table [rows, C]")
    _check(_fn("elementwise", "akas_add_rows")(_ptr(_dense(h, "h")), _ptr(_dense(table, "table")), _ptr(index), n, c,
                                              _code(table), _stream()), "add_rows")
    return h


@_flushes
def polynorm(z, coeffs, eps, out_dtype):
    """a N(z) + b N(z^2) + c N(z^3) + e per row of z [N, F]; coeffs = (a, b, c, e) float32. Powers and sums are float32."""
    n, f = z.shape
    if coeffs.dtype != torch.float32 or coeffs.numel() != 4:
        raise ValueError("polynorm takes z [N, F] and four float32 coefficients")
    out = torch.empty((n, f), dtype=out_dtype, device=z.device)
    _check(_fn("elementwise", "akas_polynorm")(_ptr(_dense(z, "z")), _ptr(coeffs), float(eps), _ptr(out), n, f, _code(z),
                                              _CODE[out_dtype], _stream()), "polynorm")
    return out


# --------------------------------------------------------------------------- mixers with a matrix state


def _rows(t: torch.Tensor, what: str):
    """(pointer, row pitch in elements) of a 2-D tensor whose rows are dense: a slice of columns of a product's result."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError(f"{what} must be two-dimensional with unit inner stride")
    return t.data_ptr(), t.stride(0)


def _slot_rows(state: torch.Tensor, what: str):
    """(pointer, slot pitch in floats) of a float32 state [slots, ...] whose every slot is dense."""
    if state.dtype != torch.float32 or not state[0].is_contiguous():
        raise ValueError(f"{what} must be float32 with a dense row per slot")
    return state.data_ptr(), state.stride(0)


@_flushes
def decay_gates(low, w_up, bias, tau):
    """sigmoid(low . w_up + bias)^(1 / tau), float32 [N, O], for low [N, R] (a slice of a product's result) and
    float32 w_up [R, O] (the up matrix of the low-rank pair, transposed)."""
    n, r = low.shape
    o = w_up.shape[1]
    if w_up.dtype != torch.float32 or bias.dtype != torch.float32 or w_up.shape[0] != r:
        raise ValueError("decay_gates takes a float32 matrix [R, O] and bias [O]")
    ptr, ld = _rows(low, "low")
    out = torch.empty((n, o), dtype=torch.float32, device=low.device)
    _check(_fn("recurrent", "akas_decay_gates")(ptr, ld, _ptr(_dense(w_up, "w_up")), _ptr(bias), _ptr(out), n, o, r, float(tau),
                                               _code(low), _stream()), "decay_gates")
    return out


@_flushes
def gla_scan(q, k, v, alpha, state, cu_seqlens, slots, heads, dim, vdim, q_scale, write=True):
    n = q.shape[0]
    if q.dtype != k.dtype or q.dtype != v.dtype or alpha.dtype != torch.float32 or not alpha.is_contiguous():
        raise ValueError("gla_scan takes q, k, v of one dtype and a dense float32 alpha")
    (qp, ldq), (kp, ldk), (vp, ldv) = _rows(q, "q"), _rows(k, "k"), _rows(v, "v")
    sp, stride = _slot_rows(state, "state")
    out = torch.empty((n, heads * vdim), dtype=torch.float32, device=q.device)
    _check(_fn("recurrent", "akas_gla_scan")(qp, ldq, kp, ldk, vp, ldv, _ptr(alpha), sp, stride, _ptr(cu_seqlens), _ptr(slots),
                                            _ptr(out), n, slots.numel(), heads, dim, vdim, float(q_scale), int(bool(write)),
                                            _code(q), _stream()), "gla_scan")
    return out


@_flushes
def causal_conv_silu(x, taps, state, cu_seqlens, seq_of_token, slots, write=True):
    n, c = x.shape
    l = taps.shape[1]
    if taps.dtype != torch.float32 or taps.shape[0] != c or not taps.is_contiguous():
        raise ValueError("causal_conv_silu takes dense float32 taps [C, L]")
    xp, ldx = _rows(x, "x")
    sp, stride = _slot_rows(state, "state")
    y = torch.empty((n, c), dtype=torch.float32, device=x.device)
    _check(_fn("recurrent", "akas_causal_conv_silu")(xp, ldx, _ptr(taps), sp, stride, _ptr(cu_seqlens), _ptr(seq_of_token),
                                                    _ptr(slots), _ptr(y), n, slots.numel(), c, l, int(bool(write)), _code(x),
                                                    _stream()), "causal_conv_silu", kernels=2 if write else 1)
    return y


@_flushes
def delta_prep(y, kv_heads, dim, q_scale, unit_eps, b, a, a_log, dt_bias):
    n = y.shape[0]
    h = b.shape[1]
    if y.dtype != torch.float32 or b.dtype != a.dtype:
        raise ValueError("delta_prep takes float32 y and b, a of one dtype")
    yp, ldy = _rows(y, "y")
    (bp, ldb), (ap, lda) = _rows(b, "b"), _rows(a, "a")
    beta = torch.empty((n, h), dtype=torch.float32, device=y.device)
    g = torch.empty_like(beta)
    _check(_fn("recurrent", "akas_delta_prep")(yp, ldy, kv_heads, dim, float(q_scale), float(unit_eps), bp, ldb, ap, lda,
                                              _ptr(a_log), _ptr(dt_bias), _ptr(beta), _ptr(g), n, h, _code(b), _stream()),
           "delta_prep")
    return beta, g


@_flushes
def delta_scan(q, k, v, beta, g, state, cu_seqlens, slots, heads, kv_heads, dim, vdim, write=True):
    n = q.shape[0]
    if any(t.dtype != torch.float32 for t in (q, k, v, beta, g)) or not beta.is_contiguous() or not g.is_contiguous():
        raise ValueError("delta_scan takes float32 inputs")
    (qp, ldq), (kp, ldk), (vp, ldv) = _rows(q, "q"), _rows(k, "k"), _rows(v, "v")
    sp, stride = _slot_rows(state, "state")
    out = torch.empty((n, heads * vdim), dtype=torch.float32, device=q.device)
    _check(_fn("recurrent", "akas_delta_scan")(qp, ldq, kp, ldk, vp, ldv, _ptr(beta), _ptr(g), sp, stride, _ptr(cu_seqlens),
                                              _ptr(slots), _ptr(out), n, slots.numel(), heads, kv_heads, dim, vdim,
                                              int(bool(write)), _stream()), "delta_scan")
    return out


@_flushes
def gated_rmsnorm(o, weight, eps, gate, heads, vdim, out_dtype, gate_activation="silu", out=None, out_scale=1.0):
    n = o.shape[0]
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape[1] != heads * vdim:
        raise ValueError("gated_rmsnorm takes dense float32 o [N, heads * vdim]")
    if gate_activation not in ("silu", "sigmoid"):
        raise ValueError(f"unknown gate activation {gate_activation!r}")
    if weight is not None and (weight.dtype != torch.float32 or weight.numel() != vdim):
        raise ValueError("gated_rmsnorm: the weight is float32 [vdim] (None: the division alone)")
    gp, ldg = _rows(gate, "gate")
    if out is None:
        out = torch.empty((n, heads * vdim), dtype=out_dtype, device=o.device)
    elif out.shape != (n, heads * vdim):
        raise ValueError("gated_rmsnorm: out must be [N, heads * vdim]")
    op, ldo = _rows(out, "out")
    _check(_fn("recurrent", "akas_gated_rmsnorm")(_ptr(o), _ptr(weight), float(eps), gp, ldg, op, n, heads, vdim,
                                                 _code(gate), _code(out), int(gate_activation == "sigmoid"),
                                                 float(out_scale), ldo, _stream()), "gated_rmsnorm")
    return out


# How the recurrence with a constant decay runs: "auto" (default), in chunks (three kernels of float32 products, see
# csrc/recurrent.cu) when some request of the step brings at least _CHUNKED_FROM tokens and the key size allows, token by
# token otherwise; "tokens": token by token always.
decay_scan_kernels = os.environ.get("AKAS_B200_DECAY_SCAN", "auto")
if decay_scan_kernels not in ("auto", "tokens"):
    raise ValueError(f"AKAS_B200_DECAY_SCAN must be auto or tokens, got {decay_scan_kernels!r}")
_CHUNKED_FROM = 48


@_flushes
def decay_scan(q, k, v, decay, state, cu_seqlens, slots, heads, dim, vdim, q_scale, activation=None, write=True, longest=None):
    """``longest``: the most tokens a request brings in this step, where the caller knows it (it chooses the kernel)."""
    n = q.shape[0]
    if q.dtype != k.dtype or q.dtype != v.dtype or decay.dtype != torch.float32 or decay.numel() != heads:
        raise ValueError("decay_scan takes q, k, v of one dtype and a float32 decay per head")
    if activation not in (None, "silu"):
        raise ValueError(f"unknown activation {activation!r}")
    (qp, ldq), (kp, ldk), (vp, ldv) = _rows(q, "q"), _rows(k, "k"), _rows(v, "v")
    sp, stride = _slot_rows(state, "state")
    out = torch.empty((n, heads * vdim), dtype=torch.float32, device=q.device)
    if decay_scan_kernels == "auto" and longest is not None and longest >= _CHUNKED_FROM:
        words = int(_fn("recurrent", "akas_decay_chunk_scratch")(n, slots.numel(), heads, dim, vdim))
        if words:
            scratch = torch.empty(words, dtype=torch.float32, device=q.device)
            _check(_fn("recurrent", "akas_decay_scan_chunked")(
                qp, ldq, kp, ldk, vp, ldv, _ptr(decay), sp, stride, _ptr(cu_seqlens), _ptr(slots), _ptr(out), _ptr(scratch), n,
                slots.numel(), heads, dim, vdim, float(q_scale), int(activation == "silu"), int(bool(write)), _code(q), _stream()),
                "decay_scan (chunks)", kernels=3)
            return out
    _check(_fn("recurrent", "akas_decay_scan")(qp, ldq, kp, ldk, vp, ldv, _ptr(decay), sp, stride, _ptr(cu_seqlens), _ptr(slots),
                                              _ptr(out), n, slots.numel(), heads, dim, vdim, float(q_scale),
                                              int(activation == "silu"), int(bool(write)), _code(q), _stream()), "decay_scan")
    return out


# --------------------------------------------------------------------------- general attention


@_flushes
def qk_norm_store(q, k, v, heads, kv_heads, dim, vdim, q_weight, k_weight, eps, k_pool, v_pool, block_table,
                  seq_of_token, positions, page_size, write=True, cos=None, sin=None, interleaved=False,
                  q_bias=None, k_bias=None, v_bias=None):
    n = q.shape[0]
    if not (q.dtype == k.dtype == v.dtype) or k_pool.dtype != v_pool.dtype:
        raise TypeError("qk_norm_store: q, k, v must have one dtype, and so must the pages")
    if q.dtype != k_pool.dtype and q.dtype != torch.float32:
        raise TypeError("qk_norm_store: q, k, v come in the pages' dtype or as float32 results of a product")
    for bias, size in ((q_bias, heads * dim), (k_bias, kv_heads * dim), (v_bias, kv_heads * vdim)):
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != size or not bias.is_contiguous()):
            raise ValueError("qk_norm_store: a bias is a dense float32 vector with one number per channel")
    rot = 0
    if cos is not None:
        rot = 2 * cos.shape[1]
        if cos.dtype != torch.float32 or sin.shape != cos.shape or cos.shape[0] != n or rot > dim:
            raise ValueError("qk_norm_store: rotary tables must be float32 [N, rot / 2] with rot <= dim")
        _dense(cos, "cos"), _dense(sin, "sin")
    (qp, ldq), (kp, ldk), (vp, ldv) = _rows(q, "q"), _rows(k, "k"), _rows(v, "v")
    out = torch.empty((n, heads * dim), dtype=k_pool.dtype, device=q.device)
    _check(_fn("attention_general", "akas_qk_norm_store")(
        qp, ldq, kp, ldk, vp, ldv, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(out), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), block_table.shape[1], _ptr(seq_of_token), _ptr(positions), page_size, n, heads, kv_heads, dim, vdim,
        int(bool(write)), _code(k_pool), _ptr(cos), _ptr(sin), rot, int(bool(interleaved)), _code(q), _ptr(q_bias), _ptr(k_bias),
        _ptr(v_bias), _stream()), "qk_norm_store")
    return out


# Which kernel runs the general attention over prompt portions in bfloat16: "mma" (default), the tensor-core kernel
# (csrc/attention_general_tc.cu) for requests that bring more than one token, the single tokens at the step's front on
# the kernel for any sizes; "plain": that kernel for everything.
general_attention = os.environ.get("AKAS_B200_GENERAL_ATTENTION", "mma")
if general_attention not in ("mma", "plain"):
    raise ValueError(f"AKAS_B200_GENERAL_ATTENTION must be mma or plain, got {general_attention!r}")


general_splits = os.environ.get("AKAS_B200_GENERAL_SPLITS", "1") != "0"  # 0: a decoding request's keys are never cut into parts


@_flushes
def attention_general(q, k_pool, v_pool, block_table, seq_of_token, positions, scale, window, keep_first, softcap,
                      r1, r2, sink, gate, page_size, ctx=None, sinks=None, out=None, out_scale=1.0, values_in_keys=0,
                      gate_channels=False):
    """``values_in_keys`` = V > 0: a key's row holds its value too, as its first V channels; ``v_pool`` is not read.
    ``gate_channels``: the gate has one logit per channel of a token's output row [N, heads * value_dim], not one per head."""
    n = q.shape[0]
    kh, d = k_pool.shape[1], k_pool.shape[3]
    if values_in_keys:
        if not 0 < values_in_keys <= d:
            raise ValueError("attention_general: the values are the first channels of the keys' rows")
        v_pool, vd, vpitch = k_pool, int(values_in_keys), d
    else:
        vd = vpitch = v_pool.shape[3]
    heads = q.shape[1] // d
    _dense(q, "q")
    if q.dtype != k_pool.dtype or (gate is not None and gate.dtype not in (q.dtype, torch.float32)):
        raise TypeError("attention_general: q and the pages must have one dtype, the gate theirs or float32")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != heads):
        raise ValueError("attention_general: sinks must be float32 [heads]")
    gp, ldg = _rows(gate, "gate") if gate is not None else (None, 0)
    if gate is not None and gate.shape != (n, heads * vd if gate_channels else heads):
        raise ValueError("attention_general: the gate is [N, heads], or with gate_channels [N, heads * value_dim]")
    channels = int(bool(gate_channels and gate is not None))
    gate_code = _code(gate) if gate is not None else _code(q)
    if out is None:
        out = torch.empty((n, heads * vd), dtype=q.dtype, device=q.device)
    elif out.shape != (n, heads * vd) or out.dtype != q.dtype:
        raise ValueError("attention_general: out must be [N, heads * value_dim] in q's dtype")
    op, ldo = _rows(out, "out")
    tail = (_ptr(sinks), float(out_scale), ldo)
    options = (float(scale), int(window or 0), int(keep_first or 0), float(softcap or 0.0), _ptr(r1), _ptr(r2),
               int(bool(sink)), gp, ldg, page_size)
    singles = n  # tokens at the front that are left to the kernel for any sizes
    lens = getattr(ctx, "query_lens", ()) if ctx is not None else ()
    if (general_attention == "mma" and q.dtype == torch.bfloat16 and lens
            and ldo % 2 == 0 and op % 4 == 0 and vpitch % 8 == 0
            and _fn("attention_general_tc", "akas_attention_general_tc_takes")(d, vd)):
        # The single tokens at the step's front (decoding requests) as one launch whose blocks hold the query heads of
        # a key/value head; then the requests from the first that brings more, as 64-query tiles. The kernel finds its
        # tiles from cu_seqlens and addresses block tables by request: both start at the launch's first request.
        first = _leading_single_tokens(ctx) if heads // kh <= 64 else 0
        launches = [(0, first, first, 1)] if first else []
        tiles = sum(-(-c // 64) for c in lens[first:])
        if tiles:
            launches.append((first, len(lens) - first, tiles, 0))
        if launches and all(0 < tiles <= 65535 for _, _, tiles, _ in launches):
            for start, requests, tiles, packed in launches:
                # single tokens: every request's keys in parts, so that a few requests with long pasts fill the GPU; the
                # parts' sums meet in a merge kernel (the count comes from sizes the host knows, as for the plain decode path)
                splits = decode_splits(requests, kh, 1, getattr(ctx, "max_context", 0) or 0) if packed and general_splits else 1
                partial = torch.empty(requests * heads * splits * (vd + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
                err = _fn("attention_general_tc", "akas_attention_general_tc")(
                    _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table[start:]), block_table.shape[1],
                    _ptr(ctx.cu_seqlens[start:]), _ptr(positions), op, *options, tiles, heads, kh, d, vd, requests,
                    packed, *tail, _ptr(partial), splits, vpitch, channels, gate_code, _stream())
                _check(err, "attention_general (tensor cores)")
            singles = 0
    if singles:
        _check(_fn("attention_general", "akas_attention_general")(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token), _ptr(positions),
            op, *options, singles, heads, kh, d, vd, _code(q), *tail, vpitch, channels, gate_code, _stream()), "attention_general")
    return out


# --------------------------------------------------------------------------- latent attention, norms without sums


@_flushes
def dynamic_tanh(x, alpha, weight, shift, out_dtype, rows=None, residual=None):
    """tanh(alpha * x) * weight + shift per element of float32 x [N, C]; ``rows``: int32 indices of the rows to take.
    With ``residual`` (dense float32 [N, C]) the result is added to it in place and it is returned."""
    c = x.shape[-1]
    if x.dtype != torch.float32 or alpha.dtype != torch.float32 or weight.numel() != c or shift.numel() != c:
        raise ValueError("dynamic_tanh takes float32 x [N, C], a float32 alpha and vectors of C numbers")
    _dense(x, "x")
    m = rows.numel() if rows is not None else x.numel() // c
    if residual is not None:
        if rows is not None or residual.dtype != torch.float32 or residual.shape != x.shape or not residual.is_contiguous():
            raise ValueError("dynamic_tanh adds to a dense float32 residual of x's shape, all rows")
        out = residual
    else:
        out = torch.empty((m, c) if rows is not None else x.shape, dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "akas_dynamic_tanh")(_ptr(x), _ptr(alpha), _ptr(weight), _ptr(shift), _ptr(out), _ptr(rows), m, c,
                                                  _CODE[out.dtype], int(residual is not None), _stream()), "dynamic_tanh")
    return out


_PLAIN_ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


@_flushes
def activation(z, kind, out_dtype):
    """act(z) element by element of a product's rows [N, F] (float32 or bfloat16, rows may be parts of wider rows),
    float32 until the one rounding to ``out_dtype``."""
    if kind not in _PLAIN_ACTIVATIONS:
        raise ValueError(f"unknown activation {kind!r}")
    n, f = z.shape
    zp, ld = _rows(z, "z")
    out = torch.empty((n, f), dtype=out_dtype, device=z.device)
    _check(_fn("elementwise", "akas_activation")(zp, ld, _code(z), _ptr(out), _CODE[out_dtype], n, f, _PLAIN_ACTIVATIONS[kind],
                                                _stream()), "activation")
    return out


_ACTIVATIONS = {"gelu_tanh": 0, "silu": 1}
_READOUT_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}  # the products' gated read-outs number them from their first, silu


@_flushes
def gated_activation(gate_up, width, bias, activation, out_dtype, residual=None, residual_bias=None):
    """act(g + b_g) * (u + b_u) of a float32 product's rows [g | u]; with ``residual`` (float32 [N, C]) the same launch
    adds ``residual_bias`` [C] to it in place: the bias of the product that will accumulate into that stream."""
    n = gate_up.shape[0]
    if gate_up.dtype != torch.float32 or gate_up.shape[1] < 2 * width:
        raise ValueError("gated_activation takes a float32 product [N, >= 2 width]")
    if activation not in _ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != 2 * width):
        raise ValueError("gated_activation: bias must be float32 [2 width]")
    gp, ld = _rows(gate_up, "gate_up")
    out = torch.empty((n, width), dtype=out_dtype, device=gate_up.device)
    c = 0
    if residual is not None:
        c = residual.shape[1]
        if (residual.dtype != torch.float32 or not residual.is_contiguous() or residual.shape[0] != n
                or residual_bias is None or residual_bias.dtype != torch.float32 or residual_bias.numel() != c):
            raise ValueError("gated_activation: residual must be dense float32 [N, C] with a float32 bias [C]")
    _check(_fn("elementwise", "akas_gated_activation")(gp, ld, _ptr(bias), _ptr(out), n, width, _ACTIVATIONS[activation],
                                                      _CODE[out_dtype], _ptr(residual), _ptr(residual_bias), c, _stream()),
           "gated_activation")
    return out


@_flushes
def latent_norm_store(proj, q_rank, kv_rank, rot, q_weight, kv_weight, eps, cos, sin, interleaved, pool, block_table,
                      seq_of_token, positions, page_size, write=True):
    n = proj.shape[0]
    if proj.dtype != torch.float32 or proj.shape[1] < q_rank + kv_rank + rot:
        raise ValueError("latent_norm_store takes the float32 product [N, >= q_rank + kv_rank + rot]")
    if pool.shape[1] != 1 or pool.shape[3] != kv_rank + rot or not pool.is_contiguous():
        raise ValueError("latent_norm_store: pages are [pages, 1, page, kv_rank + rot]")
    if (q_weight.numel() if q_weight is not None else 0) != q_rank or kv_weight.numel() != kv_rank:
        raise ValueError("latent_norm_store: one norm weight per latent channel")
    if cos is not None:
        if not rot or cos.dtype != torch.float32 or cos.shape != (n, rot // 2) or sin.shape != cos.shape:
            raise ValueError("latent_norm_store: rotary tables must be float32 [N, rot / 2]")
        _dense(cos, "cos"), _dense(sin, "sin")
    pp, ld = _rows(proj, "proj")
    out = torch.empty((n, q_rank), dtype=pool.dtype, device=proj.device)
    _check(_fn("latent", "akas_latent_norm_store")(
        pp, ld, q_rank, kv_rank, rot, _ptr(q_weight), _ptr(kv_weight), float(eps), _ptr(cos), _ptr(sin), int(bool(interleaved)),
        _ptr(out), _ptr(pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token), _ptr(positions), page_size, n,
        int(bool(write)), _code(pool), _stream()), "latent_norm_store")
    return out


@_flushes
def head_linear(x, w, heads, gate=None, cos=None, sin=None, interleaved=False):
    n = x.shape[0]
    h, o, k = w.shape
    if h != heads or x.dtype != w.dtype or not w.is_contiguous() or x.shape[1] % heads or x.shape[1] // heads < k:
        raise ValueError("head_linear takes x [N, heads * (K + T)] and dense w [heads, O, K] of one dtype")
    t = x.shape[1] // heads - k
    if cos is not None:
        if not t or cos.dtype != torch.float32 or cos.shape != (n, t // 2) or sin.shape != cos.shape:
            raise ValueError("head_linear: rotary tables must be float32 [N, T / 2]")
        _dense(cos, "cos"), _dense(sin, "sin")
    xp, ldx = _rows(x, "x")
    gp, ldg, gcode = None, 0, _F32
    if gate is not None:
        if gate.shape != (n, heads * o):
            raise ValueError("head_linear: gate must be [N, heads * O]")
        (gp, ldg), gcode = _rows(gate, "gate"), _code(gate)
    out = torch.empty((n, heads * (o + t)), dtype=x.dtype, device=x.device)
    _check(_fn("latent", "akas_head_linear")(xp, ldx, _ptr(w), _ptr(out), out.stride(0), gp, ldg, gcode, _ptr(cos), _ptr(sin),
                                            int(bool(interleaved)), n, heads, o, k, t, _code(x), _stream()), "head_linear")
    return out


# --------------------------------------------------------------------------- routed experts, parallel blocks


@_flushes
def moe_route(h, w_router, correction, groups, keep, top, scoring="softmax", renormalize=True, extra=0):
    """``extra`` = X > 0: the matrix has X more rows behind the R that compete; the sigmoids of their logits come back
    as a third result, float32 [N, X]."""
    n, c = h.shape
    r = w_router.shape[0] - int(extra)
    if scoring not in ("softmax", "sigmoid"):
        raise ValueError(f"unknown scoring {scoring!r}")
    if (w_router.dtype != torch.float32 or w_router.shape[1] != c or r < 1
            or (correction is not None and (correction.dtype != torch.float32 or correction.numel() != r))):
        raise ValueError("moe_route takes a float32 router matrix [R + extra, C] and correction [R] (or none)")
    hp, ldh = _rows(h, "h")
    chosen = torch.empty((n, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=h.device)
    extras = torch.empty((n, int(extra)), dtype=torch.float32, device=h.device) if extra else None
    _check(_fn("moe", "akas_moe_route")(hp, ldh, _ptr(_dense(w_router, "w_router")), _ptr(correction), _ptr(chosen),
                                       _ptr(weights), n, c, r, int(groups), int(keep), int(top), _code(h),
                                       int(scoring == "sigmoid"), int(bool(renormalize)), int(extra), _ptr(extras), _stream()),
           "moe_route")
    return (chosen, weights, extras) if extra else (chosen, weights)


# Which kernels run the experts in bfloat16: "auto" (default), the grouped product on the tensor cores
# (csrc/moe_grouped.cu) for steps of more than _MOE_SIMPLE_PAIRS (token, expert) pairs and sizes it takes, the
# token-by-token kernels (csrc/moe.cu) otherwise; "simple": those for everything.
moe_kernels = os.environ.get("AKAS_B200_MOE", "auto")
if moe_kernels not in ("auto", "simple"):
    raise ValueError(f"AKAS_B200_MOE must be auto or simple, got {moe_kernels!r}")
_MOE_SIMPLE_PAIRS = 64


def moe_grouped_status() -> int:
    return int(_fn("moe_grouped", "akas_moe_grouped_status")())


def _update_args(update, n, c):
    """(x, a, scale_a, scale_b, mult) of a residual update as the kernels take it (null pointers and 0 for none)."""
    if update is None:
        return None, None, None, None, 0.0
    x, a, scale_a, scale_b, mult = update
    for t in (x, a):
        if t.dtype != torch.float32 or t.shape != (n, c) or not t.is_contiguous():
            raise ValueError("a residual update takes dense float32 tensors [N, C]")
    return _ptr(x), _ptr(a), _ptr(scale_a), _ptr(scale_b), float(mult)


def _shared_args(shared, n, c):
    """(y, gate, gate's pitch) of a dense result that the experts' last kernel adds (null pointers for none)."""
    if shared is None:
        return None, None, 0
    y, gate = shared
    if y.dtype != torch.float32 or y.shape != (n, c) or not y.is_contiguous():
        raise ValueError("a shared expert's result is a dense float32 tensor [N, C]")
    if gate is None:
        return _ptr(y), None, 0
    if gate.dtype != torch.float32 or gate.shape[0] != n:
        raise ValueError("a shared expert's gate is float32, one number per token")
    return _ptr(y), _ptr(gate), gate.stride(0)


def _moe_experts_grouped(h, w_gate_up, w_down, chosen, weights, update=None, weight_input=False, shared=None):
    n, c = h.shape
    experts, f2, _ = w_gate_up.shape
    f, top = f2 // 2, chosen.shape[1]
    hp, ldh = _rows(h, "h")
    cap = int(_fn("moe_grouped", "akas_moe_grouped_rows")(n * top, experts))
    dev = h.device
    row_of_pair = torch.empty(n * top, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(cap // 128, dtype=torch.int32, device=dev)
    plan = torch.empty(4, dtype=torch.int32, device=dev)
    rows = torch.empty((cap, c), dtype=h.dtype, device=dev)
    act = torch.empty((cap, f), dtype=h.dtype, device=dev)
    y = torch.empty((cap, c), dtype=torch.float32, device=dev)
    out = torch.empty((n, c), dtype=torch.float32, device=dev) if update is None else update[0]
    _check(_fn("moe_grouped", "akas_moe_sort")(hp, ldh, _ptr(chosen), _ptr(row_of_pair), _ptr(tile_expert), _ptr(plan), _ptr(rows),
                                              n, top, c, experts, _ptr(weights) if weight_input else None, _stream()),
           "moe_sort", kernels=2)
    gemm = _fn("moe_grouped", "akas_moe_grouped_gemm")
    _check(gemm(_ptr(rows), _ptr(w_gate_up), _ptr(act), _ptr(tile_expert), _ptr(plan), cap, experts, f2, c, 2, _stream()),
           "grouped gate and up product")
    _check(gemm(_ptr(act), _ptr(w_down), _ptr(y), _ptr(tile_expert), _ptr(plan), cap, experts, c, f, 1, _stream()),
           "grouped down product")
    _check(_fn("moe_grouped", "akas_moe_combine")(hp, ldh, _ptr(y), _ptr(row_of_pair), None if weight_input else _ptr(weights),
                                                 _ptr(out), n, top, c, *_update_args(update, n, c), *_shared_args(shared, n, c),
                                                 _stream()), "moe_combine")
    return out


@_flushes
def moe_experts(h, w_gate_up, w_down, chosen, weights, update=None, weight_input=False, shared=None):
    """``weight_input``: the weight multiplies the expert's input, sum_k expert(w_k h), where otherwise it multiplies the
    result. ``shared`` = (y float32 [N, C], gate float32 [N, 1] or None): y times its gate is added to the sum.
    The weighted sum of the chosen experts' results, float32 [N, C]. With ``update`` = (x, a, scale_a, scale_b, mult)
    the sum is not returned but added into the residual stream by the last kernel: x += mult * (scale_a * a + scale_b *
    sum), in place; returns x."""
    n, c = h.shape
    experts, f2, _ = w_gate_up.shape
    f, top = f2 // 2, chosen.shape[1]
    if w_gate_up.dtype != h.dtype or w_down.dtype != h.dtype or w_down.shape != (experts, c, f) or w_gate_up.shape[2] != c:
        raise ValueError("moe_experts takes h [N, C], w_gate_up [E, 2 F, C] and w_down [E, C, F] of one dtype")
    hp, ldh = _rows(h, "h")
    if (moe_kernels == "auto" and h.dtype == torch.bfloat16 and n * top > _MOE_SIMPLE_PAIRS and ldh % 8 == 0 and hp % 16 == 0
            and _fn("moe_grouped", "akas_moe_grouped_takes")(c, f, experts)):
        _dense(w_gate_up, "w_gate_up"), _dense(w_down, "w_down")
        return _moe_experts_grouped(h, w_gate_up, w_down, chosen, weights, update, weight_input, shared)
    act = torch.empty((n * top, f), dtype=h.dtype, device=h.device)
    out = torch.empty((n, c), dtype=torch.float32, device=h.device) if update is None else update[0]
    _check(_fn("moe", "akas_moe_gate_up")(hp, ldh, _ptr(_dense(w_gate_up, "w_gate_up")), _ptr(chosen), _ptr(act), n, top, c, f,
                                         experts, _code(h), _ptr(weights) if weight_input else None, _stream()), "moe_gate_up")
    _check(_fn("moe", "akas_moe_down")(hp, ldh, _ptr(_dense(w_down, "w_down")), _ptr(chosen), None if weight_input else _ptr(weights),
                                      _ptr(act), _ptr(out), n, top, c, f, experts, _code(h), *_update_args(update, n, c),
                                      *_shared_args(shared, n, c), _stream()), "moe_down")
    return out


@_flushes
def scaled_add(x, a, scale_a, b, scale_b, mult):
    """x += mult * (scale_a * a + scale_b * b) in place on float32 x [N, C]; scales float32 [C] (None: ones); b may be None."""
    n, c = x.shape
    for t in (x, a) + ((b,) if b is not None else ()):
        if t.dtype != torch.float32 or t.shape != (n, c) or not t.is_contiguous():
            raise ValueError("scaled_add takes dense float32 tensors [N, C]")
    _check(_fn("elementwise", "akas_scaled_add")(_ptr(x), _ptr(a), _ptr(scale_a), _ptr(b), _ptr(scale_b) if b is not None else None,
                                                float(mult), n, c, _stream()), "scaled_add")
    return x


# --------------------------------------------------------------------------- sampling


@_flushes
def argmax(logits):
    m, v = logits.shape
    out = torch.empty((m,), dtype=torch.int32, device=logits.device)
    parts = max(1, min(64, v // 1024, 592 // max(m, 1)))  # slices of the vocabulary, at least 1024 entries each
    part_val = torch.empty((m, parts), dtype=torch.float32, device=logits.device)
    part_idx = torch.empty((m, parts), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "akas_argmax")(_ptr(_dense(logits, "logits")), _ptr(out), _ptr(part_val), _ptr(part_idx), m,
                                         v, parts, _stream()), "argmax", kernels=2)
    return out


@_flushes
def adjust_logits(logits, softcap, penalty, history):
    """In place on float32 logits [M, V]: softcap (float32 [M], 0 = none), then the repetition penalty (float32 [M],
    1 = none) on the tokens of ``history`` (int32 [M, W], -1 where empty)."""
    m, v = logits.shape
    if logits.dtype != torch.float32 or history.dtype != torch.int32 or history.shape[0] != m:
        raise ValueError("adjust_logits takes float32 logits [M, V] and an int32 history [M, W]")
    _check(_fn("sampling", "akas_adjust_logits")(_ptr(_dense(logits, "logits")), _ptr(_dense(softcap, "softcap")),
                                                 _ptr(_dense(penalty, "penalty")), _ptr(_dense(history, "history")),
                                                 history.shape[1], m, v, _stream()), "adjust_logits")
    return logits


@_flushes
def sample(logits, temperature, top_k, top_p, uniform):
    m, v = logits.shape
    out = torch.empty((m,), dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "akas_sample")(_ptr(_dense(logits, "logits")), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                         _ptr(uniform), _ptr(out), m, v, _stream()), "sample")
    return out
