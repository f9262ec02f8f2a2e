"""Loads the compiled CUDA library and calls its `extern "C"` functions on torch tensors.

There is no fallback: if the library cannot be built or loaded, or a function reports an
error, an exception says so. Tensors are passed as raw device pointers with their sizes;
launches go to torch's current CUDA stream, so they order with torch's own work and can
be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_int64, c_uint64, c_void_p
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


_lib = None
launches = 0      # kernels launched through this module since import (a graph replay counts its kernels too)


def _signatures(lib) -> None:
    P, I, L, F = c_void_p, c_int, c_int64, c_float
    sig = {
        "xs_embed": [P, I, P, P, I, I, F, P],
        "xs_logit_cap": [P, L, F, P],
        "xs_add_rmsnorm": [P, P, I, P, P, P, I, P, I, I, F, F, P],
        "xs_silu_mul": [P, P, I, I, I, L, I, P],
        "xs_gated_act": [P, P, I, I, I, L, I, I, P],
        "xs_logit_scale": [P, L, F, P],
        "xs_side_gate": [P, L, P, P, L, I, I, I, I, P],
        "xs_rmsnorm_rows": [P, L, P, P, L, I, I, F, I, P],
        "xs_sigmoid_mul": [P, L, P, L, I, I, I, P],
        "xs_cast_rows": [P, L, P, L, I, I, I, P],
        "xs_lightning_scan": [P, L, I, I, I, P, P, P, P, P, I, I, I, I, I, P, P, I, P, P],
        "xs_zero_rows": [P, P, I, L, P],
        "xs_gemm_generic": [P, P, P, P, I, I, I, I, I, L, L, L, P],
        "xs_qk_norm_rope_store": [P, L, P, P, P, I, P, P, P, P, P, I, I, I, I, I, F, I, I, P],
        "xs_attention_generic": [P, P, P, I, P, P, P, L, P, I, I, I, I, I, F, I, I, P],
        "xs_short_conv": [P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
        "xs_attention_mma": [P, P, P, I, P, P, P, L, P, P, L, I, I, I, I, I, I, I, F, I, I, P],
        "xs_attention_tc": [P, P, L, P, I, P, P, P, L, P, I, I, I, I, I, I, I, F, I, I, P, P],
        "xs_gemm_small_m": [P, P, P, P, P, I, I, I, I, L, L, L, I, I, P, L, P],
        "xs_gemm_small_m_normed": [P, P, P, P, P, I, I, I, I, L, L, L, I, I, P, L, P, I, I, F, P, P, L, P, P],
        "xs_gemm_small_m_ex": [P, P, P, P, P, I, I, I, I, L, L, L, I, I, P, L, P, I, I, F, P, P, L, P,
                               P, P, P, P, P, P, I, I, P, P, P, P],
        "xs_gemm_small_m_rope": [P, P, P, P, I, I, I, L, L, L, P, I, I, F, P, P, P, I, P, P, P, P, P, I, I, I, I, F, P],
        "xs_attention_mma_merged": [P, P, P, I, P, P, P, L, P, P, L, P, L, P, I, I, I, I, I, I, I, F, I, I, P],
        "xs_gemm_tc": [P, P, P, P, I, I, I, I, I, L, L, L, I, P, L, P, P],
        "xs_argmax": [P, L, I, I, P, P, P],
        "xs_sample": [P, L, I, I, P, P, P, P, P, P, I, P, P],
        "xs_apply_penalties": [P, L, I, I, P, P, P, P, P, P, P],
        "xs_note_tokens": [P, P, I, I, P, P, I, P],
        "xs_add_layernorm": [P, P, I, P, P, P, I, P, I, I, F, F, P],
        "xs_grouped_rmsnorm": [P, P, P, I, I, I, I, F, P, L, I, P],
        "xs_clamped_glu": [P, P, I, I, I, L, F, F, F, I, P],
        "xs_gemm_tc_clamped": [P, P, P, I, I, I, I, L, L, L, F, F, F, P, P],
        "xs_gemm_tc_gelu": [P, P, P, I, I, I, I, L, L, L, P, P],
        "xs_moe_route": [P, I, I, I, I, F, P, P, P],
        "xs_moe_logits": [P, L, P, P, I, I, I, I, P],
        "xs_moe_plan": [P, I, I, I, I, P, P, P, P],
        "xs_moe_gather": [P, L, P, I, P, I, I, P],
        "xs_gemm_tc_grouped": [P, P, P, I, I, P, I, I, I, I, I, L, L, F, F, F, P, P],
        "xs_moe_gemm": [P, L, P, P, L, P, I, P, I, I, I, I, F, F, F, I, I, P],
        "xs_moe_combine": [P, P, P, P, I, I, I, P, P, I, P, L, I, P],
        "xs_relu_squared": [P, P, I, L, P],
        "xs_embed_pair": [P, P, I, P, P, P, P, P, P, P, P, P, I, I, F, I, ctypes.c_longlong, ctypes.c_longlong, F, P],
        "xs_mlstm_scan": [P, L, I, I, I, P, L, P, P, P, P, P, P, P, I, I, I, I, F, F, I, P, P, I, P, P, P],
        "xs_latent_prepare": [P, L, P, L, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, I, P],
        "xs_latent_attention_generic": [P, L, L, P, P, P, I, P, P, P, L, P, P, L, L, I, I, I, I, I, F, I, I, P],
        "xs_gemm_batched": [P, L, L, P, L, L, P, L, L, I, I, I, I, I, P],
        "xs_latent_attention_mma": [P, L, L, P, P, P, I, P, P, P, L, P, P, L, L, P, L, I, I, I, I, I, I, I, F, I, I, P],
        "xs_mamba2_conv": [P, L, I, P, P, P, P, P, P, P, I, I, I, I, I, P],
        "xs_embed_pos": [P, P, I, P, P, P, I, I, F, P],
        "xs_causal_conv": [P, L, P, P, P, P, P, P, L, I, I, I, I, I, I, I, I, P],
        "xs_gated_add": [P, P, I, P, L, P, I, I, P],
        "xs_depth_average": [P, L, P, I, P, L, P],
        "xs_rmsnorm_accumulate": [P, I, P, P, I, I, F, F, I, P],
        "xs_gated_delta_scan": [P, L, I, I, I, P, L, P, P, P, P, P, P, I, I, I, I, I, F, F, I, I, P],
        "xs_moe_route_grouped": [P, I, I, I, I, P, I, I, I, F, I, I, I, P, P, P],
        "xs_mamba2_scan": [P, P, L, I, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
        "xs_mamba2_scan_chunked": [P, P, L, I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    lib.xs_last_error.restype = ctypes.c_char_p
    lib.xs_last_error.argtypes = []
    lib.xs_uniform.restype = c_double
    lib.xs_uniform.argtypes = [c_uint64, c_uint64]
    lib.xs_abi_version.restype = c_int
    lib.xs_attention_mma_scratch_bytes.restype = c_int64
    lib.xs_attention_mma_scratch_bytes.argtypes = [c_int64, c_int, c_int]
    lib.xs_attention_mma_supports.restype = c_int
    lib.xs_attention_mma_supports.argtypes = [c_int, c_int, c_int]
    lib.xs_attention_tc_supports.restype = c_int
    lib.xs_attention_tc_supports.argtypes = [c_int, c_int, c_int]
    lib.xs_attention_mma_decode_slots.restype = c_int
    lib.xs_attention_mma_decode_slots.argtypes = [c_int, c_int64]
    lib.xs_gemm_small_m_supports.restype = c_int
    lib.xs_gemm_small_m_supports.argtypes = [c_int, c_int, c_int64, c_int64]
    lib.xs_gemm_tc_supports.restype = c_int
    lib.xs_gemm_tc_supports.argtypes = [c_int, c_int, c_int, c_int64, c_int64]
    lib.xs_gemm_tc_tile_n.restype = c_int
    lib.xs_gemm_tc_tile_n.argtypes = [c_int]
    lib.xs_gemm_tc_scratch_bytes.restype = c_int64
    lib.xs_gemm_tc_scratch_bytes.argtypes = [c_int, c_int, c_int]
    lib.xs_moe_tile_rows.restype = c_int
    lib.xs_moe_tile_rows.argtypes = []
    lib.xs_moe_max_tiles.restype = c_int
    lib.xs_moe_max_tiles.argtypes = [c_int, c_int]
    lib.xs_latent_attention_mma_supports.restype = c_int
    lib.xs_latent_attention_mma_supports.argtypes = [c_int, c_int, c_int]
    lib.xs_latent_attention_mma_ctas_per_sm.restype = c_int
    lib.xs_latent_attention_mma_ctas_per_sm.argtypes = [c_int, c_int, c_int, c_int]
    lib.xs_latent_attention_mma_scratch_bytes.restype = c_int64
    lib.xs_latent_attention_mma_scratch_bytes.argtypes = [c_int64, c_int, c_int]
    lib.xs_moe_max_tiles_of.restype = c_int
    lib.xs_moe_max_tiles_of.argtypes = [c_int, c_int, c_int]
    lib.xs_gemm_small_m_ksplit.restype = c_int
    lib.xs_gemm_small_m_ksplit.argtypes = [c_int, c_int, c_int, c_int]
    lib.xs_gemm_small_m_scratch_bytes.restype = c_int64
    lib.xs_gemm_small_m_scratch_bytes.argtypes = [c_int, c_int, c_int]


class _Watched:
    """The library behind two debugging switches (the reference has the same pair for its own backend,
    XS_SYCL_PROFILE and XS_SYCL_SYNC, src/backend/sycl/sycl_backend.cpp:351-353, 2520-2570):

    XS_PROFILE=1  CUDA events around every launch; `profile_report()` (also printed at exit) sums the device time by
                  kernel function and by its sizes (the call's integer arguments).
    XS_SYNC=1     the device is waited for after every launch, and an error that shows up there is raised with the
                  name and the sizes of the launch it belongs to, instead of surfacing at some later call.

    Both run every step kernel by kernel (no CUDA graphs: engine/model.py) and cost time; neither is on by default."""

    def __init__(self, lib, profile: bool, sync: bool):
        self._lib, self._profile, self._sync = lib, profile, sync
        self.spans = []         # (name, sizes, start event, end event)
        self._name = lib._name

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        argtypes = getattr(fn, "argtypes", None)
        if not name.startswith("xs_") or not argtypes or argtypes[-1] is not c_void_p or fn.restype is not c_int:
            return fn           # not a launch (a query, a switch)

        def call(*args):
            sizes = tuple(a for a, t in zip(args, argtypes) if t in (c_int, c_int64) and isinstance(a, int) and abs(a) < (1 << 40))
            capturing = torch.cuda.is_current_stream_capturing()
            if self._profile and not capturing:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                rc = fn(*args)
                end.record()
                self.spans.append((name, sizes, start, end))
            else:
                rc = fn(*args)
            if self._sync and not capturing and rc == 0:
                try:
                    torch.cuda.synchronize()
                except RuntimeError as e:
                    raise KernelError(f"{name}{sizes}: the device reported an error after this launch: {e}") from None
            return rc

        call.__name__ = name
        setattr(self, name, call)
        return call


def profile_report(reset: bool = True, file=None) -> dict:
    """{(kernel function, sizes): (launches, total microseconds)} of the launches made under XS_PROFILE=1 since
    the last report, printed as a table (largest first) to `file` (standard error)."""
    import sys
    lib = _lib
    if not isinstance(lib, _Watched) or not lib.spans:
        return {}
    torch.cuda.synchronize()
    table = {}
    for name, sizes, start, end in lib.spans:
        n, us = table.get((name, sizes), (0, 0.0))
        table[(name, sizes)] = (n + 1, us + start.elapsed_time(end) * 1e3)
    if reset:
        lib.spans = []
    out = file or sys.stderr
    total = sum(us for _, us in table.values())
    print(f"[xpu_serve_b200 profile] {sum(n for n, _ in table.values())} launches, {total:.0f} us on the device", file=out)
    for (name, sizes), (n, us) in sorted(table.items(), key=lambda kv: -kv[1][1]):
        print(f"  {us:10.1f} us {100 * us / max(total, 1e-9):5.1f} %  x{n:<5d} {name} {sizes}", file=out)
    return table


def load(verbose: bool = True):
    """The library handle, built first if its file is missing."""
    global _lib
    if _lib is None:
        path = _build.build(verbose=verbose)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the CUDA library {path} cannot be loaded: {e}") from None
        _signatures(lib)
        # tuning switches, read once (defaults are what measured best on B200)
        if "XS_ATTN_DECODE_STAGES" in os.environ:
            lib.xs_attention_mma_set_decode_stages(int(os.environ["XS_ATTN_DECODE_STAGES"]))
        if os.environ.get("XS_NO_ONE_ROUND", "0") == "1":
            lib.xs_gemm_small_m_set_one_round(0)
        if "XS_ATTN_PREFETCH_BLOCKS" in os.environ:
            lib.xs_attention_mma_set_prefetch_blocks(int(os.environ["XS_ATTN_PREFETCH_BLOCKS"]))
        if os.environ.get("XS_NO_PDL", "0") == "1":
            lib.xs_set_pdl(0)
        if os.environ.get("XS_TC_NO_PAIR", "0") == "1":
            lib.xs_gemm_tc_set_pair(0)
        if "XS_ATTN_TMA_CARVEOUT" in os.environ:
            lib.xs_attention_mma_set_tma_carveout(int(os.environ["XS_ATTN_TMA_CARVEOUT"]))
        if "XS_ATTN_DECODE_TMA" in os.environ:        # "0": cp.async kernel for every head size; "n" (2..6): that many stages
            n = int(os.environ["XS_ATTN_DECODE_TMA"])
            lib.xs_attention_mma_set_decode_tma(1 if n > 0 else 0, n)
        profile, sync = os.environ.get("XS_PROFILE", "0") == "1", os.environ.get("XS_SYNC", "0") == "1"
        if profile or sync:
            lib = _Watched(lib, profile, sync)
            if profile:
                import atexit
                atexit.register(profile_report)
        _lib = lib
    return _lib


def watched() -> bool:
    """Whether XS_PROFILE or XS_SYNC is on (steps then run kernel by kernel, without CUDA graphs)."""
    return os.environ.get("XS_PROFILE", "0") == "1" or os.environ.get("XS_SYNC", "0") == "1"


def loaded_path() -> Optional[str]:
    return None if _lib is None else _lib._name


def _check(rc: int, kernels: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(_lib.xs_last_error().decode("utf-8", "replace"))
    launches += kernels


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (inside a graph capture: the capturing stream). Asked of torch's C layer directly
    where it offers that: `torch.cuda.current_stream()` builds a Python object per call, a hundred times a step."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32, bfloat16 are)") from None


def _need(t: torch.Tensor, what: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, is {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def uniform(seed: int, counter: int) -> float:
    """The uniform in [0, 1) that the sampling kernel derives from (seed, counter)."""
    return float(load().xs_uniform(seed & (2 ** 64 - 1), counter & (2 ** 64 - 1)))


# ------------------------------------------------------------------ wrappers
def embed(table: torch.Tensor, ids: torch.Tensor, h: torch.Tensor, scale: float = 1.0) -> None:
    """h[t] = table[ids[t]] * scale, float32."""
    _need(table, "embedding table"); _need(ids, "ids", torch.int32); _need(h, "h", torch.float32)
    T, H = h.shape
    _check(load().xs_embed(table.data_ptr(), _code(table), ids.data_ptr(), h.data_ptr(), T, H, float(scale), _stream()))


def logit_cap(logits: torch.Tensor, cap: float) -> None:
    """logits = cap * tanh(logits / cap), in place."""
    _need(logits, "logits", torch.float32)
    _check(load().xs_logit_cap(logits.data_ptr(), logits.numel(), float(cap), _stream()))


def add_rmsnorm(h: torch.Tensor, m: Optional[torch.Tensor], post_w: Optional[torch.Tensor],
                w: Optional[torch.Tensor], y: Optional[torch.Tensor], rows: Optional[torch.Tensor], eps: float,
                eps_post: Optional[float] = None) -> None:
    """h += post(m) (if m); y = RMSNorm(h, w) (if w), over `rows` of h when given."""
    _need(h, "h", torch.float32)
    H = h.shape[-1]
    n = h.shape[0] if rows is None else rows.numel()
    if m is not None:
        _need(m, "m")
        if m.shape != h.shape:
            raise KernelError(f"m is {tuple(m.shape)}, h is {tuple(h.shape)}")
    for v, name in ((post_w, "post_w"), (w, "w")):
        if v is not None:
            _need(v, name, torch.float32)
            if v.numel() != H:
                raise KernelError(f"{name} has {v.numel()} elements for rows of {H}")
    if y is not None:
        _need(y, "y")
        if y.shape[0] < n or y.shape[-1] != H:
            raise KernelError(f"y is {tuple(y.shape)} for {n} rows of {H}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _check(load().xs_add_rmsnorm(h.data_ptr(), _ptr(m), F32 if m is None else _code(m), _ptr(post_w), _ptr(w),
                                 _ptr(y), F32 if y is None else _code(y), _ptr(rows), n, H,
                                 float(eps if eps_post is None else eps_post), float(eps), _stream()))


def silu_mul(gu: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> None:
    """out = silu(gate) * up. interleave 0: a row of gu is [gate | up]; 8: blocks of 8 gate, 8 up columns."""
    _need(out, "out", gu.dtype)
    if not gu.is_cuda or gu.dim() != 2 or gu.stride(1) != 1:
        raise KernelError("gate_up must be a CUDA matrix with contiguous rows")
    T, F = out.shape
    if gu.shape[0] != T or gu.shape[1] < 2 * F:
        raise KernelError(f"gate_up is {tuple(gu.shape)} for an output of {tuple(out.shape)}")
    _check(load().xs_silu_mul(gu.data_ptr(), out.data_ptr(), _code(gu), T, F, gu.stride(0), int(interleave), _stream()))


GATE_ACTS = {"silu": 0, "gelu_tanh": 1}


def gated_act(gu: torch.Tensor, out: torch.Tensor, act: str = "silu", interleave: int = 0) -> None:
    """out = act(gate) * up with act "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))); the layouts
    of `silu_mul`."""
    if act not in GATE_ACTS:
        raise KernelError(f"gated_act: activation '{act}' ({', '.join(GATE_ACTS)})")
    _need(out, "out", gu.dtype)
    if not gu.is_cuda or gu.dim() != 2 or gu.stride(1) != 1:
        raise KernelError("gate_up must be a CUDA matrix with contiguous rows")
    T, F = out.shape
    if gu.shape[0] != T or gu.shape[1] < 2 * F:
        raise KernelError(f"gate_up is {tuple(gu.shape)} for an output of {tuple(out.shape)}")
    _check(load().xs_gated_act(gu.data_ptr(), out.data_ptr(), _code(gu), T, F, gu.stride(0), int(interleave), GATE_ACTS[act], _stream()))


def logit_scale(logits: torch.Tensor, scale: float) -> None:
    """logits *= scale, in place."""
    _need(logits, "logits", torch.float32)
    _check(load().xs_logit_scale(logits.data_ptr(), logits.numel(), float(scale), _stream()))


def zero_rows(state: torch.Tensor, slots: torch.Tensor) -> None:
    _need(state, "state"); _need(slots, "slots", torch.int32)
    row_bytes = state[0].numel() * state.element_size()
    _check(load().xs_zero_rows(state.data_ptr(), slots.data_ptr(), slots.numel(), row_bytes, _stream()))


def gemm_generic(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """out[M, N] = x[M, K] . w[N, K]^T (+ bias). Rows may be strided; columns are contiguous."""
    for t, name in ((x, "x"), (w, "w"), (out, "out")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm: {name} must be a CUDA matrix with contiguous rows")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or x.dtype != w.dtype:
        raise KernelError(f"gemm: x {tuple(x.shape)} {x.dtype}, w {tuple(w.shape)} {w.dtype}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    _check(load().xs_gemm_generic(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), _code(x), _code(out),
                                  M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()))


def qk_norm_rope_store(qkv: torch.Tensor, q_out: torch.Tensor, pool: Optional[torch.Tensor],
                       page_table: Optional[torch.Tensor], seq_of_token: torch.Tensor, positions: torch.Tensor,
                       q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], rope: Optional[torch.Tensor],
                       heads: int, kv_heads: int, head_dim: int, page_size: int, eps: float, write_kv: bool) -> None:
    _need(q_out, "q_out", qkv.dtype)
    if qkv.stride(1) != 1:
        raise KernelError("qkv rows must be contiguous")
    T = qkv.shape[0]
    width = (heads + (2 * kv_heads if write_kv else 0)) * head_dim
    if qkv.shape[1] < width:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, needs {width} columns")
    if write_kv:
        _need(pool, "cache", qkv.dtype); _need(page_table, "page table", torch.int32)
        if tuple(pool.shape[1:]) != (2, kv_heads, page_size, head_dim):
            raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {head_dim}]")
    for v, name in ((q_w, "q_norm"), (k_w, "k_norm")):
        if v is not None:
            _need(v, name, torch.float32)
            if v.numel() != head_dim:
                raise KernelError(f"{name} has {v.numel()} elements for heads of {head_dim}")
    if rope is not None:
        _need(rope, "rope table", torch.float32)
        if tuple(rope.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"rope table is {tuple(rope.shape)}, expected [*, {head_dim // 2}, 2]")
    P = 0 if page_table is None else page_table.shape[1]
    _check(load().xs_qk_norm_rope_store(
        qkv.data_ptr(), qkv.stride(0), q_out.data_ptr(), _ptr(pool), _ptr(page_table), P, seq_of_token.data_ptr(),
        positions.data_ptr(), _ptr(q_w), _ptr(k_w), _ptr(rope), T, heads, kv_heads, head_dim, page_size, float(eps),
        1 if write_kv else 0, _code(qkv), _stream()))


def attention_generic(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, seq_of_token: torch.Tensor,
                      positions: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, kv_heads: int,
                      page_size: int, scale: float, window: int) -> None:
    _need(q, "q"); _need(out, "out", q.dtype); _need(pool, "cache", q.dtype); _need(page_table, "page table", torch.int32)
    T, heads, D = q.shape
    if tuple(pool.shape[1:]) != (2, kv_heads, page_size, D):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {D}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < heads:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {heads} heads")
        ld_gate = gate.stride(0)
    _check(load().xs_attention_generic(
        q.data_ptr(), pool.data_ptr(), page_table.data_ptr(), page_table.shape[1], seq_of_token.data_ptr(),
        positions.data_ptr(), _ptr(gate), ld_gate, out.data_ptr(), T, heads, kv_heads, D, page_size, float(scale),
        int(window), _code(q), _stream()))


def attention_mma_supports(head_dim: int, page_size: int, group: int) -> bool:
    return bool(load().xs_attention_mma_supports(head_dim, page_size, group))


def attention_mma_decode_slots(head_dim: int, tiles: int) -> int:
    """CTAs of the decode attention kernel that run at one time on the device when `tiles` = sequences x kv heads
    (the kernel keeps fewer stages, and so more CTAs an SM, when the tiles alone overfill the device)."""
    return int(load().xs_attention_mma_decode_slots(head_dim, tiles))


def attention_mma_scratch_bytes(rows: int, head_dim: int, splits: int) -> int:
    return int(load().xs_attention_mma_scratch_bytes(rows, head_dim, splits))


def attention_mma(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, cu_seqlens: torch.Tensor,
                  kv_lens: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor,
                  scratch: Optional[torch.Tensor], n_seqs: int, max_q_len: int, kv_heads: int, page_size: int,
                  scale: float, window: int, splits: int, counters: Optional[torch.Tensor] = None,
                  bounded_waits: bool = False) -> None:
    """Tensor-core attention over the paged bfloat16 cache. `scratch`: a byte buffer of at least
    attention_mma_scratch_bytes(tokens * heads, head_dim, splits) when splits > 1. `counters`: at least
    n_seqs * kv_heads zeroed int32 words that the kernel leaves zeroed; with them a decode step (one token a
    sequence) merges its key splits inside the attention kernel instead of in a second one. `bounded_waits`: a decode
    step at head size 64 may take the kernel that the TMA unit feeds; its waits are bounded, and one that gives up sets
    gemm_tc_status(device), which the caller then has to look at (tc_status_unread)."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pool, "cache", torch.bfloat16)
    _need(page_table, "page table", torch.int32)
    T, heads, D = q.shape
    if tuple(pool.shape[1:]) != (2, kv_heads, page_size, D):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {D}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < heads:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {heads} heads")
        ld_gate = gate.stride(0)
    sbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    merged = counters is not None and splits > 1 and max_q_len == 1 and heads // kv_heads <= 16
    if merged:
        _need(counters, "counters", torch.int32)
        if counters.numel() < n_seqs * kv_heads:
            raise KernelError(f"attention: {counters.numel()} counters for {n_seqs} sequences of {kv_heads} kv heads")
    tma = bounded_waits and max_q_len == 1 and D == 64 and heads // kv_heads <= 16
    if tma:
        mark_bounded(q.device)
    _check(load().xs_attention_mma_merged(
        q.data_ptr(), pool.data_ptr(), page_table.data_ptr(), page_table.shape[1], cu_seqlens.data_ptr(),
        kv_lens.data_ptr(), _ptr(gate), ld_gate, out.data_ptr(), _ptr(scratch), sbytes, _ptr(counters) if merged else None,
        pool.shape[0] if tma else 0, gemm_tc_status(q.device).data_ptr() if tma else None,
        T, n_seqs, max_q_len, heads, kv_heads, D, page_size, float(scale), int(window), int(splits), _stream()),
        kernels=2 if splits > 1 and not merged else 1)


def attention_tc_supports(head_dim: int, page_size: int, group: int) -> bool:
    return bool(load().xs_attention_tc_supports(head_dim, page_size, group))


def attention_tc(q: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor, cu_seqlens: torch.Tensor,
                 kv_lens: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, n_seqs: int, max_q_len: int,
                 kv_heads: int, page_size: int, scale: float, window: int, max_kv_len: int = 0) -> None:
    """Attention for prompts on the tcgen05 tensor cores (head size 64): the same operation as attention_mma with
    one key split. A wait that gives up inside the kernel sets gemm_tc_status(device). `max_kv_len` (the longest
    sequence's keys, 0 if unknown) only picks the order in which the kernel's CTAs start."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pool, "cache", torch.bfloat16)
    _need(page_table, "page table", torch.int32)
    T, heads, D = q.shape
    if tuple(pool.shape[1:]) != (2, kv_heads, page_size, D):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {D}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < heads:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {heads} heads")
        ld_gate = gate.stride(0)
    mark_bounded(q.device)
    _check(load().xs_attention_tc(
        q.data_ptr(), pool.data_ptr(), pool.shape[0], page_table.data_ptr(), page_table.shape[1], cu_seqlens.data_ptr(),
        kv_lens.data_ptr(), _ptr(gate), ld_gate, out.data_ptr(), T, n_seqs, max_q_len, heads, kv_heads, D, page_size,
        float(scale), int(window), int(max_kv_len), gemm_tc_status(q.device).data_ptr(), _stream()))


def gemm_small_m_supports(M: int, K: int, ldx: int, ldw: int) -> bool:
    return bool(load().xs_gemm_small_m_supports(M, K, ldx, ldw))


def gemm_small_m_ksplit(M: int, N: int, K: int, sms: int) -> int:
    """The number of K slices the kernel prefers for this shape on a device with `sms` SMs."""
    return int(load().xs_gemm_small_m_ksplit(M, N, K, sms))


def gemm_small_m_scratch_bytes(M: int, N: int, ksplit: int) -> int:
    return int(load().xs_gemm_small_m_scratch_bytes(M, N, ksplit))


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, swiglu=False, ksplit: int = 1,
                 scratch: Optional[torch.Tensor] = None, in_ssq: Optional[torch.Tensor] = None, in_width: int = 0,
                 in_eps: float = 0.0, next_w: Optional[torch.Tensor] = None, next_x: Optional[torch.Tensor] = None,
                 out_ssq: Optional[torch.Tensor] = None, conv: Optional[dict] = None,
                 argmax: Optional[tuple] = None) -> None:
    """out[M, N] = x . w^T (+ bias) for M <= 16, bfloat16 operands; or residual (float32) += the product;
    or, with swiglu, out[M, N / 2] = silu(gate) * up for a weight stacked as blocks of 8 gate and 8 up rows
    (swiglu="relu_squared": out[M, N] = max(product, 0)^2 instead; swiglu="gelu_tanh": the gated form with the tanh form
    of gelu on the gate).
    ksplit > 1 cuts K over several CTAs; `scratch` is then a zero-initialised byte buffer of at least
    gemm_small_m_scratch_bytes, kept (whole) from call to call.

    RMSNorm across the product: with `residual`, `next_w` [N] and `next_x` [M, N] bfloat16, the kernel also
    leaves next_x = bfloat16(residual * next_w) and, in `out_ssq` [ceil(N / 16), 16] float32, each tile's
    sums of squares of the new residual values per row. A product given that `out_ssq` as `in_ssq` (with the
    residual's width and the norm's eps) and that `next_x` as x scales its result by each row's
    1 / sqrt(mean square + eps): together they are norm(residual) . w^T without a norm kernel between.

    Work behind the product, in the same kernel: `conv` = dict(taps [k, H] float32, bias [H] or None, state
    [slots, k - 1, H] bfloat16, slots [M] int32, out [M, H] bfloat16, counters: H / 16 zeroed int32 words, left
    zeroed): the product is a short-convolution layer's in_proj for one token a sequence, out = [B | C | X], and the
    gated convolution with its state update follows. `argmax` = (out [M] int32, keys: 16 zeroed int64 words,
    counter: one zeroed int32 word; both left zeroed): each row's column of the largest output."""
    for t, name in ((x, "x"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.bfloat16:
            raise KernelError(f"gemm (few rows): {name} must be a bfloat16 CUDA matrix with contiguous rows")
    M, K = x.shape
    N = w.shape[0]
    target = residual if residual is not None else out
    if w.shape[1] != K or target is None or tuple(target.shape) != (M, N // 2 if swiglu in (True, "gelu_tanh") else N) or target.stride(1) != 1:
        raise KernelError(f"gemm (few rows): x {tuple(x.shape)}, w {tuple(w.shape)}, out "
                          f"{None if target is None else tuple(target.shape)}")
    if residual is not None and residual.dtype != torch.float32:
        raise KernelError("gemm (few rows): the residual must be float32")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    in_tiles = 0
    if in_ssq is not None:
        _need(in_ssq, "in_ssq", torch.float32)
        if in_ssq.dim() != 2 or in_ssq.shape[1] != 16 or not in_ssq.is_contiguous() or in_width <= 0:
            raise KernelError(f"gemm (few rows): sums of squares {tuple(in_ssq.shape)} over a width of {in_width}")
        in_tiles = in_ssq.shape[0]
    ld_next = 0
    if next_x is not None or next_w is not None or out_ssq is not None:
        if next_x is not None:
            _need(next_w, "next_w", torch.float32); _need(next_x, "next_x", torch.bfloat16)
            if tuple(next_x.shape) != (M, N) or next_x.stride(1) != 1 or next_w.numel() != N or not next_w.is_contiguous():
                raise KernelError(f"gemm (few rows): next_x {tuple(next_x.shape)}, next_w {tuple(next_w.shape)} for [{M}, {N}]")
            ld_next = next_x.stride(0)
        _need(out_ssq, "out_ssq", torch.float32)
        if tuple(out_ssq.shape) != ((N + 15) // 16, 16) or not out_ssq.is_contiguous():
            raise KernelError(f"gemm (few rows): out_ssq is {tuple(out_ssq.shape)}, expected [{(N + 15) // 16}, 16]")
    cv = [None] * 6 + [0, 0]
    if conv is not None:
        taps, state, slots, cout, counters = conv["taps"], conv["state"], conv["slots"], conv["out"], conv["counters"]
        k, H = taps.shape
        _need(taps, "taps", torch.float32); _need(state, "state", torch.bfloat16); _need(slots, "slots", torch.int32)
        _need(cout, "conv out", torch.bfloat16); _need(counters, "conv counters", torch.int32)
        if conv.get("bias") is not None:
            _need(conv["bias"], "conv bias", torch.float32)
        if (N != 3 * H or tuple(state.shape[1:]) != (k - 1, H) or slots.numel() < M or tuple(cout.shape) != (M, H)
                or counters.numel() < H // 16 or out is None or out.dtype != torch.bfloat16):
            raise KernelError(f"gemm (few rows): convolution of {k} taps over {H} channels behind a product of {N} columns, "
                              f"state {tuple(state.shape)}, out {tuple(cout.shape)}")
        cv = [taps.data_ptr(), _ptr(conv.get("bias")), state.data_ptr(), slots.data_ptr(), cout.data_ptr(),
              counters.data_ptr(), int(k), int(H)]
    am = [None, None, None]
    if argmax is not None:
        a_out, keys, counter = argmax
        _need(a_out, "argmax out", torch.int32); _need(keys, "argmax keys", torch.int64); _need(counter, "argmax counter", torch.int32)
        if a_out.numel() < M or keys.numel() < 16 or M > 16:
            raise KernelError(f"gemm (few rows): argmax of {M} rows into {a_out.numel()} words")
        am = [keys.data_ptr(), counter.data_ptr(), a_out.data_ptr()]
    _check(load().xs_gemm_small_m_ex(
        x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(out), _ptr(residual), F32 if out is None else _code(out), M, N, K,
        x.stride(0), w.stride(0), target.stride(0), 2 if swiglu == "relu_squared" else 3 if swiglu == "gelu_tanh" else 1 if swiglu else 0, int(ksplit), _ptr(scratch),
        0 if scratch is None else scratch.numel() * scratch.element_size(), _ptr(in_ssq), in_tiles, int(in_width),
        float(in_eps), _ptr(next_w), _ptr(next_x), ld_next, _ptr(out_ssq), *cv, *am, _stream()))


def gemm_small_m_rope(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor],
                      q_out: torch.Tensor, pool: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                      seq_of_token: torch.Tensor, positions: torch.Tensor, q_w: Optional[torch.Tensor],
                      k_w: Optional[torch.Tensor], rope: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int,
                      page_size: int, eps: float, in_ssq: Optional[torch.Tensor] = None, in_width: int = 0,
                      in_eps: float = 0.0) -> None:
    """An attention layer's q/k/v product for one token a sequence (M <= 16, bfloat16) with what qk_norm_rope_store does
    behind it in the same kernel: out [M, N] = x . w^T (+ bias) as gemm_small_m leaves it (its columns behind the heads,
    the head gate's, are what the caller still reads), and from its columns (heads x head_dim of q, then, with `pool`,
    kv_heads x head_dim of k and of v): per-head RMSNorm (q_w, k_w), rotation by `rope` [positions, head_dim / 2, 2],
    queries to q_out [M, heads, head_dim], keys and raw values into the cache's pages. Head sizes 32, 64, 128."""
    for t, name in ((x, "x"), (w, "w"), (out, "out"), (q_out, "q_out")):
        _need(t, name, torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    width = (heads + (2 * kv_heads if pool is not None else 0)) * head_dim
    if (x.stride(1) != 1 or w.stride(1) != 1 or w.shape[1] != K or tuple(out.shape) != (M, N) or out.stride(1) != 1
            or N < width or tuple(q_out.shape) != (M, heads, head_dim) or not q_out.is_contiguous()
            or head_dim not in (32, 64, 128) or M > 16):
        raise KernelError(f"gemm (few rows) with rotation: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, "
                          f"q_out {tuple(q_out.shape)}, {heads} + 2 x {kv_heads} heads of {head_dim}")
    _need(seq_of_token, "seq_of_token", torch.int32); _need(positions, "positions", torch.int32)
    if seq_of_token.numel() < M or positions.numel() < M:
        raise KernelError("gemm (few rows) with rotation: a sequence and a position per row")
    P_ = 0
    if pool is not None:
        _need(pool, "cache", torch.bfloat16); _need(page_table, "page table", torch.int32)
        if tuple(pool.shape[1:]) != (2, kv_heads, page_size, head_dim):
            raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 2, {kv_heads}, {page_size}, {head_dim}]")
        P_ = page_table.shape[1]
    for v, name in ((q_w, "q_norm"), (k_w, "k_norm")):
        if v is not None:
            _need(v, name, torch.float32)
            if v.numel() != head_dim:
                raise KernelError(f"{name} has {v.numel()} elements for heads of {head_dim}")
    if rope is not None:
        _need(rope, "rope table", torch.float32)
        if tuple(rope.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"rope table is {tuple(rope.shape)}, expected [*, {head_dim // 2}, 2]")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    in_tiles = 0
    if in_ssq is not None:
        _need(in_ssq, "in_ssq", torch.float32)
        if in_ssq.dim() != 2 or in_ssq.shape[1] != 16 or not in_ssq.is_contiguous() or in_width <= 0:
            raise KernelError(f"gemm (few rows): sums of squares {tuple(in_ssq.shape)} over a width of {in_width}")
        in_tiles = in_ssq.shape[0]
    _check(load().xs_gemm_small_m_rope(
        x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), out.stride(0),
        _ptr(in_ssq), in_tiles, int(in_width), float(in_eps), q_out.data_ptr(), _ptr(pool), _ptr(page_table), P_,
        seq_of_token.data_ptr(), positions.data_ptr(), _ptr(q_w), _ptr(k_w), _ptr(rope), heads, kv_heads, head_dim,
        page_size, float(eps), _stream()))


EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_RELU_SQ = 0, 1, 2, 3
_tc_status = {}


def gemm_tc_supports(T: int, N: int, K: int, ldx: int, ldw: int) -> bool:
    return bool(load().xs_gemm_tc_supports(T, N, K, ldx, ldw))


def gemm_tc_scratch_bytes(T: int, N: int, ksplit: int) -> int:
    return int(load().xs_gemm_tc_scratch_bytes(T, N, ksplit))


def gemm_tc_status(device) -> torch.Tensor:
    """The device word that the tcgen05 kernels set non-zero when one of their waits gave up."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _tc_status:
        _tc_status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_status[device]


# Devices on which a kernel with bounded waits (the tcgen05 kernels, decode attention fed by the TMA unit) was launched
# since the status word was last looked at. Whoever next waits for the device anyway (the generation loop for its
# tokens, trace replay for its logits) reads the word with what it waits for and hands it to `tc_status_read`.
_tc_unread = set()


bounded_launches = 0      # launches of kernels with bounded waits since import (a graph's capture counts its own)


def mark_bounded(device) -> None:
    """A kernel with bounded waits was launched (or a graph that holds one replayed) on `device`."""
    global bounded_launches
    bounded_launches += 1
    _tc_unread.add(gemm_tc_status(device).device)


def tc_status_unread(device) -> bool:
    return gemm_tc_status(device).device in _tc_unread


def tc_status_read(value: int, device) -> None:
    """`value`: the status word as copied from the device after every tcgen05 kernel launched so far has run.
    Non-zero: a bounded wait inside such a kernel gave up, so what the step wrote (activations, keys and
    values in the cache) is partly computed: the word is cleared and the step fails."""
    word = gemm_tc_status(device)
    _tc_unread.discard(word.device)
    if int(value) != 0:
        word.zero_()
        raise KernelError(f"a tcgen05 kernel gave up waiting (status {int(value)}): this step's results and what it "
                          f"wrote to the cache are not valid")


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            epilogue: int = EPI_STORE, ksplit: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """x[T, K] . w[N, K]^T on tcgen05 tensor cores (bfloat16 operands). epilogue EPI_STORE: out[T, N] bfloat16 or
    float32; EPI_RESIDUAL: out float32 += product; EPI_SWIGLU: out[T, N / 2] = silu(gate) * up for a weight stacked
    in blocks of 8 gate and 8 up rows; EPI_RELU_SQ: out = max(product, 0)^2."""
    for t, name in ((x, "x"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.bfloat16:
            raise KernelError(f"gemm (tcgen05): {name} must be a bfloat16 CUDA matrix with contiguous rows")
    T, K = x.shape
    N = w.shape[0]
    cols = N // 2 if epilogue == EPI_SWIGLU else N
    if w.shape[1] != K or tuple(out.shape) != (T, cols) or out.stride(1) != 1:
        raise KernelError(f"gemm (tcgen05): x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    mark_bounded(x.device)
    _check(load().xs_gemm_tc(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), _code(out), int(epilogue), T, N, K,
                             x.stride(0), w.stride(0), out.stride(0), int(ksplit), _ptr(scratch),
                             0 if scratch is None else scratch.numel() * scratch.element_size(),
                             gemm_tc_status(x.device).data_ptr(), _stream()))


def short_conv(bcx: torch.Tensor, w_t: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
               all_single: bool = False) -> None:
    """`all_single`: every sequence brings exactly one token (lets one kernel also move the state)."""
    _need(out, "out", bcx.dtype); _need(state, "state", bcx.dtype); _need(w_t, "taps", torch.float32)
    T, H = out.shape
    K = w_t.shape[0]
    if bcx.stride(1) != 1 or bcx.shape[0] != T or bcx.shape[1] < 3 * H or w_t.shape[1] != H:
        raise KernelError(f"short_conv: bcx {tuple(bcx.shape)}, taps {tuple(w_t.shape)}, out {tuple(out.shape)}")
    if tuple(state.shape[1:]) != (K - 1, H):
        raise KernelError(f"short_conv: state is {tuple(state.shape)}, expected [*, {K - 1}, {H}]")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    _check(load().xs_short_conv(bcx.data_ptr(), bcx.stride(0), w_t.data_ptr(), _ptr(bias), state.data_ptr(),
                                seq_of_token.data_ptr(), cu_seqlens.data_ptr(), slots.data_ptr(), out.data_ptr(),
                                T, slots.numel(), H, K, _code(bcx), 1 if all_single else 0, _stream()),
           kernels=1 if all_single and bcx.dtype == torch.bfloat16 and H % 8 == 0 and K <= 8 else 2)


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = index of the largest of row i, the lowest index among equals."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    n, V = logits.shape
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch.numel() < n:       # zeroed words the wide-row path works in and leaves zeroed
        scratch = _argmax_scratch[logits.device] = torch.zeros(max(n, 256), dtype=torch.int64, device=logits.device)
    _check(load().xs_argmax(logits.data_ptr(), logits.stride(0), n, V, out.data_ptr(), scratch.data_ptr(), _stream()),
           kernels=2 if V >= 16384 else 1)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor, out: torch.Tensor,
           advance: bool = False) -> None:
    """A seeded draw per row from (seed, counter). `advance`: every row's counter goes up by one inside the kernel
    (greedy rows' too), so that a generation loop needs no launch of its own for that."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    n, V = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                        (seeds, "seeds", torch.int64), (counters, "counters", torch.int64)):
        _need(t, name, dt)
        if t.numel() < n:
            raise KernelError(f"{name} has {t.numel()} entries for {n} rows")
    _check(load().xs_sample(logits.data_ptr(), logits.stride(0), n, V, temperature.data_ptr(), top_k.data_ptr(),
                            top_p.data_ptr(), min_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(),
                            1 if advance else 0, out.data_ptr(), _stream()))


def apply_penalties(logits: torch.Tensor, seen: torch.Tensor, gen_count: torch.Tensor, state_rows: torch.Tensor,
                    repetition: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(seen, "seen", torch.uint8); _need(gen_count, "counts", torch.int32)
    n, V = logits.shape
    _check(load().xs_apply_penalties(logits.data_ptr(), logits.stride(0), n, V, seen.data_ptr(), gen_count.data_ptr(),
                                     state_rows.data_ptr(), repetition.data_ptr(), presence.data_ptr(),
                                     frequency.data_ptr(), _stream()))


def note_tokens(tokens: torch.Tensor, rows_of_token: torch.Tensor, seen: torch.Tensor, gen_count: torch.Tensor,
                generated: bool) -> None:
    _need(tokens, "tokens", torch.int32); _need(rows_of_token, "rows", torch.int32)
    V = seen.shape[1]
    _check(load().xs_note_tokens(tokens.data_ptr(), rows_of_token.data_ptr(), tokens.numel(), V, seen.data_ptr(),
                                 gen_count.data_ptr(), 1 if generated else 0, _stream()))


# ------------------------------------------------ layer norm, grouped unit norm, clamped gated unit
def add_layernorm(h: torch.Tensor, m: Optional[torch.Tensor], post_w: Optional[torch.Tensor],
                  w: Optional[torch.Tensor], y: Optional[torch.Tensor], rows: Optional[torch.Tensor], eps: float,
                  eps_post: Optional[float] = None) -> None:
    """h += LN(m, post_w) (m alone without post_w), if m; y = LN(h, w) (if w), over `rows` of h when given; LN is the
    layer norm with a weight and no bias."""
    _need(h, "h", torch.float32)
    H = h.shape[-1]
    n = h.shape[0] if rows is None else rows.numel()
    if m is not None:
        _need(m, "m")
        if m.shape != h.shape:
            raise KernelError(f"m is {tuple(m.shape)}, h is {tuple(h.shape)}")
    for v, name in ((post_w, "post_w"), (w, "w")):
        if v is not None:
            _need(v, name, torch.float32)
            if v.numel() != H:
                raise KernelError(f"{name} has {v.numel()} elements for rows of {H}")
    if y is not None:
        _need(y, "y")
        if y.shape[0] < n or y.shape[-1] != H:
            raise KernelError(f"y is {tuple(y.shape)} for {n} rows of {H}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _check(load().xs_add_layernorm(h.data_ptr(), _ptr(m), F32 if m is None else _code(m), _ptr(post_w), _ptr(w),
                                   _ptr(y), F32 if y is None else _code(y), _ptr(rows), n, H,
                                   float(eps if eps_post is None else eps_post), float(eps), _stream()))


def grouped_rmsnorm(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, groups: int, eps: float,
                    gate: Optional[torch.Tensor] = None, gate_act: str = "sigmoid") -> None:
    """y[t, g] = x[t, g] / sqrt(mean(x[t, g]^2) + eps) * w[g] for the `groups` equal parts g of a row; x float32.
    `gate` (y's element type, rows at least as wide as x's, contiguous columns): y is also multiplied by sigmoid(gate),
    or by silu(gate) with gate_act "silu"."""
    if gate_act not in ("sigmoid", "silu"):
        raise KernelError(f"grouped_rmsnorm: gate activation '{gate_act}' (sigmoid, silu)")
    _need(x, "x", torch.float32); _need(w, "w", torch.float32); _need(y, "y")
    if y.shape != x.shape or w.numel() != x.shape[1]:
        raise KernelError(f"grouped_rmsnorm: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if gate is not None and (gate.dtype != y.dtype or gate.stride(1) != 1 or gate.shape[0] != x.shape[0] or gate.shape[1] < x.shape[1]):
        raise KernelError(f"grouped_rmsnorm: gate {tuple(gate.shape)} {gate.dtype} for y {tuple(y.shape)} {y.dtype}")
    _check(load().xs_grouped_rmsnorm(x.data_ptr(), w.data_ptr(), y.data_ptr(), _code(y), x.shape[0], x.shape[1],
                                     int(groups), float(eps), _ptr(gate), 0 if gate is None else gate.stride(0),
                                     1 if gate_act == "silu" else 0, _stream()))


def clamped_glu(gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, shift: float, interleave: int = 0) -> None:
    """out = g * sigmoid(alpha g) * (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit); a row of gu is
    [gate | up], or with interleave 8 blocks of 8 gate and 8 up columns."""
    _need(out, "out", gu.dtype)
    if not gu.is_cuda or gu.dim() != 2 or gu.stride(1) != 1:
        raise KernelError("gate_up must be a CUDA matrix with contiguous rows")
    T, F = out.shape
    if gu.shape[0] != T or gu.shape[1] < 2 * F:
        raise KernelError(f"gate_up is {tuple(gu.shape)} for an output of {tuple(out.shape)}")
    _check(load().xs_clamped_glu(gu.data_ptr(), out.data_ptr(), _code(gu), T, F, gu.stride(0), float(limit), float(alpha),
                                 float(shift), int(interleave), _stream()))


def gemm_tc_clamped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, shift: float) -> None:
    """The tcgen05 product with the clamped gated unit in its epilogue: w [2 F, K] stacked in blocks of 8 gate and 8 up
    rows, out[T, F] = g * sigmoid(alpha g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    for t, name in ((x, "x"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.bfloat16:
            raise KernelError(f"gemm (tcgen05): {name} must be a bfloat16 CUDA matrix with contiguous rows")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (T, N // 2) or out.stride(1) != 1:
        raise KernelError(f"gemm (tcgen05): x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    mark_bounded(x.device)
    _check(load().xs_gemm_tc_clamped(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), T, N, K, x.stride(0), w.stride(0),
                                     out.stride(0), float(limit), float(alpha), float(shift), gemm_tc_status(x.device).data_ptr(),
                                     _stream()))


def gemm_tc_gelu(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """The tcgen05 product with the gated gelu in its epilogue: w [2 F, K] stacked in blocks of 8 gate and 8 up rows,
    out[T, F] = gelu_tanh(gate) * up."""
    for t, name in ((x, "x"), (w, "w")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != torch.bfloat16:
            raise KernelError(f"gemm (tcgen05): {name} must be a bfloat16 CUDA matrix with contiguous rows")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (T, N // 2) or out.stride(1) != 1:
        raise KernelError(f"gemm (tcgen05): x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    mark_bounded(x.device)
    _check(load().xs_gemm_tc_gelu(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), T, N, K, x.stride(0), w.stride(0),
                                  out.stride(0), gemm_tc_status(x.device).data_ptr(), _stream()))


# ------------------------------------------------------------------------------- routed experts
def moe_max_tiles(rows: int, experts: int) -> int:
    """The most row tiles that `rows` rows over `experts` experts can make (what the products' grids are sized by)."""
    return int(load().xs_moe_max_tiles(rows, experts))


def moe_logits(x: torch.Tensor, w: torch.Tensor, logits: torch.Tensor) -> None:
    """logits[t, e] = x[t] . w[e], float32 sums (not rounded) of the products of x's and w's element type."""
    _need(w, "router weight", x.dtype); _need(logits, "router logits", torch.float32)
    T, K = x.shape
    E = w.shape[0]
    if x.stride(1) != 1 or w.shape[1] != K or tuple(logits.shape) != (T, E):
        raise KernelError(f"moe_logits: x {tuple(x.shape)}, w {tuple(w.shape)}, logits {tuple(logits.shape)}")
    _check(load().xs_moe_logits(x.data_ptr(), x.stride(0), w.data_ptr(), logits.data_ptr(), T, E, K, _code(x), _stream()))


def moe_route(logits: torch.Tensor, top: int, ids: torch.Tensor, wts: torch.Tensor, experts: Optional[int] = None,
              scale: float = 1.0) -> None:
    """Per row of float32 logits: the `top` largest (ties: the lower index) into ids, their softmax times `scale` into
    wts. `experts`: only the first so many columns of a row are router logits (default: all)."""
    _need(logits, "router logits", torch.float32); _need(ids, "ids", torch.int32); _need(wts, "weights", torch.float32)
    T, ld = logits.shape
    E = ld if experts is None else int(experts)
    if ids.numel() < T * top or wts.numel() < T * top:
        raise KernelError(f"moe_route: {T} tokens x top {top} do not fit ids {ids.numel()} / weights {wts.numel()}")
    _check(load().xs_moe_route(logits.data_ptr(), ld, T, E, int(top), float(scale), ids.data_ptr(), wts.data_ptr(), _stream()))


def moe_route_grouped(logits: torch.Tensor, top: int, ids: torch.Tensor, wts: torch.Tensor, experts: Optional[int] = None,
                      correction: Optional[torch.Tensor] = None, groups: int = 1, keep: int = 1, group_top: int = 2,
                      scale: float = 1.0, renorm: bool = False, score: str = "sigmoid", real: Optional[int] = None) -> None:
    """Per row of float32 logits: scores s = sigmoid(logit), choice scores c = s + correction; the experts stand in
    `groups` equal groups of neighbours, of which the `keep` with the largest sum of their `group_top` largest choice
    scores stay open; the `top` open experts with the largest c (ties: the lower index) go into ids, their s (times
    `scale`; divided by their sum with `renorm`) into wts. `score` "softmax": s is the softmax over all `experts` logits
    instead. `real`: only the first so many experts have weights; a choice of a later one is written as id -1 (its input
    passes, times its weight)."""
    _need(logits, "router logits", torch.float32); _need(ids, "ids", torch.int32); _need(wts, "weights", torch.float32)
    if score not in ("sigmoid", "softmax"):
        raise KernelError(f"moe_route_grouped: score '{score}' (sigmoid, softmax)")
    T, ld = logits.shape
    E = ld if experts is None else int(experts)
    if correction is not None:
        _need(correction, "correction", torch.float32)
        if correction.numel() != E:
            raise KernelError(f"moe_route_grouped: a correction of {correction.numel()} entries for {E} experts")
    if ids.numel() < T * top or wts.numel() < T * top:
        raise KernelError(f"moe_route_grouped: {T} tokens x top {top} do not fit ids {ids.numel()} / weights {wts.numel()}")
    _check(load().xs_moe_route_grouped(logits.data_ptr(), ld, T, E, int(top), _ptr(correction), int(groups), int(keep),
                                       int(group_top), float(scale), 1 if renorm else 0, 1 if score == "softmax" else 0,
                                       E if real is None else int(real), ids.data_ptr(), wts.data_ptr(), _stream()))


def moe_max_tiles_of(rows: int, experts: int, tile_rows: int) -> int:
    """The same for tiles of `tile_rows` rows with every expert's rows padded to whole tiles."""
    return int(load().xs_moe_max_tiles_of(rows, experts, tile_rows))


def moe_plan(ids: torch.Tensor, experts: int, place: torch.Tensor, source: torch.Tensor, meta: torch.Tensor,
             tile_rows: int = 0) -> None:
    """Sorts the rows (token, choice) by expert: place[row] = its place in that order, source[place] = row, and meta =
    [tiles, -, -, -, (expert, first place, rows) per tile]. tile_rows > 0: tiles of that many rows and every expert's
    rows padded to whole tiles (source, which then has tile_rows * moe_max_tiles_of places, is -1 where no row stands)."""
    n = ids.numel()
    for t, name in ((ids, "ids"), (place, "place"), (source, "source"), (meta, "meta")):
        _need(t, name, torch.int32)
    tiles = moe_max_tiles_of(n, experts, tile_rows) if tile_rows else moe_max_tiles(n, experts)
    if place.numel() < n or source.numel() < (tiles * tile_rows if tile_rows else n) or meta.numel() < 4 + 3 * tiles:
        raise KernelError("moe_plan: an output is too small")
    _check(load().xs_moe_plan(ids.data_ptr(), n, int(experts), int(tile_rows), source.numel(), place.data_ptr(),
                              source.data_ptr(), meta.data_ptr(), _stream()))


def moe_gather(x: torch.Tensor, source: torch.Tensor, top: int, sorted_rows: torch.Tensor) -> None:
    """sorted_rows[r] = x[source[r] // top], zeros where source[r] < 0 (bfloat16 rows of a multiple of 8 elements)."""
    _need(sorted_rows, "sorted rows", torch.bfloat16); _need(source, "source", torch.int32)
    if x.dtype != torch.bfloat16 or x.stride(1) != 1 or sorted_rows.shape[1] != x.shape[1] or sorted_rows.shape[0] != source.numel():
        raise KernelError(f"moe_gather: x {tuple(x.shape)}, sorted {tuple(sorted_rows.shape)}, {source.numel()} places")
    _check(load().xs_moe_gather(x.data_ptr(), x.stride(0), source.data_ptr(), int(top), sorted_rows.data_ptr(),
                                sorted_rows.shape[0], x.shape[1], _stream()))


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, meta: torch.Tensor, max_tiles: int, glu: bool,
                    clamp=None, relu_squared: bool = False) -> None:
    """out[r] = w[expert of r's tile] . x[r] on tcgen05 tensor cores for the padded row tiles (128 rows) of a plan.
    w: [experts, N, K] bfloat16; with `glu` each expert's rows come in blocks of 8 gate and 8 up rows and
    out[r] = silu(gate) * up has N / 2 columns; `clamp` (limit, alpha, shift): the clamped unit's activation instead,
    g * sigmoid(alpha g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit). `relu_squared` (without
    `glu`): out[r] = max(product, 0)^2."""
    limit, alpha, shift = (0.0, 1.0, 0.0) if clamp is None else clamp
    if glu and relu_squared:
        raise KernelError("gemm (tcgen05, grouped): one activation at a time")
    _need(x, "x", torch.bfloat16); _need(w, "expert weights", torch.bfloat16); _need(out, "out", torch.bfloat16)
    E, N, K = w.shape
    if x.shape[1] != K or out.shape[0] != x.shape[0] or out.shape[1] != (N // 2 if glu else N) or x.shape[0] < 128 * max_tiles:
        raise KernelError(f"gemm (tcgen05, grouped): x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    mark_bounded(x.device)
    _check(load().xs_gemm_tc_grouped(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out),
                                     EPI_SWIGLU if glu else EPI_RELU_SQ if relu_squared else EPI_STORE,
                                     meta.data_ptr(), int(max_tiles), x.shape[0], E, N, K, x.stride(0), out.stride(0),
                                     float(limit), float(alpha), float(shift), gemm_tc_status(x.device).data_ptr(), _stream()))


def moe_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, meta: torch.Tensor, rows: int, source: Optional[torch.Tensor],
             top: int, glu: bool, clamp=None) -> None:
    """out[place] = w[expert of place] . x[source[place] // top] (x[place] without `source`) for the `rows` sorted
    places of a plan. w: [experts, N, K], or [experts, 2 N, K] with `glu` (gate rows first; out = silu(gate) * up, or
    with `clamp` (limit, alpha, shift) the clamped unit's activation)."""
    limit, alpha, shift = (0.0, 1.0, 0.0) if clamp is None else clamp
    for t, name in ((x, "x"), (out, "out")):
        if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"moe_gemm: {name} must be a CUDA matrix with contiguous rows")
    _need(w, "expert weights", x.dtype)
    E, N, K = w.shape
    if glu:
        N //= 2
    if x.shape[1] != K or out.shape[1] != N or out.shape[0] < rows or out.dtype != x.dtype:
        raise KernelError(f"moe_gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(load().xs_moe_gemm(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), _ptr(source), int(top),
                              meta.data_ptr(), moe_max_tiles(rows, E), N, K, 1 if glu else 0, float(limit), float(alpha), float(shift),
                              _code(x), _code(out), _stream()))


def moe_combine(rows_out: torch.Tensor, place: torch.Tensor, wts: torch.Tensor, y: torch.Tensor, top: int,
                shared: Optional[torch.Tensor] = None, shared_gate: Optional[torch.Tensor] = None,
                passed: Optional[torch.Tensor] = None) -> None:
    """y[t] = sum_k wts[t, k] * rows_out[place[t, k]], summed in float32 in the order of k. `shared` [T, H] (a unit that
    every token uses) starts the sum, times sigmoid(shared_gate[t, 0]) when `shared_gate` (float32, one row a token whose
    first column is the gate's logit) is given. `passed` [T, H] (the tokens' inputs): a choice whose place is -1 adds its
    weight times the token's input (an expert that hands its input through)."""
    _need(rows_out, "expert outputs", y.dtype); _need(y, "y")
    T, H = y.shape
    ld_gate = 0
    if passed is not None and (passed.dtype != y.dtype or passed.stride(1) != 1 or tuple(passed.shape) != (T, H)):
        raise KernelError(f"moe_combine: passed inputs {tuple(passed.shape)} {passed.dtype} for y {tuple(y.shape)}")
    if shared is not None:
        _need(shared, "shared unit's output", y.dtype)
        if tuple(shared.shape) != (T, H):
            raise KernelError(f"moe_combine: shared {tuple(shared.shape)} for y {tuple(y.shape)}")
        if shared_gate is not None:
            if shared_gate.dtype != torch.float32 or shared_gate.dim() != 2 or shared_gate.shape[0] != T or shared_gate.stride(1) != 1:
                raise KernelError(f"moe_combine: gate logits {tuple(shared_gate.shape)} {shared_gate.dtype} for {T} tokens")
            ld_gate = shared_gate.stride(0)
    _check(load().xs_moe_combine(rows_out.data_ptr(), place.data_ptr(), wts.data_ptr(), y.data_ptr(), T, H, int(top),
                                 _ptr(shared), _ptr(shared_gate) if shared is not None else None, ld_gate, _ptr(passed),
                                 0 if passed is None else passed.stride(0), _code(y), _stream()))


def relu_squared(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(x, 0)^2, elementwise."""
    _need(x, "x"); _need(out, "out", x.dtype)
    if out.shape != x.shape:
        raise KernelError(f"relu_squared: x {tuple(x.shape)}, out {tuple(out.shape)}")
    _check(load().xs_relu_squared(x.data_ptr(), out.data_ptr(), _code(x), x.numel(), _stream()))


def embed_pair(table: torch.Tensor, pair: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
               cu_seqlens: torch.Tensor, slots: torch.Tensor, last_token: torch.Tensor, inv_freq: torch.Tensor,
               norm_w: Optional[torch.Tensor], h: torch.Tensor, scale: float, buckets: int, mul_prev: int, mul_cur: int,
               eps: float) -> None:
    """h[t] = RMSNorm(table[tok] * scale + pair[bucket of (previous token, tok)] + sine/cosine of the position, norm_w)
    in float32 (no norm without norm_w). bucket = (prev * mul_prev + tok * mul_cur) mod buckets, and row `buckets` for a
    sequence's first token. `last_token` (int32, one word a slot) holds each sequence's last token between steps: it is
    read for a step's first token of a sequence and then takes the sequence's last token of this step.
    inv_freq: ceil(width / 2) float32 frequencies; entries 2i and 2i + 1 of a row get sin and cos of position * inv_freq[i]."""
    _need(table, "embedding table"); _need(pair, "pair table", table.dtype); _need(ids, "ids", torch.int32)
    _need(h, "h", torch.float32); _need(last_token, "last tokens", torch.int32); _need(inv_freq, "frequencies", torch.float32)
    T, H = h.shape
    if table.shape[1] != H or tuple(pair.shape) != (buckets + 1, H) or inv_freq.numel() < (H + 1) // 2:
        raise KernelError(f"embed_pair: table {tuple(table.shape)}, pair table {tuple(pair.shape)} for {buckets} buckets, width {H}")
    if norm_w is not None:
        _need(norm_w, "norm weight", torch.float32)
        if norm_w.numel() != H:
            raise KernelError(f"embed_pair: norm weight of {norm_w.numel()} for width {H}")
    _check(load().xs_embed_pair(table.data_ptr(), pair.data_ptr(), _code(table), ids.data_ptr(), positions.data_ptr(),
                                seq_of_token.data_ptr(), cu_seqlens.data_ptr(), slots.data_ptr(), last_token.data_ptr(),
                                inv_freq.data_ptr(), _ptr(norm_w), h.data_ptr(), T, H, float(scale), int(buckets),
                                int(mul_prev), int(mul_cur), float(eps), _stream()))


def mlstm_copies(vdim: int) -> int:
    """How many copies of a head's n and m the recurrence kernel keeps (one per block of value columns)."""
    return int(load().xs_mlstm_copies(int(vdim)))


def mlstm_scan(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, gates: torch.Tensor, i_bias: torch.Tensor,
               f_bias: torch.Tensor, s_state: torch.Tensor, nm_state: torch.Tensor, cu_seqlens: torch.Tensor,
               slots: torch.Tensor, y: torch.Tensor, heads: int, dim: int, vdim: int, cap: float, q_scale: float,
               chunks=None) -> None:
    """The mLSTM recurrence over a step's tokens, sequence by sequence from each slot's state (csrc/mlstm.cu). qkv: rows
    with q [heads * dim] at column q_col, k at k_col, v [heads * vdim] at v_col; gates: float32 rows [input gates' |
    forget gates'] pre-activations without biases; s_state [slots, heads, dim, vdim], nm_state [slots, heads,
    mlstm_copies(vdim), dim + 1] float32; y [T, heads * vdim] float32. `chunks` (chunk list [n, 3] int32: sequence, first
    token, tokens; first chunk of each sequence [sequences + 1] int32; scratch [n, heads, dim, vdim] and [n, heads,
    mlstm_copies(vdim), dim + 2] float32): the chunks run side by side in two passes with a carry between them."""
    _need(gates, "gates", torch.float32); _need(y, "y", torch.float32); _need(s_state, "state", torch.float32)
    _need(nm_state, "normaliser state", torch.float32); _need(i_bias, "input gate bias", torch.float32)
    _need(f_bias, "forget gate bias", torch.float32)
    if not qkv.is_cuda or qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("mlstm: qkv must be a CUDA matrix with contiguous rows")
    T = qkv.shape[0]
    if (max(q_col, k_col) + heads * dim > qkv.shape[1] or v_col + heads * vdim > qkv.shape[1] or gates.shape[0] != T
            or gates.shape[1] < 2 * heads or tuple(y.shape) != (T, heads * vdim)):
        raise KernelError(f"mlstm: qkv {tuple(qkv.shape)}, gates {tuple(gates.shape)}, y {tuple(y.shape)} for {heads} heads of {dim} / {vdim}")
    if tuple(s_state.shape[1:]) != (heads, dim, vdim) or tuple(nm_state.shape[1:]) != (heads, mlstm_copies(vdim), dim + 1):
        raise KernelError(f"mlstm: state {tuple(s_state.shape)} / {tuple(nm_state.shape)} for {heads} heads of {dim} / {vdim}")
    if i_bias.numel() != heads or f_bias.numel() != heads:
        raise KernelError(f"mlstm: gate biases of {i_bias.numel()} / {f_bias.numel()} for {heads} heads")
    chunk_args = (None, None, 0, None, None)
    if chunks is not None:
        chunk_seq, first_chunk, s_chunk, nm_chunk = chunks
        n = chunk_seq.shape[0]
        _need(chunk_seq, "chunk list", torch.int32); _need(first_chunk, "first chunks", torch.int32)
        _need(s_chunk, "chunk states", torch.float32); _need(nm_chunk, "chunk normalisers", torch.float32)
        if (tuple(s_chunk.shape) != (n, heads, dim, vdim) or tuple(nm_chunk.shape) != (n, heads, mlstm_copies(vdim), dim + 2)
                or first_chunk.numel() != cu_seqlens.numel()):
            raise KernelError(f"mlstm: chunk scratch {tuple(s_chunk.shape)} / {tuple(nm_chunk.shape)} for {n} chunks")
        chunk_args = (chunk_seq.data_ptr(), first_chunk.data_ptr(), n, s_chunk.data_ptr(), nm_chunk.data_ptr())
    _check(load().xs_mlstm_scan(qkv.data_ptr(), qkv.stride(0), int(q_col), int(k_col), int(v_col), gates.data_ptr(),
                                gates.stride(0), i_bias.data_ptr(), f_bias.data_ptr(), s_state.data_ptr(), nm_state.data_ptr(),
                                cu_seqlens.data_ptr(), slots.data_ptr(), y.data_ptr(), cu_seqlens.numel() - 1, heads, dim, vdim,
                                float(cap), float(q_scale), _code(qkv), *chunk_args, _stream()),
           kernels=3 if chunks is not None else 1)


# ----------------------------------------------------------------------------- latent attention
def latent_prepare(down: torch.Tensor, q: torch.Tensor, norm_w: torch.Tensor, table: Optional[torch.Tensor],
                   positions: torch.Tensor, seq_of_token: torch.Tensor, page_table: torch.Tensor, pool: torch.Tensor,
                   q_rot: torch.Tensor, heads: int, dim: int, rot_dim: int, rank: int, dims: int, page_size: int,
                   eps: float, write_kv: bool = True) -> None:
    """From the down-projection [T, rank + rot_dim] and the queries [T, heads * (dim + rot_dim)]: the cache row
    [unit-RMS(down[:rank]) * norm_w | rotated down[rank:]] at each token's position, and every head's rotated query part
    into q_rot [T, heads, rot_dim]. table: [positions, dims / 2, 2] (cos, sin)."""
    _need(q_rot, "q_rot", q.dtype); _need(pool, "cache", q.dtype); _need(norm_w, "latent norm weight", torch.float32)
    _need(page_table, "page table", torch.int32)
    T = q.shape[0]
    if down.stride(1) != 1 or q.stride(1) != 1 or down.shape[1] < rank + rot_dim or q.shape[1] < heads * (dim + rot_dim):
        raise KernelError(f"latent_prepare: down {tuple(down.shape)}, q {tuple(q.shape)}")
    if tuple(pool.shape[1:]) != (1, 1, page_size, rank + rot_dim):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 1, 1, {page_size}, {rank + rot_dim}]")
    if table is not None:
        _need(table, "rotation table", torch.float32)
        if tuple(table.shape[1:]) != (dims // 2, 2):
            raise KernelError(f"rotation table is {tuple(table.shape)}, expected [*, {dims // 2}, 2]")
    _check(load().xs_latent_prepare(down.data_ptr(), down.stride(0), q.data_ptr(), q.stride(0), norm_w.data_ptr(),
                                    _ptr(table), positions.data_ptr(), seq_of_token.data_ptr(), page_table.data_ptr(),
                                    page_table.shape[1], pool.data_ptr(), q_rot.data_ptr(), T, heads, dim, rot_dim, rank,
                                    dims if table is not None else 0, page_size, float(eps), 1 if write_kv else 0, _code(q),
                                    _stream()))


def latent_attention_generic(q_lat: torch.Tensor, q_rot: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor,
                             seq_of_token: torch.Tensor, positions: torch.Tensor, gate: Optional[torch.Tensor],
                             sink: Optional[torch.Tensor], out: torch.Tensor, page_size: int, scale: float,
                             window: int) -> None:
    """q_lat, out: [T, heads, rank] views (any token and head strides, contiguous channels); q_rot [T, heads, rot_dim]."""
    T, H, R = q_lat.shape
    Dr = q_rot.shape[2]
    _need(q_rot, "q_rot", q_lat.dtype); _need(pool, "cache", q_lat.dtype); _need(page_table, "page table", torch.int32)
    if q_lat.stride(2) != 1 or out.stride(2) != 1 or tuple(out.shape) != (T, H, R) or out.dtype != q_lat.dtype:
        raise KernelError(f"latent attention: q {tuple(q_lat.shape)}, out {tuple(out.shape)}")
    if tuple(pool.shape[1:]) != (1, 1, page_size, R + Dr):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 1, 1, {page_size}, {R + Dr}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != q_lat.dtype or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < H:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {H} heads")
        ld_gate = gate.stride(0)
    if sink is not None:
        _need(sink, "sink", torch.float32)
    _check(load().xs_latent_attention_generic(
        q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_rot.data_ptr(), pool.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], seq_of_token.data_ptr(), positions.data_ptr(), _ptr(gate), ld_gate, _ptr(sink), out.data_ptr(),
        out.stride(0), out.stride(1), T, H, R, Dr, page_size, float(scale), int(window), _code(q_lat), _stream()))


def latent_attention_mma_supports(rank: int, rot_dim: int, page_size: int) -> bool:
    return bool(load().xs_latent_attention_mma_supports(rank, rot_dim, page_size))


def latent_attention_mma_ctas_per_sm(max_q_len: int, heads: int, rank: int, rot_dim: int) -> int:
    """CTAs of the kernel that share an SM for steps of at most `max_q_len` tokens a sequence (the tile of single tokens
    with few heads is smaller)."""
    return int(load().xs_latent_attention_mma_ctas_per_sm(max_q_len, heads, rank, rot_dim))


def latent_attention_mma_scratch_bytes(rows: int, rank: int, splits: int) -> int:
    return int(load().xs_latent_attention_mma_scratch_bytes(rows, rank, splits))


def latent_attention_mma(q_lat: torch.Tensor, q_rot: torch.Tensor, pool: torch.Tensor, page_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, kv_lens: torch.Tensor, gate: Optional[torch.Tensor],
                         sink: Optional[torch.Tensor], out: torch.Tensor, scratch: Optional[torch.Tensor], n_seqs: int,
                         max_q_len: int, page_size: int, scale: float, window: int, splits: int) -> None:
    """Latent attention on tensor cores over the bfloat16 cache. q_lat, out: [T, heads, rank] views; q_rot [T, heads,
    rot_dim]. With splits > 1 every sequence's key pages are cut over that many CTAs and `scratch` (bytes, at least
    latent_attention_mma_scratch_bytes(T * heads, rank, splits)) takes their partial results."""
    T, H, R = q_lat.shape
    Dr = q_rot.shape[2]
    _need(q_rot, "q_rot", torch.bfloat16); _need(pool, "cache", torch.bfloat16); _need(page_table, "page table", torch.int32)
    if q_lat.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or q_lat.stride(2) != 1 or out.stride(2) != 1 or tuple(out.shape) != (T, H, R):
        raise KernelError(f"latent attention (mma): q {tuple(q_lat.shape)} {q_lat.dtype}, out {tuple(out.shape)} {out.dtype}")
    if tuple(pool.shape[1:]) != (1, 1, page_size, R + Dr):
        raise KernelError(f"cache is {tuple(pool.shape)}, expected [*, 1, 1, {page_size}, {R + Dr}]")
    ld_gate = 0
    if gate is not None:
        if gate.dtype != torch.bfloat16 or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < H:
            raise KernelError(f"gate is {tuple(gate.shape)} {gate.dtype} for {T} tokens of {H} heads")
        ld_gate = gate.stride(0)
    if sink is not None:
        _need(sink, "sink", torch.float32)
    _check(load().xs_latent_attention_mma(
        q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_rot.data_ptr(), pool.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], cu_seqlens.data_ptr(), kv_lens.data_ptr(), _ptr(gate), ld_gate, _ptr(sink), out.data_ptr(),
        out.stride(0), out.stride(1), _ptr(scratch), 0 if scratch is None else scratch.numel() * scratch.element_size(),
        T, n_seqs, max_q_len, H, R, Dr, page_size, float(scale), int(window), int(splits), _stream()),
        kernels=2 if splits > 1 else 1)


def gemm_batched(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = x[b] . w[b]^T for [batch, M, K], [batch, N, K] and [batch, M, N] views with contiguous last dimensions
    and any row and batch strides."""
    B, M, K = x.shape
    N = w.shape[1]
    if w.shape != (B, N, K) or out.shape != (B, M, N) or x.dtype != w.dtype or out.dtype != x.dtype:
        raise KernelError(f"gemm_batched: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    for t in (x, w, out):
        if not t.is_cuda or t.stride(2) != 1:
            raise KernelError("gemm_batched: operands must be CUDA tensors with contiguous last dimensions")
    _check(load().xs_gemm_batched(x.data_ptr(), x.stride(1), x.stride(0), w.data_ptr(), w.stride(1), w.stride(0),
                                  out.data_ptr(), out.stride(1), out.stride(0), B, M, N, K, _code(x), _stream()))


# -------------------------------------------------------------------------------------- mamba-2
def mamba2_conv(proj: torch.Tensor, col0: int, taps_w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(causal depthwise conv of proj[:, col0:col0 + C] + bias), inputs before the step from `state`
    [*, taps - 1, C], which is then moved on. taps_w: [C, taps], the last column the current token's."""
    _need(out, "out", proj.dtype); _need(state, "state", proj.dtype); _need(taps_w, "taps", torch.float32)
    T, C = out.shape
    taps = taps_w.shape[1]
    if proj.stride(1) != 1 or proj.shape[0] != T or proj.shape[1] < col0 + C or taps_w.shape[0] != C:
        raise KernelError(f"mamba2_conv: proj {tuple(proj.shape)}, taps {tuple(taps_w.shape)}, out {tuple(out.shape)}")
    if taps > 1 and tuple(state.shape[1:]) != (taps - 1, C):
        raise KernelError(f"mamba2_conv: state is {tuple(state.shape)}, expected [*, {taps - 1}, {C}]")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    _check(load().xs_mamba2_conv(proj.data_ptr(), proj.stride(0), int(col0), taps_w.data_ptr(), _ptr(bias), state.data_ptr(),
                                 seq_of_token.data_ptr(), cu_seqlens.data_ptr(), slots.data_ptr(), out.data_ptr(), T,
                                 slots.numel(), C, taps, _code(proj), _stream()), kernels=2 if taps > 1 else 1)


def mamba2_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
                d_skip: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, y: torch.Tensor,
                heads: int, vdim: int, n_state: int, groups: int, chunks=None) -> None:
    """The recurrence over a step's tokens; y [T, heads * vdim] float32 takes y_t * silu(z_t). state: [*, heads,
    n_state, vdim] float32. `chunks` = (chunk_seq [n, 3] int32, first_chunk [n_seqs + 1] int32, chunk_state, chunk_decay)
    runs long pieces chunk by chunk side by side."""
    _need(xbc, "xbc", proj.dtype); _need(state, "state", torch.float32); _need(y, "y", torch.float32)
    for t, name in ((dt_bias, "dt_bias"), (a_log, "A_log"), (d_skip, "D")):
        _need(t, name, torch.float32)
        if t.numel() != heads:
            raise KernelError(f"mamba2_scan: {name} has {t.numel()} entries for {heads} heads")
    if tuple(state.shape[1:]) != (heads, n_state, vdim):
        raise KernelError(f"mamba2_scan: state is {tuple(state.shape)}, expected [*, {heads}, {n_state}, {vdim}]")
    if xbc.shape[1] != heads * vdim + 2 * groups * n_state or proj.stride(1) != 1 or proj.shape[1] < dt_col + heads:
        raise KernelError(f"mamba2_scan: xbc {tuple(xbc.shape)}, proj {tuple(proj.shape)}")
    n_seqs = slots.numel()
    if chunks is None:
        _check(load().xs_mamba2_scan(xbc.data_ptr(), proj.data_ptr(), proj.stride(0), int(dt_col), dt_bias.data_ptr(),
                                     a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu_seqlens.data_ptr(),
                                     slots.data_ptr(), y.data_ptr(), n_seqs, heads, vdim, n_state, groups, _code(proj),
                                     _stream()))
        return
    chunk_seq, first_chunk, chunk_state, chunk_decay = chunks
    _need(chunk_seq, "chunk_seq", torch.int32); _need(first_chunk, "first_chunk", torch.int32)
    _need(chunk_state, "chunk_state", torch.float32); _need(chunk_decay, "chunk_decay", torch.float32)
    n = chunk_seq.shape[0]
    if chunk_state.numel() < n * heads * n_state * vdim or chunk_decay.numel() < n * heads:
        raise KernelError("mamba2_scan: the chunks' scratch is too small")
    _check(load().xs_mamba2_scan_chunked(xbc.data_ptr(), proj.data_ptr(), proj.stride(0), int(dt_col), dt_bias.data_ptr(),
                                         a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu_seqlens.data_ptr(),
                                         slots.data_ptr(), y.data_ptr(), chunk_state.data_ptr(), chunk_decay.data_ptr(),
                                         chunk_seq.data_ptr(), first_chunk.data_ptr(), n, n_seqs, heads, vdim, n_state,
                                         groups, _code(proj), _stream()), kernels=3)


# ------------------------------------------------------------------------- a layer's frame
def embed_pos(table: torch.Tensor, rows: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, h: torch.Tensor,
              scale: float = 1.0) -> None:
    """h[t] = table[ids[t]] * scale + rows[positions[t]], float32."""
    _need(table, "embedding table"); _need(rows, "position rows", table.dtype); _need(ids, "ids", torch.int32)
    _need(positions, "positions", torch.int32); _need(h, "h", torch.float32)
    T, H = h.shape
    if table.shape[1] != H or rows.shape[1] != H:
        raise KernelError(f"embed_pos: table {tuple(table.shape)}, rows {tuple(rows.shape)}, h {tuple(h.shape)}")
    _check(load().xs_embed_pos(table.data_ptr(), rows.data_ptr(), _code(table), ids.data_ptr(), positions.data_ptr(),
                               h.data_ptr(), T, H, float(scale), _stream()))


def side_gate(x: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, offset: int) -> None:
    """x[t, j] = gelu_tanh(x[t, j]) * table[ids[t], offset + j], in place; x [T, d] (contiguous columns) and table
    [vocab, *] of one element type."""
    _need(ids, "ids", torch.int32); _need(table, "side table", x.dtype)
    T, d = x.shape
    if not x.is_cuda or x.stride(1) != 1 or table.dim() != 2 or table.stride(1) != 1 or offset < 0 or offset + d > table.shape[1] \
            or ids.numel() < T:
        raise KernelError(f"side_gate: x {tuple(x.shape)}, columns {offset} + {d} of a table {tuple(table.shape)}")
    _check(load().xs_side_gate(x.data_ptr(), x.stride(0), ids.data_ptr(), table.data_ptr(), table.stride(0), int(offset), T, d,
                               _code(x), _stream()))


def rmsnorm_rows(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, eps: float) -> None:
    """y[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w for views x, y [T, n] (any row strides, contiguous columns) of one element
    type; the sum and the scale in float32."""
    _need(w, "w", torch.float32)
    T, n = x.shape
    if not x.is_cuda or x.stride(1) != 1 or y.stride(1) != 1 or tuple(y.shape) != (T, n) or y.dtype != x.dtype or w.numel() != n:
        raise KernelError(f"rmsnorm_rows: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    _check(load().xs_rmsnorm_rows(x.data_ptr(), x.stride(0), w.data_ptr(), y.data_ptr(), y.stride(0), T, n, float(eps), _code(x), _stream()))


def sigmoid_mul(o: torch.Tensor, g: torch.Tensor) -> None:
    """o *= sigmoid(g), elementwise over views [T, n] (any row strides, contiguous columns) of one element type."""
    T, n = o.shape
    if not o.is_cuda or o.stride(1) != 1 or g.stride(1) != 1 or tuple(g.shape) != (T, n) or g.dtype != o.dtype:
        raise KernelError(f"sigmoid_mul: o {tuple(o.shape)} {o.dtype}, g {tuple(g.shape)} {g.dtype}")
    _check(load().xs_sigmoid_mul(o.data_ptr(), o.stride(0), g.data_ptr(), g.stride(0), T, n, _code(o), _stream()))


def cast_rows(src: torch.Tensor, dst: torch.Tensor) -> None:
    """dst = src for views [T, n] (any row strides, contiguous columns): float32 into dst's element type."""
    _need(src, "src", torch.float32)
    T, n = src.shape
    if src.dim() != 2 or src.stride(1) != 1 or dst.stride(1) != 1 or tuple(dst.shape) != (T, n):
        raise KernelError(f"cast_rows: src {tuple(src.shape)}, dst {tuple(dst.shape)}")
    _check(load().xs_cast_rows(src.data_ptr(), src.stride(0), dst.data_ptr(), dst.stride(0), T, n, _code(dst), _stream()))


def lightning_scan(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor,
                   cu_seqlens: torch.Tensor, slots: torch.Tensor, y: torch.Tensor, heads: int, dim: int, vdim: int,
                   chunks=None) -> None:
    """The decayed linear recurrence S <- decay_h S + k v^T, o = S^T q over a step's tokens, sequence by sequence from each
    slot's state (csrc/lightning.cu); q, k, v are silu of qkv's columns from q_col (heads * dim), k_col (heads * dim) and
    v_col (heads * vdim) on. decay [heads] float32; state [slots, heads, dim, vdim] float32; y [T, heads * vdim] float32.
    `chunks` (chunk list [n, 3] int32: sequence, first token, tokens; first chunk of each sequence [sequences + 1] int32;
    scratch [n, heads, dim, vdim] float32): the chunks run side by side in two passes with a carry between them."""
    _need(decay, "decay", torch.float32); _need(state, "state", torch.float32); _need(y, "y", torch.float32)
    if not qkv.is_cuda or qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("lightning: qkv must be a CUDA matrix with contiguous rows")
    T = qkv.shape[0]
    if (max(q_col, k_col) + heads * dim > qkv.shape[1] or v_col + heads * vdim > qkv.shape[1] or tuple(y.shape) != (T, heads * vdim)
            or decay.numel() != heads or tuple(state.shape[1:]) != (heads, dim, vdim)):
        raise KernelError(f"lightning: qkv {tuple(qkv.shape)}, y {tuple(y.shape)}, state {tuple(state.shape)} for {heads} heads of {dim} x {vdim}")
    chunk_args = (None, None, 0, None)
    if chunks is not None:
        chunk_seq, first_chunk, chunk_state = chunks
        n = chunk_seq.shape[0]
        _need(chunk_seq, "chunk list", torch.int32); _need(first_chunk, "first chunks", torch.int32)
        _need(chunk_state, "chunk states", torch.float32)
        if tuple(chunk_state.shape) != (n, heads, dim, vdim) or first_chunk.numel() != cu_seqlens.numel():
            raise KernelError(f"lightning: chunk scratch {tuple(chunk_state.shape)} for {n} chunks")
        chunk_args = (chunk_seq.data_ptr(), first_chunk.data_ptr(), n, chunk_state.data_ptr())
    _check(load().xs_lightning_scan(qkv.data_ptr(), qkv.stride(0), int(q_col), int(k_col), int(v_col), decay.data_ptr(),
                                    state.data_ptr(), cu_seqlens.data_ptr(), slots.data_ptr(), y.data_ptr(), cu_seqlens.numel() - 1,
                                    int(heads), int(dim), int(vdim), _code(qkv), *chunk_args, _stream()),
           kernels=3 if chunks is not None else 1)


def causal_conv(x: torch.Tensor, taps_w: torch.Tensor, state: torch.Tensor, seq_of_token: torch.Tensor,
                cu_seqlens: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, act: str = "none",
                residual: bool = False, all_single: bool = False) -> None:
    """out[t, c] = (x[t, c] with `residual`) + act(sum_j taps_w[c, j] * x[t - (n - 1) + j, c]) within each sequence, the
    inputs before the step from `state` [*, n - 1, C] (x's element type), which is then moved on. act: "none" | "silu".
    `all_single`: every sequence brings exactly one token (the one kernel then also moves the state)."""
    if act not in ("none", "silu"):
        raise KernelError(f"causal_conv: activation '{act}' (none, silu)")
    _need(taps_w, "taps", torch.float32); _need(state, "state", x.dtype)
    T, C = out.shape
    taps = taps_w.shape[1]
    if (x.dim() != 2 or x.stride(1) != 1 or out.stride(1) != 1 or out.dtype != x.dtype or x.shape[0] != T or x.shape[1] < C
            or taps_w.shape[0] != C):
        raise KernelError(f"causal_conv: x {tuple(x.shape)}, taps {tuple(taps_w.shape)}, out {tuple(out.shape)}")
    if taps > 1 and tuple(state.shape[1:]) != (taps - 1, C):
        raise KernelError(f"causal_conv: state is {tuple(state.shape)}, expected [*, {taps - 1}, {C}]")
    _check(load().xs_causal_conv(x.data_ptr(), x.stride(0), taps_w.data_ptr(), state.data_ptr(), seq_of_token.data_ptr(),
                                 cu_seqlens.data_ptr(), slots.data_ptr(), out.data_ptr(), out.stride(0), T, slots.numel(), C,
                                 taps, 1 if act == "silu" else 0, 1 if residual else 0, 1 if all_single else 0, _code(x), _stream()),
           kernels=2 if taps > 1 and not all_single else 1)


def gated_add(h: torch.Tensor, branch: torch.Tensor, logits: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """h += branch * sigmoid(logits + bias): h float32 [T, W]; logits float32 rows at least W wide."""
    _need(h, "h", torch.float32); _need(branch, "branch")
    T, W = h.shape
    if tuple(branch.shape) != (T, W) or logits.dtype != torch.float32 or logits.shape[0] != T or logits.shape[1] < W or logits.stride(1) != 1:
        raise KernelError(f"gated_add: h {tuple(h.shape)}, branch {tuple(branch.shape)}, gate {tuple(logits.shape)} {logits.dtype}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != W:
            raise KernelError(f"gated_add: a bias of {bias.numel()} entries for rows of {W}")
    _check(load().xs_gated_add(h.data_ptr(), branch.data_ptr(), _code(branch), logits.data_ptr(), logits.stride(0), _ptr(bias),
                               T, W, _stream()))


def depth_average(history: torch.Tensor, coef: torch.Tensor, terms: int, out: torch.Tensor) -> None:
    """out = sum over j < terms of coef[j] * history[j]; history [n, T, W] float32, out [T, W] float32 (it may be a later
    plane of `history`)."""
    _need(history, "history", torch.float32); _need(coef, "coefficients", torch.float32); _need(out, "out", torch.float32)
    if history.dim() != 3 or history.shape[0] < terms or coef.numel() != terms or out.shape != history.shape[1:]:
        raise KernelError(f"depth_average: history {tuple(history.shape)}, {coef.numel()} coefficients for {terms} terms, "
                          f"out {tuple(out.shape)}")
    _check(load().xs_depth_average(history.data_ptr(), history.stride(0), coef.data_ptr(), int(terms), out.data_ptr(),
                                   out.numel(), _stream()))


def rmsnorm_accumulate(x: torch.Tensor, w: torch.Tensor, acc: torch.Tensor, eps: float, scale: float, add: bool) -> None:
    """acc = (acc if add else 0) + scale * x / sqrt(mean(x^2) + eps) * w, row by row, float32."""
    _need(x, "x"); _need(w, "w", torch.float32); _need(acc, "acc", torch.float32)
    T, W = x.shape
    if tuple(acc.shape) != (T, W) or w.numel() != W:
        raise KernelError(f"rmsnorm_accumulate: x {tuple(x.shape)}, w {tuple(w.shape)}, acc {tuple(acc.shape)}")
    _check(load().xs_rmsnorm_accumulate(x.data_ptr(), _code(x), w.data_ptr(), acc.data_ptr(), T, W, float(eps), float(scale),
                                        1 if add else 0, _stream()))


def gated_delta_scan(qkv: torch.Tensor, q_col: int, k_col: int, v_col: int, ab: torch.Tensor, a_log: torch.Tensor,
                     dt_bias: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, y: torch.Tensor,
                     heads: int, key_heads: int, dim: int, vdim: int, q_scale: float, unit_eps: float) -> None:
    """The gated delta rule over a step's tokens (csrc/gated_delta.cu). qkv: rows with q (key_heads * dim), k (likewise) and
    v (heads * vdim) from the given columns on; ab float32 rows [a: heads | b: heads | ...]; state [*, heads, dim, vdim]
    float32; y [T, heads * vdim] float32."""
    _need(ab, "gate inputs", torch.float32); _need(state, "state", torch.float32); _need(y, "y", torch.float32)
    _need(a_log, "A_log", torch.float32); _need(dt_bias, "dt_bias", torch.float32)
    T = y.shape[0]
    if (qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[0] != T or ab.shape[0] != T or ab.shape[1] < 2 * heads
            or y.shape[1] != heads * vdim or a_log.numel() != heads or dt_bias.numel() != heads
            or max(q_col, k_col) + key_heads * dim > qkv.shape[1] or v_col + heads * vdim > qkv.shape[1]):
        raise KernelError(f"gated_delta_scan: qkv {tuple(qkv.shape)}, gates {tuple(ab.shape)}, y {tuple(y.shape)}")
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"gated_delta_scan: state is {tuple(state.shape)}, expected [*, {heads}, {dim}, {vdim}]")
    _check(load().xs_gated_delta_scan(qkv.data_ptr(), qkv.stride(0), int(q_col), int(k_col), int(v_col), ab.data_ptr(),
                                      ab.stride(0), a_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(),
                                      cu_seqlens.data_ptr(), slots.data_ptr(), y.data_ptr(), slots.numel(), int(heads),
                                      int(key_heads), int(dim), int(vdim), float(q_scale), float(unit_eps), int(T), _code(qkv), _stream()))
