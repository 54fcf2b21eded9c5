"""Tensor-level entry points of the hand-written kernels.

Each function checks shapes, dtypes and layout on the host, then calls the C
launcher of the compiled library on the current CUDA stream.  A size that a
kernel does not take is refused here with a `KernelError` that says why; there
is no other route for the same work (no library attention, no CPU path).
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import build

PAGE_TOKENS = 64

_P, _I, _L, _F, _U, _D = c_void_p, c_int, c_longlong, c_float, c_ulonglong, c_double

# library, symbol -> argument types (the stream is always last)
_SIGNATURES = {
    "gtg_embed": ("elementwise", [_I, _P, _P, _P, _I, _I, _I, _F, _P]),
    "gtg_add_rmsnorm": ("elementwise", [_I, _P, _P, _P, _F, _P, _P, _I, _I, _P]),
    "gtg_swiglu": ("elementwise", [_I, _P, _P, _I, _I, _I, _P]),
    "gtg_rmsnorm_rows": ("elementwise", [_P, _P, _F, _I, _I, _P]),
    "gtg_scale": ("elementwise", [_P, _L, _F, _P]),
    "gtg_rope_table": ("elementwise", [_P, _P, _P, _I, _I, _D, _P]),
    "gtg_rope_kv_store": ("elementwise", [_I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P, _L, _P, _I, _P, _P, _P, _I, _P]),
    "gtg_add_layernorm": ("elementwise", [_I, _P, _P, _P, _P, _F, _P, _P, _I, _I, _P]),
    "gtg_activation": ("elementwise", [_I, _P, _I, _I, _I, _I, _P]),
    "gtg_softcap": ("elementwise", [_P, _L, _F, _P]),
    "gtg_hidden_concat": ("elementwise", [_I, _P, _P, _P, _P, _I, _I, _P]),
    "gtg_causal_conv_silu": ("ssm", [_I, _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "gtg_conv_state_update": ("ssm", [_I, _P, _I, _P, _P, _P, _I, _I, _I, _P]),
    "gtg_ssm_scan": ("ssm", [_I, _P, _I, _P, _I, _P, _I, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_causal_conv_step": ("ssm", [_I, _P, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _P]),
    "gtg_gated_rmsnorm": ("ssm", [_I, _P, _I, _P, _I, _P, _F, _P, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_simt": ("gemm_f32", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P]),
    "gtg_advance": ("elementwise", [_P, _P, _P, _P, _I, _P]),
    "gtg_check_cache_access": ("elementwise", [_I, _I, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _P, _P]),
    "gtg_gemm_f32": ("gemm_f32", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_mma": ("gemm_bf16_mma", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_skinny": ("gemm_bf16_skinny", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_skinny_status": ("gemm_bf16_skinny", []),
    "gtg_gemm_bf16_skinny_test_hooks": ("gemm_bf16_skinny", [_I]),
    "gtg_gemm_bf16_tcgen05_test_hooks": ("gemm_bf16_tcgen05", [_I]),
    "gtg_gemm_bf16_swapab_test_hooks": ("gemm_bf16_swapab", [_I]),
    "gtg_attention_tcgen05_test_hooks": ("attention_tcgen05", [_I]),
    "gtg_gemm_bf16_tcgen05": ("gemm_bf16_tcgen05", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_tcgen05_add": ("gemm_bf16_tcgen05", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_tcgen05_status": ("gemm_bf16_tcgen05", []),
    "gtg_gemm_bf16_tcgen05_qkv_rope": ("gemm_bf16_tcgen05", [_P, _I, _P, _I, _P, _I, _I, _I, _P, _P, _P, _P, _P, _I,
                                                             _P, _P, _L, _I, _I, _P]),
    "gtg_gemm_bf16_swapab": ("gemm_bf16_swapab", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P]),
    "gtg_gemm_bf16_swapab_scratch_floats": ("gemm_bf16_swapab", [_I, _I, _I]),
    "gtg_gemm_bf16_swapab_status": ("gemm_bf16_swapab", []),
    "gtg_attention_simple": ("attention_simple", [_I, _P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P, _P,
                                                  _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _I, _F, _P, _P]),
    "gtg_qkv_conv_finish": ("attention_prep", [_I, _P, _I, _P, _P, _I, _P, _P, _P, _P, _F, _P, _I, _I, _P, _I, _P, _P, _L, _P, _I,
                                               _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_delta_prepare": ("delta", [_P, _I, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _F, _F, _P]),
    "gtg_delta_scan_supports": ("delta", [_I, _I]),
    "gtg_delta_scan": ("delta", [_P, _I, _P, _I, _P, _I, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_head_norm_gate": ("delta", [_I, _P, _I, _P, _I, _P, _F, _P, _I, _I, _I, _I, _P]),
    "gtg_rmsnorm_add": ("elementwise", [_I, _I, _P, _P, _P, _F, _P, _P, _I, _I, _P]),
    "gtg_round_rows": ("elementwise", [_I, _P, _P, _L, _P]),
    "gtg_swiglu_bias": ("elementwise", [_I, _P, _P, _P, _P, _I, _I, _I, _P]),
    "gtg_add_bias": ("elementwise", [_I, _P, _P, _P, _I, _I, _P]),
    "gtg_sigmoid_gate": ("elementwise", [_I, _P, _I, _P, _I, _I, _I, _I, _P]),
    "gtg_gemm_simt_batched": ("gemm_f32", [_I, _P, _I, _L, _P, _I, _L, _P, _I, _L, _I, _I, _I, _I, _P]),
    "gtg_gemm_bf16_grouped": ("gemm_bf16_grouped", [_P, _I, _L, _P, _I, _P, _I, _L, _P, _P, _I, _L, _I, _I, _I, _I, _I, _I,
                                                    _I, _P, _I, _L, _P]),
    "gtg_latent_prepare": ("latent", [_I, _P, _I, _P, _I, _P, _P, _F, _P, _L, _P, _I, _P, _P, _P, _P, _I,
                                      _I, _I, _I, _I, _I, _I, _P, _I, _I, _P]),
    "gtg_expanded_attention_supports": ("latent", [_I, _I, _I]),
    "gtg_expanded_attention_bf16": ("latent", [_P, _I, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P]),
    "gtg_latent_spread": ("latent", [_P, _I, _P, _I, _I, _I, _I, _I, _I, _P]),
    "gtg_latent_attention_supports": ("latent", [_I, _I]),
    "gtg_latent_status": ("latent", []),
    "gtg_latent_test_hooks": ("latent", [_I]),
    "gtg_latent_attention_bf16": ("latent", [_P, _I, _P, _I, _P, _L, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _I, _P, _P]),
    "gtg_latent_attention_splits": ("latent", [_I, _I, _I, _I, _I, _I]),
    "gtg_moe_gather": ("experts", [_P, _I, _P, _I, _P, _I, _I, _P]),
    "gtg_gemm_bf16_tcgen05_grouped": ("gemm_bf16_tcgen05", [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P]),
    "gtg_moe_route": ("experts", [_I, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "gtg_moe_gather_scaled": ("experts", [_I, _P, _I, _P, _I, _P, _P, _I, _I, _P]),
    "gtg_attention_masked_supports": ("attention_masked", [_I, _I]),
    "gtg_attention_masked_scratch_floats": ("attention_masked", [_I, _I, _I, _I]),
    "gtg_attention_masked_splits": ("attention_masked", [_I, _I, _I, _I, _I, _I, _I]),
    "gtg_attention_masked_bf16": ("attention_masked", [_P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                                       _F, _I, _I, _P, _I, _P, _F, _I, _P]),
    "gtg_hyper_norm": ("hyper", [_I, _I, _P, _P, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _P]),
    "gtg_qkv_finish": ("attention_prep", [_I, _P, _I, _P, _P, _I, _I, _F, _P, _P, _F, _P, _I, _P, _P, _P, _L, _P, _I, _P, _P, _P,
                                          _I, _I, _I, _I, _I, _P]),
    "gtg_moe_arrange": ("experts", [_P, _I, _I, _I, _I, _P, _P, _P, _P]),
    "gtg_moe_product_simt": ("experts", [_I, _I, _P, _I, _P, _I, _P, _I, _L, _P, _I, _P, _I, _I, _I, _P]),
    "gtg_moe_combine": ("experts", [_I, _P, _I, _P, _P, _P, _I, _I, _I, _P]),
    "gtg_attention_bf16_supports": ("attention_bf16", [_I]),
    "gtg_attention_decode_scratch_floats": ("attention_bf16", [_I, _I, _I, _I]),
    "gtg_attention_decode_plan": ("attention_bf16", [_I, _I, _I, _I, _I, _L, _I, _P, _P]),
    "gtg_attention_prefill_bf16": ("attention_bf16", [_P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P, _P,
                                                      _I, _I, _I, _I, _I, _F, _I, _P]),
    "gtg_attention_decode_rope_bf16": ("attention_bf16", [_P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P,
                                                          _I, _I, _I, _I, _F, _I, _I, _P, _P, _P, _P, _I, _I, _I, _P]),
    "gtg_attention_decode_bf16": ("attention_bf16", [_P, _I, _P, _I, _P, _P, _L, _P, _I, _P, _P,
                                                     _I, _I, _I, _I, _F, _I, _I, _P, _I, _I, _P]),
    "gtg_attention_tcgen05_supports": ("attention_tcgen05", [_I]),
    "gtg_attention_tcgen05_status": ("attention_tcgen05", []),
    "gtg_attention_prefill_tcgen05": ("attention_tcgen05", [_P, _I, _I, _P, _I, _P, _P, _L, _I, _P, _I, _P, _P, _P,
                                                            _I, _I, _I, _I, _I, _F, _I, _I, _P, _F, _I, _P]),
    "gtg_argmax": ("sampling", [_P, _I, _I, _I, _P, _P]),
    "gtg_sample_temperature": ("sampling", [_P, _I, _I, _I, _F, _U, _P, _P, _P, _P]),
}
_RESTYPES = {"gtg_attention_decode_scratch_floats": c_longlong,
             "gtg_attention_masked_scratch_floats": c_longlong,
             "gtg_gemm_bf16_swapab_scratch_floats": c_longlong}

_FUNCS = {}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_chained = False


def _apply_chained(lib) -> None:
    setter = getattr(lib, "gtg_set_chained_launch", None)
    if setter is not None:
        setter.argtypes, setter.restype = [c_int], None
        setter(1 if _chained else 0)


class chained_launches:
    """Within this context the small kernels of a step are launched so that each
    may begin (up to the point where it needs its predecessor's results) while
    the one before it is still running -- programmatic dependent launch.  It is
    meant for decode steps, where launch and drain gaps are a large share of the
    time; the launches may be recorded into a CUDA graph."""

    def __init__(self, on: bool = True):
        self.on = bool(on)

    def __enter__(self):
        global _chained
        self.before = _chained
        _chained = self.on
        for lib in build._LOADED.values():
            _apply_chained(lib)
        return self

    def __exit__(self, *exc):
        global _chained
        _chained = self.before
        for lib in build._LOADED.values():
            _apply_chained(lib)


def _fn(symbol: str):
    f = _FUNCS.get(symbol)
    if f is None:
        lib_name, argtypes = _SIGNATURES[symbol]
        if not torch.cuda.is_available():
            raise KernelError(f"{symbol}: no CUDA device; this library runs on the GPU only "
                              f"and has no CPU path")
        lib = build.library(lib_name)
        _apply_chained(lib)
        f = getattr(lib, symbol)
        f.argtypes = argtypes
        f.restype = _RESTYPES.get(symbol, c_int)
        _FUNCS[symbol] = f
    return f


_CODES = {-1: "bad argument", -2: "size not supported by this kernel"}


_launches = 0


def launch_count() -> int:
    """How many kernel launchers of this library have been called so far (a
    launcher that is recorded into a CUDA graph counts once, when recorded)."""
    return _launches


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        if code in _CODES:
            raise KernelError(f"{what}: {_CODES[code]}")
        raise KernelError(f"{what}: CUDA error {code} (cudaError_t)")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Called once per launch: the direct binding
    costs a fraction of a microsecond, `torch.cuda.current_stream()` many."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _rows2d(t: torch.Tensor, name: str) -> None:
    _need(t.dim() == 2 and t.stride(1) == 1, f"{name} must be 2-D with a unit inner stride, "
                                             f"got shape {tuple(t.shape)} strides {t.stride()}")


# ------------------------------------------------- the debug pass over cache addresses
_checked = False
_ACCESS_FAULTS = {1: "a token names a sequence outside the batch", 2: "a sequence's slot is outside the cache",
                  3: "a position or a run of tokens is negative", 4: "a position lies beyond the block table's row",
                  5: "the block table names a page outside the cache"}


class checked_access:
    """Within this context every kernel that finds keys and values through the block
    table is preceded by a pass over the same indices (sequence -> slot -> table row
    -> page); the first index that would leave its array is reported as a
    `KernelError` and the kernel is not launched.  The stand-in for a memory
    checker: it costs a kernel and a synchronisation per call, so it is for
    debugging, not for serving, and a step under it is not recorded as a graph."""

    def __init__(self, on: bool = True):
        self.on = bool(on)

    def __enter__(self):
        global _checked
        self.before, _checked = _checked, self.on
        return self

    def __exit__(self, *exc):
        global _checked
        _checked = self.before


def _check_access(what: str, mode: int, kv, slots, positions=None, token_seq=None, start_pos=None,
                  cu_seqlens=None, n_items: Optional[int] = None) -> None:
    if not _checked or kv is None:
        return
    n_seqs = slots.numel()
    if n_items is None:
        n_items = n_seqs
    flag = torch.zeros(2, dtype=torch.int32, device=slots.device)
    code = _fn("gtg_check_cache_access")(mode, int(n_items), _ptr(token_seq), _ptr(slots), _ptr(positions),
                                         _ptr(start_pos), _ptr(cu_seqlens), n_seqs, _ptr(kv.block_table),
                                         kv.table_stride, kv.block_table.shape[0], kv.k.shape[0], _ptr(flag), _stream())
    if code != 0:
        raise KernelError(f"{what}: the access check could not run (code {code})")
    bad, item = flag.tolist()
    if bad:
        unit = "token" if mode == 0 else "sequence"
        raise KernelError(f"{what}: {_ACCESS_FAULTS.get(bad, bad)} ({unit} {item} of the step); the kernel was not launched")


# ------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[n,:] (float32) = table[tokens[n],:] * scale."""
    N, (V, H) = tokens.numel(), table.shape
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous(), "embed: tokens must be contiguous int32")
    _need(table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32
          and tuple(out.shape) == (N, H), "embed: out must be contiguous float32 [N, H]")
    _check(_fn("gtg_embed")(_dt(table), _ptr(tokens), _ptr(table), _ptr(out), N, H, V, float(scale), _stream()), "embed")


def add_rmsnorm(residual: torch.Tensor, pending: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """residual (+= pending); out = rmsnorm(residual) * weight.  With `rows` only
    those rows are read (nothing is written back) and out has len(rows) rows."""
    H = residual.shape[1]
    R = rows.numel() if rows is not None else residual.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: residual must be contiguous float32")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == H,
          "add_rmsnorm: weight must be float32 [H]")
    _need(out.is_contiguous() and tuple(out.shape) == (R, H), "add_rmsnorm: out must be contiguous [rows, H]")
    if pending is not None:
        _need(pending.dtype == out.dtype and pending.is_contiguous() and pending.shape == residual.shape,
              "add_rmsnorm: pending must match the residual's shape and out's dtype")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.is_contiguous(), "add_rmsnorm: rows must be contiguous int32")
    _check(_fn("gtg_add_rmsnorm")(_dt(out), _ptr(residual), _ptr(pending), _ptr(weight), float(eps),
                                  _ptr(out), _ptr(rows), R, H, _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[m,i] = act(gate_up[m,i]) * gate_up[m,I+i], act = silu or another of `ACTIVATIONS`."""
    _need(activation in ACTIVATIONS, f"swiglu: activation {activation!r} is not known; known: {sorted(ACTIVATIONS)}")
    M, two_i = gate_up.shape
    _need(two_i % 2 == 0 and gate_up.is_contiguous() and out.is_contiguous()
          and tuple(out.shape) == (M, two_i // 2) and out.dtype == gate_up.dtype,
          "swiglu: gate_up [M, 2I] and out [M, I] must be contiguous and of one dtype")
    _check(_fn("gtg_swiglu")(_dt(out), _ptr(gate_up), _ptr(out), M, two_i // 2, ACTIVATIONS[activation], _stream()), "swiglu")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor, amplitude: float = 1.0) -> None:
    """out[n,i] = amplitude * (cos, sin)(positions[n] * inv_freq[i]), angle and functions in float64."""
    N, half = positions.numel(), inv_freq.numel()
    _need(positions.dtype == torch.int32 and positions.is_contiguous(), "rope_table: positions must be int32")
    _need(inv_freq.dtype == torch.float64 and inv_freq.is_contiguous(), "rope_table: inv_freq must be float64")
    _need(out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (N, half, 2),
          "rope_table: out must be float32 [N, half, 2]")
    _check(_fn("gtg_rope_table")(_ptr(positions), _ptr(inv_freq), _ptr(out), N, half, float(amplitude), _stream()), "rope_table")


ROTARY_PAIRINGS = {"half": 0, "interleaved": 1}


def rope_kv_store(qkv: torch.Tensor, cos_sin: Optional[torch.Tensor], n_heads: int, n_kv_store: int,
                  head_dim: int, kv, token_seq: torch.Tensor, slots: torch.Tensor,
                  positions: torch.Tensor, pairing: str = "half", rotary_dim: Optional[int] = None,
                  values_from_keys: bool = False) -> None:
    """Rotate the query heads of qkv in place; rotate the key heads and copy the
    value heads into the cache `kv` at each token's (slot, position).  With
    n_kv_store == 0 only queries are rotated and `kv` may be None.  `pairing`:
    "half" rotates channel i with i + rotary_dim/2, "interleaved" 2i with 2i+1;
    the first `rotary_dim` channels of a head rotate (default: all), the rest
    pass unchanged.  Any other layout is refused.  With `values_from_keys` qkv
    holds query and key heads only, and the value stored for a head is its key
    as projected, before the rotation."""
    _rows2d(qkv, "rope_kv_store: qkv")
    N = qkv.shape[0]
    _need(head_dim % 2 == 0, "rope_kv_store: head_dim must be even")
    _need(pairing in ROTARY_PAIRINGS, f"rope_kv_store: pairing {pairing!r} is not supported; "
                                      f"supported: {sorted(ROTARY_PAIRINGS)}")
    rot = head_dim if rotary_dim is None else int(rotary_dim)
    _need(rot % 2 == 0 and 0 < rot <= head_dim,
          f"rope_kv_store: rotary_dim {rot} must be even and between 2 and head_dim {head_dim}")
    _need(qkv.shape[1] >= (n_heads + (1 if values_from_keys else 2) * n_kv_store) * head_dim,
          "rope_kv_store: qkv is too narrow")
    if cos_sin is not None:
        _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
              and tuple(cos_sin.shape) == (N, rot // 2, 2), "rope_kv_store: cos_sin must be float32 [N, rotary_dim/2, 2]")
    for name, t in (("token_seq", token_seq), ("slots", slots), ("positions", positions)):
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"rope_kv_store: {name} must be contiguous int32")
    if n_kv_store > 0:
        _need(kv is not None and kv.k.dtype == qkv.dtype and kv.head_dim == head_dim
              and kv.n_kv_heads == n_kv_store, "rope_kv_store: cache entry does not match the heads to store")
        _check_access("rope_kv_store", 0, kv, slots, positions, token_seq, n_items=N)
        args = (_ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table), kv.table_stride)
    else:
        args = (None, None, 0, None, 0)
    _check(_fn("gtg_rope_kv_store")(_dt(qkv), _ptr(qkv), qkv.stride(0), _ptr(cos_sin), n_heads, n_kv_store,
                                    head_dim, rot, ROTARY_PAIRINGS[pairing], 1 if values_from_keys else 0, *args, _ptr(token_seq), _ptr(slots), _ptr(positions),
                                    N, _stream()), "rope_kv_store")


def advance(tokens: torch.Tensor, positions: torch.Tensor, steps: torch.Tensor,
            sampled: torch.Tensor) -> None:
    """tokens <- sampled; positions += 1; steps += 1 (between decode steps that stay on the device)."""
    B = tokens.numel()
    for name, t in (("tokens", tokens), ("positions", positions), ("steps", steps), ("sampled", sampled)):
        _need(t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= B, f"advance: {name} must be int32 [B]")
    _check(_fn("gtg_advance")(_ptr(tokens), _ptr(positions), _ptr(steps), _ptr(sampled), B, _stream()), "advance")



def add_layernorm(residual: torch.Tensor, pending: Optional[torch.Tensor], weight: torch.Tensor,
                  bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
                  rows: Optional[torch.Tensor] = None) -> None:
    """residual (+= pending); out = (residual - mean) / sqrt(var + eps) * weight + bias.
    With `rows` only those rows are read (nothing is written back)."""
    H = residual.shape[1]
    R = rows.numel() if rows is not None else residual.shape[0]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_layernorm: residual must be contiguous float32")
    for name, t in (("weight", weight), ("bias", bias)):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == H),
              f"add_layernorm: {name} must be float32 [H]")
    _need(weight is not None, "add_layernorm: a weight is needed")
    _need(out.is_contiguous() and tuple(out.shape) == (R, H), "add_layernorm: out must be contiguous [rows, H]")
    if pending is not None:
        _need(pending.dtype == out.dtype and pending.is_contiguous() and pending.shape == residual.shape,
              "add_layernorm: pending must match the residual's shape and out's dtype")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.is_contiguous(), "add_layernorm: rows must be contiguous int32")
    _check(_fn("gtg_add_layernorm")(_dt(out), _ptr(residual), _ptr(pending), _ptr(weight), _ptr(bias), float(eps),
                                    _ptr(out), _ptr(rows), R, H, _stream()), "add_layernorm")


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}
# gate activations whose product act(gate) * up the products' epilogues form, and the epilogue's name
GATED_EPILOGUES = {"silu": "swiglu", "gelu_tanh": "gated_gelu_tanh", "relu2": "gated_relu2"}
EPILOGUE_GATED = 32           # a product's epilogue code from here on: the gated product with activation (code - 32) on the gate
EPILOGUE_ACTIVATION = 16      # a product's epilogue code from here on: the plain product, then activation (code - 16)


def activation(x: torch.Tensor, kind: str) -> None:
    """x <- f(x) in place, evaluated in float: "relu2" (relu squared), "gelu_tanh", "silu"."""
    _rows2d(x, "activation: x")
    _need(kind in ACTIVATIONS, f"activation: {kind!r} is not known; known: {sorted(ACTIVATIONS)}")
    _check(_fn("gtg_activation")(_dt(x), _ptr(x), x.stride(0), x.shape[0], x.shape[1], ACTIVATIONS[kind], _stream()),
           "activation")


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), in place (float32)."""
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "softcap: logits must be contiguous float32")
    _need(cap > 0, "softcap: the cap must be positive")
    _check(_fn("gtg_softcap")(_ptr(logits), logits.numel(), float(cap), _stream()), "softcap")


def scale(x: torch.Tensor, factor: float) -> None:
    """x <- factor * x in place (float32): a multiplier on the logits."""
    _need(x.dtype == torch.float32 and x.is_contiguous(), "scale: x must be contiguous float32")
    _check(_fn("gtg_scale")(_ptr(x), x.numel(), float(factor), _stream()), "scale")


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """x[n] <- x[n] / sqrt(mean(x[n]^2) + eps) * weight, in place on float32 rows: a norm
    that changes the hidden state itself (the one directly behind the token embedding)."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "rmsnorm_rows: x must be contiguous float32 [N, H]")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == x.shape[1],
          "rmsnorm_rows: weight must be float32 [H]")
    _check(_fn("gtg_rmsnorm_rows")(_ptr(x), _ptr(weight), float(eps), x.shape[0], x.shape[1], _stream()), "rmsnorm_rows")


def hidden_concat(residual: torch.Tensor, pending: Optional[torch.Tensor], other: torch.Tensor,
                  out: torch.Tensor) -> None:
    """out[:, :H] = residual (+ pending); out[:, H:] = other (float32 [N, H])."""
    N, H = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and other.dtype == torch.float32
          and other.is_contiguous() and other.shape == residual.shape,
          "hidden_concat: residual and other must be contiguous float32 of one shape")
    _need(out.is_contiguous() and tuple(out.shape) == (N, 2 * H), "hidden_concat: out must be contiguous [N, 2H]")
    if pending is not None:
        _need(pending.dtype == out.dtype and pending.is_contiguous() and pending.shape == residual.shape,
              "hidden_concat: pending must match the residual's shape and out's dtype")
    _check(_fn("gtg_hidden_concat")(_dt(out), _ptr(residual), _ptr(pending), _ptr(other), _ptr(out), N, H, _stream()),
           "hidden_concat")


def rmsnorm_add(update: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor,
                image: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> None:
    """residual += rmsnorm(update (+ bias)) * weight, in float: the norm on a
    sublayer's output.  `update` is float32 or of the activation dtype; `image`,
    if given, receives the new residual rounded to the activation dtype."""
    N, H = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "rmsnorm_add: residual must be contiguous float32")
    _need(update.is_contiguous() and update.shape == residual.shape, "rmsnorm_add: update must be contiguous [N, H]")
    for name, t in (("weight", weight), ("bias", bias)):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == H),
              f"rmsnorm_add: {name} must be float32 [H]")
    if image is not None:
        _need(image.is_contiguous() and image.shape == residual.shape, "rmsnorm_add: image must be contiguous [N, H]")
        dt = _dt(image)
    else:
        dt = _dt(update)
    _need(update.dtype == torch.float32 or _dt(update) == dt, "rmsnorm_add: update must be float32 or of the image's dtype")
    _check(_fn("gtg_rmsnorm_add")(dt, 1 if update.dtype == torch.float32 else 0, _ptr(update), _ptr(bias), _ptr(weight),
                                  float(eps), _ptr(residual), _ptr(image), N, H, _stream()), "rmsnorm_add")


HYPER_MAX_COPIES = 8


def hyper_norm(copies: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
               seed: Optional[torch.Tensor] = None, update: Optional[torch.Tensor] = None,
               mix: Optional[torch.Tensor] = None, out_w: Optional[torch.Tensor] = None,
               in_w: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """The hidden state in S copies, float32 [N, S, H].  With `update` y [N, H] (float32 or
    out's dtype) first x_t <- sum_s mix[s, t] x_s + out_w[t] y, all copies at once; then
    out = rmsnorm(sum_t in_w[t] x_t) * weight (in_w None: the plain sum).  With `seed`
    [N, H] the copies are made: each is the seed's row.  With `rows` only those
    tokens are read, nothing is written back, and out has len(rows) rows."""
    _need(copies.dtype == torch.float32 and copies.is_contiguous() and copies.dim() == 3,
          "hyper_norm: the copies must be contiguous float32 [N, S, H]")
    N, S, H = copies.shape
    R = rows.numel() if rows is not None else N
    _need(S <= HYPER_MAX_COPIES, f"hyper_norm: at most {HYPER_MAX_COPIES} copies, got {S}")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == H, "hyper_norm: weight must be float32 [H]")
    _need(out.is_contiguous() and tuple(out.shape) == (R, H), "hyper_norm: out must be contiguous [rows, H]")
    _need(seed is None or (seed.dtype == torch.float32 and seed.is_contiguous() and tuple(seed.shape) == (N, H) and update is None),
          "hyper_norm: the seed must be contiguous float32 [N, H], without an update")
    if update is not None:
        _need(update.is_contiguous() and tuple(update.shape) == (N, H) and update.dtype in (torch.float32, out.dtype),
              "hyper_norm: the update must be contiguous [N, H], float32 or of out's dtype")
        _need(mix is not None and out_w is not None and mix.dtype == out_w.dtype == torch.float32 and mix.is_contiguous()
              and out_w.is_contiguous() and tuple(mix.shape) == (S, S) and out_w.numel() == S,
              "hyper_norm: an update needs mix float32 [S, S] and out_w float32 [S]")
    _need(in_w is None or (in_w.dtype == torch.float32 and in_w.is_contiguous() and in_w.numel() == S), "hyper_norm: in_w must be float32 [S]")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.is_contiguous(), "hyper_norm: rows must be contiguous int32")
    _check(_fn("gtg_hyper_norm")(_dt(out), 1 if (update is not None and update.dtype == torch.float32) else 0, _ptr(copies), _ptr(seed),
                                 _ptr(update), _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(weight), float(eps), _ptr(out), _ptr(rows),
                                 R, S, H, _stream()), "hyper_norm")


def qkv_finish(sums: torch.Tensor, bias: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor], n_heads: int, kv,
               q_out: torch.Tensor, token_seq, slots, positions, *, unit_norm: bool = False, eps: float = 0.0,
               v_first: Optional[torch.Tensor] = None, v_keep: Optional[torch.Tensor] = None, blend: float = 0.0,
               gate_out: Optional[torch.Tensor] = None, store: bool = True) -> None:
    """From the float sums of a fused projection [N, q | k | v | gate]: biases added, the first
    channels of query and key heads rotated (half-split pairs, as many as the table has),
    optionally each head divided by its root mean square, values blended with `v_first`
    ((1 - blend) v + blend v_first; float32 [N, n_kv * value_dim]) or kept in `v_keep`
    unblended, gate columns turned into sigmoid factors (`gate_out` float32 [N, n_heads]);
    queries to `q_out`, keys and values into the cache `kv` (its head_dim and value_dim)."""
    _rows2d(sums, "qkv_finish: sums"); _rows2d(q_out, "qkv_finish: q_out")
    N = sums.shape[0]
    hd, vd, n_kv = kv.head_dim, kv.value_dim, kv.n_kv_heads
    biased = n_heads * hd + n_kv * (hd + vd)
    width = biased + (n_heads if gate_out is not None else 0)
    _need(sums.dtype == torch.float32 and sums.shape[1] >= width, f"qkv_finish: sums must be float32 with {width} columns at least")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == biased), "qkv_finish: bias must be float32 [q | k | v]")
    rot = 0
    if cos_sin is not None:
        _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[0] == N and cos_sin.shape[2] == 2,
              "qkv_finish: the rotation table must be float32 [N, pairs, 2]")
        rot = 2 * cos_sin.shape[1]
        _need(rot <= hd, "qkv_finish: more rotated channels than a head has")
    _need(q_out.dtype == kv.k.dtype and q_out.shape[0] == N and q_out.shape[1] >= n_heads * hd, "qkv_finish: q_out must be [N, n_heads * head_dim] of the cache's dtype")
    for t, name in ((v_first, "v_first"), (v_keep, "v_keep")):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == (N, n_kv * vd)), f"qkv_finish: {name} must be float32 [N, n_kv * value_dim]")
    _need(gate_out is None or (gate_out.dtype == torch.float32 and gate_out.is_contiguous() and tuple(gate_out.shape) == (N, n_heads)),
          "qkv_finish: gate_out must be float32 [N, n_heads]")
    _int32("qkv_finish", token_seq, slots, positions)
    if store:
        _check_access("qkv_finish", 0, kv, slots, positions, token_seq, n_items=N)
    _check(_fn("gtg_qkv_finish")(_dt(q_out), _ptr(sums), sums.stride(0), _ptr(bias), _ptr(cos_sin), rot, 1 if unit_norm else 0, float(eps),
                                 _ptr(v_first), _ptr(v_keep), float(blend), _ptr(q_out), q_out.stride(0), _ptr(gate_out),
                                 _ptr(kv.k) if store else None, _ptr(kv.v) if store else None, kv.page_stride, _ptr(kv.block_table),
                                 kv.table_stride, _ptr(token_seq), _ptr(slots), _ptr(positions), N, n_heads, n_kv, hd, vd, _stream()),
           "qkv_finish")


def round_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32) rounded to out's dtype."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == x.shape,
          "round_rows: x float32 and out, both contiguous and of one shape")
    _check(_fn("gtg_round_rows")(_dt(out), _ptr(x), _ptr(out), x.numel(), _stream()), "round_rows")


def swiglu_bias(gate_up: torch.Tensor, gate_bias: Optional[torch.Tensor], up_bias: Optional[torch.Tensor],
                out: torch.Tensor) -> None:
    """out[m,i] = silu(gate_up[m,i] + gate_bias[i]) * (gate_up[m,I+i] + up_bias[i]) from a
    product's float32 sums [M, 2I]."""
    _rows2d(out, "swiglu_bias: out")
    M, two_i = gate_up.shape
    I = two_i // 2
    _need(gate_up.dtype == torch.float32 and gate_up.is_contiguous() and two_i % 2 == 0 and tuple(out.shape) == (M, I),
          "swiglu_bias: gate_up must be contiguous float32 [M, 2I] and out [M, I]")
    for name, t in (("gate_bias", gate_bias), ("up_bias", up_bias)):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == I), f"swiglu_bias: {name} must be float32 [I]")
    _check(_fn("gtg_swiglu_bias")(_dt(out), _ptr(gate_up), _ptr(gate_bias), _ptr(up_bias), _ptr(out), out.stride(0), M, I,
                                  _stream()), "swiglu_bias")


def add_bias(x: torch.Tensor, bias: torch.Tensor, out: torch.Tensor) -> None:
    """out = x + bias, x a product's float32 sums [M, N], out float32 or the activation dtype."""
    M, N = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == x.shape,
          "add_bias: x float32 and out, both contiguous [M, N]")
    _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == N, "add_bias: bias must be float32 [N]")
    _check(_fn("gtg_add_bias")(_dt(out), _ptr(x), _ptr(bias), _ptr(out), M, N, _stream()), "add_bias")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x *= sigmoid(gate) in place, evaluated in float; the logits are of x's dtype or float32."""
    _rows2d(x, "sigmoid_gate: x"); _rows2d(gate, "sigmoid_gate: gate")
    _need(x.shape == gate.shape and gate.dtype in (x.dtype, torch.float32), "sigmoid_gate: x and gate must agree in shape, gate of x's dtype or float32")
    _check(_fn("gtg_sigmoid_gate")(_dt(x), _ptr(x), x.stride(0), _ptr(gate), gate.stride(0), x.shape[0], x.shape[1],
                                   1 if gate.dtype == torch.float32 else 0, _stream()), "sigmoid_gate")


def qkv_conv_finish(sums: torch.Tensor, bias: Optional[torch.Tensor], conv_w: Optional[torch.Tensor],
                    conv_state: Optional[torch.Tensor], cu_seqlens, q_norm: Optional[torch.Tensor],
                    k_norm: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor], interleaved: bool,
                    n_heads: int, n_kv: int, head_dim: int, value_dim: int, kv, q_out: torch.Tensor,
                    token_seq, slots, positions, store: bool = True, one_token_each: bool = False) -> None:
    """Between the fused projection and the attention, for mixers whose q, k and v pass a
    short causal convolution over time: of the float32 sums [N, >= q | k | v] (n_kv key and
    value heads; 0: queries only) add the bias [q | k | v], convolve every channel over the
    last taps tokens (conv_w float32 [taps, C], oldest tap first; earlier steps' raw sums from
    conv_state float32 [slots, taps-1, C]; None: no convolution), norm every query and key
    head with q_norm / k_norm (float32 [head_dim]; None: no norm), rotate the head's first
    2 * cos_sin.shape[1] channels (2i with 2i+1 if `interleaved`, else i with i + half),
    write queries to q_out and, with `store`, keys and values to the cache.  The state is
    not changed: `conv_state_update` over the same sums follows.  `one_token_each`: a decode
    step (the form that shares a run of rows between neighbouring tokens is then not taken)."""
    _rows2d(sums, "qkv_conv_finish: sums"); _rows2d(q_out, "qkv_conv_finish: q_out")
    N = sums.shape[0]
    C = n_heads * head_dim + n_kv * (head_dim + value_dim)
    _need(sums.dtype == torch.float32 and sums.shape[1] >= C, "qkv_conv_finish: sums must be float32 rows of q | k | v")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C),
          "qkv_conv_finish: bias must be float32 [q | k | v]")
    taps = 1
    if conv_w is not None:
        taps = conv_w.shape[0]
        _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and tuple(conv_w.shape) == (taps, C),
              "qkv_conv_finish: conv_w must be float32 [taps, q | k | v]")
        _need(taps == 1 or (conv_state is not None and conv_state.dtype == torch.float32 and conv_state.is_contiguous()
                            and tuple(conv_state.shape[1:]) == (taps - 1, C)),
              "qkv_conv_finish: conv_state must be float32 [slots, taps-1, q | k | v]")
    for name, t in (("q_norm", q_norm), ("k_norm", k_norm)):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == head_dim),
              f"qkv_conv_finish: {name} must be float32 [head_dim]")
    rot = 0
    if cos_sin is not None:
        _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.dim() == 3 and cos_sin.shape[0] == N
              and cos_sin.shape[2] == 2, "qkv_conv_finish: cos_sin must be float32 [N, pairs, 2]")
        rot = 2 * cos_sin.shape[1]
        _need(rot <= head_dim, "qkv_conv_finish: more rotated channels than a head has")
    _need(q_out.shape[0] == N and q_out.shape[1] >= n_heads * head_dim, "qkv_conv_finish: q_out is too narrow")
    store = bool(store and n_kv > 0)
    if store:
        _need(kv.k.dtype == q_out.dtype and kv.n_kv_heads == n_kv and kv.head_dim == head_dim and kv.value_dim == value_dim,
              "qkv_conv_finish: the cache entry does not match the heads")
    _int32("qkv_conv_finish", cu_seqlens, token_seq, slots, positions)
    if store:
        _check_access("qkv_conv_finish", 0, kv, slots, positions, token_seq, n_items=N)
    _check(_fn("gtg_qkv_conv_finish")(_dt(q_out), _ptr(sums), sums.stride(0), _ptr(bias), _ptr(conv_w), taps, _ptr(conv_state),
                                      _ptr(cu_seqlens), _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(cos_sin), rot,
                                      1 if interleaved else 0, _ptr(q_out), q_out.stride(0),
                                      _ptr(kv.k) if store else None, _ptr(kv.v) if store else None,
                                      kv.page_stride if store else 0, _ptr(kv.block_table) if store else None,
                                      kv.table_stride if store else 0, _ptr(token_seq), _ptr(slots), _ptr(positions),
                                      N, n_heads, n_kv, head_dim, value_dim, 1 if one_token_each else 0, _stream()),
           "qkv_conv_finish")


# ------------------------------------------------------------- the gated delta rule
DELTA_MAX_KEY_DIM = 512       # most key channels a head of the delta rule's state may have (16 rows a lane, 32 lanes)


def delta_scan_supports(key_dim: int, value_dim: int) -> bool:
    return bool(_fn("gtg_delta_scan_supports")(int(key_dim), int(value_dim)))


def delta_prepare(qk: torch.Tensor, decay: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                  beta_in: torch.Tensor, beta: torch.Tensor, n_heads: int, n_groups: int, key_dim: int,
                  unit_eps: float, q_scale: float) -> None:
    """Per token, in place on float32 rows: every query and key head of qk ([N, >= 2 * n_groups *
    key_dim], queries then keys) becomes x / sqrt(sum(x^2) + unit_eps), queries also times
    q_scale; decay [N, n_heads * key_dim] becomes exp(-exp(a_log[h]) softplus(decay + dt_bias));
    beta [N, n_heads] = sigmoid(beta_in [N, n_heads])."""
    _rows2d(qk, "delta_prepare: qk"); _rows2d(decay, "delta_prepare: decay"); _rows2d(beta_in, "delta_prepare: beta_in")
    N = qk.shape[0]
    _need(qk.dtype == decay.dtype == beta_in.dtype == beta.dtype == torch.float32, "delta_prepare: float32 rows only")
    _need(qk.shape[1] >= 2 * n_groups * key_dim and tuple(decay.shape) == (N, n_heads * key_dim)
          and tuple(beta_in.shape) == (N, n_heads) and tuple(beta.shape) == (N, n_heads) and beta.is_contiguous(),
          "delta_prepare: qk [N, 2 groups * d], decay [N, heads * d], beta_in and beta [N, heads]")
    _need(dt_bias.dtype == torch.float32 and dt_bias.is_contiguous() and dt_bias.numel() == n_heads * key_dim
          and a_log.dtype == torch.float32 and a_log.is_contiguous() and a_log.numel() == n_heads,
          "delta_prepare: dt_bias float32 [heads * d], a_log float32 [heads]")
    _check(_fn("gtg_delta_prepare")(_ptr(qk), qk.stride(0), _ptr(decay), decay.stride(0), _ptr(dt_bias), _ptr(a_log),
                                    _ptr(beta_in), beta_in.stride(0), _ptr(beta), N, n_heads, n_groups, key_dim,
                                    float(unit_eps), float(q_scale), _stream()), "delta_prepare")


def delta_scan(qk: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
               out: torch.Tensor, cu_seqlens, slots, n_seqs: int, n_heads: int, n_groups: int, key_dim: int,
               value_dim: int, one_token_each: bool = False) -> None:
    """The gated delta rule, token by token, all float32: per head h (queries and keys of
    group h // (n_heads / n_groups)), S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T;
    out = S^T q.  qk [N, >= 2 groups * d] (queries, then keys), v [N, heads * dv], decay
    [N, heads * d], beta [N, heads]; state [slots, heads, d, dv], read and left per
    sequence; out [N, heads * dv].  `one_token_each`: row b is sequence b's only token (a
    decode step), which a kernel of its own serves where the sizes allow."""
    for name, t in (("qk", qk), ("v", v), ("decay", decay), ("out", out)):
        _rows2d(t, f"delta_scan: {name}")
        _need(t.dtype == torch.float32, f"delta_scan: {name} must be float32")
    N = qk.shape[0]
    _need(qk.shape[1] >= 2 * n_groups * key_dim and tuple(v.shape) == (N, n_heads * value_dim)
          and tuple(decay.shape) == (N, n_heads * key_dim) and tuple(out.shape) == (N, n_heads * value_dim),
          "delta_scan: qk [N, 2 groups * d], v and out [N, heads * dv], decay [N, heads * d]")
    _need(beta.dtype == torch.float32 and beta.is_contiguous() and tuple(beta.shape) == (N, n_heads),
          "delta_scan: beta must be contiguous float32 [N, heads]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (n_heads, key_dim, value_dim),
          "delta_scan: state must be float32 [slots, heads, d, dv]")
    _need(delta_scan_supports(key_dim, value_dim), f"delta_scan: a state of {key_dim} x {value_dim} a head is not supported")
    _int32("delta_scan", cu_seqlens, slots)
    _check(_fn("gtg_delta_scan")(_ptr(qk), qk.stride(0), _ptr(v), v.stride(0), _ptr(decay), decay.stride(0), _ptr(beta),
                                 _ptr(state), _ptr(out), out.stride(0), _ptr(cu_seqlens), _ptr(slots), int(n_seqs),
                                 n_heads, n_groups, key_dim, value_dim, 1 if one_token_each and N == n_seqs else 0, _stream()),
           "delta_scan")


def head_norm_gate(y: torch.Tensor, gate_logits: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                   n_heads: int) -> None:
    """out[n, h, :] = y[n, h, :] / sqrt(mean(y[n, h, :]^2) + eps) * weight * sigmoid(gate_logits[n, h, :]):
    y and gate_logits float32 [N, heads * dv], weight float32 [dv] shared by the heads."""
    _rows2d(y, "head_norm_gate: y"); _rows2d(gate_logits, "head_norm_gate: gate"); _rows2d(out, "head_norm_gate: out")
    N, width = y.shape
    _need(width % n_heads == 0, "head_norm_gate: the row is not a whole number of heads")
    dv = width // n_heads
    _need(y.dtype == torch.float32 and gate_logits.dtype == torch.float32 and tuple(gate_logits.shape) == (N, width)
          and tuple(out.shape) == (N, width), "head_norm_gate: y and gate float32 [N, heads * dv], out of that shape")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == dv,
          "head_norm_gate: weight must be float32 [dv]")
    _check(_fn("gtg_head_norm_gate")(_dt(out), _ptr(y), y.stride(0), _ptr(gate_logits), gate_logits.stride(0), _ptr(weight),
                                     float(eps), _ptr(out), out.stride(0), N, n_heads, dv, _stream()), "head_norm_gate")


# ------------------------------------------------------------- recurrent mixers
def _int32(name: str, *tensors) -> None:
    for t in tensors:
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name}: index tensors must be contiguous int32")


def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     conv_state: torch.Tensor, out: torch.Tensor, token_seq, cu_seqlens, slots,
                     n_seqs: Optional[int] = None, update_state: bool = False, one_token_each: bool = False,
                     pairs: Optional[torch.Tensor] = None) -> None:
    """out[n, c] = silu(bias[c] + sum_j weight[j, c] x[n - (taps-1-j), c]) (weight is
    held tap by tap, [taps, C]; the last tap is the current token's) within each
    sequence of the packed rows; what precedes a sequence's first row of the step
    comes from conv_state[slot] ([taps-1, C] float32, oldest first).  With
    `update_state` the state is then left as `conv_state_update` leaves it (one
    kernel does both when every sequence brings one token: `one_token_each`).
    With `pairs` (float32 [n, Q, 2]) only the first C - 2Q channels go to `out`;
    the rest, two runs U and V of Q channels, are left as float (U_q, V_q) side
    by side, which is how `ssm_scan` reads a recurrence's B and C."""
    _rows2d(x, "causal_conv_silu: x"); _rows2d(out, "causal_conv_silu: out")
    n, C = x.shape
    taps = weight.shape[0]
    n_plain = C
    if pairs is not None:
        _need(pairs.dtype == torch.float32 and pairs.is_contiguous() and pairs.dim() == 3 and pairs.shape[0] == n
              and pairs.shape[2] == 2 and 2 * pairs.shape[1] <= C, "causal_conv_silu: pairs must be float32 [n, Q, 2]")
        n_plain = C - 2 * pairs.shape[1]
    _need(out.dtype == x.dtype and tuple(out.shape) == (n, n_plain), "causal_conv_silu: out must be [n, plain channels] of x's dtype")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.dim() == 2 and weight.shape[1] == C,
          "causal_conv_silu: weight must be float32 [taps, C]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == C),
          "causal_conv_silu: bias must be float32 [C]")
    _need(conv_state.dtype == torch.float32 and conv_state.is_contiguous()
          and tuple(conv_state.shape[1:]) == (taps - 1, C), "causal_conv_silu: conv_state must be float32 [slots, taps-1, C]")
    _int32("causal_conv_silu", token_seq, cu_seqlens, slots)
    if update_state and one_token_each:
        _need(n == slots.numel(), "causal_conv_silu: one token each means as many rows as sequences")
        _check(_fn("gtg_causal_conv_step")(_dt(x), _ptr(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(conv_state),
                                           _ptr(out), out.stride(0), _ptr(slots), n, C, taps, n_plain, _ptr(pairs), _stream()),
               "causal_conv_silu(step)")
        return
    _check(_fn("gtg_causal_conv_silu")(_dt(x), _ptr(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(conv_state),
                                       _ptr(out), out.stride(0), _ptr(token_seq), _ptr(cu_seqlens), _ptr(slots),
                                       n, C, taps, n_plain, _ptr(pairs), _stream()), "causal_conv_silu")
    if update_state:
        conv_state_update(x, conv_state, cu_seqlens, slots, slots.numel() if n_seqs is None else n_seqs)


def conv_state_update(x: torch.Tensor, conv_state: torch.Tensor, cu_seqlens, slots, n_seqs: int) -> None:
    """conv_state[slot] <- the last taps-1 inputs of each sequence, this step's rows included."""
    _rows2d(x, "conv_state_update: x")
    C = x.shape[1]
    keep = conv_state.shape[1]
    _need(conv_state.dtype == torch.float32 and conv_state.is_contiguous() and conv_state.shape[2] == C,
          "conv_state_update: conv_state must be float32 [slots, taps-1, C]")
    _int32("conv_state_update", cu_seqlens, slots)
    _check(_fn("gtg_conv_state_update")(_dt(x), _ptr(x), x.stride(0), _ptr(conv_state), _ptr(cu_seqlens), _ptr(slots),
                                        int(n_seqs), C, keep + 1, _stream()), "conv_state_update")


def ssm_scan(x: torch.Tensor, bc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
             skip: torch.Tensor, state: torch.Tensor, y: torch.Tensor, cu_seqlens, slots, n_seqs: int,
             heads: int, groups: int, n_state: int, head_dim: int, one_token_each: bool = False) -> None:
    """The state-space recurrence with a scalar decay per head, token by token:
    x [n, heads*P]; bc float32 [n, groups*N, 2], (B_n, C_n) side by side;
    dt_raw [n, heads]; dt = softplus(dt_raw + dt_bias), S <- exp(-exp(a_log) dt) S + dt B x^T,
    y = S^T C + skip * x.  state: float32 [slots, heads, N, P], read and left
    per sequence; y: float32 [n, heads*P].  `one_token_each`: row b is sequence
    b's only token (a decode step), which a kernel of its own serves."""
    _rows2d(x, "ssm_scan: x"); _rows2d(dt_raw, "ssm_scan: dt_raw"); _rows2d(y, "ssm_scan: y")
    n = x.shape[0]
    inner = heads * head_dim
    _need(x.shape[1] == inner and dt_raw.dtype == x.dtype and tuple(dt_raw.shape) == (n, heads),
          "ssm_scan: x must be [n, heads*P] and dt_raw [n, heads] of one dtype")
    _need(bc.dtype == torch.float32 and bc.is_contiguous() and tuple(bc.shape) == (n, groups * n_state, 2),
          "ssm_scan: bc must be contiguous float32 [n, groups*N, 2]")
    _need(y.dtype == torch.float32 and tuple(y.shape) == (n, inner), "ssm_scan: y must be float32 [n, heads*P]")
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("skip", skip)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == heads, f"ssm_scan: {name} must be float32 [heads]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, n_state, head_dim),
          "ssm_scan: state must be float32 [slots, heads, N, P]")
    _int32("ssm_scan", cu_seqlens, slots)
    _check(_fn("gtg_ssm_scan")(_dt(x), _ptr(x), x.stride(0), _ptr(bc), groups * n_state, _ptr(dt_raw), dt_raw.stride(0),
                               _ptr(dt_bias), _ptr(a_log), _ptr(skip), _ptr(state), _ptr(y), y.stride(0),
                               _ptr(cu_seqlens), _ptr(slots), int(n_seqs), heads, groups, n_state, head_dim,
                               1 if one_token_each and n == n_seqs else 0, _stream()), "ssm_scan")


def gated_rmsnorm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                  parts: int = 1) -> None:
    """out = rmsnorm_parts(y * silu(z)) * weight: the row is cut into `parts` equal
    pieces, each divided by its own root mean square.  y float32; z, out the
    activation dtype."""
    _rows2d(y, "gated_rmsnorm: y"); _rows2d(z, "gated_rmsnorm: z"); _rows2d(out, "gated_rmsnorm: out")
    n, width = y.shape
    _need(y.dtype == torch.float32 and z.dtype == out.dtype and tuple(z.shape) == (n, width) and tuple(out.shape) == (n, width),
          "gated_rmsnorm: y float32, z and out of one dtype, all [n, width]")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == width,
          "gated_rmsnorm: weight must be float32 [width]")
    _need(parts >= 1 and width % parts == 0, f"gated_rmsnorm: {parts} pieces do not divide a row of {width}")
    _check(_fn("gtg_gated_rmsnorm")(_dt(out), _ptr(y), y.stride(0), _ptr(z), z.stride(0), _ptr(weight), float(eps),
                                    _ptr(out), out.stride(0), n, width, int(parts), _stream()), "gated_rmsnorm")


# ---------------------------------------------------------------- matrix products
SKINNY_MAX_ROWS = 128         # most rows the weight-streaming kernels take (beyond: the prompt-sized product)
STREAM_MAX_ROWS = 16          # up to here: warp-level MMA fed by bulk copies; beyond: tcgen05 with swapped operands
WARP_LEVEL_MAX_ROWS = 64      # most rows the warp-level kernel takes when asked for by name
TILED_KIND = "tcgen05"        # what "auto" uses beyond SKINNY_MAX_ROWS rows


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """The weight layout of the fused SwiGLU epilogue: rows in blocks of 8 gate
    features followed by the same 8 up features.  gate, up: [I, K] with I % 8 == 0."""
    i, k = gate.shape
    _need(up.shape == gate.shape and i % 8 == 0, "interleave_gate_up: equal shapes with a multiple of 8 rows")
    return torch.stack([gate.reshape(i // 8, 8, k), up.reshape(i // 8, 8, k)], dim=1).reshape(2 * i, k).contiguous()


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, kind: str = "auto",
           epilogue: str = "none") -> None:
    """out[M,N] = x[M,K] . w[N,K]^T.  float32 operands take the true 32-bit
    kernel; bfloat16 operands accumulate in float and write bfloat16 or float32.
    `kind` picks the bfloat16 kernel: "auto" (by the number of rows), "skinny"
    (weight streaming, up to 64 rows), "swapab" (weight streaming on tcgen05 with
    the tokens as the N dimension, up to 128 rows), "tcgen05" (TMA + tensor memory)
    or "tiled" (warp-level MMA).  epilogue="swiglu" (bfloat16, not "tiled"): w is laid out by
    `interleave_gate_up` and out[M, N/2] = silu(gate) * up, computed from the
    float accumulators; epilogue="gated_gelu_tanh" | "gated_relu2": the same with that
    activation on the gate.  epilogue="relu2" | "gelu_tanh" | "silu": out[M, N] is that
    activation of the product, applied to the float sums inside the tensor-core
    kernels, by the `activation` kernel behind the others."""
    _rows2d(x, "linear: x"); _rows2d(w, "linear: w"); _rows2d(out, "linear: out")
    M, K = x.shape
    N = w.shape[0]
    if epilogue in ACTIVATIONS:
        fused = (x.dtype == torch.bfloat16 and kind != "tiled" and K % 8 == 0 and x.stride(0) % 8 == 0
                 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                 and out.data_ptr() % 16 == 0 and out.stride(0) % (4 if out.dtype == torch.float32 else 8) == 0)
        if not fused:
            linear(x, w, out, kind=kind)
            activation(out, epilogue)
            return
    gated = epilogue in GATED_EPILOGUES.values()
    _need(epilogue == "none" or gated or epilogue in ACTIVATIONS, f"linear: unknown epilogue {epilogue!r}")
    n_out = N // 2 if gated else N
    _need(w.shape[1] == K and tuple(out.shape) == (M, n_out),
          f"linear: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} (epilogue {epilogue})")
    if x.dtype == torch.float32:
        _need(epilogue == "none", "linear: the float32 product has no fused epilogue")
        _need(w.dtype == torch.float32 and out.dtype == torch.float32, "linear: float32 x needs float32 w and out")
        _check(_fn("gtg_gemm_f32")(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                                   M, N, K, _stream()), "linear(float32)")
        return
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear: operands must both be bfloat16 or both float32")
    _need(out.dtype in (torch.bfloat16, torch.float32), "linear: out must be bfloat16 or float32")
    if kind == "auto" and epilogue == "none" and not (
            K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
            and out.stride(0) % (4 if out.dtype == torch.float32 else 8) == 0):
        # a shape the tensor-core products cannot address: the plain walk, float accumulation
        _check(_fn("gtg_gemm_bf16_simt")(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                                         1 if out.dtype == torch.float32 else 0, M, N, K, _stream()),
               "linear(bfloat16, plain)")
        return
    _need(K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0,
          f"linear(bfloat16): the inner size {K} and the row strides must be multiples of 8")
    # few rows (a decode step): stream the weights once; many rows: tiled product
    if kind == "auto":
        kind = "skinny" if M <= STREAM_MAX_ROWS else "swapab" if M <= SKINNY_MAX_ROWS else TILED_KIND
    symbol = {"skinny": "gtg_gemm_bf16_skinny", "tiled": "gtg_gemm_bf16_mma", "swapab": "gtg_gemm_bf16_swapab",
              "tcgen05": "gtg_gemm_bf16_tcgen05"}.get(kind)
    _need(symbol is not None, f"linear: unknown kind {kind!r}")
    if kind in ("skinny", "swapab"):
        most = WARP_LEVEL_MAX_ROWS if kind == "skinny" else SKINNY_MAX_ROWS
        _need(M <= most, f"linear: the weight-streaming kernel {kind!r} takes at most {most} rows")
    out_f32 = 1 if out.dtype == torch.float32 else 0
    epi_code = (1 if epilogue == "swiglu" else EPILOGUE_GATED + ACTIVATIONS[epilogue[len("gated_"):]] if gated
                else EPILOGUE_ACTIVATION + ACTIVATIONS[epilogue] if epilogue in ACTIVATIONS else 0)
    if kind == "tiled":
        _need(epilogue == "none", "linear: the warp-level kernel has no fused epilogue")
        code = _fn(symbol)(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                           out_f32, M, N, K, _stream())
    elif kind == "swapab":
        if gated:
            _need(N % 16 == 0, f"linear: the fused SwiGLU needs a multiple of 16 rows of w, got {N}")
        scratch = torch.empty(int(_fn("gtg_gemm_bf16_swapab_scratch_floats")(M, N, K)), dtype=torch.float32,
                              device=x.device)
        code = _fn(symbol)(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                           out_f32, M, N, K, epi_code, _ptr(scratch), _stream())
    else:
        if gated:
            _need(N % 16 == 0, f"linear: the fused SwiGLU needs a multiple of 16 rows of w, got {N}")
        code = _fn(symbol)(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0),
                           out_f32, M, N, K, epi_code, _stream())
    _check(code, "linear(bfloat16)")


def _grouped_ok(a: torch.Tensor, w: torch.Tensor, K: int, *strides: int) -> bool:
    """Whether the warp-level tensor-core product can address these bfloat16 operands."""
    return (a.dtype == torch.bfloat16 and K % 8 == 0 and all(s % 8 == 0 for s in strides)
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def linear_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None) -> None:
    """out[m, h, :] = x[m, h, :] . w[h]^T for every head h: x [M, heads, K], w
    [heads, N, K], out [M, heads, N]; x and out may be views whose heads lie side
    by side in wider rows (any row and head stride, unit channel stride).  With
    `gate` (laid out like out) the result is multiplied by sigmoid(gate), in
    float: in the product's epilogue on the tensor-core route, by a kernel of
    its own behind the plain product."""
    _need(x.dim() == 3 and w.dim() == 3 and out.dim() == 3 and x.stride(2) == 1 and out.stride(2) == 1 and w.is_contiguous(),
          "linear_heads: x [M, heads, K], w contiguous [heads, N, K], out [M, heads, N] with unit channel strides")
    M, heads, K = x.shape
    N = w.shape[1]
    _need(tuple(w.shape) == (heads, N, K) and tuple(out.shape) == (M, heads, N),
          f"linear_heads: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)}")
    _need(x.dtype == w.dtype == out.dtype, "linear_heads: one dtype for x, w and out")
    if gate is not None:
        _need(gate.shape == out.shape and gate.dtype == out.dtype and gate.stride(2) == 1, "linear_heads: gate must be laid out like out")
    if M == 0:
        return
    if _grouped_ok(x, w, K, x.stride(0), x.stride(1)):
        g = (_ptr(gate), gate.stride(0), gate.stride(1)) if gate is not None else (None, 0, 0)
        _check(_fn("gtg_gemm_bf16_grouped")(_ptr(x), x.stride(0), x.stride(1), None, 0, _ptr(w), K, N * K, None, _ptr(out),
                                            out.stride(0), out.stride(1), 0, heads, M, N, K, 128 if M > 64 else 64,
                                            2 if gate is not None else 0, *g, _stream()), "linear_heads(bfloat16)")
        return
    _check(_fn("gtg_gemm_simt_batched")(_dt(x), _ptr(x), x.stride(0), x.stride(1), _ptr(w), K, N * K, _ptr(out),
                                        out.stride(0), out.stride(1), heads, M, N, K, _stream()), "linear_heads")
    if gate is not None:
        for h in range(heads):
            sigmoid_gate(out[:, h], gate[:, h])


def linear_add_residual(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> bool:
    """residual[M,N] += bfloat16(x[M,K] . w[N,K]^T): the product of a prompt step
    adds its result to a float32 residual stream in its epilogue (tensor reductions,
    each element once), rounded as it would be if it were stored first -- what
    `linear` into a bfloat16 update followed by the norm kernel's addition gives,
    without the update's trip through memory.  False, with nothing done, for
    operands the tensor-memory kernel does not take this way (few rows, float32
    operands, rows the tensor copies cannot address); the caller then uses `linear`."""
    if not (x.dim() == 2 and w.dim() == 2 and residual.dim() == 2):
        return False
    M, K = x.shape
    N = w.shape[0]
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.float32
            and M > SKINNY_MAX_ROWS and w.shape[1] == K and tuple(residual.shape) == (M, N)
            and x.stride(1) == 1 and w.stride(1) == 1 and residual.stride(1) == 1
            and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and residual.stride(0) % 4 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and residual.data_ptr() % 16 == 0):
        return False
    code = _fn("gtg_gemm_bf16_tcgen05_add")(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(residual),
                                            residual.stride(0), M, N, K, _stream())
    if code == -2:
        return False
    _check(code, "linear_add_residual")
    return True


def qkv_rope_fused_supports(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, cos_sin, n_heads: int,
                            n_kv_heads: int, head_dim: int, kv) -> bool:
    """Whether `linear_qkv_rope` takes these operands: a prompt-sized bfloat16
    product (more rows than the weight-streaming kernels take), heads of 64
    channels, a rotation table, and operands the tensor copies can address."""
    return (cos_sin is not None and kv is not None and head_dim == 64 and x.shape[0] > SKINNY_MAX_ROWS
            and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
            and kv.k.dtype == torch.bfloat16 and kv.head_dim == 64 and kv.n_kv_heads == n_kv_heads
            and w.shape[0] == (n_heads + 2 * n_kv_heads) * 64 and qkv.shape[1] == w.shape[0]
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and qkv.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and qkv.data_ptr() % 16 == 0
            and kv.page_stride % 8 == 0)


def linear_qkv_rope(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, cos_sin: torch.Tensor, n_heads: int,
                    n_kv_heads: int, kv, token_seq: torch.Tensor, slots: torch.Tensor,
                    positions: torch.Tensor) -> None:
    """The query/key/value projection of a prompt with rotation and cache store in
    its epilogue (heads of 64 channels): qkv[:, :n_heads*64] = rotated queries;
    rotated keys and the values go into `kv` at each token's (slot, position); the
    key and value columns of qkv are not written.  What `linear` followed by
    `rope_kv_store` computes, with the rotation applied to the float accumulators."""
    _rows2d(x, "linear_qkv_rope: x"); _rows2d(w, "linear_qkv_rope: w"); _rows2d(qkv, "linear_qkv_rope: qkv")
    _need(qkv_rope_fused_supports(x, w, qkv, cos_sin, n_heads, n_kv_heads, 64, kv),
          "linear_qkv_rope: operands not supported (see qkv_rope_fused_supports)")
    M, K = x.shape
    _need(w.shape[1] == K and qkv.shape[0] == M, "linear_qkv_rope: shapes do not agree")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and tuple(cos_sin.shape) == (M, 32, 2),
          "linear_qkv_rope: cos_sin must be float32 [M, 32, 2]")
    for name, t in (("token_seq", token_seq), ("slots", slots), ("positions", positions)):
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"linear_qkv_rope: {name} must be contiguous int32")
    _check_access("linear_qkv_rope", 0, kv, slots, positions, token_seq, n_items=M)
    _check(_fn("gtg_gemm_bf16_tcgen05_qkv_rope")(
        _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(qkv), qkv.stride(0), M, K, _ptr(cos_sin),
        _ptr(token_seq), _ptr(slots), _ptr(positions), _ptr(kv.block_table), kv.table_stride,
        _ptr(kv.k), _ptr(kv.v), kv.page_stride, n_heads, n_kv_heads, _stream()), "linear_qkv_rope")


def bounded_wait_failures() -> int:
    """Non-zero if a kernel ever gave up a bounded wait on its own asynchronous
    copies (it then returned without a result).  Reading it synchronises."""
    total = 0
    for symbol in ("gtg_gemm_bf16_skinny_status", "gtg_gemm_bf16_tcgen05_status", "gtg_gemm_bf16_swapab_status",
                   "gtg_attention_tcgen05_status", "gtg_latent_status"):
        if _SIGNATURES[symbol][0] in build._LOADED:        # only libraries that have run can have failed
            total += int(_fn(symbol)())
    return total


WAITING_LIBRARIES = ("gemm_bf16_skinny", "gemm_bf16_tcgen05", "gemm_bf16_swapab", "attention_tcgen05", "latent")


def wait_test_hooks(library: str, test_waits: bool) -> None:
    """For tests of the give-up path only.  While set, every launch of `library`
    (one of WAITING_LIBRARIES) takes the test form of its kernel: the same code
    compiled so that it issues none of its asynchronous copies -- the barriers it
    waits on then never complete -- and so that a wait polls a thousand times
    before it gives up.  A kernel launched so returns without a result and
    `bounded_wait_failures()` reads non-zero.  The call synchronises the device and
    clears the library's status word; False restores normal operation."""
    _need(library in WAITING_LIBRARIES, f"wait_test_hooks: {library!r} has no bounded waits; known: {WAITING_LIBRARIES}")
    code = int(_fn(f"gtg_{library}_test_hooks")(1 if test_waits else 0))
    if code != 0:
        raise KernelError(f"wait_test_hooks({library}): CUDA error {code}")


# ----------------------------------------------------------------------- attention
def attention_bf16_supports(head_dim: int) -> bool:
    return bool(_fn("gtg_attention_bf16_supports")(head_dim))


def attention_simple(q: torch.Tensor, out: torch.Tensor, kv, token_seq, slots, positions,
                     n_heads: int, scale: float, window: int = 0, value_dim: Optional[int] = None,
                     chunk: int = 0, gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                     sinks: Optional[torch.Tensor] = None, gate_logits: Optional[torch.Tensor] = None) -> None:
    """One warp per (token, head): the float32 path's attention, for prompts and
    decode steps alike.  `value_dim`: a value is the first so many channels of a
    row of the value plane (default: all of them), and a head of `out` is that wide.
    `chunk` > 0: a token sees the keys of its own stretch of `chunk` positions only.
    `gate`: float32 [N, n_heads], a factor on each head's output; `gate_logits`: float32
    rows of n_heads * value width logits (any row stride) whose sigmoids multiply the
    output channel by channel.  `softcap` c > 0: scores become c tanh(score / c).
    `sinks`: float32 [n_heads]; exp(sinks[h]) joins head h's softmax denominator."""
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    N = q.shape[0]
    vrow = kv.value_dim
    vd = vrow if value_dim is None else int(value_dim)
    _need(kv.k.dtype == q.dtype == out.dtype, "attention: q, out and the cache must share a dtype")
    _need(kv.head_dim <= 2048 and 0 < vd <= min(vrow, 1024),
          f"attention: head_dim {kv.head_dim} exceeds 2048 or the value width {vd} exceeds 1024 or the stored row")
    _need(gate is None or (gate.dtype == torch.float32 and gate.is_contiguous() and tuple(gate.shape) == (N, n_heads)),
          "attention: gate must be contiguous float32 [N, n_heads]")
    _need(q.shape[1] >= n_heads * kv.head_dim and out.shape[1] >= n_heads * vd, "attention: q or out is too narrow")
    gate_ld = 0
    if gate_logits is not None:
        _need(gate is None, "attention: a gate per head or logits per channel, not both")
        _rows2d(gate_logits, "attention: gate_logits")
        _need(gate_logits.dtype == torch.float32 and tuple(gate_logits.shape) == (N, n_heads * vd),
              "attention: gate_logits must be float32 [N, n_heads * value width]")
        gate, gate_ld = gate_logits, gate_logits.stride(0)
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads),
          "attention: sinks must be contiguous float32 [n_heads]")
    _need(softcap >= 0, "attention: the cap on the scores must not be negative")
    _check_access("attention_simple", 0, kv, slots, positions, token_seq, n_items=N)
    _check(_fn("gtg_attention_simple")(_dt(q), _ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                       _ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table),
                                       kv.table_stride, _ptr(token_seq), _ptr(slots), _ptr(positions),
                                       N, n_heads, kv.n_kv_heads, kv.head_dim, vd, vrow, float(scale), int(window),
                                       int(chunk), _ptr(gate), int(gate_ld), float(softcap), _ptr(sinks), _stream()),
           "attention_simple")


def attention_general(q: torch.Tensor, out: torch.Tensor, kv, ctx, n_heads: int, scale: float, window: int = 0,
                      chunk: int = 0, gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                      gate_logits: Optional[torch.Tensor] = None) -> None:
    """Attention for mixers whose keys and values differ in size, whose keys are seen
    within stretches of `chunk` positions, or whose heads carry a gate: `ctx` is the
    step's context (rows, positions, sequences).  out[n, h] = gate[n, h] *
    softmax(q . K * scale over the visible keys) V.  bfloat16 heads of a multiple of 8
    channels up to 128 take the tensor-core kernel (`attention_masked_bf16`); float32
    and other widths the plain one; steps that bring more than one token a sequence, with
    keys and values of 64 or 128 channels alike, the prompt attention on tcgen05.
    `softcap` c > 0: scores become c tanh(score / c) after the scale.  `gate_logits`: float32
    rows [N, n_heads * value width] whose sigmoids multiply the output channel by channel."""
    if (q.dtype == torch.bfloat16 and not ctx.is_decode and kv.value_dim == kv.head_dim and attention_tcgen05_supports(kv)
            and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0):
        # the logits' sigmoids multiply the output in a kernel of their own here: in this kernel's epilogue a thread
        # holds a query's row and reads its 64 or 128 logits alone, which cost the kernel 37 us of 94 at 2,048 tokens
        # against 10 us for the pass over rows
        attention_prefill_tcgen05(q, out, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos, ctx.n_seqs, ctx.max_q_len, n_heads, scale,
                                  window, chunk, gate, softcap=softcap)
        if gate_logits is not None:
            sigmoid_gate(out[:, : n_heads * kv.value_dim], gate_logits)
        return
    if q.dtype == torch.bfloat16 and attention_masked_supports(kv) and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and scale > 0:
        splits = int(_fn("gtg_attention_masked_splits")(ctx.n_seqs, ctx.max_q_len, n_heads, kv.n_kv_heads, ctx.max_kv_len,
                                                        int(window), int(chunk)))
        scratch = None
        if splits > 1:
            scratch = ctx.rt.empty(int(_fn("gtg_attention_masked_scratch_floats")(q.shape[0], n_heads, kv.value_dim, splits)),
                                   dtype=torch.float32)
        attention_masked_bf16(q, out, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos, ctx.n_seqs, ctx.max_q_len, n_heads, scale,
                              window, chunk, gate, splits, scratch, softcap=softcap, gate_logits=gate_logits)
        return
    attention_simple(q, out, kv, ctx.token_seq, ctx.slots, ctx.positions, n_heads, scale, window, chunk=chunk, gate=gate,
                     softcap=softcap, gate_logits=gate_logits)


def attention_masked_supports(kv) -> bool:
    return (kv.k.dtype == torch.bfloat16 and bool(_fn("gtg_attention_masked_supports")(kv.head_dim, kv.value_dim))
            and kv.page_stride % 8 == 0)


def attention_masked_bf16(q, out, kv, cu_seqlens, slots, start_pos, n_seqs: int, max_q_len: int, n_heads: int, scale: float,
                          window: int = 0, chunk: int = 0, gate: Optional[torch.Tensor] = None, n_splits: int = 1,
                          scratch: Optional[torch.Tensor] = None, softcap: float = 0.0,
                          gate_logits: Optional[torch.Tensor] = None) -> None:
    """The tensor-core form of `attention_general`: rows are (token, query head of a group)
    pairs, a block of 64 rows reads each page once for the group.  Prompts, portions and
    decode steps alike; `n_splits` > 1 cuts every tile's pages into that many shares, merged
    through `scratch` (float32, `gtg_attention_masked_scratch_floats`).  `softcap` and
    `gate_logits` as in `attention_simple`."""
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    N = q.shape[0]
    gate_ld = 0
    if gate_logits is not None:
        _need(gate is None, "attention: a gate per head or logits per channel, not both")
        _rows2d(gate_logits, "attention: gate_logits")
        _need(gate_logits.dtype == torch.float32 and tuple(gate_logits.shape) == (N, n_heads * kv.value_dim),
              "attention: gate_logits must be float32 [N, n_heads * value width]")
        gate, gate_ld = gate_logits, gate_logits.stride(0)
    _need(softcap >= 0, "attention: the cap on the scores must not be negative")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16, "attention_masked_bf16: bfloat16 only")
    _need(q.shape[1] >= n_heads * kv.head_dim and out.shape[1] >= n_heads * kv.value_dim, "attention: q or out is too narrow")
    _need(gate is None or gate_ld > 0 or (gate.dtype == torch.float32 and gate.is_contiguous() and tuple(gate.shape) == (N, n_heads)),
          "attention: gate must be contiguous float32 [N, n_heads]")
    _need(scale > 0, "attention_masked_bf16: the scale must be positive")
    _int32("attention", cu_seqlens, slots, start_pos)
    if n_splits > 1:
        need = int(_fn("gtg_attention_masked_scratch_floats")(N, n_heads, kv.value_dim, n_splits))
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
              f"attention_masked_bf16: {n_splits} shares need {need} floats of scratch")
    _check_access("attention_masked_bf16", 2, kv, slots, start_pos=start_pos, cu_seqlens=cu_seqlens)
    _check(_fn("gtg_attention_masked_bf16")(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv.k), _ptr(kv.v), kv.page_stride,
                                            _ptr(kv.block_table), kv.table_stride, _ptr(cu_seqlens), _ptr(slots), _ptr(start_pos),
                                            int(n_seqs), int(max_q_len), N, n_heads, kv.n_kv_heads, kv.head_dim, kv.value_dim,
                                            float(scale), int(window), int(chunk), _ptr(gate), int(n_splits), _ptr(scratch),
                                            float(softcap), int(gate_ld), _stream()),
           "attention_masked_bf16")


def attention_prefill_bf16(q, out, kv, cu_seqlens, slots, start_pos, n_seqs: int, max_q_len: int,
                           n_heads: int, scale: float, window: int = 0) -> None:
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16,
          "attention_prefill_bf16: bfloat16 only")
    _need(attention_bf16_supports(kv.head_dim),
          f"attention_prefill_bf16: head_dim {kv.head_dim} is not a multiple of 16 up to 128")
    _check_access("attention_prefill_bf16", 2, kv, slots, start_pos=start_pos, cu_seqlens=cu_seqlens, n_items=n_seqs)
    _check(_fn("gtg_attention_prefill_bf16")(_ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                             _ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table),
                                             kv.table_stride, _ptr(cu_seqlens), _ptr(slots), _ptr(start_pos),
                                             n_seqs, max_q_len, n_heads, kv.n_kv_heads, kv.head_dim,
                                             float(scale), int(window), _stream()), "attention_prefill_bf16")


def attention_tcgen05_supports(kv) -> bool:
    """The tensor-core prompt attention serves heads of 64 or 128 channels whose
    keys and values lie page by page as [k|v][head][token][channel]."""
    hd = kv.head_dim
    return (kv.k.dtype == torch.bfloat16 and hd in (64, 128)
            and kv.page_stride == 2 * kv.n_kv_heads * 64 * hd
            and kv.v.data_ptr() - kv.k.data_ptr() == kv.n_kv_heads * 64 * hd * 2)


def attention_prefill_tcgen05(q, out, kv, cu_seqlens, slots, start_pos, n_seqs: int, max_q_len: int,
                              n_heads: int, scale: float, window: int = 0, chunk: int = 0,
                              gate: Optional[torch.Tensor] = None, softcap: float = 0.0,
                              gate_logits: Optional[torch.Tensor] = None) -> None:
    """Prompt attention on tcgen05 (128 queries x one head per thread block).  `chunk` > 0:
    a query sees the keys of its own stretch of `chunk` positions only; `gate`: float32
    [N, n_heads], a factor on each head's output.  `softcap` and `gate_logits` as in
    `attention_simple`."""
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    gate_ld = 0
    if gate_logits is not None:
        _need(gate is None, "attention: a gate per head or logits per channel, not both")
        _rows2d(gate_logits, "attention: gate_logits")
        _need(gate_logits.dtype == torch.float32 and tuple(gate_logits.shape) == (q.shape[0], n_heads * kv.head_dim),
              "attention: gate_logits must be float32 [N, n_heads * value width]")
        gate, gate_ld = gate_logits, gate_logits.stride(0)
    _need(softcap >= 0, "attention: the cap on the scores must not be negative")
    _need(gate is None or gate_ld > 0 or (gate.dtype == torch.float32 and gate.is_contiguous() and tuple(gate.shape) == (q.shape[0], n_heads)),
          "attention: gate must be contiguous float32 [N, n_heads]")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "attention_prefill_tcgen05: bfloat16 only")
    _need(attention_tcgen05_supports(kv),
          "attention_prefill_tcgen05: needs head_dim 64 or 128 and keys and values of a page side by side")
    _check_access("attention_prefill_tcgen05", 2, kv, slots, start_pos=start_pos, cu_seqlens=cu_seqlens, n_items=n_seqs)
    _check(_fn("gtg_attention_prefill_tcgen05")(_ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0),
                                                _ptr(kv.k), _ptr(kv.v), kv.page_stride, kv.k.shape[0],
                                                _ptr(kv.block_table), kv.table_stride, _ptr(cu_seqlens),
                                                _ptr(slots), _ptr(start_pos), n_seqs, max_q_len, n_heads,
                                                kv.n_kv_heads, kv.head_dim, float(scale), int(window), int(chunk),
                                                _ptr(gate), float(softcap), int(gate_ld), _stream()),
           "attention_prefill_tcgen05")


def attention_decode_plan(n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int, max_kv_len: int,
                          window: int = 0, total_kv_len: int = 0):
    """(n_splits, chunk_pages, ring_pages) for `attention_decode_bf16`: into how
    many thread blocks the keys of the longest sequence's (sequence, key/value
    head) pairs are split, how many pages one split takes (a shorter sequence
    then takes as many splits as its own pages need), and which form of the
    kernel runs: the one with three pages in its ring and more blocks to an SM,
    or, for a batch that brings about one block per place on the device, the one
    with four.  `total_kv_len` is the batch's keys altogether (0: all sequences
    as long as the longest).  The library estimates, for every chunk size, the
    waves of blocks on this device (its multiprocessor count and the kernel's
    own occupancy, from the runtime) and the time the memory needs, and takes
    the least.  The choice depends on the batch's lengths and the window, never
    on the data."""
    chunk, ring = c_int(0), c_int(0)
    n = int(_fn("gtg_attention_decode_plan")(n_seqs, n_heads, n_kv_heads, head_dim, int(max_kv_len),
                                             int(total_kv_len), int(window), ctypes.byref(chunk), ctypes.byref(ring)))
    if n < 1:
        raise KernelError(f"attention_decode_plan: {_CODES.get(n, n)}")
    return n, int(chunk.value), int(ring.value)


def attention_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(_fn("gtg_attention_decode_scratch_floats")(n_seqs, n_heads, head_dim, n_splits))


def attention_decode_bf16(q, out, kv, slots, positions, n_heads: int, scale: float, window: int,
                          n_splits: int, scratch: Optional[torch.Tensor], unrotated=None,
                          chunk_pages: int = 0, ring_pages: int = 0) -> None:
    """Attention of one new token per sequence over the cache (keys split over
    `n_splits` thread blocks per head group).  Normally q is rotated and the new
    keys and values are in the cache (`rope_kv_store`).  With
    unrotated=(cos_sin, k_new, v_new, store) the kernel does that work itself: q
    and k_new come as the projection wrote them, cos_sin float32 [B, hd/2, 2] or
    None rotates them, and the new key and value are attended to and, if `store`,
    written to the cache; k_new None for a layer that reads another's cache.
    With `chunk_pages` (from `attention_decode_plan`; 0: every sequence is cut into
    n_splits equal parts) a sequence is cut into as many equal parts as give parts
    of about that many pages, at most n_splits: shorter sequences take fewer splits.
    Blocks start sequence by sequence in batch order: with very unequal lengths, put
    the long sequences first.  `ring_pages` (from the plan; 0: the default) picks
    the form of the kernel; the result does not depend on it."""
    _rows2d(q, "attention: q"); _rows2d(out, "attention: out")
    B = q.shape[0]
    _need(chunk_pages >= 0, "attention_decode_bf16: chunk_pages must not be negative")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kv.k.dtype == torch.bfloat16,
          "attention_decode_bf16: bfloat16 only")
    _need(attention_bf16_supports(kv.head_dim),
          f"attention_decode_bf16: head_dim {kv.head_dim} is not a multiple of 16 up to 128")
    _check_access("attention_decode_bf16", 1, kv, slots, positions, n_items=B)
    if n_splits > 1:
        need = attention_decode_scratch_floats(B, n_heads, kv.head_dim, n_splits)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
              and scratch.numel() >= need, f"attention_decode_bf16: scratch needs {need} floats")
    if unrotated is not None:
        cos_sin, k_new, v_new, store = unrotated
        hd = kv.head_dim
        if cos_sin is not None:
            _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and tuple(cos_sin.shape) == (B, hd // 2, 2),
                  "attention_decode_bf16: cos_sin must be float32 [B, hd/2, 2]")
        if k_new is not None:
            for name, t in (("k_new", k_new), ("v_new", v_new)):
                _need(t is not None and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1
                      and t.stride(0) == q.stride(0) and tuple(t.shape) == (B, kv.n_kv_heads * hd),
                      f"attention_decode_bf16: {name} must be bfloat16 [B, n_kv * hd] with q's row stride")
        _check(_fn("gtg_attention_decode_rope_bf16")(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv.k), _ptr(kv.v), kv.page_stride,
            _ptr(kv.block_table), kv.table_stride, _ptr(slots), _ptr(positions), B, n_heads, kv.n_kv_heads,
            kv.head_dim, float(scale), int(window), int(n_splits), _ptr(scratch), _ptr(cos_sin),
            _ptr(k_new), _ptr(v_new) if k_new is not None else None, 1 if store else 0,
            int(chunk_pages), int(ring_pages), _stream()),
            "attention_decode_bf16")
        return
    _check(_fn("gtg_attention_decode_bf16")(_ptr(q), q.stride(0), _ptr(out), out.stride(0),
                                            _ptr(kv.k), _ptr(kv.v), kv.page_stride, _ptr(kv.block_table),
                                            kv.table_stride, _ptr(slots), _ptr(positions), B, n_heads,
                                            kv.n_kv_heads, kv.head_dim, float(scale), int(window),
                                            int(n_splits), _ptr(scratch), int(chunk_pages), int(ring_pages),
                                            _stream()),
           "attention_decode_bf16")


# ---------------------------------------------------------- attention through a latent
def latent_prepare(q: torch.Tensor, dkv: Optional[torch.Tensor], cos_sin: torch.Tensor, norm_weight: Optional[torch.Tensor],
                   eps: float, kv, token_seq, slots, positions, q_full: Optional[torch.Tensor], n_heads: int, dim: int,
                   rot: int, rank: int, rows_out: Optional[torch.Tensor] = None, pairing: str = "interleaved") -> None:
    """Per token: with a down projection `dkv` [N, rank + rot], the latent
    rmsnorm(dkv[:, :rank]) * norm_weight and the rotated dkv[:, rank:] go into the
    token's cache row [rank + rot] of `kv`; and every head's rotated query part
    q[:, h, dim:] goes to q_full[:, h, rank:] (q [N, heads * (dim + rot)], q_full
    [N, heads * (rank + rot)]).  Of a rotated part's channels the first 2 P turn,
    pairs (2i, 2i+1), or (i, i + P) with `pairing` "half", by cos_sin [N, P, 2]; the rest pass unchanged.  Without q_full the
    rotated query parts are written back into q.  `rows_out` [N, rank + rot], with a down
    projection, receives every token's cache row once more, token by token."""
    _rows2d(q, "latent_prepare: q")
    N = q.shape[0]
    _need(rot % 2 == 0 and rot > 0, "latent_prepare: an even number of rotated channels is needed")
    _need(pairing in ROTARY_PAIRINGS, f"latent_prepare: pairing {pairing!r} is not known; known: {sorted(ROTARY_PAIRINGS)}")
    _need(q.shape[1] == n_heads * (dim + rot), "latent_prepare: q must be [N, heads*(dim+rot)]")
    if q_full is not None:
        _rows2d(q_full, "latent_prepare: q_full")
        _need(tuple(q_full.shape) == (N, n_heads * (rank + rot)) and q.dtype == q_full.dtype,
              "latent_prepare: q_full must be [N, heads*(rank+rot)] of q's dtype")
    if rows_out is not None:
        _rows2d(rows_out, "latent_prepare: rows_out")
        _need(dkv is not None and tuple(rows_out.shape) == (N, rank + rot) and rows_out.dtype == q.dtype,
              "latent_prepare: rows_out needs a down projection and must be [N, rank+rot] of q's dtype")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.dim() == 3 and cos_sin.shape[0] == N
          and cos_sin.shape[2] == 2 and 2 * cos_sin.shape[1] <= rot, "latent_prepare: cos_sin must be float32 [N, pairs <= rot/2, 2]")
    rdims = 2 * cos_sin.shape[1]
    _int32("latent_prepare", token_seq, slots, positions)
    if dkv is not None:
        _rows2d(dkv, "latent_prepare: dkv")
        _need(tuple(dkv.shape) == (N, rank + rot) and dkv.dtype == q.dtype, "latent_prepare: dkv must be [N, rank+rot] of q's dtype")
        _need(kv is not None and kv.k.dtype == q.dtype and kv.n_kv_heads == 1 and kv.head_dim == rank + rot,
              "latent_prepare: the cache entry must hold one head of rank + rot channels")
        _need(norm_weight is not None and norm_weight.dtype == torch.float32 and norm_weight.is_contiguous()
              and norm_weight.numel() == rank, "latent_prepare: norm_weight must be float32 [rank]")
        _check_access("latent_prepare", 0, kv, slots, positions, token_seq, n_items=N)
        args = (_ptr(kv.k), kv.page_stride, _ptr(kv.block_table), kv.table_stride)
    else:
        args = (None, 0, None, 0)
    _check(_fn("gtg_latent_prepare")(_dt(q), _ptr(q), q.stride(0), _ptr(dkv), dkv.stride(0) if dkv is not None else 0,
                                     _ptr(cos_sin), _ptr(norm_weight), float(eps), *args, _ptr(token_seq), _ptr(slots),
                                     _ptr(positions), _ptr(q_full), q_full.stride(0) if q_full is not None else 0, N, n_heads, dim,
                                     rot, rdims, rank, _ptr(rows_out), rows_out.stride(0) if rows_out is not None else 0,
                                     ROTARY_PAIRINGS[pairing], _stream()),
           "latent_prepare")


def latent_attention_supports(kv, rank: int) -> bool:
    """Whether the tensor-core attention over latent rows takes this cache entry:
    bfloat16 rows of a multiple of 16 channels, a multiple of 8 (up to 512) of them values."""
    return (kv is not None and kv.k.dtype == torch.bfloat16 and kv.n_kv_heads == 1 and kv.page_stride % 8 == 0
            and bool(_fn("gtg_latent_attention_supports")(kv.head_dim, int(rank))))


def latent_attention_plan(n_seqs: int, max_q_len: int, n_heads: int, head_dim: int, rank: int, max_kv_len: int,
                          window: int = 0):
    """(n_splits, scratch floats per token) for `latent_attention_bf16`: into how many
    runs the keys of a block of query rows are cut so that a step with few rows
    (a decode step) still fills the device; 1 for prompts.  It depends on the
    step's sizes only, never on the data."""
    splits = int(_fn("gtg_latent_attention_splits")(n_seqs, max_q_len, n_heads, head_dim, int(max_kv_len), int(window)))
    if rank % 2:
        splits = 1
    return splits, (splits * n_heads * (rank + 2) if splits > 1 else 0)


def latent_attention_bf16(q: torch.Tensor, out: torch.Tensor, kv, cu_seqlens, slots, start_pos, n_seqs: int,
                          max_q_len: int, n_heads: int, rank: int, scale: float, window: int = 0,
                          n_splits: int = 1, scratch: Optional[torch.Tensor] = None,
                          sinks: Optional[torch.Tensor] = None) -> None:
    """Attention of every (token, head) of the step over its sequence's cache rows
    (one shared head of kv.head_dim channels, the first `rank` of which are the
    values): q [N, heads * head_dim] folded query rows, out [N, heads * rank].
    Causal, over the last `window` keys (0: all).  Prompts, portions and single
    tokens alike.  With n_splits > 1 (`latent_attention_plan`) the keys are cut into
    runs whose results a second kernel merges; `scratch` then holds N times the
    plan's floats per token.  `sinks`: float32 [n_heads]; exp(sinks[h]) joins head h's
    softmax denominator without a key or a value."""
    _rows2d(q, "latent_attention: q"); _rows2d(out, "latent_attention: out")
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads),
          "latent_attention_bf16: sinks must be contiguous float32 [n_heads]")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and latent_attention_supports(kv, rank),
          "latent_attention_bf16: bfloat16 rows of a multiple of 16 channels, a multiple of 8 of them values")
    _need(q.shape[1] == n_heads * kv.head_dim and out.shape[1] == n_heads * rank and q.stride(0) % 8 == 0
          and out.stride(0) % 2 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 4 == 0,
          "latent_attention_bf16: q [N, heads * head_dim] and out [N, heads * rank], aligned rows")
    _int32("latent_attention_bf16", cu_seqlens, slots, start_pos)
    if n_splits > 1:
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
              and scratch.numel() >= n_splits * q.shape[0] * n_heads * (rank + 2), "latent_attention_bf16: scratch is too small")
    _check_access("latent_attention_bf16", 2, kv, slots, start_pos=start_pos, cu_seqlens=cu_seqlens, n_items=n_seqs)
    _check(_fn("gtg_latent_attention_bf16")(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kv.k), kv.page_stride,
                                            _ptr(kv.block_table), kv.table_stride, _ptr(cu_seqlens), _ptr(slots), _ptr(start_pos),
                                            int(n_seqs), int(max_q_len), n_heads, kv.head_dim, int(rank), float(scale), int(window),
                                            int(n_splits), _ptr(scratch) if n_splits > 1 else None, q.shape[0], _ptr(sinks), _stream()),
           "latent_attention_bf16")


def expanded_attention_supports(dim: int, rot: int, v_dim: int) -> bool:
    """Whether `expanded_attention_bf16` takes heads of dim + rot key channels and v_dim value channels."""
    return bool(_fn("gtg_expanded_attention_supports")(int(dim), int(rot), int(v_dim)))


def latent_spread(k_rot: torch.Tensor, runs: torch.Tensor, n_heads: int, offset: int) -> None:
    """runs[n, h, offset : offset + rot] = k_rot[n, :] for every head: the one rotated key
    part of a token into its place in every head's run (runs [N, heads * per], bfloat16)."""
    _rows2d(k_rot, "latent_spread: k_rot"); _rows2d(runs, "latent_spread: runs")
    N, rot = k_rot.shape
    _need(runs.shape[0] == N and runs.shape[1] % n_heads == 0 and k_rot.dtype == torch.bfloat16 and runs.dtype == torch.bfloat16,
          "latent_spread: bfloat16 k_rot [N, rot] and runs [N, heads * per]")
    _check(_fn("gtg_latent_spread")(_ptr(k_rot), k_rot.stride(0), _ptr(runs), runs.stride(0), N, n_heads, runs.shape[1] // n_heads,
                                    int(offset), rot, _stream()), "latent_spread")


def expanded_attention_bf16(q: torch.Tensor, runs: torch.Tensor, out: torch.Tensor, cu_seqlens, n_seqs: int, max_q_len: int,
                            n_heads: int, dim: int, rot: int, v_dim: int, scale: float, window: int = 0,
                            sinks: Optional[torch.Tensor] = None) -> None:
    """Attention of a step whose sequences all start at their first token, over the
    step's own rows with keys and values per head: q [N, heads * (dim + rot)] (a
    head's rotated part last, rotated); runs [N, heads * (dim + v_dim + rot)], per
    token and head [unrotated key | value | rotated key part] -> out [N, heads *
    v_dim].  Causal within each sequence, over the last `window` keys (0: all).  `sinks`:
    float32 [n_heads], as in `latent_attention_bf16`."""
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == n_heads),
          "expanded_attention_bf16: sinks must be contiguous float32 [n_heads]")
    for name, t in (("q", q), ("runs", runs), ("out", out)):
        _rows2d(t, f"expanded_attention: {name}")
        _need(t.dtype == torch.bfloat16, "expanded_attention_bf16: bfloat16 only")
    N = q.shape[0]
    _need(q.shape[1] == n_heads * (dim + rot) and tuple(runs.shape) == (N, n_heads * (dim + v_dim + rot))
          and tuple(out.shape) == (N, n_heads * v_dim), "expanded_attention_bf16: shapes do not agree")
    _need(expanded_attention_supports(dim, rot, v_dim), "expanded_attention_bf16: head sizes not supported")
    _int32("expanded_attention_bf16", cu_seqlens)
    _check(_fn("gtg_expanded_attention_bf16")(_ptr(q), q.stride(0), _ptr(runs), runs.stride(0), _ptr(out), out.stride(0),
                                              _ptr(cu_seqlens), int(n_seqs), int(max_q_len), n_heads, dim, rot, v_dim, float(scale),
                                              int(window), _ptr(sinks), _stream()), "expanded_attention_bf16")


# ------------------------------------------------------------------ routed experts
MOE_TILE_ROWS = 64


MOE_SCORING = {"softmax_chosen": 0, "sigmoid": 1}


def moe_route(x: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], chosen: torch.Tensor,
              weights: torch.Tensor, scoring: str = "softmax_chosen") -> None:
    """Router logits x . router^T + bias in float; chosen[n, :] = the `top` largest
    (ties: the lower index), weights[n, :] = softmax over those logits alone
    ("softmax_chosen") or each chosen logit's own sigmoid ("sigmoid")."""
    _need(scoring in MOE_SCORING, f"moe_route: scoring {scoring!r} is not known; known: {sorted(MOE_SCORING)}")
    _rows2d(x, "moe_route: x")
    N, H = x.shape
    E, top = router.shape[0], chosen.shape[1]
    _need(router.dtype == torch.float32 and router.is_contiguous() and tuple(router.shape) == (E, H), "moe_route: router must be float32 [E, H]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == E), "moe_route: bias must be float32 [E]")
    _need(chosen.dtype == torch.int32 and chosen.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()
          and tuple(chosen.shape) == (N, top) and tuple(weights.shape) == (N, top) and 0 < top <= E,
          "moe_route: chosen int32 [N, top] and weights float32 [N, top]")
    _check(_fn("gtg_moe_route")(_dt(x), _ptr(x), x.stride(0), _ptr(router), _ptr(bias), _ptr(chosen), _ptr(weights), N, H, E, top,
                                MOE_SCORING[scoring], _stream()), "moe_route")


def moe_tiles_cap(n_items: int, n_experts: int, tile: int = MOE_TILE_ROWS) -> int:
    """Tiles of `tile` rows that hold any assignment of n_items (token, expert) pairs."""
    return (n_items + tile - 1) // tile + n_experts


def moe_arrange(chosen: torch.Tensor, n_experts: int, row_item: torch.Tensor, item_row: torch.Tensor,
                tile_expert: torch.Tensor, tile: int = MOE_TILE_ROWS) -> None:
    """Order the (token, expert) pairs by expert, every expert's rows padded to whole
    tiles: row_item[row] = pair or -1, item_row[pair] = row, tile_expert[tile] = expert or -1."""
    n_items = chosen.numel()
    cap = tile_expert.numel()
    _int32("moe_arrange", chosen, row_item, item_row, tile_expert)
    _need(cap >= moe_tiles_cap(n_items, n_experts, tile) and row_item.numel() == cap * tile and item_row.numel() == n_items,
          "moe_arrange: tile_expert [tiles], row_item [tiles * tile], item_row [pairs]")
    _check(_fn("gtg_moe_arrange")(_ptr(chosen), n_items, n_experts, tile, cap, _ptr(row_item), _ptr(item_row), _ptr(tile_expert),
                                  _stream()), "moe_arrange")


def moe_gather(x: torch.Tensor, row_item: torch.Tensor, item_div: int, out: torch.Tensor,
               weights: Optional[torch.Tensor] = None) -> None:
    """out[row, :] = x[row_item[row] // item_div, :], zeros for padding rows: the inputs of a
    step's (token, expert) pairs in arranged order (bfloat16, a multiple of 8 channels).
    With `weights` (float32, one per pair) a row is weights[pair] * x[token, :], the product
    in float and rounded once; that form takes either dtype and any width."""
    _rows2d(x, "moe_gather: x")
    if weights is not None or x.dtype != torch.bfloat16 or x.shape[1] % 8 or x.stride(0) % 8:
        _need(out.dtype == x.dtype and out.is_contiguous() and tuple(out.shape) == (row_item.numel(), x.shape[1]),
              "moe_gather: out must be contiguous [rows, H] of x's dtype")
        _need(weights is None or (weights.dtype == torch.float32 and weights.is_contiguous()),
              "moe_gather: weights must be contiguous float32, one per pair")
        _int32("moe_gather", row_item)
        _check(_fn("gtg_moe_gather_scaled")(_dt(x), _ptr(x), x.stride(0), _ptr(row_item), int(item_div), _ptr(weights), _ptr(out),
                                            out.shape[0], x.shape[1], _stream()), "moe_gather")
        return
    _need(x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.is_contiguous()
          and tuple(out.shape) == (row_item.numel(), x.shape[1]), "moe_gather: bfloat16 x [N, H] and out [rows, H]")
    _int32("moe_gather", row_item)
    _check(_fn("gtg_moe_gather")(_ptr(x), x.stride(0), _ptr(row_item), int(item_div), _ptr(out), out.shape[0], x.shape[1], _stream()),
           "moe_gather")


def moe_product_fused_supports(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `moe_product` runs these operands on the tensor cores (where it can
    apply the gated silu in its epilogue)."""
    return w.dim() == 3 and _grouped_ok(a, w, w.shape[2], a.stride(0), w.shape[1] * w.shape[2])


def moe_product(a: torch.Tensor, row_item: torch.Tensor, item_div: int, w: torch.Tensor, tile_expert: torch.Tensor,
                out: torch.Tensor, epilogue: str = "none") -> None:
    """out[row, :] = a[source(row), :] . w[expert of the row's tile]^T over arranged
    rows.  item_div > 0: the source is the pair's token, row_item[row] // item_div
    (a holds tokens); 0: the row itself (a holds arranged rows, zeros in its padding
    rows: `moe_gather`), which in tiles of 128 takes the prompt-sized tensor-memory
    product.  w [E, N, K].  The tile is out's rows over tile_expert's length: 64, or 128 on the tensor
    cores.  epilogue="swiglu" (tensor cores only: `moe_product_fused_supports`):
    every w[e] is laid out by `interleave_gate_up` and out [rows, N/2] = silu(gate) * up.
    epilogue="relu2" | "gelu_tanh" | "silu": that activation of the product, applied to the float
    sums inside the tensor-core kernels, by the `activation` kernel behind the plain one."""
    _rows2d(a, "moe_product: a"); _rows2d(out, "moe_product: out")
    E, N, K = w.shape
    cap = tile_expert.numel()
    tile = out.shape[0] // max(cap, 1)
    _need(epilogue in ("none", "swiglu") or epilogue in ACTIVATIONS, f"moe_product: unknown epilogue {epilogue!r}")
    if epilogue in ACTIVATIONS and not moe_product_fused_supports(a, w):
        # the plain product has no epilogue: the activation runs behind it
        moe_product(a, row_item, item_div, w, tile_expert, out)
        activation(out, epilogue)
        return
    n_out = N // 2 if epilogue == "swiglu" else N
    epi_code = 1 if epilogue == "swiglu" else EPILOGUE_ACTIVATION + ACTIVATIONS[epilogue] if epilogue in ACTIVATIONS else 0
    _need(w.is_contiguous() and a.dtype == w.dtype and a.shape[1] == K, "moe_product: a [*, K] and contiguous w [E, N, K] of one dtype")
    _need(tuple(out.shape) == (cap * tile, n_out) and out.dtype in (a.dtype, torch.float32), "moe_product: out must be [tiles * tile, N]")
    _need(item_div > 0 or a.shape[0] == out.shape[0], "moe_product: a must hold the arranged rows")
    _int32("moe_product", row_item, tile_expert)
    if moe_product_fused_supports(a, w):
        _need(tile in (64, 128), f"moe_product: tiles of 64 or 128 rows, not {tile}")
        _need(epilogue != "swiglu" or N % 16 == 0, "moe_product: the fused gated silu needs a multiple of 16 rows per expert")
        if (tile == 128 and item_div == 0 and out.data_ptr() % 16 == 0
                and out.stride(0) % (4 if out.dtype == torch.float32 else 8) == 0):
            # arranged rows in tiles of 128: the prompt-sized product (tensor copies, tensor memory)
            _check(_fn("gtg_gemm_bf16_tcgen05_grouped")(_ptr(a), a.stride(0), _ptr(w), K, _ptr(out), out.stride(0),
                                                        1 if out.dtype == torch.float32 else 0, cap * tile, N, K,
                                                        epi_code, _ptr(tile_expert), E, _stream()),
                   "moe_product(tcgen05)")
            return
        _check(_fn("gtg_gemm_bf16_grouped")(_ptr(a), a.stride(0), 0, _ptr(row_item), int(item_div), _ptr(w), K, N * K,
                                            _ptr(tile_expert), _ptr(out), out.stride(0), 0, 1 if out.dtype == torch.float32 else 0,
                                            1, cap * tile, N, K, tile, epi_code, None, 0, 0, _stream()),
               "moe_product(bfloat16)")
        return
    _need(epilogue == "none" and tile == MOE_TILE_ROWS, "moe_product: the plain product has tiles of 64 rows and no epilogue")
    _check(_fn("gtg_moe_product_simt")(_dt(a), 1 if out.dtype == torch.float32 else 0, _ptr(a), a.stride(0), _ptr(row_item),
                                       int(item_div), _ptr(w), K, N * K, _ptr(tile_expert), cap, _ptr(out), out.stride(0), N, K,
                                       _stream()), "moe_product")


def moe_combine(y: torch.Tensor, item_row: torch.Tensor, weights: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[t, :] = sum_k weights[t, k] * y[item_row[t * top + k], :] (float sums, k in
    order; out float32 or bfloat16).  weights None: the plain sum of a token's rows."""
    _rows2d(y, "moe_combine: y")
    N = out.shape[0]
    top = item_row.numel() // max(N, 1)
    H = y.shape[1]
    _need(y.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (N, H) and item_row.numel() == N * top
          and (weights is None or (weights.dtype == torch.float32 and weights.is_contiguous() and tuple(weights.shape) == (N, top))),
          "moe_combine: y float32 [rows, H], weights float32 [N, top], out [N, H]")
    _int32("moe_combine", item_row)
    _check(_fn("gtg_moe_combine")(_dt(out), _ptr(y), y.stride(0), _ptr(item_row), _ptr(weights), _ptr(out), N, H, top, _stream()),
           "moe_combine")


# ------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the maximum of logits[r,:]."""
    _rows2d(logits, "argmax: logits")
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= R and out.is_contiguous(),
          "argmax: logits float32, out int32 [R]")
    _check(_fn("gtg_argmax")(_ptr(logits), logits.stride(0), R, V, _ptr(out), _stream()), "argmax")


def sample_temperature(logits: torch.Tensor, temperature: float, seed: int, sequence_ids: torch.Tensor,
                       steps: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] ~ softmax(logits[r,:] / temperature), drawn with the uniform that
    (seed, sequence_ids[r], steps[r]) determine."""
    _rows2d(logits, "sample: logits")
    R, V = logits.shape
    _need(temperature > 0, "sample_temperature: the temperature must be positive (0 means greedy: use argmax)")
    for name, t in (("sequence_ids", sequence_ids), ("steps", steps), ("out", out)):
        _need(t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= R, f"sample: {name} must be int32 [R]")
    _check(_fn("gtg_sample_temperature")(_ptr(logits), logits.stride(0), R, V, float(temperature),
                                         int(seed) & (2**64 - 1), _ptr(sequence_ids), _ptr(steps),
                                         _ptr(out), _stream()), "sample_temperature")
