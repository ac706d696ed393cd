"""Python face of the CUDA kernels: loads the shared library built from
``csrc/`` and wraps each exported entry point.  Every wrapper checks dtypes,
shapes and contiguity, launches on torch's current stream and raises on a launch
error.  There is no fallback: without a CUDA device or without the library these
functions raise.

Matrix products in bfloat16 go to the vendor library through ``torch.mm`` (the
reference's ``nn.Linear`` does the same, batchspec/models/modules/attention/base.py:32-39);
float32 products use this package's own FFMA kernel so that no reduced-precision
mode can slip in.
"""
from __future__ import annotations

import ctypes
import sys
import threading
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

_lib = None
_lock = threading.Lock()
_launches = 0          # kernels of this package launched (for the benchmark's count)

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t}")


_SIGNATURES = {
    "bspec_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "bspec_add_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_float,
                          c_int, c_void_p, c_int, c_void_p],
    "bspec_gather_rows_add": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                              c_void_p],
    "bspec_residual_update": [c_void_p, c_void_p, c_int, c_float, c_void_p, c_longlong, c_void_p, c_int, c_void_p],
    "bspec_gelu_tanh_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_bigram_add": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_scale": [c_void_p, c_longlong, c_float, c_void_p],
    "bspec_gate_mul": [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_void_p],
    "bspec_lightning_recurrence": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_longlong, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_scan_conv": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_selective_scan": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                             c_longlong, c_float, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_relu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_qkv_prepare": [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float,
                          c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                          c_longlong, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "bspec_attention_masked": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                               c_longlong, c_float, c_int, c_void_p, c_longlong, c_longlong, c_float, c_int, c_void_p],
    "bspec_delta_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                            c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                            c_int, c_int, c_int, c_float, c_float, c_void_p],
    "bspec_delta_recurrence": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p,
                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_gated_rmsnorm": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                            c_float, c_int, c_void_p],
    "bspec_rope_kv_append": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p],
    "bspec_rope_inplace": [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_float,
                           c_void_p],
    "bspec_add_layernorm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float,
                            c_void_p],
    "bspec_clamped_glu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "bspec_gelu_erf": [c_void_p, c_int, c_longlong, c_void_p],
    "bspec_relu_squared": [c_void_p, c_int, c_longlong, c_void_p],
    "bspec_stream_expand": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "bspec_stream_norm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                          c_int, c_int, c_float, c_void_p, c_void_p],
    "bspec_stream_gather": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                            c_void_p],
    "bspec_tanh_softcap": [c_void_p, c_longlong, c_float, c_void_p],
    "bspec_latent_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
                             c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_longlong, c_void_p],
    "bspec_latent_attention_generic": [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p,
                                       c_longlong, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_longlong, c_int, c_void_p,
                                       c_void_p],
    "bspec_latent_attention_mma_supported": [c_int, c_int],
    "bspec_latent_attention_mma_rows": [c_int, c_int, c_int, c_int],
    "bspec_latent_attention_mma_smem": [c_int, c_int, c_int, c_int],
    "bspec_latent_attention_mma": [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_void_p,
                                   c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_longlong,
                                   c_void_p, c_float, c_int, c_void_p, c_void_p],
    "bspec_gate_heads": [c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_moe_route": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                        c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "bspec_moe_plan": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                       c_void_p, c_void_p],
    "bspec_moe_grouped": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_void_p],
    "bspec_moe_skinny": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                         c_int, c_void_p],
    "bspec_moe_skinny_mma": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                             c_int, c_int, c_void_p],
    "bspec_moe_gather": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    "bspec_moe_combine": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "bspec_sgemm_tn_batched": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                               c_longlong, c_longlong, c_longlong, c_int, c_void_p],
    "bspec_attention_generic": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p],
    "bspec_attention_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p],
    "bspec_attention_bf16_masked": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                    c_longlong, c_void_p, c_float, c_void_p],
    "bspec_attention_prefill_tc_masked": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                          c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "bspec_attention_prefill_tc_capped": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int,
                                          c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p],
    "bspec_gemm_tc_plan": [c_int, c_int, c_int, c_int, c_void_p],
    "bspec_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "bspec_gemm_tc_act": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "bspec_gemm_tc_clamped_glu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int,
                                  c_void_p],
    "bspec_gemm_tc_qkv_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong,
                               c_void_p],
    "bspec_attention_prefill_tc": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_float,
                                   c_int, c_int, c_void_p, c_void_p],
    "bspec_sgemm_tn": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p],
    "bspec_pick_slices": [c_int],
    "bspec_argmax": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "bspec_sample": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ulonglong, c_void_p,
                     c_void_p, c_void_p, c_void_p, c_void_p],
}


_features = None       # features of the loaded library: a frozenset, or None for the library of all files


def load_library(features=None):
    """Load (building on first use) the kernel library.  Raises if it cannot.

    ``features`` None: the loaded library if there is one, else the library of all files.  A tuple of names of
    ``csrc.build.FEATURES``: a library that has at least the core and those (what is loaded already, if it does;
    else one is built and loaded, and the wrappers call into it from then on)."""
    global _lib, _features
    if _lib is not None and (features is None or _features is None or set(features) <= _features):
        return _lib
    with _lock:
        if _lib is not None and (features is None or _features is None or set(features) <= _features):
            return _lib
        from ..csrc.build import FEATURES, LIB_NAME, library_path
        want = None if features is None else frozenset(features) | (_features or frozenset())
        if want is not None and want == frozenset(FEATURES):
            want = None
        path = library_path(build=True, features=None if want is None else tuple(sorted(want)))
        if path.name == LIB_NAME:
            want = None                               # the library of all files served the request
        lib = ctypes.CDLL(str(path))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                if want is None:
                    raise KernelError(f"{path} has no entry point {name}")
                continue                              # an entry point of a feature this library was built without
            fn.argtypes = argtypes
            fn.restype = c_longlong if name == "bspec_gemm_tc_plan" else c_int
        _lib, _features = lib, want
        from . import debug
        debug.apply_environment(sys.modules[__name__], lib)
        global _BOUNDS_ACTIVE
        from ..csrc.build import bounds_requested
        _BOUNDS_ACTIVE = bounds_requested()
    return _lib


def require(*features) -> None:
    """Make sure the loaded library has these features (a part calls this when it is built)."""
    load_library(features=tuple(features))


_BOUNDS_ACTIVE = False


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel of the library (on by default)."""
    lib = load_library()
    lib.bspec_set_pdl.argtypes = [c_int]
    lib.bspec_set_pdl.restype = None
    lib.bspec_set_pdl(int(bool(on)))


_TRACE_SETTERS = ["bspec_trace_set_attention_tcgen05", "bspec_trace_set_elementwise", "bspec_trace_set_attention_generic", "bspec_trace_set_attention_bf16",
                  "bspec_trace_set_gemm_fp32", "bspec_trace_set_sampling", "bspec_trace_set_gemm_tcgen05", "bspec_trace_set_latent",
                  "bspec_trace_set_moe", "bspec_trace_set_latent_mma", "bspec_trace_set_delta",
                  "bspec_trace_set_state_mixers", "bspec_trace_set_streams"]
TRACE_KERNEL_NAMES = {1: "embed", 2: "add_rmsnorm", 3: "gather_rows_add", 4: "silu_mul", 5: "rope_kv_append",
                      6: "rope_inplace", 7: "attn_generic", 8: "attn_decode", 9: "attn_prefill", 10: "sgemm",
                      11: "sample_threshold", 12: "sample_pick", 13: "sample_final", 14: "add_layernorm", 15: "clamped_glu",
                      16: "gelu_erf", 17: "tanh_softcap", 18: "residual_update", 19: "qkv_prepare", 60: "delta_prepare",
                      61: "delta_recurrence", 62: "gated_rmsnorm", 63: "bigram_add", 64: "scale", 65: "lightning_recurrence",
                      66: "scan_conv", 67: "selective_scan", 70: "stream_expand", 71: "stream_norm", 72: "stream_gather", 20: "gemm_tcgen05", 30: "attn_prefill_tc", 40: "latent_prepare",
                      41: "latent_attn_generic", 42: "gate_heads", 43: "latent_attn_mma", 44: "latent_attn_join",
                      50: "moe_route", 51: "moe_plan", 52: "moe_grouped", 53: "moe_gather", 54: "moe_combine", 55: "moe_skinny", 56: "moe_skinny_mma", 57: "moe_rank", 58: "moe_offsets", 59: "moe_place"}


def set_trace(buf: Optional[torch.Tensor], count: Optional[torch.Tensor]) -> None:
    """Tuning aid.  ``buf`` int64 [capacity, 3] and ``count`` int32 [2] = {0, capacity} on the device: from now on
    block 0 of every kernel appends (kernel id, start ns, ns at which its wait on the predecessor returned).
    ``None`` switches it off.  Set it before capturing a graph that should record."""
    lib = load_library()
    for name in _TRACE_SETTERS:
        fn = getattr(lib, name, None)
        if fn is None:
            continue                                  # a file of a feature the loaded library was built without
        fn.argtypes = [c_void_p, c_void_p]
        fn.restype = c_int
        _check(fn(_ptr(buf), _ptr(count)), name)


def library_file() -> str:
    load_library()
    from ..csrc.build import library_path
    return str(library_path(build=False, features=None if _features is None else tuple(sorted(_features))))


def launch_count() -> int:
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels of this package launched by a CUDA-graph replay."""
    global _launches
    _launches += int(n)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("batchspec_b200 kernels run on a CUDA device only; got a tensor on " + str(t.device))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = [None]


def _stream() -> int:
    """Handle of torch's current stream on the current device.  Asked for at every launch (a graph capture
    switches streams), so through the one call that does nothing else."""
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index[0] is None:
        _device_index[0] = torch.cuda.current_device()
    return _raw_stream(_device_index[0])


def _check(err: int, name: str) -> None:
    global _launches
    _launches += 1
    if err != 0:
        raise KernelError(f"{name}: CUDA error {err}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------- rows

def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    _require_cuda(ids, table, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous()
    n, d = out.shape
    assert table.shape[1] == d and ids.numel() == n
    _check(load_library().bspec_embed(ids.data_ptr(), table.data_ptr(), _dtype_code(table.dtype), out.data_ptr(),
                                      n, d, table.shape[0], float(scale), _stream()), "embed")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, delta_scale: float = 1.0, exact: bool = False,
                delta_vec: Optional[torch.Tensor] = None) -> None:
    """resid += delta_scale * delta_vec * delta (if delta is given; ``delta_vec`` float32 [d], a factor per column, or
    None); out = the RMS-normalised rows times ``weight`` ([d], or one number for all columns).  ``exact``: the
    product with the weight is taken in float32 and the result rounded once; otherwise the normalised row is cast
    to the output type first and multiplied there."""
    _require_cuda(resid, delta, weight, out, delta_vec)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous()
    n, d = resid.shape
    assert out.shape == resid.shape and weight.numel() in (d, 1)
    assert delta_vec is None or (delta_vec.dtype == torch.float32 and delta_vec.numel() == d and delta_vec.is_contiguous())
    w_scalar = int(weight.numel() == 1 and d != 1)
    if delta is not None:
        assert delta.shape == resid.shape and delta.is_contiguous()
    dd = _dtype_code(delta.dtype) if delta is not None else _dtype_code(out.dtype)
    _check(load_library().bspec_add_rmsnorm(resid.data_ptr(), _ptr(delta), dd, weight.data_ptr(),
                                            _dtype_code(weight.dtype), out.data_ptr(), _dtype_code(out.dtype),
                                            n, d, float(eps), float(delta_scale), int(bool(exact)), _ptr(delta_vec),
                                            w_scalar, _stream()),
           "add_rmsnorm")


def gather_rows_add(resid: torch.Tensor, pending: Optional[torch.Tensor], rows: torch.Tensor,
                    out: torch.Tensor, scale: float = 1.0, vec: Optional[torch.Tensor] = None) -> None:
    """out[i] = resid[rows[i]] + scale * vec * pending[rows[i]] (``vec`` float32 [d], a factor per column, or None)."""
    _require_cuda(resid, pending, rows, out, vec)
    assert vec is None or (vec.dtype == torch.float32 and vec.numel() == out.shape[1] and vec.is_contiguous())
    assert resid.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32
    assert resid.is_contiguous() and out.is_contiguous() and (pending is None or pending.is_contiguous())
    pd = _dtype_code(pending.dtype) if pending is not None else F32
    _check(load_library().bspec_gather_rows_add(resid.data_ptr(), _ptr(pending), pd, rows.data_ptr(), out.data_ptr(),
                                                out.shape[0], out.shape[1], resid.shape[0], float(scale), _ptr(vec),
                                                _stream()),
           "gather_rows_add")


def residual_update(resid: torch.Tensor, pending: Optional[torch.Tensor], scale: float = 1.0,
                    extra: Optional[torch.Tensor] = None, vec: Optional[torch.Tensor] = None) -> None:
    """In place on the float32 residual: resid += scale * vec * pending (if given; ``vec`` float32 [d], a factor per
    column, or None) + extra (if given, float32)."""
    _require_cuda(resid, pending, extra, vec)
    assert vec is None or (vec.dtype == torch.float32 and vec.numel() == resid.shape[-1] and vec.is_contiguous())
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    assert pending is None or (pending.shape == resid.shape and pending.is_contiguous())
    assert extra is None or (extra.shape == resid.shape and extra.is_contiguous() and extra.dtype == torch.float32)
    if pending is None and extra is None:
        return
    _check(load_library().bspec_residual_update(resid.data_ptr(), _ptr(pending),
                                                _dtype_code(pending.dtype) if pending is not None else F32,
                                                float(scale), _ptr(extra), resid.numel(), _ptr(vec), resid.shape[-1],
                                                _stream()), "residual_update")


def add_layernorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor,
                  eps: float, out: torch.Tensor) -> None:
    """resid += delta (if given), out = (resid - mean) / sqrt(var + eps) * weight + bias, in float32."""
    _require_cuda(resid, delta, weight, bias, out)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous()
    n, d = resid.shape
    assert out.shape == resid.shape and weight.numel() == d and bias.numel() == d and weight.dtype == bias.dtype
    if delta is not None:
        assert delta.shape == resid.shape and delta.is_contiguous()
    dd = _dtype_code(delta.dtype) if delta is not None else _dtype_code(out.dtype)
    _check(load_library().bspec_add_layernorm(resid.data_ptr(), _ptr(delta), dd, weight.data_ptr(), bias.data_ptr(),
                                              _dtype_code(weight.dtype), out.data_ptr(), _dtype_code(out.dtype),
                                              n, d, float(eps), _stream()), "add_layernorm")


def clamped_glu(u: torch.Tensor, out: torch.Tensor, alpha: float, limit: float, group: int = 0) -> None:
    """out = g * sigmoid(alpha * g) * (up + 1) with g = min(gate, limit), up = clamp(up, -limit, limit); the column
    layouts of ``silu_mul``."""
    _require_cuda(u, out)
    n, inter = out.shape
    assert u.shape == (n, 2 * inter) and u.dtype == out.dtype and u.is_contiguous() and out.is_contiguous()
    _check(load_library().bspec_clamped_glu(u.data_ptr(), out.data_ptr(), _dtype_code(u.dtype), n, inter, int(group),
                                            float(alpha), float(limit), _stream()), "clamped_glu")


def tanh_softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """In place on float32: cap * tanh(x / cap)."""
    _require_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(load_library().bspec_tanh_softcap(x.data_ptr(), x.numel(), float(cap), _stream()), "tanh_softcap")
    return x


def gelu_erf_(x: torch.Tensor) -> torch.Tensor:
    """In place: 0.5 x (1 + erf(x / sqrt 2))."""
    _require_cuda(x)
    assert x.is_contiguous()
    _check(load_library().bspec_gelu_erf(x.data_ptr(), _dtype_code(x.dtype), x.numel(), _stream()), "gelu_erf")
    return x


def relu_squared_(x: torch.Tensor) -> torch.Tensor:
    """In place max(x, 0)^2, float32 arithmetic."""
    _require_cuda(x)
    assert x.is_contiguous()
    _check(load_library().bspec_relu_squared(x.data_ptr(), _dtype_code(x.dtype), x.numel(), _stream()), "relu_squared")
    return x


# ---------------------------------------------------------------------------- several residual streams

def _stream_args(x, pending, vec, mixw):
    n, S, d = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    if pending is not None:
        assert pending.shape == (n, d) and pending.is_contiguous()
        assert mixw is not None and mixw.dtype == torch.float32 and mixw.numel() == S * S + S and mixw.is_contiguous()
        assert vec is None or (vec.dtype == torch.float32 and vec.numel() == d and vec.is_contiguous())
    return n, S, d


def stream_expand(src: torch.Tensor, streams: int) -> torch.Tensor:
    """[n, d] float32 -> [n, streams, d]: every stream starts as the same row."""
    require("streams")
    _require_cuda(src)
    assert src.dtype == torch.float32 and src.is_contiguous()
    n, d = src.shape
    x = torch.empty((n, streams, d), dtype=torch.float32, device=src.device)
    _check(load_library().bspec_stream_expand(src.data_ptr(), x.data_ptr(), n, streams, d, _stream()), "stream_expand")
    return x


def stream_norm(x: torch.Tensor, pending: Optional[torch.Tensor], vec: Optional[torch.Tensor],
                mixw: Optional[torch.Tensor], read: Optional[torch.Tensor], weight: Optional[torch.Tensor] = None,
                eps: float = 0.0, out: Optional[torch.Tensor] = None, expand: Optional[torch.Tensor] = None) -> None:
    """x [n, S, d] float32, in place: if ``pending`` [n, d] is given it joins all streams at once,
    x_t <- sum_s mix[s, t] x_s + write[t] * vec * pending, ``mixw`` = [mix (S x S, from x to) | write (S)] float32 and
    ``vec`` a float32 factor per column or None.  If ``read`` (float32 [S]) is given, out = RMS norm of
    u = sum_s read[s] x_s times ``weight``, float32 arithmetic and one rounding.  ``expand`` (float32 [n, d]): x holds
    nothing yet; every stream starts as that row and is written (a step's first norm, which so spares a kernel that
    only copies the embedding S times)."""
    require("streams")
    _require_cuda(x, pending, vec, mixw, read, weight, out, expand)
    n, S, d = _stream_args(x, pending, vec, mixw)
    assert expand is None or (expand.dtype == torch.float32 and expand.shape == (n, d) and expand.is_contiguous())
    if read is not None:
        assert read.dtype == torch.float32 and read.numel() == S and read.is_contiguous()
        assert weight.numel() == d and out.shape == (n, d) and out.is_contiguous()
    elif pending is None and expand is None:
        return
    _check(load_library().bspec_stream_norm(
        x.data_ptr(), _ptr(pending), _dtype_code(pending.dtype) if pending is not None else F32, _ptr(vec), _ptr(mixw),
        _ptr(read), _ptr(weight), _dtype_code(weight.dtype) if weight is not None else F32, _ptr(out),
        _dtype_code(out.dtype) if out is not None else F32, n, S, d, float(eps), _ptr(expand), _stream()), "stream_norm")


def stream_gather(x: torch.Tensor, pending: Optional[torch.Tensor], vec: Optional[torch.Tensor],
                  mixw: Optional[torch.Tensor], rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = the sum over the streams of row rows[i] of x [n, S, d], after ``pending`` has joined them as in
    ``stream_norm`` (x itself is not changed)."""
    _require_cuda(x, pending, vec, mixw, rows, out)
    n, S, d = _stream_args(x, pending, vec, mixw)
    assert rows.dtype == torch.int32 and out.dtype == torch.float32 and out.shape == (rows.numel(), d) and out.is_contiguous()
    _check(load_library().bspec_stream_gather(
        x.data_ptr(), _ptr(pending), _dtype_code(pending.dtype) if pending is not None else F32, _ptr(vec), _ptr(mixw),
        rows.data_ptr(), out.data_ptr(), out.shape[0], S, d, n, _stream()), "stream_gather")


GLU_FUSION = True
GLU_GROUP = 8      # gate/up interleave of weights prepared for the fused epilogues: 8 gate rows, then their 8 up rows


def silu_mul(u: torch.Tensor, out: torch.Tensor, group: int = 0) -> None:
    """out = silu(gate) * up.  ``group`` 0: u = [gate | up]; G > 0: blocks of G gate columns and their G up columns."""
    _require_cuda(u, out)
    n, inter = out.shape
    assert u.shape == (n, 2 * inter) and u.dtype == out.dtype and u.is_contiguous() and out.is_contiguous()
    _check(load_library().bspec_silu_mul(u.data_ptr(), out.data_ptr(), _dtype_code(u.dtype), n, inter, int(group),
                                         _stream()), "silu_mul")


def relu_mul(u: torch.Tensor, out: torch.Tensor, group: int = 0) -> None:
    """out = relu(gate) * up; the column layouts of ``silu_mul``."""
    _require_cuda(u, out)
    n, inter = out.shape
    assert u.shape == (n, 2 * inter) and u.dtype == out.dtype and u.is_contiguous() and out.is_contiguous()
    _check(load_library().bspec_relu_mul(u.data_ptr(), out.data_ptr(), _dtype_code(u.dtype), n, inter, int(group),
                                         _stream()), "relu_mul")


def gelu_tanh_mul(u: torch.Tensor, out: torch.Tensor, group: int = 0) -> None:
    """out = gelu(gate) * up with gelu(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); the column layouts of
    ``silu_mul``."""
    _require_cuda(u, out)
    n, inter = out.shape
    assert u.shape == (n, 2 * inter) and u.dtype == out.dtype and u.is_contiguous() and out.is_contiguous()
    _check(load_library().bspec_gelu_tanh_mul(u.data_ptr(), out.data_ptr(), _dtype_code(u.dtype), n, inter, int(group),
                                              _stream()), "gelu_tanh_mul")


GATED_ACTIVATIONS = {"silu": (1, silu_mul), "relu": (3, relu_mul), "gelu_tanh": (4, gelu_tanh_mul)}   # epilogue kind, kernel


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """In place on float32: x *= factor."""
    _require_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(load_library().bspec_scale(x.data_ptr(), x.numel(), float(factor), _stream()), "scale")
    return x


def bigram_add(resid: torch.Tensor, table: torch.Tensor, prev: torch.Tensor, ctx, buckets: int, mul_prev: int,
               mul_cur: int, vocab: int) -> None:
    """resid[t] += table[(previous token * mul_prev + token * mul_cur) mod buckets], and table[buckets] for the token
    at position 0.  ``prev`` int32 [slots, >= 1]: the last token of every request's earlier steps; it is read for a
    portion's first token and then set to the portion's last token."""
    _require_cuda(resid, table, prev)
    n, d = resid.shape
    assert resid.dtype == torch.float32 and resid.is_contiguous() and table.is_contiguous()
    assert table.shape == (buckets + 1, d) and prev.dtype == torch.int32 and prev.stride(-1) == 1
    _check(load_library().bspec_bigram_add(resid.data_ptr(), ctx.token_ids.data_ptr(), ctx.positions.data_ptr(),
                                           ctx.tok_entry.data_ptr(), ctx.qo_indptr.data_ptr(),
                                           ctx.state_slots.data_ptr(), prev.data_ptr(), prev.stride(0),
                                           table.data_ptr(), _dtype_code(table.dtype), n, d, int(vocab), int(buckets),
                                           int(mul_prev), int(mul_cur), _stream()), "bigram_add")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GLU_GROUP) -> torch.Tensor:
    """[I, d] gate and up rows -> [2I, d] in blocks of ``group`` gate rows followed by their up rows."""
    inter, d = gate.shape
    assert inter % group == 0 and up.shape == gate.shape
    return torch.stack([gate.view(inter // group, group, d), up.view(inter // group, group, d)], dim=1).reshape(2 * inter, d).contiguous()


def linear_glu(x: torch.Tensor, w13: torch.Tensor, group: int = GLU_GROUP, activation: str = "silu") -> torch.Tensor:
    """act(x Wg^T) * (x Wu^T), act = silu, relu or gelu_tanh, for bfloat16 with ``w13`` interleaved by
    ``interleave_gate_up``: one kernel with the activation in the GEMM's epilogue for decode-sized steps, vendor GEMM +
    activation kernel otherwise."""
    epilogue, kernel = GATED_ACTIVATIONS[activation]
    _require_cuda(x, w13)
    M, K = x.shape
    N = w13.shape[0]
    inter = N // 2
    if (GLU_FUSION and x.dtype == torch.bfloat16 and K % 8 == 0 and M > 0 and group == GLU_GROUP
            and x.is_contiguous() and (TC_GEMM == "all" or (TC_GEMM == "auto" and M <= TC_GEMM_MAX_M))):
        out = torch.empty((M, inter), dtype=x.dtype, device=x.device)
        _check(load_library().bspec_gemm_tc(x.data_ptr(), w13.data_ptr(), out.data_ptr(), M, N, K, 0,
                                            epilogue,
                                            _status_word(x.device).data_ptr(), sm_count(x.device), _stream()), "gemm_tc_glu")
        return out
    u = linear(x, w13)
    out = torch.empty((M, inter), dtype=x.dtype, device=x.device)
    kernel(u, out, group)
    return out


def linear_clamped_glu(x: torch.Tensor, w13: torch.Tensor, alpha: float, limit: float, group: int = GLU_GROUP) -> torch.Tensor:
    """g sigmoid(alpha g) (u + 1) with g = min(x Wg^T, limit), u = clamp(x Wu^T, -limit, limit), for ``w13`` interleaved
    by ``interleave_gate_up``: one kernel with the activation in the product's epilogue for decode-sized bfloat16
    steps, else product + activation kernel."""
    _require_cuda(x, w13)
    M, K = x.shape
    N = w13.shape[0]
    inter = N // 2
    out = torch.empty((M, inter), dtype=x.dtype, device=x.device)
    if (GLU_FUSION and x.dtype == torch.bfloat16 and K % 8 == 0 and M > 0 and group == GLU_GROUP and N % 16 == 0
            and x.is_contiguous() and (TC_GEMM == "all" or (TC_GEMM == "auto" and M <= TC_GEMM_MAX_M))):
        _check(load_library().bspec_gemm_tc_clamped_glu(x.data_ptr(), w13.data_ptr(), out.data_ptr(), M, N, K,
                                                        float(alpha), float(limit), _status_word(x.device).data_ptr(),
                                                        sm_count(x.device), _stream()), "gemm_tc_clamped_glu")
        return out
    clamped_glu(linear(x, w13), out, alpha, limit, group)
    return out


def rope_frequency_table(freqs: torch.Tensor, device) -> torch.Tensor:
    """The form in which the rotary kernels take their frequencies: float32 [2, n], the leading parts of the
    float64 values in row 0 and the remainders in row 1 (their sum is the float64 value to 2^-48).  The kernels
    form the angle position * frequency in float64 from it."""
    f = freqs.detach().to("cpu", torch.float64).reshape(-1)
    hi = f.to(torch.float32)
    lo = (f - hi.to(torch.float64)).to(torch.float32)
    return torch.stack([hi, lo]).contiguous().to(device)


def rope_kv_append(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                   inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, positions: torch.Tensor,
                   tok_entry: torch.Tensor, kv_indptr: torch.Tensor, kv_indices: torch.Tensor, cache: torch.Tensor,
                   page_size: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k, and write k and v of every token into the cache
    page of its position.  ``inv_freq``: a ``rope_frequency_table`` of rotary_dim / 2 frequencies.
    ``cache``: one layer's pages, any shape with
    2 * n_kv_heads * page_size * head_dim elements per page, laid out
    [page][k|v][kv head][row][dim]."""
    _require_cuda(qkv, positions, cache)
    n = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert cache.dtype == qkv.dtype and cache.is_contiguous()
    assert positions.dtype == torch.int32 and tok_entry.dtype == torch.int32
    if rotary_dim:
        assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, rotary_dim // 2) and inv_freq.is_contiguous()
    _check(load_library().bspec_rope_kv_append(
        qkv.data_ptr(), _dtype_code(qkv.dtype), n, n_heads, n_kv_heads, head_dim, _ptr(inv_freq), int(rotary_dim),
        int(bool(interleaved)), positions.data_ptr(), tok_entry.data_ptr(), kv_indptr.data_ptr(),
        kv_indices.data_ptr(), cache.data_ptr(), int(page_size), int(bool(write_kv)), cache.shape[0], _stream()),
        "rope_kv_append")


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                 interleaved: bool = False, magnitude: float = 1.0) -> None:
    """x: [n, H, w] view whose last dim is dense; rows and heads may be strided, and the first ``rotary_dim`` numbers
    of every head are rotated (a view of the rotated part of wider heads has a head stride larger than its width).
    ``inv_freq``: a ``rope_frequency_table``.  ``magnitude`` multiplies cosine and sine."""
    _require_cuda(x, positions, inv_freq)
    n, H, hd = x.shape
    assert x.stride(2) == 1 and hd >= rotary_dim and positions.dtype == torch.int32
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, rotary_dim // 2) and inv_freq.is_contiguous()
    _check(load_library().bspec_rope_inplace(x.data_ptr(), _dtype_code(x.dtype), n, x.stride(0), H, x.stride(1),
                                             inv_freq.data_ptr(), int(rotary_dim), int(bool(interleaved)),
                                             positions.data_ptr(), float(magnitude), _stream()), "rope_inplace")


# ---------------------------------------------------------------------------- attention

# Which attention kernels may run; tests switch these to compare kernels with each other (see also kernels/debug.py)
USE_TMA_ATTENTION = True
USE_TC_ATTENTION = True         # tcgen05 kernel for long prompt portions
BALANCED_ATTENTION = True       # equal shares of key tiles over a fixed grid for decode
FORCE_GENERIC_ATTENTION = False      # tests set this to compare the tensor-core kernels with the generic one
_sm_counts = {}


def sm_count(device=None) -> int:
    """Number of SMs of ``device`` (default: the current one), asked once per device."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _sm_counts:
        _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_counts[idx]


_tile_counters = {}               # device -> zeroed int32 buffers kept alive (graphs hold their addresses)


def attention_splits(n_entries: int, n_kv_heads: int, group: int, max_q_len: int, max_kv_len: int,
                     ctas_per_sm: int = 3) -> int:
    """How many ways the split-key kernel cuts each request's keys.  Every CTA pays a prologue and, with more
    than one split, a join, so long chunks are preferred: if chunks of at least 128 keys give no more CTAs than
    fit on the device at once, use them all (small batches: fill the SMs); otherwise chunks of at least 512
    keys, one split if that already keeps four fifths of the last wave busy, else the count that wastes the
    least of it.  1 when the step also holds long portions (they go to the 64-row kernel, which fills the
    device by itself)."""
    short = max(1, 16 // group)
    if max_q_len > short:
        return 1
    row_tiles = -(-(max_q_len * group) // 16)
    base = max(1, n_entries * n_kv_heads * row_tiles)
    slots = sm_count() * ctas_per_sm
    fine = min(64, max(1, -(-max_kv_len // 128)))
    if base * fine <= slots:
        return fine
    eff = lambda s: (base * s) / (-(-(base * s) // slots) * slots)
    if eff(1) >= 0.8:
        return 1
    best, best_eff = 1, eff(1)
    for s in range(2, min(64, max(1, max_kv_len // 512)) + 1):
        if eff(s) > best_eff + 1e-9:
            best, best_eff = s, eff(s)
    return best


_work_counters = {}               # device -> two zeroed ints: the prompt attention kernel's item counter


def _work_counter(device) -> torch.Tensor:
    if device not in _work_counters:
        _work_counters[device] = torch.zeros((2,), dtype=torch.int32, device=device)
    return _work_counters[device]


def _counters(device, n: int) -> torch.Tensor:
    bufs = _tile_counters.setdefault(device, [])
    if not bufs or bufs[-1].numel() < n:
        bufs.append(torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device))
    return bufs[-1]


def _attention_plan(device, ctx, tables, n_heads: int, n_kv_heads: int, head_dim: int):
    """Which bfloat16 attention kernels a step launches for layers of these sizes, with their scratch and the
    addresses of the step's metadata (kept alive by ``ctx`` and ``tables``)."""
    group = n_heads // n_kv_heads
    short = max(1, 16 // group)
    # the TMA-fed split-key kernels (page sizes 8..64) fit two CTAs per SM, the plain one three
    tma = USE_TMA_ATTENTION and tables.page_size % 8 == 0 and 64 % tables.page_size == 0
    # Equal shares of all key tiles over a fixed grid (cut on the device from the step's lengths): n_splits is
    # then only the most partial results a row tile may be left in, and the scratch is indexed by request.
    balanced = int(tma and BALANCED_ATTENTION and ctx.n_entries <= 512 and not ctx.extras.get("attn_splits"))
    if balanced:
        n_splits = min(64, max(16, -(-4 * sm_count(device) // (ctx.n_entries * n_kv_heads)) + 2))
    else:
        n_splits = ctx.extras.get("attn_splits") or attention_splits(ctx.n_entries, n_kv_heads, group, ctx.max_q_len,
                                                                     ctx.max_kv_len, 2 if tma else 3)
    run_decode = int(ctx.extras.get("min_q_len", 1) <= short)
    run_prefill = int(ctx.max_q_len > short)
    o_part = ml_part = counters = None
    if n_splits > 1 and run_decode:
        rows = ctx.n_entries * min(ctx.max_q_len, short) if balanced else ctx.n_tokens
        o_part = torch.empty((rows * n_heads * n_splits * head_dim,), dtype=torch.float32, device=device)
        ml_part = torch.empty((rows * n_heads * n_splits * 2,), dtype=torch.float32, device=device)
        row_tiles = -(-(min(ctx.max_q_len, short) * group) // 16)
        counters = _counters(device, ctx.n_entries * n_kv_heads * row_tiles)
        ctx.extras[("attention scratch", n_heads, n_kv_heads, head_dim, id(tables))] = (o_part, ml_part)   # alive
    elif n_splits > 1:
        n_splits = 1                         # no short request in the step: the split-key kernel does not run
    prefill_tc = bool(run_prefill and tma and USE_TC_ATTENTION and head_dim == 128)
    return (tma, balanced, n_splits, short, run_decode, run_prefill, prefill_tc, _ptr(o_part), _ptr(ml_part),
            _ptr(counters), _status_word(device).data_ptr(), ctx.qo_indptr.data_ptr(), ctx.positions.data_ptr(),
            ctx.tok_entry.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(),
            _ptr(getattr(ctx, "kv_len", None)))


def sink_table(sink: torch.Tensor) -> torch.Tensor:
    """The form in which the tensor-core attention kernels take softmax sinks: float32, times log2(e)."""
    return (sink.to(torch.float32) * 1.4426950408889634).contiguous()


def gate_mul(x: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, factor: float = 1.0) -> None:
    """out = x * sigmoid(gate) * factor.  ``x`` [n, w] contiguous; ``gate`` a float32 view [n, w] of rows that may be
    wider, or None for no gate; ``out`` a view [n, w] of rows that may be wider."""
    _require_cuda(x, gate, out)
    n, w = x.shape
    assert x.is_contiguous() and out.shape == x.shape and out.stride(1) == 1 and out.dtype == x.dtype
    assert gate is None or (gate.dtype == torch.float32 and gate.shape == x.shape and gate.stride(1) == 1)
    _check(load_library().bspec_gate_mul(x.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                         out.data_ptr(), out.stride(0), _dtype_code(x.dtype), n, w, float(factor),
                                         _stream()), "gate_mul")


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, ctx, tables, n_heads: int,
                    n_kv_heads: int, head_dim: int, scale: float, window: int = 0, chunk: int = 0,
                    sink: Optional[torch.Tensor] = None, sink_l2: Optional[torch.Tensor] = None,
                    softcap: float = 0.0) -> None:
    """Causal attention of the step's tokens over their requests' cached keys.
    ``qkv``: [n, >= n_heads*head_dim] rows with the (already rotated) query heads
    first.  ``ctx`` gives qo_indptr / positions / n_entries / max_q_len, ``tables``
    the block tables of the cache group.  bfloat16 with head_dim 64/128/256 runs
    on the tensor-core kernels; everything else on the generic float32-math kernel.
    ``window`` > 0 keeps the last ``window`` keys, ``chunk`` > 0 the keys of the query's own chunk of ``chunk``
    positions (one of the two at most).  ``sink`` (float32 per query head, with ``sink_l2`` its ``sink_table``) adds
    exp(sink) to the softmax denominator.  ``softcap`` c > 0 turns a scaled score s into c tanh(s / c)."""
    _require_cuda(qkv, out, cache, sink, sink_l2)
    assert qkv.stride(1) == 1 and out.is_contiguous() and out.dtype == qkv.dtype == cache.dtype
    assert not (window and chunk) and window >= 0 and chunk >= 0
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads and sink_l2 is not None
                            and sink_l2.dtype == torch.float32 and sink_l2.numel() == n_heads)
    mask = int(window) if window else -int(chunk)      # the kernels take a chunk mask as a negative window
    lib = load_library()
    if qkv.dtype == torch.bfloat16 and head_dim in (64, 128, 256) and not FORCE_GENERIC_ATTENTION:
        # Everything that depends on the step and the layer's sizes only is worked out once per step (all layers of
        # a model ask the same question), the scratch included: the layers run one after the other on one stream.
        key = ("attention", n_heads, n_kv_heads, head_dim, id(tables), BALANCED_ATTENTION, USE_TMA_ATTENTION)
        plan = ctx.extras.get(key)
        if plan is None:
            plan = ctx.extras[key] = _attention_plan(qkv.device, ctx, tables, n_heads, n_kv_heads, head_dim)
        (tma, balanced, n_splits, short, run_decode, run_prefill, prefill_tc, o_part, ml_part, counters, status, qo, pos,
         tok_entry, kv_indptr, kv_indices, kv_len) = plan
        if prefill_tc:
            # long portions on the tcgen05 kernel; what is left for the call below are the short requests
            _check(lib.bspec_attention_prefill_tc_capped(
                qkv.data_ptr(), qkv.stride(0), out.data_ptr(), status, cache.shape[0], cache.data_ptr(), qo, pos,
                kv_indptr, kv_indices, ctx.n_entries, qkv.shape[0], ctx.max_q_len, n_heads, n_kv_heads, head_dim,
                tables.page_size,
                float(scale), mask, short + 1, _work_counter(qkv.device).data_ptr(), _ptr(sink_l2), float(softcap),
                _stream()),
                "attention_prefill_tc")
            run_prefill = 0
            if not run_decode:
                return
        _check(lib.bspec_attention_bf16_masked(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), o_part, ml_part, counters, status,
            cache.shape[0] if tma else 0, cache.data_ptr(), qo, pos, tok_entry, kv_indptr, kv_indices, ctx.n_entries,
            ctx.n_tokens, ctx.max_q_len, n_heads, n_kv_heads, head_dim, tables.page_size, float(scale), mask,
            n_splits, short, run_decode, run_prefill, balanced, kv_len, cache.shape[0], _ptr(sink_l2), float(softcap),
            _stream()),
            "attention_bf16")
        global _launches
        _launches += 1 if run_decode and run_prefill else 0
        return
    _check(lib.bspec_attention_masked(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), cache.data_ptr(), _dtype_code(qkv.dtype),
        ctx.qo_indptr.data_ptr(), ctx.positions.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(),
        ctx.n_entries, ctx.max_q_len, n_heads, n_kv_heads, head_dim, head_dim, tables.page_size, float(scale),
        int(window), int(chunk), _ptr(sink), cache.shape[0], float(softcap), 0, None, 0, out.stride(0), 1.0, 0, _stream()),
        "attention_generic")


def qkv_prepare(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, v_dim: int,
                bias: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
                magnitude: float, norm_eps: float, positions: torch.Tensor, tok_entry: torch.Tensor,
                kv_indptr: torch.Tensor, kv_indices: torch.Tensor, cache: torch.Tensor, page_size: int,
                write_kv: bool = True, q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None,
                norm_first: bool = False) -> torch.Tensor:
    """From the float32 rows [q | k | v] of the fused projection: bias, rotation of the first ``rotary_dim`` numbers
    of every q and k head (cosine and sine times ``magnitude``), division of every q and k head by its root mean
    square (``norm_eps`` > 0; times ``q_norm`` / ``k_norm``, a weight per number of a head shared by the heads, when
    given; before the rotation with ``norm_first``, else after it), in float32; returns q [n, n_heads * head_dim] in the cache's dtype and writes k and v
    into the cache page of each token's position.  Page layout: [k: kv head, row, head_dim | v: kv head, row, v_dim].
    ``qkv`` may be a view of the leading columns of wider rows.  ``v_dim`` 0: no values (the keys serve as values)
    and a page holds keys only."""
    _require_cuda(qkv, cache, positions)
    n = qkv.shape[0]
    assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and cache.is_contiguous()
    assert qkv.shape[1] == (n_heads + n_kv_heads) * head_dim + n_kv_heads * v_dim
    assert positions.dtype == torch.int32 and tok_entry.dtype == torch.int32
    if bias is not None:
        assert bias.numel() == qkv.shape[1] and bias.is_contiguous()
    if rotary_dim:
        assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, rotary_dim // 2) and inv_freq.is_contiguous()
    if q_norm is not None or k_norm is not None:
        assert q_norm is not None and k_norm is not None and q_norm.dtype == k_norm.dtype and norm_eps > 0
        assert q_norm.numel() == head_dim and k_norm.numel() == head_dim and q_norm.is_contiguous() and k_norm.is_contiguous()
    q = torch.empty((n, n_heads * head_dim), dtype=cache.dtype, device=qkv.device)
    _check(load_library().bspec_qkv_prepare(
        qkv.data_ptr(), qkv.stride(0), n, n_heads, n_kv_heads, head_dim, v_dim, _ptr(bias),
        _dtype_code(bias.dtype) if bias is not None else F32, _ptr(inv_freq), int(rotary_dim), int(bool(interleaved)),
        float(magnitude), float(norm_eps), positions.data_ptr(), tok_entry.data_ptr(), kv_indptr.data_ptr(),
        kv_indices.data_ptr(), q.data_ptr(), cache.data_ptr(), _dtype_code(cache.dtype), int(page_size),
        int(bool(write_kv)), cache.shape[0], _ptr(q_norm), _ptr(k_norm),
        _dtype_code(q_norm.dtype) if q_norm is not None else F32, int(bool(norm_first)), _stream()), "qkv_prepare")
    return q


def masked_attention(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, ctx, tables, n_heads: int,
                     n_kv_heads: int, head_dim: int, v_dim: int, scale: float, window: int = 0, chunk: int = 0,
                     sink: Optional[torch.Tensor] = None, softcap: float = 0.0, values_are_keys: bool = False,
                     gate: Optional[torch.Tensor] = None, out_scale: float = 1.0, gate_per_head: bool = False) -> None:
    """Causal attention with optional masks and sink over pages laid out [k | v] with values of size ``v_dim``:
    ``window`` > 0 keeps the last ``window`` keys, ``chunk`` > 0 the keys of the query's own chunk of positions;
    ``sink`` (float32 per query head) adds exp(sink) to the softmax denominator; ``softcap`` c > 0 turns a scaled
    score s into c tanh(s / c); ``values_are_keys``: pages hold keys only and a key is its own value;  ``gate``
    (a float32 view [n, n_heads * v_dim] of rows that may be wider; [n, n_heads] with ``gate_per_head``, one logit for
    all numbers of a head): the output is multiplied by sigmoid(gate);
    ``out_scale`` multiplies it.  ``out`` may be a view of the leading columns of wider rows.  float32 arithmetic."""
    _require_cuda(q, out, cache, sink, gate)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == q.dtype == cache.dtype
    assert out.shape == (q.shape[0], n_heads * v_dim) and (not values_are_keys or v_dim == head_dim)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads and sink.is_contiguous())
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and
                            gate.shape == ((q.shape[0], n_heads) if gate_per_head else out.shape))
    _check(load_library().bspec_attention_masked(
        q.data_ptr(), q.stride(0), out.data_ptr(), cache.data_ptr(), _dtype_code(q.dtype), ctx.qo_indptr.data_ptr(),
        ctx.positions.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(), ctx.n_entries,
        ctx.max_q_len, n_heads, n_kv_heads, head_dim, v_dim, tables.page_size, float(scale), int(window), int(chunk),
        _ptr(sink), cache.shape[0], float(softcap), int(bool(values_are_keys)), _ptr(gate),
        gate.stride(0) if gate is not None else 0, out.stride(0), float(out_scale), int(bool(gate_per_head)), _stream()),
        "attention_masked")


# ---------------------------------------------------------------------------- gated delta rule

def delta_prepare(proj: torch.Tensor, b_off: int, a_off: int, conv: torch.Tensor, a_log: torch.Tensor,
                  dt_bias: torch.Tensor, state: torch.Tensor, tail_off: int, ctx, n_heads: int, n_kv_heads: int,
                  dim: int, v_dim: int, taps: int, q_scale: float, unit_eps: float):
    """(mix float32 [n, C], gates float32 [n, 2 H]) from the float32 rows of the fused projection
    [q | k | v | ... b at b_off | a at a_off]: short causal convolution and silu of the C = 2 G dim + H v_dim
    channels (inputs before the portion come from ``state[slot, tail_off:]``), unit length of every q and k head
    (q times ``q_scale``), beta = sigmoid(b) and the decay exp(-exp(A_log) softplus(a + dt_bias))."""
    _require_cuda(proj, conv, state)
    n, ld = proj.shape
    C = 2 * n_kv_heads * dim + n_heads * v_dim
    assert proj.dtype == torch.float32 and proj.is_contiguous() and state.dtype == torch.float32 and state.is_contiguous()
    assert conv.shape == (C, taps) and conv.is_contiguous() and conv.dtype == a_log.dtype == dt_bias.dtype
    assert a_log.numel() == n_heads and dt_bias.numel() == n_heads
    assert tail_off + (taps - 1) * C <= state.shape[1] and max(b_off, a_off) + n_heads <= ld and C <= ld
    mix = torch.empty((n, C), dtype=torch.float32, device=proj.device)
    gates = torch.empty((n, 2 * n_heads), dtype=torch.float32, device=proj.device)
    _check(load_library().bspec_delta_prepare(
        proj.data_ptr(), n, ld, int(b_off), int(a_off), conv.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(),
        _dtype_code(conv.dtype), state.data_ptr(), state.stride(0), int(tail_off), ctx.qo_indptr.data_ptr(),
        ctx.tok_entry.data_ptr(), ctx.state_slots.data_ptr(), mix.data_ptr(), gates.data_ptr(), n_heads, n_kv_heads,
        dim, v_dim, taps, float(q_scale), float(unit_eps), _stream()), "delta_prepare")
    return mix, gates


def delta_recurrence(mix: torch.Tensor, gates: torch.Tensor, proj: torch.Tensor, state: torch.Tensor, tail_off: int,
                     ctx, n_heads: int, n_kv_heads: int, dim: int, v_dim: int, taps: int) -> torch.Tensor:
    """The gated delta rule over every entry's portion, per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  ``state[slot, :tail_off]`` holds S as [head, value column, key row padded to a multiple of 4] and is read and written;
    ``state[slot, tail_off:]`` receives the portion's last ``taps - 1`` projection rows.  Returns o float32
    [n, H * v_dim]."""
    _require_cuda(mix, gates, proj, state)
    n = mix.shape[0]
    assert state.stride(0) % 4 == 0 and dim <= 256 and tail_off >= n_heads * v_dim * (-(-dim // 4) * 4)
    out = torch.empty((n, n_heads * v_dim), dtype=torch.float32, device=mix.device)
    _check(load_library().bspec_delta_recurrence(
        mix.data_ptr(), gates.data_ptr(), proj.data_ptr(), proj.shape[1], state.data_ptr(), state.stride(0),
        int(tail_off), ctx.qo_indptr.data_ptr(), ctx.state_slots.data_ptr(), out.data_ptr(), ctx.n_entries, n_heads,
        n_kv_heads, dim, v_dim, taps, _stream()), "delta_recurrence")
    return out


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, n_heads: int, v_dim: int,
                  out_dtype: torch.dtype, gate_act: str = "silu") -> torch.Tensor:
    """o float32 [n, H * V]; gate a float32 view [n, H * V] of rows that may be wider.  Returns
    o / rms_V(o) * weight * act(gate) in ``out_dtype``, act = "silu" or "sigmoid".  With H = 1 the norm runs over the
    whole row."""
    assert gate_act in ("silu", "sigmoid")
    _require_cuda(o, gate, weight)
    n = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous() and gate.dtype == torch.float32 and gate.stride(1) == 1
    assert gate.shape == o.shape == (n, n_heads * v_dim) and weight.numel() == v_dim
    out = torch.empty((n, n_heads * v_dim), dtype=out_dtype, device=o.device)
    _check(load_library().bspec_gated_rmsnorm(o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(),
                                              _dtype_code(weight.dtype), out.data_ptr(), _dtype_code(out_dtype), n,
                                              n_heads, v_dim, float(eps), int(gate_act == "sigmoid"), _stream()),
           "gated_rmsnorm")
    return out


# ---------------------------------------------------------------------------- lightning attention, selective scan

def lightning_recurrence(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: torch.Tensor,
                         state: torch.Tensor, ctx, n_heads: int, dim: int, v_dim: int) -> torch.Tensor:
    """Linear attention with a fixed decay per head over every entry's portion: S <- decay_h S + k v^T, o = S^T q, with
    q, k, v = silu of the float32 columns of ``proj`` at ``q_off`` / ``k_off`` (H * dim each) and ``v_off`` (H * v_dim).
    ``state[slot]`` holds S as [head, value column, key row] float32 and is read and written.  Returns o float32
    [n, H * v_dim]."""
    _require_cuda(proj, decay, state)
    n, ld = proj.shape
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and state.dtype == torch.float32 and state.stride(1) == 1
    assert decay.dtype == torch.float32 and decay.numel() == n_heads and decay.is_contiguous()
    assert state.shape[1] >= n_heads * v_dim * dim and dim <= 256
    assert max(q_off, k_off) + n_heads * dim <= ld and v_off + n_heads * v_dim <= ld
    out = torch.empty((n, n_heads * v_dim), dtype=torch.float32, device=proj.device)
    _check(load_library().bspec_lightning_recurrence(
        proj.data_ptr(), proj.stride(0), int(q_off), int(k_off), int(v_off), decay.data_ptr(), state.data_ptr(),
        state.stride(0), ctx.qo_indptr.data_ptr(), ctx.state_slots.data_ptr(), out.data_ptr(), ctx.n_entries, n_heads,
        dim, v_dim, _stream()), "lightning_recurrence")
    return out


def scan_conv(xz: torch.Tensor, conv: torch.Tensor, bias: torch.Tensor, state: torch.Tensor, tail_off: int, ctx,
              inner: int, taps: int, run_dtype: torch.dtype):
    """silu(bias + causal convolution over ``taps`` inputs) of the first ``inner`` float32 columns of ``xz``, per
    channel; inputs before a portion come from ``state[slot, tail_off:]`` ([(taps-1), inner], oldest first).  Returns
    the result as float32 [n, inner] and in ``run_dtype`` (the same tensor when that is float32)."""
    _require_cuda(xz, conv, bias, state)
    n = xz.shape[0]
    assert xz.dtype == torch.float32 and xz.stride(1) == 1 and xz.shape[1] >= inner
    assert conv.shape == (inner, taps) and conv.is_contiguous() and bias.numel() == inner and conv.dtype == bias.dtype
    assert state.dtype == torch.float32 and tail_off + (taps - 1) * inner <= state.shape[1]
    xc = torch.empty((n, inner), dtype=torch.float32, device=xz.device)
    xr = xc if run_dtype == torch.float32 else torch.empty((n, inner), dtype=run_dtype, device=xz.device)
    _check(load_library().bspec_scan_conv(
        xz.data_ptr(), xz.stride(0), conv.data_ptr(), bias.data_ptr(), _dtype_code(conv.dtype), state.data_ptr(),
        state.stride(0), int(tail_off), ctx.qo_indptr.data_ptr(), ctx.tok_entry.data_ptr(), ctx.state_slots.data_ptr(),
        xc.data_ptr(), None if xr is xc else xr.data_ptr(), _dtype_code(run_dtype), n, inner, taps, _stream()),
        "scan_conv")
    return xc, xr


def scan_decay_table(a_log: torch.Tensor) -> torch.Tensor:
    """What the scan kernel reads instead of ``a_log`` [inner, N]: A = -exp(a_log), float32, laid out [N, inner] like
    the state, so that a step's decay is exp(dt A) with nothing else to compute or to read from scattered places.
    Made once when the weights are bound."""
    return (-torch.exp(a_log.to(torch.float32))).t().contiguous()


def selective_scan(xz: torch.Tensor, xc: torch.Tensor, dt_raw: torch.Tensor, bc: torch.Tensor, a_log: torch.Tensor,
                   d_skip: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, tail_off: int, ctx,
                   out: torch.Tensor, out_scale: float, inner: int, n_state: int, taps: int,
                   decay_table: Optional[torch.Tensor] = None) -> None:
    """The selective scan over every entry's portion.  Per channel c and state n, with dt = softplus(dt_raw + dt_bias)
    and A = -exp(a_log): S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c;
    out[t, c] = y_c silu(z_c) out_scale.  ``xz`` float32 [n, >= 2 inner] = [x before the convolution | z]; ``xc``
    float32 [n, inner] after it; ``bc`` float32 [n, 2 N] = [B | C]; ``state[slot]`` = [S as [N, inner] | the
    convolution's last taps-1 inputs at ``tail_off``], read and written.  ``out``: a view [n, inner] of rows that may
    be wider, float32 or bfloat16.  ``decay_table``: ``scan_decay_table(a_log)`` kept by the caller (made here when
    absent)."""
    if decay_table is None:
        decay_table = scan_decay_table(a_log)
    _require_cuda(xz, xc, dt_raw, bc, decay_table, d_skip, dt_bias, state, out)
    n = xz.shape[0]
    f32 = torch.float32
    assert xz.dtype == f32 and xz.stride(1) == 1 and xz.shape[1] >= 2 * inner
    assert xc.dtype == f32 and xc.is_contiguous() and xc.shape == (n, inner)
    assert dt_raw.dtype == f32 and dt_raw.is_contiguous() and dt_raw.shape == (n, inner)
    assert bc.dtype == f32 and bc.stride(1) == 1 and bc.shape == (n, 2 * n_state)
    assert decay_table.shape == (n_state, inner) and decay_table.is_contiguous() and decay_table.dtype == f32
    assert d_skip.dtype == dt_bias.dtype and d_skip.numel() == dt_bias.numel() == inner
    assert state.dtype == f32 and tail_off >= n_state * inner and tail_off + (taps - 1) * inner <= state.shape[1]
    assert out.shape == (n, inner) and out.stride(1) == 1
    _check(load_library().bspec_selective_scan(
        xz.data_ptr(), xz.stride(0), xc.data_ptr(), dt_raw.data_ptr(), bc.data_ptr(), bc.stride(0),
        decay_table.data_ptr(), d_skip.data_ptr(), dt_bias.data_ptr(), _dtype_code(d_skip.dtype), state.data_ptr(), state.stride(0),
        int(tail_off), ctx.qo_indptr.data_ptr(), ctx.state_slots.data_ptr(), out.data_ptr(), _dtype_code(out.dtype),
        out.stride(0), float(out_scale), ctx.n_entries, inner, n_state, taps, _stream()), "selective_scan")


# ---------------------------------------------------------------------------- matrix products

# Which bfloat16 products run on this package's tcgen05 kernel: "auto" (those with at most TC_GEMM_MAX_M rows),
# "all", or "none".  Measured on B200 in whole decode steps of 1B to 8B models: with up to 8 tokens the kernel (weights
# on the accumulator rows, K slices joined inside a cluster, the gate/up activation in its epilogue, weight tiles
# fetched before the wait on the kernel before) beats the vendor library by 2 to 12 %; from 16 tokens on the library
# wins, by 1 to 15 % (the join of the slices grows with the tokens), so larger steps go to the library.
TC_GEMM = "auto"
TC_GEMM_MAX_M = 8
_status = {}


def _status_word(device) -> torch.Tensor:
    if device not in _status:
        _status[device] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _status[device]


def _raise_status(dev, code: int) -> None:
    with torch.inference_mode():          # the words may have been made inside inference mode (by a step)
        _status[dev].zero_()
        for bufs in _tile_counters.values():
            for b in bufs:
                b.zero_()
        for b in _work_counters.values():
            b.zero_()
    raise KernelError(f"a kernel on {dev} gave up a bounded wait (code {code}: GEMM 1 = stage never freed, "
                      f"2 = operands never arrived, 3 = accumulator never completed; decode attention 11/13 = stage "
                      f"never freed, 12/14 = keys never arrived; prompt attention 21/22 the same, 31-41 = a role of "
                      f"the tensor-core prompt kernel).  The results of the steps "
                      f"since the last check are not valid.")


def check_status() -> None:
    """Raise if a kernel of this package gave up on a bounded wait (synchronises); in a checked build
    (``BSPEC_BOUNDS=1``) also if an index was found outside its range."""
    for dev, t in _status.items():
        code = int(t.item())
        if code:
            _raise_status(dev, code)
    check_bounds()


_BOUNDS_REPORTS = ["bspec_bounds_report_state_mixers", "bspec_bounds_report_elementwise", "bspec_bounds_report_gemm_tcgen05",
                   "bspec_bounds_report_attention_generic", "bspec_bounds_report_attention_bf16",
                   "bspec_bounds_report_latent", "bspec_bounds_report_latent_mma", "bspec_bounds_report_delta",
                   "bspec_bounds_report_streams"]
BOUNDS_CODES = {101: "token id (embedding)", 102: "row (gather)", 103: "block-table slot (rotary + cache append)",
                104: "page id (rotary + cache append)", 105: "block-table slot (q/k/v product's epilogue)",
                106: "page id (q/k/v product's epilogue)", 107: "page id (attention over plain loads)",
                108: "page id (bfloat16 attention over plain loads)", 109: "block-table slot (latent entry append)",
                110: "page id (latent entry append)", 111: "page id (latent attention over plain loads)",
                112: "page id (latent attention on the tensor cores)", 113: "block-table slot (q/k/v preparation)",
                114: "page id (q/k/v preparation)"}


def bounds_reports() -> list:
    """Checked build only (the library built with ``BSPEC_BOUNDS=1`` in the environment): what the kernels of the
    current device recorded since the last call, as (source file, what, value, limit, block); the records are
    cleared.  Empty in an ordinary build.  Waits for the device."""
    lib = load_library()
    found = []
    for name in _BOUNDS_REPORTS:
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = [ctypes.POINTER(c_int * 4)]
        fn.restype = c_int
        rec = (c_int * 4)()
        r = fn(ctypes.byref(rec))
        if r < 0:
            raise KernelError(f"{name} failed with CUDA error {-r}")
        if r == 1 and rec[0]:
            found.append((name[len("bspec_bounds_report_"):], BOUNDS_CODES.get(rec[0], str(rec[0])), rec[1], rec[2], rec[3]))
    return found


def bounds_build() -> bool:
    """Whether the loaded library is the checked build."""
    load_library()
    return _BOUNDS_ACTIVE


def check_bounds() -> None:
    """Raise if the checked build recorded an index outside its range (no-op in an ordinary build)."""
    if not _BOUNDS_ACTIVE:
        return
    found = bounds_reports()
    if found:
        raise KernelError("the checked build found indices outside their ranges (the accesses were skipped): " +
                          "; ".join(f"{src}: {what} {value} not in [0, {limit}) in block {block}"
                                    for src, what, value, limit, block in found))


_status_host = {}


def status_to_host_async() -> None:
    """Enqueue, on the current stream, a copy of the status word into pinned host memory: whoever synchronises
    with the stream next (to read a step's tokens or logits) calls ``raise_if_gave_up`` afterwards, so that a step
    whose kernels gave up a wait is never taken for a result, at no extra synchronisation."""
    for dev, t in _status.items():
        if dev not in _status_host:
            _status_host[dev] = torch.zeros((1,), dtype=torch.int32).pin_memory()
        _status_host[dev].copy_(t, non_blocking=True)


def raise_if_gave_up() -> None:
    """After a synchronisation that followed ``status_to_host_async``: raise if the copy shows a wait given up."""
    for dev, h in _status_host.items():
        code = int(h[0])
        if code:
            with torch.inference_mode():
                h.zero_()
            torch.cuda.synchronize(dev)
            _raise_status(dev, code)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T on the tcgen05 kernel (bfloat16 operands, float32 accumulation)."""
    lib = load_library()
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    if K % 8 != 0 or M <= 0:
        raise KernelError(f"gemm_tc: sizes M={M} N={N} K={K} are not supported (K must be a multiple of 8)")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(lib.bspec_gemm_tc(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, int(out_dtype == torch.float32), 0,
                             _status_word(x.device).data_ptr(), sm_count(x.device), _stream()), "gemm_tc")
    return out


PLAIN_ACTIVATIONS = {"relu2": (1, relu_squared_), "gelu": (0, gelu_erf_)}     # epilogue kind (0: none), in-place kernel


def linear_act(x: torch.Tensor, w: torch.Tensor, activation: str) -> torch.Tensor:
    """act(x w^T) with a plain activation on every output (``PLAIN_ACTIVATIONS``): one kernel with the activation in
    the tcgen05 product's epilogue for decode-sized bfloat16 steps when the epilogue knows it, else the product and
    the in-place activation kernel."""
    epilogue, kernel = PLAIN_ACTIVATIONS[activation]
    _require_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    if (epilogue and GLU_FUSION and x.dtype == torch.bfloat16 and K % 8 == 0 and M > 0 and x.is_contiguous()
            and w.is_contiguous() and (TC_GEMM == "all" or (TC_GEMM == "auto" and M <= TC_GEMM_MAX_M))):
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
        _check(load_library().bspec_gemm_tc_act(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, 0, epilogue,
                                                _status_word(x.device).data_ptr(), sm_count(x.device), _stream()),
               "gemm_tc_act")
        return out
    return kernel(linear(x, w))


FUSE_QKV_ROPE = True       # decode-sized steps: rotary encoding and the cache append in the q/k/v product's epilogue


def linear_qkv_rope(x: torch.Tensor, wqkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                    inv_freq: torch.Tensor, rotary_dim: int, interleaved: bool, positions: torch.Tensor,
                    tok_entry: torch.Tensor, kv_indptr: torch.Tensor, kv_indices: torch.Tensor, cache: torch.Tensor,
                    page_size: int, write_kv: bool = True) -> Optional[torch.Tensor]:
    """x [M, K] @ [Wq; Wk; Wv]^T with the rotary encoding of q and k and the write of k and v into their cache
    pages done in the product's epilogue, for bfloat16 steps of at most ``TC_GEMM_MAX_M`` tokens and heads of
    128 rotated over their whole width.  Returns [M, (Hq + 2 Hkv) * 128] whose q columns hold the rotated queries
    (its k and v columns are not written), or None when the sizes are not these: the caller then runs the product,
    ``rope_kv_append`` and so on one after the other."""
    M, K = x.shape
    N = wqkv.shape[0]
    if not (FUSE_QKV_ROPE and TC_GEMM != "none" and x.dtype == torch.bfloat16
            and cache.dtype == torch.bfloat16 and head_dim == 128 and rotary_dim == 128 and 0 < M <= TC_GEMM_MAX_M
            and K % 8 == 0 and N == (n_heads + 2 * n_kv_heads) * 128 and x.is_contiguous() and wqkv.is_contiguous()):
        return None
    _require_cuda(x, wqkv, cache, positions)
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, 64) and inv_freq.is_contiguous()
    assert cache.is_contiguous() and positions.dtype == torch.int32 and tok_entry.dtype == torch.int32
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    _check(load_library().bspec_gemm_tc_qkv_rope(
        x.data_ptr(), wqkv.data_ptr(), out.data_ptr(), M, N, K, _status_word(x.device).data_ptr(), sm_count(x.device),
        inv_freq.data_ptr(), positions.data_ptr(), tok_entry.data_ptr(), kv_indptr.data_ptr(), kv_indices.data_ptr(),
        cache.data_ptr(), n_heads, n_kv_heads, int(page_size), int(bool(interleaved)), int(bool(write_kv)),
        cache.shape[0], _stream()), "gemm_tc_qkv_rope")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T -> [M, N] in ``out_dtype`` (default: x's dtype)."""
    _require_cuda(x, w)
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype, (x.shape, w.shape, x.dtype, w.dtype)
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32 and x.stride(1) == 1 and w.stride(1) == 1
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _check(load_library().bspec_sgemm_tn(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0),
                                             w.stride(0), N, _stream()), "sgemm_tn")
        return out
    if (K % 8 == 0 and M > 0 and x.is_contiguous() and w.is_contiguous()
            and (TC_GEMM == "all" or (TC_GEMM == "auto" and M <= TC_GEMM_MAX_M))):
        return gemm_tc(x, w, out_dtype)
    if out_dtype == x.dtype:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def linear_batched(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [B, M, K] (rows and batches may be strided, K dense) times w [B, N, K]^T -> [B, M, N] contiguous: one product
    per head.  bfloat16 on the vendor library's batched product, float32 on this package's FFMA kernel."""
    _require_cuda(x, w)
    B, M, K = x.shape
    N = w.shape[1]
    assert w.shape == (B, N, K) and x.dtype == w.dtype and x.stride(2) == 1 and w.is_contiguous()
    if x.dtype == torch.float32:
        out = torch.empty((B, M, N), dtype=torch.float32, device=x.device)
        _check(load_library().bspec_sgemm_tn_batched(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(1),
                                                     K, N, x.stride(0), N * K, M * N, B, _stream()), "sgemm_tn_batched")
        return out
    return torch.bmm(x, w.transpose(1, 2))


# ---------------------------------------------------------------------------- latent attention

def latent_prepare(down: torch.Tensor, q_off: int, q_rank: int, kv_off: int, kv_rank: int, rot_dim: int,
                   wq: torch.Tensor, wkv: torch.Tensor, eps: float, inv_freq: torch.Tensor, magnitude: float,
                   positions: torch.Tensor, tok_entry: torch.Tensor, kv_indptr: torch.Tensor, kv_indices: torch.Tensor,
                   cache: torch.Tensor, page_size: int, write_kv: bool = True) -> torch.Tensor:
    """From the float32 rows of the down projections: the RMS-normalised query latent (returned, [n, q_rank] in the
    cache's dtype) and the cache entry of every token, [normalised key/value latent | rotated key part], written
    to the page of its position.  Rotation: adjacent pairs, ``magnitude`` on cosine and sine."""
    _require_cuda(down, cache, positions)
    n, ld = down.shape
    assert down.dtype == torch.float32 and down.is_contiguous() and cache.is_contiguous()
    assert wq.dtype == wkv.dtype and wq.numel() == q_rank and wkv.numel() == kv_rank
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, rot_dim // 2) and inv_freq.is_contiguous()
    assert q_off + q_rank <= ld and kv_off + kv_rank + rot_dim <= ld
    cq = torch.empty((n, q_rank), dtype=cache.dtype, device=down.device)
    _check(load_library().bspec_latent_prepare(
        down.data_ptr(), n, ld, q_off, q_rank, kv_off, kv_rank, rot_dim, wq.data_ptr(), wkv.data_ptr(),
        _dtype_code(wq.dtype), float(eps), inv_freq.data_ptr(), float(magnitude), positions.data_ptr(),
        tok_entry.data_ptr(), kv_indptr.data_ptr(), kv_indices.data_ptr(), cq.data_ptr(), cache.data_ptr(),
        _dtype_code(cache.dtype), int(page_size), int(bool(write_kv)), cache.shape[0], _stream()), "latent_prepare")
    return cq


FORCE_GENERIC_LATENT = False       # tests set this to compare the tensor-core kernel with the generic one


def latent_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, ctx, tables,
                     n_heads: int, kv_rank: int, rot_dim: int, scale: float, rotate=None, window: int = 0,
                     sink: Optional[torch.Tensor] = None) -> None:
    """Causal softmax attention in the latent space over the paged entries [c | kr].  ``q_lat`` [H, n, kv_rank] and
    ``q_rot`` [n, H, rot_dim] are views with a dense last dim; ``out`` [H, n, kv_rank] receives sum_j p_j c_j per
    head.  ``rotate`` None: ``q_rot`` is already rotated.  ``rotate`` = (``rope_frequency_table``, magnitude):
    it is not, and is rotated by adjacent pairs on the way, inside the tensor-core kernel as it loads the queries,
    or in place by the rotation kernel before the generic one.  ``window`` > 0: a query sees its own entry and the
    ``window - 1`` before it.  ``sink`` (float32 per head): exp(sink) joins the softmax denominator."""
    _require_cuda(q_lat, q_rot, out, cache, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == n_heads and sink.is_contiguous())
    H, n, R = q_lat.shape
    assert H == n_heads and R == kv_rank and q_rot.shape == (n, H, rot_dim) and out.shape == (H, n, R)
    assert q_lat.stride(2) == 1 and q_rot.stride(2) == 1 and out.stride(2) == 1
    assert q_lat.dtype == q_rot.dtype == out.dtype == cache.dtype and cache.is_contiguous()
    lib = load_library()
    if (q_lat.dtype == torch.bfloat16 and not FORCE_GENERIC_LATENT and latent_mma_supported(kv_rank, rot_dim)
            and out.stride(2) == 1 and out.stride(1) % 2 == 0 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0):
        # Few rows and many entries (decode): the key tiles of a request are cut into shares for more CTAs.  The
        # count depends on the step's shape alone (entries, longest portion, longest allowed request), so a
        # captured step keeps it; shares that get no tile leave at once.
        rows = lib.bspec_latent_attention_mma_rows(ctx.max_q_len, n_heads, kv_rank, rot_dim)       # rows of a CTA's tile
        row_tiles = -(-(ctx.max_q_len * n_heads) // rows)
        n_splits = 1
        if ctx.max_q_len * n_heads <= 256:
            # as many shares as fill the CTAs that are resident at once (one wave), at least 256 keys each
            smem = lib.bspec_latent_attention_mma_smem(rows, kv_rank, rot_dim, 0) + 1024
            slots = sm_count(q_lat.device) * max(1, min(4, (227 * 1024) // smem))
            keys = min(ctx.max_kv_len, window + ctx.max_q_len) if window > 0 else ctx.max_kv_len
            n_splits = max(1, min(64, slots // (ctx.n_entries * row_tiles), -(-keys // 256)))
        o_part = ml_part = None
        if n_splits > 1:
            o_part = torch.empty((n * H * n_splits * R,), dtype=torch.float32, device=q_lat.device)
            ml_part = torch.empty((n * H * n_splits * 2,), dtype=torch.float32, device=q_lat.device)
        _check(lib.bspec_latent_attention_mma(
            q_lat.data_ptr(), q_lat.stride(1), q_lat.stride(0), q_rot.data_ptr(), q_rot.stride(0), q_rot.stride(1),
            out.data_ptr(), out.stride(1), out.stride(0), cache.data_ptr(), ctx.qo_indptr.data_ptr(),
            ctx.positions.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(), ctx.n_entries, n,
            ctx.max_q_len, n_heads, kv_rank, rot_dim, tables.page_size, float(scale), n_splits, _ptr(o_part),
            _ptr(ml_part), cache.shape[0], rotate[0].data_ptr() if rotate else None,
            float(rotate[1]) if rotate else 1.0, int(window), _ptr(sink), _stream()), "latent_attention_mma")
        if n_splits > 1:
            count_launches(1)
        return
    if rotate:
        rope_inplace(q_rot, ctx.positions, rotate[0], rot_dim, True, rotate[1])
    _check(lib.bspec_latent_attention_generic(
        q_lat.data_ptr(), q_lat.stride(1), q_lat.stride(0), q_rot.data_ptr(), q_rot.stride(0), q_rot.stride(1),
        out.data_ptr(), out.stride(1), out.stride(0), cache.data_ptr(), _dtype_code(cache.dtype),
        ctx.qo_indptr.data_ptr(), ctx.positions.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(),
        ctx.n_entries, ctx.max_q_len, n_heads, kv_rank, rot_dim, tables.page_size, float(scale), cache.shape[0],
        int(window), _ptr(sink), _stream()), "latent_attention_generic")


def latent_mma_supported(kv_rank: int, rot_dim: int) -> bool:
    """Whether the tensor-core latent attention kernel takes these sizes (else the generic kernel runs)."""
    return bool(load_library().bspec_latent_attention_mma_supported(int(kv_rank), int(rot_dim)))


def gate_heads(v: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, h*V + j] = v[h, t, j] * sigmoid(gate[t, h]).  ``v`` [H, n, V] with a dense last dim; ``gate`` a float32
    view [n, H] of rows that may be wider."""
    _require_cuda(v, gate, out)
    H, n, V = v.shape
    assert gate.dtype == torch.float32 and gate.shape == (n, H) and gate.stride(1) == 1 and v.stride(2) == 1
    assert out.shape == (n, H * V) and out.is_contiguous() and out.dtype == v.dtype
    _check(load_library().bspec_gate_heads(v.data_ptr(), v.stride(0), v.stride(1), gate.data_ptr(), gate.stride(0),
                                           out.data_ptr(), _dtype_code(v.dtype), n, H, V, _stream()), "gate_heads")


# ---------------------------------------------------------------------------- routed feed-forward

MOE_LIBRARY_GROUPED = True       # bfloat16 steps with many rows per expert: the vendor library's grouped product
MOE_LIBRARY_MIN_ROWS = 32        # ... from this many (token, choice) rows per expert on average
MOE_ROUTE_FUSED_MAX = 0          # up to this many tokens the router's logits are formed inside its kernel (else: a product)
MOE_SKINNY_MMA = True            # ... its tensor-core form, for inner sizes that are multiples of 32
MOE_SKINNY = True                # bfloat16 steps with fewer rows per expert: the weight-streaming kernel


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], n_groups: int, keep: int,
              top: int, scale: float, softmax_top: bool = False):
    """(expert ids int32 [n, top], weights float32 [n, top]) of every token; the rule is in ``csrc/moe.cu``.
    ``softmax_top``: the logits plus ``correction`` (a bias) choose, and the weights are the softmax over the chosen
    logits alone; otherwise sigmoid scores."""
    _require_cuda(h, router)
    n, d = h.shape
    E = router.shape[0]
    assert router.shape == (E, d) and router.dtype == h.dtype and h.is_contiguous() and router.is_contiguous()
    ids = torch.empty((n, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=h.device)
    # many tokens: the logits as one matrix product with float32 accumulation and output; few: inside the kernel
    logits = linear(h, router, out_dtype=torch.float32) if n > MOE_ROUTE_FUSED_MAX else None
    _check(load_library().bspec_moe_route(h.data_ptr(), _dtype_code(h.dtype), n, d, router.data_ptr(), _ptr(correction),
                                          _dtype_code(correction.dtype) if correction is not None else F32, E,
                                          int(n_groups), int(keep), int(top), float(scale), ids.data_ptr(),
                                          wts.data_ptr(), _ptr(logits), int(bool(softmax_top)), _stream()), "moe_route")
    return ids, wts


def moe_experts(h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                out_dtype: torch.dtype, glu: bool = False) -> torch.Tensor:
    """sum_k wts[t, k] * Wdown[e] gelu(Wup[e] h[t]) with e = ids[t, k].  ``w_up`` [E, ff, d], ``w_down`` [E, d, ff].
    ``glu``: the experts are gated, Wdown[e] (silu(Wgate[e] h) * (Wup[e] h)), and ``w_up`` holds [gate; up] as
    [E, 2 ff, d]; the first product then leaves its result as it is, and this package's grouped kernels form
    silu(gate) * up while they stage the rows of the second product (the vendor's grouped product is followed by
    ``silu_mul`` instead).
    The (token, choice) rows are sorted by expert on the device; no count is read on the host."""
    _require_cuda(h, ids, wts, w_up, w_down)
    lib = load_library()
    n, d = h.shape
    E, ff_up, _ = w_up.shape
    ff = ff_up // 2 if glu else ff_up                 # the down projection's inner size
    act = 0 if glu else 1                             # the first product's epilogue: 1 = gelu
    act_down = 2 if glu else 0                        # the second product's operand: 2 = silu(gate) * up of [gate | up] rows
    top = ids.shape[1]
    slots = n * top
    assert w_up.shape == (E, ff_up, d) and w_down.shape == (E, d, ff) and w_up.is_contiguous() and w_down.is_contiguous()
    assert not glu or ff_up == 2 * ff

    def gated(u):
        if not glu:
            return u
        m = torch.empty((slots, ff), dtype=u.dtype, device=u.device)
        silu_mul(u, m)
        return m
    assert h.is_contiguous() and ids.is_contiguous() and wts.is_contiguous() and h.dtype == w_up.dtype == w_down.dtype
    dev, code = h.device, _dtype_code(h.dtype)
    library = (MOE_LIBRARY_GROUPED and h.dtype == torch.bfloat16 and slots >= MOE_LIBRARY_MIN_ROWS * E
               and d % 8 == 0 and ff % 8 == 0 and hasattr(torch, "_grouped_mm"))
    # few rows per expert in bfloat16: tiles of 8 rows on the kernel that streams the experts' weights
    skinny = (not library and MOE_SKINNY and h.dtype == torch.bfloat16 and slots < 32 * E and d % 8 == 0
              and ff % 8 == 0 and 16 * max(d, ff_up) <= 200 * 1024)
    # ... on the tensor cores when both inner sizes are multiples of 32 and 16 token rows fit shared memory
    skinny_mma = skinny and MOE_SKINNY_MMA and d % 32 == 0 and ff % 32 == 0
    # 16 token rows per tile while they leave room for three CTAs per SM and there are that many rows per expert
    mma_rows = 16 if (32 * max(d, ff_up) <= 72 * 1024 and slots > 4 * E) else 8
    BM = (mma_rows if skinny_mma else 8) if skinny else (64 if slots >= 32 * E else 16)
    max_tiles = min(slots, slots // BM + E)
    many = slots > 2048                   # the plan in three kernels over all SMs (needs counters and ranks)
    meta = torch.empty((2 * slots + E + 1 + 3 * max_tiles + 1 + (E + slots if many else 0),), dtype=torch.int32, device=dev)
    perm, inv = meta[:slots], meta[slots:2 * slots]
    offsets = meta[2 * slots:2 * slots + E + 1]
    tiles = meta[2 * slots + E + 1:2 * slots + E + 1 + 3 * max_tiles]
    at = 2 * slots + E + 1 + 3 * max_tiles
    n_tiles = meta[at:at + 1]
    counts, rank = (meta[at + 1:at + 1 + E], meta[at + 1 + E:]) if many else (None, None)
    _check(lib.bspec_moe_plan(ids.data_ptr(), slots, E, BM, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(),
                              tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, _ptr(counts), _ptr(rank), _stream()),
           "moe_plan")
    if many:
        count_launches(2)
    if library:
        rows = torch.empty((slots, d), dtype=h.dtype, device=dev)
        _check(lib.bspec_moe_gather(h.data_ptr(), code, perm.data_ptr(), top, rows.data_ptr(), slots, d, _stream()),
               "moe_gather")
        ends = offsets[1:]
        u = torch._grouped_mm(rows, w_up.transpose(1, 2), offs=ends)
        u = gated(u) if glu else gelu_erf_(u)
        y = torch._grouped_mm(u, w_down.transpose(1, 2), offs=ends)
    elif skinny_mma:
        u = torch.empty((slots, ff_up), dtype=h.dtype, device=dev)
        y = torch.empty((slots, d), dtype=torch.float32, device=dev)
        _check(lib.bspec_moe_skinny_mma(h.data_ptr(), perm.data_ptr(), top, w_up.data_ptr(), u.data_ptr(), code, ff_up, d,
                                        tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, act, mma_rows, _stream()), "moe_skinny_mma_up")
        _check(lib.bspec_moe_skinny_mma(u.data_ptr(), None, top, w_down.data_ptr(), y.data_ptr(), F32, d, ff,
                                        tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, act_down, mma_rows, _stream()), "moe_skinny_mma_down")
    elif skinny:
        u = torch.empty((slots, ff_up), dtype=h.dtype, device=dev)
        y = torch.empty((slots, d), dtype=torch.float32, device=dev)
        _check(lib.bspec_moe_skinny(h.data_ptr(), perm.data_ptr(), top, w_up.data_ptr(), u.data_ptr(), code, ff_up, d,
                                    tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, act, _stream()), "moe_skinny_up")
        _check(lib.bspec_moe_skinny(u.data_ptr(), None, top, w_down.data_ptr(), y.data_ptr(), F32, d, ff,
                                    tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, act_down, _stream()), "moe_skinny_down")
    else:
        u = torch.empty((slots, ff_up), dtype=h.dtype, device=dev)
        y = torch.empty((slots, d), dtype=torch.float32, device=dev)
        _check(lib.bspec_moe_grouped(h.data_ptr(), perm.data_ptr(), top, w_up.data_ptr(), u.data_ptr(), code, code, ff_up,
                                     d, tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, BM, act, _stream()),
               "moe_grouped_up")
        _check(lib.bspec_moe_grouped(u.data_ptr(), None, top, w_down.data_ptr(), y.data_ptr(), code, F32, d, ff,
                                     tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, BM, act_down, _stream()),
               "moe_grouped_down")
    out = torch.empty((n, d), dtype=out_dtype, device=dev)
    _check(lib.bspec_moe_combine(y.data_ptr(), _dtype_code(y.dtype), inv.data_ptr(), wts.data_ptr(), top,
                                 out.data_ptr(), _dtype_code(out_dtype), n, d, _stream()), "moe_combine")
    return out


# ---------------------------------------------------------------------------- sampling

def _pick_scratch(logits: torch.Tensor):
    rows, vocab = logits.shape
    nb = load_library().bspec_pick_slices(vocab)
    part_v = torch.empty((rows * nb,), dtype=torch.float32, device=logits.device)
    part_i = torch.empty((rows * nb,), dtype=torch.int32, device=logits.device)
    return part_v, part_i


def argmax(logits: torch.Tensor) -> torch.Tensor:
    _require_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    if logits.shape[0] == 0:
        return out
    part_v, part_i = _pick_scratch(logits)
    _check(load_library().bspec_argmax(logits.data_ptr(), logits.shape[0], logits.shape[1], part_v.data_ptr(),
                                       part_i.data_ptr(), out.data_ptr(), _stream()), "argmax")
    count_launches(1)
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           stream_id: torch.Tensor, counter: torch.Tensor, seed: int,
           threshold_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-row parameters on the device: temperature f32 (<= 0: greedy), top_k i32
    (<= 0: off), top_p f32 (<= 0 or >= 1: off), stream_id i64 and counter i64 (the
    random stream of the row's request and the index of the draw in it).
    ``threshold_out`` (int32 [rows]) receives each row's threshold: the ordered key
    (sign bit flipped for positive floats, all bits for negative) of the smallest
    logit that stays in the top-k / top-p set, 0 where nothing is cut."""
    _require_cuda(logits, temperature, top_k, top_p, stream_id, counter)
    rows = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert temperature.dtype == torch.float32 and top_k.dtype == torch.int32 and top_p.dtype == torch.float32
    assert stream_id.dtype == torch.int64 and counter.dtype == torch.int64
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if rows == 0:
        return out
    part_v, part_i = _pick_scratch(logits)
    threshold = threshold_out if threshold_out is not None else torch.empty((rows,), dtype=torch.int32, device=logits.device)
    assert threshold.dtype == torch.int32 and threshold.numel() == rows and threshold.is_cuda
    _check(load_library().bspec_sample(logits.data_ptr(), rows, logits.shape[1], temperature.data_ptr(),
                                       top_k.data_ptr(), top_p.data_ptr(), stream_id.data_ptr(), counter.data_ptr(),
                                       int(seed) & 0xFFFFFFFFFFFFFFFF, threshold.data_ptr(), part_v.data_ptr(),
                                       part_i.data_ptr(), out.data_ptr(), _stream()), "sample")
    count_launches(3)
    return out
