"""ctypes binding of libgact_b200.so (declared in include/gact_b200.h).

The library is required: importing this module without it raises, and nothing in the package falls back to
a CPU or pure-PyTorch implementation of the kernels.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libgact_b200.so"

F32, F16, BF16 = 0, 1, 2
DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
RNG_CURAND, RNG_FAST, RNG_RTN, RNG_EXTERNAL = 0, 1, 2, 3
RNG_CODE = {"curand": RNG_CURAND, "fast": RNG_FAST, "rtn": RNG_RTN, "external": RNG_EXTERNAL}
GROUP = 256

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python gact-icml_b200/build.py` "
        "(nvcc, sm_100a).  gact has no fallback path.")

lib = C.CDLL(str(LIB_PATH))

_vp, _i, _i64, _u64, _d = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_double
_SIGNATURES = {
    "gact_version": ([], _i),
    "gact_error_string": ([_i], C.c_char_p),
    "gact_packed_bytes": ([_i64, _i], _i64),
    "gact_quantize": ([_vp, _i, _i64, _i, _u64, _i, _vp, _i, _vp, _vp, _vp, _vp], _i),
    "gact_pipeline_error": ([], _i),
    "gact_pipeline_error_reset": ([], _i),
    "gact_pipeline_test_hook": ([C.c_uint32, _i], None),
    "gact_dequantize": ([_vp, _vp, _vp, _i, _i64, _i, _vp, _vp], _i),
    "gact_minimax": ([_vp, _i, _i64, _vp, _vp, _vp], _i),
    "gact_mask_words": ([_i64], _i64),
    "gact_mask_pack": ([_vp, _i64, _vp, _vp, _vp], _i),
    "gact_mask_unpack": ([_vp, _i64, _vp, _vp], _i),
    "gact_fingerprint": ([_vp, _i, _i64, _vp, _vp], _i),
    "gact_sq_diffs3_scratch_bytes": ([], _i64),
    "gact_sq_diffs3": ([_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i, _vp, _vp, _vp], _i),
    "gact_sq_diffs3_noalloc": ([_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i, _vp, _vp], _i),
    "gact_sensitivity": ([_vp, _d, _vp, _i, _vp], _i),
    "gact_calc_precision": ([_vp, _vp, _vp, _i, _d, _vp, _vp], _i),
    "gact_calc_precision_host": ([_vp, _vp, _vp, _i, _d], _i),
}
for _name, (_args, _res) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _res


# The two calls every saved tensor makes.  gact/_fastcall.so (csrc/fastcall.c, built by build.py) hands the integer
# arguments to the same C entry points without ctypes' per-argument conversion (1.8 us -> 0.3 us per call); when
# it was not built the ctypes functions serve.
try:
    from gact import _fastcall
    quantize_call, dequantize_call = _fastcall.quantize, _fastcall.dequantize
except ImportError:
    _fastcall = None
    quantize_call, dequantize_call = lib.gact_quantize, lib.gact_dequantize


class GactError(RuntimeError):
    pass


def check(status: int, what: str) -> None:
    """Raise like the reference's TORCH_CHECK does (RuntimeError) on a non-zero status; argument errors
    become ValueError."""
    if status == 0:
        return
    msg = f"{what}: {lib.gact_error_string(status).decode()} (status {status})"
    if status in (1, 2, 5, 6, 9):
        raise ValueError(msg)
    raise GactError(msg)


def check_pipeline(where: str) -> None:
    """Raise if a bounded wait of the quantize kernel's bulk-copy pipeline ever ran out on the current device:
    the tiles that warp had not written hold stale bytes, so training must not go on as if nothing had happened.
    Reads one word from the device (synchronises); called where the host waits anyway.  The word is cleared
    so that the next check reports new trouble only."""
    err = lib.gact_pipeline_error()
    if err > 0:
        lib.gact_pipeline_error_reset()
        raise GactError(f"{where}: a bulk copy of gact_quantize did not arrive within its wait limit "
                        f"(pipeline error {err}); compressed activations of this step are incomplete")


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor!")       # same wording as the reference's check


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """cudaStream_t of torch's current stream on the current device."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def guard_and_stream(t: torch.Tensor):
    """(context, cudaStream_t) for a library call on tensor t: one current-device query serves both."""
    cur = torch.cuda.current_device()
    idx = t.device.index
    if idx == cur:
        return _NO_GUARD, (_raw_stream(cur) if _raw_stream is not None else torch.cuda.current_stream().cuda_stream)
    return torch.cuda.device(t.device), torch.cuda.current_stream(t.device).cuda_stream


def device_guard(t: torch.Tensor):
    """Context that makes the tensor's device current for the duration of a library call.  The hooks almost
    always run with the right device already current, in which case this costs one comparison."""
    if t.device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(t.device)
