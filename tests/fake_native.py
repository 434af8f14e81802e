"""A stand-in for ``gact._native`` that runs on host memory, for CPU tests of the host-side logic.

The C ABI takes raw pointers, so the same calls work on CPU tensors when the functions behind them are the CPU
oracle's.  Only tests use this; the product always talks to libgact_b200.so.
"""
import contextlib
import ctypes as C

import numpy as np
import torch

import oracle

_o = oracle.lib()
GROUP = 256


class FakeLib:
    pipeline_error = 0          # tests set this to see the Python layer react

    def gact_version(self):
        return 100

    def gact_pipeline_error(self):
        return self.pipeline_error

    def gact_pipeline_error_reset(self):
        FakeLib.pipeline_error = 0
        return 0

    def gact_error_string(self, st):
        return b"fake"

    def gact_packed_bytes(self, n, bits):
        if bits not in (1, 2, 4, 8) or n < 0:
            return -1
        return oracle.sizes(n, bits)[2]

    def gact_mask_words(self, n):
        return (n + 511) // 512 * 16

    def gact_quantize(self, x, dtype, n, bits, seed, mode, noise, fma, packed, qmin, qscale, stream):
        return _o.oracle_quantize(x, dtype, n, bits, seed, mode, noise, fma, packed, qmin, qscale)

    def gact_dequantize(self, packed, qmin, qscale, dtype, n, bits, out, stream):
        return _o.oracle_dequantize(packed, qmin, qscale, dtype, n, bits, out)

    def gact_minimax(self, x, dtype, n, mn, mx, stream):
        return _o.oracle_minimax(x, dtype, n, mn, mx)

    def gact_mask_pack(self, x, n, words, flag, stream):
        _o.oracle_mask_pack(x, n, words)
        if flag:
            arr = np.ctypeslib.as_array((C.c_uint8 * n).from_address(x))
            if (arr > 1).any():
                C.c_int.from_address(flag).value = 1
        return 0

    def gact_mask_unpack(self, words, n, out, stream):
        return _o.oracle_mask_unpack(words, n, out)

    def gact_sq_diffs3_scratch_bytes(self):
        return 64

    def gact_sq_diffs3(self, g0, g1, g2, P, seg_ptr, seg_off, seg_len, nseg, scratch, out3, stream):
        if nseg:
            ptrs = (C.c_uint64 * nseg).from_address(seg_ptr)
            lens = (C.c_int64 * nseg).from_address(seg_len)
            flat = np.concatenate([np.ctypeslib.as_array((C.c_float * lens[k]).from_address(ptrs[k])) for k in range(nseg)])
            flat = np.ascontiguousarray(flat)
            g2 = flat.ctypes.data
        return _o.oracle_sq_diffs3(g0, g1, g2, P, out3)

    def gact_sensitivity(self, d3, scale, Cout, L, stream):
        d = np.ctypeslib.as_array((C.c_double * (3 * L)).from_address(d3)).reshape(L, 3)
        out = (C.c_float * L).from_address(Cout)
        for l in range(L):
            out[l] = oracle.sensitivity([np.float32(v * scale) for v in d[l]])
        return 0

    def gact_calc_precision(self, b, Cp, w, L, target, status, stream):
        st = _o.oracle_calc_precision(b, Cp, w, L, target)
        if status:
            C.c_int.from_address(status).value = 8 if st else 0
        return 0


class FakeNative:
    """Drop-in for the module object ``gact._native``."""
    F32, F16, BF16 = 0, 1, 2
    DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    RNG_CURAND, RNG_FAST, RNG_RTN, RNG_EXTERNAL = 0, 1, 2, 3
    RNG_CODE = {"curand": 0, "fast": 1, "rtn": 2, "external": 3}
    GROUP = 256
    lib = FakeLib()
    quantize_call = lib.gact_quantize
    dequantize_call = lib.gact_dequantize

    @staticmethod
    def check(status, what):
        if status:
            raise RuntimeError(f"{what}: status {status}")

    GactError = RuntimeError

    @staticmethod
    def check_pipeline(where):
        if FakeNative.lib.gact_pipeline_error() > 0:
            FakeNative.lib.gact_pipeline_error_reset()
            raise RuntimeError(f"{where}: pipeline error")

    @staticmethod
    def require_cuda(t, name):
        return None

    @staticmethod
    def stream_ptr():
        return 0

    @staticmethod
    def device_guard(t):
        return contextlib.nullcontext()

    @staticmethod
    def guard_and_stream(t):
        return contextlib.nullcontext(), 0


def install(monkeypatch):
    """Route gact.ops / gact.autoprec / gact.quantizer to the host-memory stand-in."""
    import gact.ops
    import gact.autoprec
    import gact.quantizer
    monkeypatch.setattr(gact.ops, "nv", FakeNative)
    monkeypatch.setattr(gact.autoprec, "nv", FakeNative)
    import gact.controller
    monkeypatch.setattr(gact.controller, "_nv", FakeNative)
    monkeypatch.setattr(gact.quantizer, "_hooks", None)        # the native hooks only take CUDA tensors
    monkeypatch.setattr(gact.quantizer.Quantizer, "_on_device", staticmethod(lambda t: True))
