"""Python front-end of the CPU oracle (``gact_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline / reference arm import this package, and
only as the checker.  The product (``gact``) never does, and has no CPU fallback.

All functions take and return CPU torch tensors.  16-bit floats travel as their bit patterns; the C code
does its own fp16 / bf16 rounding in software.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "gact_oracle.c"
_LIB = _HERE / "libgact_oracle.so"

GROUP = 256
DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
RNG_MODES = {"curand": 0, "fast": 1, "rtn": 2, "external": 3}

_lib = None


def build(force: bool = False) -> Path:
    """Compile the C restatement with gcc (a second or two).  OpenMP is used when the compiler has it (it only
    spreads independent groups over the host cores); otherwise the oracle runs on one thread."""
    if force or not _LIB.exists() or _LIB.stat().st_mtime < _SRC.stat().st_mtime:
        base = ["-O2", "-fPIC", "-std=c11", "-ffp-contract=off", "-fno-fast-math", "-shared", "-o", str(_LIB), str(_SRC), "-lm"]
        compilers = [c for c in (os.environ.get("CC"), "/usr/bin/gcc", "gcc") if c]
        for extra in (["-fopenmp"], []):
            for cc in compilers:
                if subprocess.run([cc] + extra + base, capture_output=True).returncode == 0:
                    return _LIB
        raise RuntimeError("could not compile oracle/gact_oracle.c with any of %s" % compilers)
    return _LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB))
        c = ctypes
        L.oracle_quantize.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_int, c.c_uint64, c.c_int, c.c_void_p,
                                      c.c_int, c.c_void_p, c.c_void_p, c.c_void_p]
        L.oracle_dequantize.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int64, c.c_int, c.c_void_p]
        L.oracle_minimax.argtypes = [c.c_void_p, c.c_int, c.c_int64, c.c_void_p, c.c_void_p]
        L.oracle_mask_pack.argtypes = [c.c_void_p, c.c_int64, c.c_void_p]
        L.oracle_mask_unpack.argtypes = [c.c_void_p, c.c_int64, c.c_void_p]
        L.oracle_calc_precision.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64, c.c_double]
        L.oracle_sq_diffs3.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64, c.c_void_p]
        L.oracle_curand_uniform.argtypes = [c.c_uint64, c.c_uint64, c.c_uint32]
        L.oracle_curand_uniform.restype = c.c_float
        L.oracle_fast_noise.argtypes = [c.c_uint64, c.c_int64]
        L.oracle_fast_noise.restype = c.c_float
        L.oracle_philox4x32_10.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p]
        L.oracle_philox4x32_r.argtypes = [c.c_void_p, c.c_void_p, c.c_int, c.c_void_p]
        L.oracle_float_to_half.argtypes = [c.c_float]
        L.oracle_float_to_half.restype = c.c_uint16
        L.oracle_half_to_float.argtypes = [c.c_uint16]
        L.oracle_half_to_float.restype = c.c_float
        L.oracle_float_to_bf16.argtypes = [c.c_float]
        L.oracle_float_to_bf16.restype = c.c_uint16
        L.oracle_check_half_reciprocal.restype = c.c_int64
        L.oracle_check_markstein.argtypes = [c.c_uint32, c.c_int]
        L.oracle_check_markstein.restype = c.c_int64
        _lib = L
    return _lib


def _cpu(t: torch.Tensor) -> torch.Tensor:
    assert t.device.type == "cpu", "the oracle works on CPU tensors"
    return t.contiguous()


def sizes(n: int, bits: int):
    """(G, R, packed_bytes) for n elements: G groups of 256, R row-blocks of 8/bits groups."""
    G = (n + GROUP - 1) // GROUP
    wpt = 8 // bits
    R = (G + wpt - 1) // wpt
    return G, R, R * GROUP


def scale_dtype(dtype):
    """Storage type of the per-group scale: the input type, except fp32 for bf16 inputs."""
    return torch.float32 if dtype == torch.bfloat16 else dtype


def quantize(x: torch.Tensor, bits: int, seed: int, rng_mode: str = "curand", noise: torch.Tensor | None = None,
             fma: bool = True):
    """-> (packed uint8[R*256], qmin[G] in x.dtype, qscale[G] in scale_dtype(x.dtype))."""
    x = _cpu(x)
    n = x.numel()
    G, R, nbytes = sizes(n, bits)
    packed = torch.zeros(nbytes, dtype=torch.uint8)
    qmin = torch.empty(G, dtype=x.dtype)
    qscale = torch.empty(G, dtype=scale_dtype(x.dtype))
    nz_ptr = None
    if rng_mode == "external":
        noise = _cpu(noise).to(torch.float32)
        assert noise.numel() == G * GROUP, "noise is indexed like the zero-padded input"
        nz_ptr = noise.data_ptr()
    rc = lib().oracle_quantize(x.data_ptr(), DTYPES[x.dtype], n, bits, seed & (2**64 - 1), RNG_MODES[rng_mode], nz_ptr,
                               int(fma), packed.data_ptr(), qmin.data_ptr(), qscale.data_ptr())
    if rc:
        raise ValueError(f"oracle_quantize: status {rc}")
    return packed, qmin, qscale


def dequantize(packed: torch.Tensor, qmin: torch.Tensor, qscale: torch.Tensor, n: int, bits: int) -> torch.Tensor:
    packed, qmin, qscale = _cpu(packed), _cpu(qmin), _cpu(qscale)
    out = torch.empty(n, dtype=qmin.dtype)
    rc = lib().oracle_dequantize(packed.data_ptr(), qmin.data_ptr(), qscale.data_ptr(), DTYPES[qmin.dtype], n, bits,
                                 out.data_ptr())
    if rc:
        raise ValueError(f"oracle_dequantize: status {rc}")
    return out


def minimax(x: torch.Tensor):
    x = _cpu(x)
    G = (x.numel() + GROUP - 1) // GROUP
    mn = torch.empty(G, dtype=x.dtype)
    mx = torch.empty(G, dtype=x.dtype)
    lib().oracle_minimax(x.data_ptr(), DTYPES[x.dtype], x.numel(), mn.data_ptr(), mx.data_ptr())
    return mn, mx


def op_quantize(x: torch.Tensor, q_bit: int, seed: int, **kw):
    """Same return contract as the reference's ``op_quantize`` (gact/gact/ops.py:57-59):
    ``[q_input, q_bit, q_scale, q_min]``; q_input is int8 of R*256+1 bytes whose last byte is unspecified."""
    n = x.numel()
    G = (n + GROUP - 1) // GROUP
    if q_bit == 32:
        flat = torch.zeros(G * GROUP, dtype=x.dtype)
        flat[:n] = x.reshape(-1)
        groups = flat.reshape(G, GROUP)
        q_min = groups.min(dim=-1, keepdim=True).values
        q_scale = groups.max(dim=-1, keepdim=True).values - q_min
        return [groups, 32, q_scale, q_min]
    packed, qmin, qscale = quantize(x, q_bit, seed, **kw)
    q_input = torch.zeros(packed.numel() + 1, dtype=torch.int8)
    q_input[:-1] = packed.view(torch.int8)
    return [q_input, q_bit, qscale.reshape(G, 1, 1), qmin.reshape(G, 1, 1)]


def op_dequantize(q, shape):
    """Reference ``op_dequantize`` (gact/gact/ops.py:61-69)."""
    q_input, q_bit, q_scale, q_min = q
    n = 1
    for s in shape:
        n *= int(s)
    if q_bit == 32:
        return q_input.reshape(-1)[:n].reshape(*shape).contiguous()
    packed = q_input.view(torch.uint8)[: sizes(n, q_bit)[2]]
    return dequantize(packed, q_min.reshape(-1), q_scale.reshape(-1), n, q_bit).reshape(*shape)


def mask_pack(x: torch.Tensor) -> torch.Tensor:
    x = _cpu(x).reshape(-1)
    if x.dtype == torch.bool:
        x = x.to(torch.uint8)
    assert x.dtype == torch.uint8
    words = torch.zeros((x.numel() + 511) // 512 * 16, dtype=torch.int32)
    lib().oracle_mask_pack(x.data_ptr(), x.numel(), words.data_ptr())
    return words


def mask_unpack(words: torch.Tensor, n: int) -> torch.Tensor:
    words = _cpu(words)
    out = torch.empty(n, dtype=torch.uint8)
    lib().oracle_mask_unpack(words.data_ptr(), n, out.data_ptr())
    return out


def calc_precision(b: torch.Tensor, C: torch.Tensor, w: torch.Tensor, target: float):
    """In-place greedy allocation; returns (b, status) with status 1 when the budget is unreachable."""
    assert b.dtype == torch.int32 and C.dtype == torch.float32 and w.dtype == torch.int64
    b, C, w = _cpu(b), _cpu(C), _cpu(w)
    st = lib().oracle_calc_precision(b.data_ptr(), C.data_ptr(), w.data_ptr(), b.numel(), float(target))
    return b, st


def sq_diffs3(g0, g1, g2):
    g0, g1, g2 = _cpu(g0).float(), _cpu(g1).float(), _cpu(g2).float()
    out = torch.zeros(3, dtype=torch.float64)
    lib().oracle_sq_diffs3(g0.data_ptr(), g1.data_ptr(), g2.data_ptr(), g0.numel(), out.data_ptr())
    return out


def sensitivity(d3) -> float:
    """C_l from the three squared distances (gact/gact/autoprec.py:119-126)."""
    d01, d02, d12 = (float(v) for v in d3)
    sens = max(d01, max(d02, d12) * 2)
    if sens != sens or sens in (float("inf"), float("-inf")) or sens > 1e10:
        return 1e10
    return sens


def fingerprint(t: torch.Tensor):
    """(hash of the sampled elements, sum of raw bit patterns) as the library's gact_fingerprint defines them: both
    wrapping 64-bit sums; sample i at i * (n // cnt), cnt = min(n, 100), each hashed with the splitmix64 finaliser of
    bits + 0x9E3779B97F4A7C15 * (i + 1).  The sample positions are the reference's (gact/gact/utils.py:16-24)."""
    import numpy as np
    raw = _cpu(t).reshape(-1).view({1: torch.uint8, 2: torch.int16, 4: torch.int32}[t.element_size()]).numpy()
    raw = raw.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[t.element_size()]).astype(np.uint64)
    n = raw.size
    if n == 0:
        return 0, 0
    cnt = min(n, 100)
    idx = np.arange(cnt, dtype=np.int64) * (n // cnt)
    with np.errstate(over="ignore"):
        z = raw[idx] + np.uint64(0x9E3779B97F4A7C15) * (np.arange(cnt, dtype=np.uint64) + np.uint64(1))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
        return int(z.sum(dtype=np.uint64)), int(raw.sum(dtype=np.uint64))


def threads() -> int:
    """Host threads the quantize / dequantize loops use (OpenMP)."""
    return int(lib().oracle_threads())


def set_threads(t: int) -> None:
    lib().oracle_set_threads(int(t))


def curand_uniform(seed: int, subsequence: int, draw: int) -> float:
    return float(lib().oracle_curand_uniform(seed, subsequence, draw))


def fast_noise(seed: int, elem: int) -> float:
    return float(lib().oracle_fast_noise(seed, elem))


def philox(counter, key, rounds=10):
    """Philox4x32 with the given number of rounds (10 = cuRAND's generator, 7 = what rng_mode 'fast' uses)."""
    c = (ctypes.c_uint32 * 4)(*counter)
    k = (ctypes.c_uint32 * 2)(*key)
    o = (ctypes.c_uint32 * 4)()
    if rounds == 10:
        lib().oracle_philox4x32_10(c, k, o)
    else:
        lib().oracle_philox4x32_r(c, k, rounds, o)
    return list(o)
