"""Shared helpers of the test-suite: bit-level tensor comparison and direct calls through the C ABI."""
import ctypes

import torch

GROUP = 256


def bits_of(t: torch.Tensor) -> torch.Tensor:
    """Integer view of a float tensor with every NaN collapsed to one pattern (CPU and GPU produce
    different NaN payloads; which values are NaN must still agree)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        v = t.view(torch.int32).clone()
        v[torch.isnan(t)] = 0x7FC00000
        return v
    if t.dtype in (torch.float16, torch.bfloat16):
        v = t.view(torch.int16).clone()
        v[torch.isnan(t)] = 0x7FFF
        return v
    return t


def assert_bits_equal(a: torch.Tensor, b: torch.Tensor, what: str = ""):
    a, b = bits_of(a).reshape(-1), bits_of(b).reshape(-1)
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if not torch.equal(a, b):
        bad = (a != b).nonzero().reshape(-1)
        i = int(bad[0])
        raise AssertionError(f"{what}: {bad.numel()} of {a.numel()} differ, first at {i}: {int(a[i])} vs {int(b[i])}")


def abi_quantize(x, bits, seed, rng_mode="curand", noise=None, fma=True, pad=64):
    """gact_quantize through ctypes on a CUDA tensor.  Outputs carry `pad` guard bytes/elements on both
    sides, filled with a canary that is verified after the call.  Returns (packed u8, qmin, qscale) on CPU."""
    from gact import _native as nv
    assert x.is_cuda and x.is_contiguous()
    n = x.numel()
    G = (n + GROUP - 1) // GROUP
    nbytes = nv.lib.gact_packed_bytes(n, bits)
    pk = torch.full((nbytes + 2 * pad,), 0x5A, dtype=torch.uint8, device=x.device)
    canary = torch.tensor(12345.0).to(x.dtype)
    qmin = torch.full((G + 2 * pad,), float(canary), dtype=x.dtype, device=x.device)
    sdt = torch.float32 if x.dtype == torch.bfloat16 else x.dtype       # bf16 keeps an fp32 scale
    qscale = torch.full((G + 2 * pad,), float(canary), dtype=sdt, device=x.device)
    es = x.element_size()
    nz = None
    if rng_mode == "external":
        noise = noise.to(device=x.device, dtype=torch.float32).contiguous()
        nz = noise.data_ptr()
    assert pad % 16 == 0
    st = nv.lib.gact_quantize(x.data_ptr(), nv.DTYPE_CODE[x.dtype], n, bits, seed & (2**64 - 1), nv.RNG_CODE[rng_mode], nz,
                              int(fma), pk.data_ptr() + pad, qmin.data_ptr() + pad * es, qscale.data_ptr() + pad * qscale.element_size(),
                              torch.cuda.current_stream().cuda_stream)
    assert st == 0, nv.lib.gact_error_string(st)
    torch.cuda.synchronize()
    pk, qmin, qscale = pk.cpu(), qmin.cpu(), qscale.cpu()
    assert bool((pk[:pad] == 0x5A).all()) and bool((pk[pad + nbytes:] == 0x5A).all()), "packed: guard bytes overwritten"
    for t, nm in ((qmin, "qmin"), (qscale, "qscale")):
        assert bool((t[:pad] == canary).all()) and bool((t[pad + G:] == canary).all()), f"{nm}: guard overwritten"
    return pk[pad:pad + nbytes].clone(), qmin[pad:pad + G].clone(), qscale[pad:pad + G].clone()


def abi_dequantize(packed, qmin, qscale, n, bits, device="cuda", pad=64):
    """gact_dequantize through ctypes; inputs are CPU tensors; returns the n outputs on CPU and checks that
    nothing outside [0, n) was written."""
    from gact import _native as nv
    dt = qmin.dtype
    canary = torch.tensor(-777.0).to(dt)
    out = torch.full((n + 2 * pad,), float(canary), dtype=dt, device=device)
    es = out.element_size()
    pk = packed.to(device)
    mn, sc = qmin.to(device).contiguous(), qscale.to(device).contiguous()
    st = nv.lib.gact_dequantize(pk.data_ptr(), mn.data_ptr(), sc.data_ptr(), nv.DTYPE_CODE[dt], n, bits,
                                out.data_ptr() + pad * es, torch.cuda.current_stream().cuda_stream)
    assert st == 0, nv.lib.gact_error_string(st)
    torch.cuda.synchronize()
    out = out.cpu()
    assert bool((out[:pad] == canary).all()) and bool((out[pad + n:] == canary).all()), "out: guard overwritten"
    return out[pad:pad + n].clone()
