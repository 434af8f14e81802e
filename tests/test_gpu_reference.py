"""GPU parity against the reference's own CUDA kernels, built unmodified for sm_100a by oracle/build_ref.py
(into oracle/_ref/, which travels with the repository snapshot).  Skipped when those binaries are absent.

The reference kernels need a zero-padded copy of the input viewed as (G, 1, 256); ours reads the tensor in
place.  Bit-exact: packed bytes (the reference's spare last byte excluded), min, scale, dequantized values.
"""
import pytest
import torch

import oracle
from oracle import build_ref
from helpers import abi_dequantize, abi_quantize, assert_bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    q = build_ref.load("ref_quantization")
    m = build_ref.load("ref_minimax")
    if q is None or m is None:
        pytest.skip("oracle/_ref not built (needs the reference checkout at build time)")
    return q, m


def ref_quantize(ref, x, bits, seed):
    q, m = ref
    n = x.numel()
    G = (n + 255) // 256
    flat = torch.zeros(G * 256, dtype=x.dtype, device=x.device)
    flat[:n] = x.reshape(-1)
    groups = flat.reshape(G, 256)
    mn, mx = m.minimax(groups)
    packed, scale = q.pack_single_precision(groups.view(G, 1, 256), mn.view(G, 1, 1), mx.view(G, 1, 1), bits, True, seed)
    out = q.unpack_single_precision(packed, bits, scale, mn.view(G, 1, 1), G, 1, 256)
    torch.cuda.synchronize()
    return packed, mn, scale.reshape(-1), out.reshape(-1)[:n]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("kind", ["randn", "relu", "special", "zeros_signed", "uniform"])
def test_against_reference_kernels(ref, dtype, bits, kind):
    from test_gpu_parity import make_input
    for n, seed in ((256 * 24, 0), (256 * 37 + 19, 5), (1000 * 100, 12345)):
        x_cpu = make_input(kind, n, dtype, seed=seed + 1)
        x = x_cpu.cuda()
        rpk, rmn, rsc, rout = ref_quantize(ref, x, bits, seed)
        pk, mn, sc = abi_quantize(x, bits, seed, "curand")
        tag = f"{dtype} b={bits} n={n} {kind}"
        assert_bits_equal(mn, rmn, "qmin vs reference " + tag)
        assert_bits_equal(sc, rsc, "qscale vs reference " + tag)
        assert_bits_equal(pk, rpk.cpu().view(torch.uint8)[:-1], "packed vs reference " + tag)
        out = abi_dequantize(pk, mn, sc, n, bits)
        assert_bits_equal(out, rout, "dequantized vs reference " + tag)
        # and the oracle agrees with the reference too (this is what pins the oracle)
        opk, omn, osc = oracle.quantize(x_cpu, bits, seed, "curand")
        assert_bits_equal(opk, rpk.cpu().view(torch.uint8)[:-1], "oracle packed vs reference " + tag)
        assert_bits_equal(omn, rmn, "oracle qmin vs reference " + tag)
        assert_bits_equal(osc, rsc, "oracle qscale vs reference " + tag)


def test_mask_against_reference_kernels(ref):
    """Only sizes that are multiples of 512: for other sizes the reference kernel stores past its output."""
    q, _ = ref
    from gact.ops import op_quantize_mask, op_dequantize_mask
    for n in (512, 512 * 300, 1024 * 1000):
        x = (torch.rand(n, device="cuda") < 0.4).to(torch.uint8)
        rmask = q.act_quantize_dropout_mask(x)
        ours = op_quantize_mask(x)[0]
        assert torch.equal(ours, rmask)
        rout = q.act_dequantize_dropout_mask(rmask, n)
        assert torch.equal(op_dequantize_mask([ours, x.shape]), rout)
        assert torch.equal(rout, x)


def _reference_style_quantize(ext_minimax, ext_quantization, x, q_bit, seed):
    """The data flow of the reference's op_quantize / op_dequantize (pad, group, minimax, pack; unpack, slice),
    written against whatever modules are passed in."""
    n = x.numel()
    G = (n + 255) // 256
    flat = x.reshape(1, -1)
    if G * 256 > n:
        flat = torch.cat([flat, torch.zeros([1, G * 256 - n], dtype=x.dtype, device=x.device)], dim=1)
    groups = flat.reshape(-1, 256)
    q_min, mx = ext_minimax.minimax(groups)
    q_min = q_min.reshape(G, -1, 1)
    q_input, q_scale = ext_quantization.pack_single_precision(groups.view(G, -1, 256), q_min, mx.view(G, -1, 1), q_bit, True, seed)
    out = ext_quantization.unpack_single_precision(q_input, q_bit, q_scale, q_min, G, 1, 256)
    return q_input, q_scale, q_min, out.ravel()[:n].reshape(x.shape).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_pybind_compatible_shims_against_reference_modules(ref, dtype, bits):
    """gact.cpp_extension.{minimax,quantization} are drop-ins for the reference's modules of the same names: the same
    Python, run once on the reference's modules and once on the shims, gives the same tensors."""
    import gact.cpp_extension.minimax as shim_minimax
    import gact.cpp_extension.quantization as shim_quantization
    rq, rm = ref
    for shape, seed in (((24, 256), 0), ((37, 300), 5), ((8, 17, 33), 77)):
        x = torch.randn(shape, device="cuda").to(dtype)
        a = _reference_style_quantize(rm, rq, x, bits, seed)
        b = _reference_style_quantize(shim_minimax, shim_quantization, x, bits, seed)
        assert a[0].shape == b[0].shape and a[0].dtype == b[0].dtype
        assert torch.equal(a[0][:-1], b[0][:-1])                   # the last byte is unspecified on both sides
        for i, what in ((1, "scale"), (2, "min"), (3, "dequantized")):
            assert a[i].shape == b[i].shape and a[i].dtype == b[i].dtype, what
            assert_bits_equal(b[i].reshape(-1), a[i].reshape(-1), f"{what} {dtype} b={bits} {shape}")
    m = (torch.rand(512 * 9, device="cuda") < 0.3).to(torch.uint8)
    assert torch.equal(shim_quantization.act_quantize_dropout_mask(m), rq.act_quantize_dropout_mask(m))
    w = shim_quantization.act_quantize_dropout_mask(m)
    assert torch.equal(shim_quantization.act_dequantize_dropout_mask(w, m.numel()), m)


def test_calc_precision_shim_against_reference_module():
    """The CPU-side greedy allocator of the reference (built unmodified) against gact.cpp_extension.calc_precision."""
    rc = build_ref.load("ref_calc_precision")
    if rc is None:
        pytest.skip("oracle/_ref not built")
    from gact.cpp_extension.calc_precision import calc_precision
    g = torch.Generator().manual_seed(3)
    for L in (3, 50, 700):
        C = torch.rand(L, generator=g) * 100
        C[::5] = 1.0
        w = torch.randint(1, 1 << 22, (L,), generator=g, dtype=torch.int64)
        for avg in (1.2, 2.0, 4.0, 6.5):
            target = avg * float(w.sum())
            want = rc.calc_precision(torch.full((L,), 32, dtype=torch.int32), C, w, target)
            got = calc_precision(torch.full((L,), 32, dtype=torch.int32), C, w, target)
            assert torch.equal(got, want), (L, avg)
