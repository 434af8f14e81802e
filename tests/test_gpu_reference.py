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
