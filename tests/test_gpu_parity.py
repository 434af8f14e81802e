"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle on the same inputs.

Bar: packed codes, per-group min and scale, and dequantized values are bit-exact (integer / IEEE work on
both sides; NaN payloads are normalised before comparing).
"""
import pytest
import torch

import oracle
from helpers import abi_dequantize, abi_quantize, assert_bits_equal

pytestmark = pytest.mark.gpu



@pytest.fixture(autouse=True, params=["ring", "default"])
def ring_threshold(request):
    """Every test of this module runs twice: with the ring kernel taking every tensor of at least one 32 KB chunk,
    and with the library's own choice (ring from 48 MB on, direct loads below)."""
    from gact import _native as nv
    before = nv.lib.gact_set_ring_min_chunks(1 if request.param == "ring" else 0)
    yield request.param
    nv.lib.gact_set_ring_min_chunks(before)
    assert nv.lib.gact_pipeline_error() == 0


DTYPES = [torch.float32, torch.float16, torch.bfloat16]
BITS = [1, 2, 4, 8]
# sizes: single element, around one group, ragged (n % 256 != 0), G % wpt != 0 for every width, several tiles
SIZES = [1, 255, 256, 257, 7700, 256 * 13, 256 * 64 + 5, 100 * 77]


def make_input(kind, n, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g)
    if kind == "relu":
        x = x.clamp_min(0)
    elif kind == "uniform":
        x = torch.rand(n, generator=g)
    elif kind == "large":
        x = x * 3.0e4
    elif kind == "tiny":
        x = x * 1e-6
    elif kind == "const":
        x = torch.full((n,), 1.25)
    elif kind == "special":
        x = x.clone()
        idx = torch.randperm(n, generator=g)
        k = max(1, n // 50)
        x[idx[:k]] = float("nan")
        x[idx[k:2 * k]] = float("inf")
        x[idx[2 * k:3 * k]] = float("-inf")
        x[idx[3 * k:6 * k]] = 0.0
        x[idx[6 * k:9 * k]] = -0.0
    elif kind == "zeros_signed":
        # groups whose extreme is a zero of either sign: the reported sign follows the reference's order
        x = x.abs()
        idx = torch.randperm(n, generator=g)
        x[idx[: n // 3]] = 0.0
        x[idx[n // 3: n // 2]] = -0.0
        if n > 600:
            x[256:512] = -x[256:512]          # a group that is all <= 0 with zeros at the top
            x[512:600] = 0.0
            x[600:768] = -0.0                  # a group of zeros of both signs only
    return x.to(dtype)


def check_case(x_cpu, bits, seed, rng_mode, fma=True, noise=None):
    x = x_cpu.cuda()
    pk, mn, sc = abi_quantize(x, bits, seed, rng_mode, noise=noise, fma=fma)
    opk, omn, osc = oracle.quantize(x_cpu, bits, seed, rng_mode, noise=noise, fma=fma)
    tag = f"{x_cpu.dtype} b={bits} n={x_cpu.numel()} {rng_mode}"
    assert_bits_equal(mn, omn, "qmin " + tag)
    assert_bits_equal(sc, osc, "qscale " + tag)
    assert_bits_equal(pk, opk, "packed " + tag)
    out = abi_dequantize(pk, mn, sc, x_cpu.numel(), bits)
    oout = oracle.dequantize(opk, omn, osc, x_cpu.numel(), bits)
    assert_bits_equal(out, oout, "dequantized " + tag)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bits", BITS)
def test_quantize_sizes(dtype, bits):
    for n in SIZES:
        check_case(make_input("randn", n, dtype, seed=n), bits, seed=n % 7, rng_mode="curand")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("kind", ["relu", "uniform", "large", "tiny", "const", "special", "zeros_signed"])
def test_quantize_distributions(dtype, bits, kind):
    if kind == "large" and dtype == torch.float16:
        pass  # overflows to inf in fp16: still a valid (and interesting) input
    check_case(make_input(kind, 256 * 37 + 19, dtype, seed=3), bits, seed=11, rng_mode="curand")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bits", BITS)
def test_round_to_nearest_and_external_noise(dtype, bits):
    n = 256 * 21 + 100
    x = make_input("randn", n, dtype, seed=5)
    check_case(x, bits, 0, "rtn")
    G = (n + 255) // 256
    g = torch.Generator().manual_seed(9)
    noise = torch.rand(G * 256, generator=g)
    noise[::97] = 1.0          # the value that can push a code past 2^bits - 1 (no upper clamp)
    noise[5::89] = 0.0
    check_case(x, bits, 0, "external", noise=noise)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bits", BITS)
def test_fast_noise_arrangement(dtype, bits):
    """rng_mode 'fast': the same arithmetic on a different Philox arrangement (one call per 8 elements)."""
    for n in (1, 300, 256 * 13, 256 * 64 + 5):
        check_case(make_input("randn", n, dtype, seed=n), bits, seed=n + (7 << 33), rng_mode="fast")
    check_case(make_input("special", 256 * 37 + 19, dtype, seed=3), bits, seed=11, rng_mode="fast")
    check_case(make_input("relu", 256 * 5000 + 3, dtype, seed=3), bits, seed=2, rng_mode="fast")


@pytest.mark.parametrize("bits", BITS)
def test_fp32_unfused_multiply_add(bits):
    x = make_input("randn", 256 * 40 + 3, torch.float32, seed=8)
    check_case(x, bits, 4, "curand", fma=False)
    check_case(x, bits, 4, "rtn", fma=False)


def test_seed_is_64_bit():
    x = make_input("randn", 256 * 9, torch.float32, seed=1)
    for seed in (0, 1, 2**32 - 1, 2**32, (5 << 32) + 17, 2**64 - 1):
        check_case(x, 2, seed, "curand")


def test_config1_single_tensor_round_trip():
    """fp32 32x128x768 from N(0,1) with seed 0, group 256, 2 bit, seed 0."""
    torch.manual_seed(0)
    x = torch.randn(32, 128, 768)
    check_case(x.reshape(-1), 2, 0, "curand")


def test_many_row_blocks_grid_stride():
    """More tiles than the launch has warps, so every warp loops."""
    x = make_input("relu", 256 * 40000 + 77, torch.float16, seed=2)     # 16-bit, up to 40 960 groups: tiles of 4 groups
    check_case(x, 8, 3, "curand")
    check_case(x, 1, 3, "curand")
    x = make_input("relu", 256 * 50000 + 77, torch.float16, seed=3)     # above that: tiles of 8 groups
    check_case(x, 4, 3, "curand")
    check_case(x.to(torch.bfloat16), 2, 3, "fast")


def test_minimax_entry_point():
    from gact import _native as nv
    for dtype in DTYPES:
        x_cpu = make_input("zeros_signed", 256 * 33 + 10, dtype, seed=4)
        x = x_cpu.cuda()
        G = (x.numel() + 255) // 256
        mn = torch.empty(G, dtype=dtype, device="cuda")
        mx = torch.empty(G, dtype=dtype, device="cuda")
        st = nv.lib.gact_minimax(x.data_ptr(), nv.DTYPE_CODE[dtype], x.numel(), mn.data_ptr(), mx.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
        assert st == 0
        omn, omx = oracle.minimax(x_cpu)
        assert_bits_equal(mn, omn, "min")
        assert_bits_equal(mx, omx, "max")


def test_argument_errors():
    from gact import _native as nv
    x = torch.zeros(512, device="cuda")
    pk = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    q = torch.zeros(8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    f = nv.lib.gact_quantize
    assert f(x.data_ptr(), 0, 512, 3, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 1      # bits
    assert f(x.data_ptr(), 7, 512, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 2      # dtype
    assert f(None, 0, 512, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 3              # null
    assert f(x.data_ptr() + 4, 0, 500, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 4  # alignment
    assert f(x.data_ptr(), 0, -1, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 5       # size
    assert f(x.data_ptr(), 0, 512, 2, 0, 3, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 6      # noise missing
    assert f(x.data_ptr(), 0, 0, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 0        # empty input
    torch.cuda.synchronize()


def test_more_than_2_to_31_elements(ring_threshold):
    """64-bit indexing: a 4.3 GB fp16 tensor; the far end is checked against the oracle (round to nearest has no
    index-dependent noise, so a slice that starts on a row-block boundary can be checked on its own)."""
    if ring_threshold == "ring":
        pytest.skip("round to nearest never takes the ring kernel")
    from gact.ops import quantize_pack, dequantize_and_unpack
    n = (1 << 31) + 256 * 12 + 100
    free, _ = torch.cuda.mem_get_info()
    if free < 14 * (1 << 30):
        pytest.skip("not enough free device memory")
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.empty(n, dtype=torch.float16, device="cuda")
    step = 1 << 28
    for i in range(0, n, step):
        x[i:i + step] = torch.randn(min(step, n - i), device="cuda", generator=g).half()
    q, sc, mn = quantize_pack(x, 2, 0, rng_mode="rtn")
    G = (n + 255) // 256
    start_g = (G - 1024) // 4 * 4                        # a row-block boundary near the end
    tail = x[start_g * 256:].cpu()
    opk, omn, osc = oracle.quantize(tail, 2, 0, "rtn")
    assert torch.equal(q[start_g // 4 * 256:-1].cpu().view(torch.uint8), opk)
    assert_bits_equal(mn.reshape(-1)[start_g:], omn, "min")
    assert_bits_equal(sc.reshape(-1)[start_g:], osc, "scale")
    y = dequantize_and_unpack(q, (n,), 2, sc, mn)
    want = oracle.dequantize(opk, omn, osc, tail.numel(), 2)
    assert_bits_equal(y[start_g * 256:], want, "dequantized tail")
    first = oracle.quantize(x[:256 * 64].cpu(), 2, 0, "rtn")[0]
    assert torch.equal(q[:first.numel()].cpu().view(torch.uint8), first)
    del x, y, q
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", BITS)
def test_above_the_ring_threshold(dtype, bits, ring_threshold):
    """50 MB tensors: the size from which the library picks the ring kernel by itself, plus a ragged tail."""
    if ring_threshold == "ring":
        pytest.skip("same kernel either way at this size")
    n = 1536 * 16384 + 3 * 16384 + 1000
    x = make_input("relu", n, dtype, seed=bits)
    check_case(x, bits, 5, "fast")
    if bits in (2, 8):
        check_case(x, bits, 5, "curand")
