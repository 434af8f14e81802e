"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle on the same inputs.

Bar: packed codes, per-group min and scale, and dequantized values are bit-exact (integer / IEEE work on
both sides; NaN payloads are normalised before comparing).
"""
import pytest
import torch

import oracle
from helpers import abi_dequantize, abi_quantize, assert_bits_equal

pytestmark = pytest.mark.gpu



@pytest.fixture(autouse=True)
def no_wait_ran_out():
    """The fp16 / bf16 kernel waits for its bulk copies with a bound; none of these tests may ever hit it."""
    from gact import _native as nv
    yield
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


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bits", BITS)
def test_kinds_of_group_side_by_side(dtype, bits):
    """The 16-bit kernel treats three kinds of group differently (plain; guarded: a NaN, an infinity or an
    overflowing range; special: scale +inf or not positive) and runs tiles of plain groups through a copy of the code
    pass without per-group tests.  Here every kind sits next to every other, tile by tile (tiles of 4 and 8 groups)."""
    g = torch.Generator().manual_seed(17)

    def group(kind):
        x = torch.randn(256, generator=g)
        if kind == 1:
            x[7] = float("nan")
        elif kind == 2:
            x[:] = float("nan")
        elif kind == 3:
            x[200] = float("inf")
        elif kind == 4:
            x[31] = float("-inf")
        elif kind == 5:
            x[0], x[255] = 60000.0, -60000.0           # the range overflows half precision
        elif kind == 6:
            x[:] = 1.25                                # fp16: scale +inf
        elif kind == 7:
            x = 1.0 + x * 1e-7                         # a range of a few ulps, or none
        elif kind == 8:
            x[3], x[4], x[100] = float("nan"), float("inf"), float("-inf")
        elif kind == 9:
            x = x.clamp_min(0)
        elif kind == 10:
            x[::2] = float("nan")
        return x

    order = [0] * 8 + list(range(11)) + [0] * 5 + [1, 0, 0, 0, 0, 0, 0, 0] + [0, 0, 0, 0, 6, 0, 0, 0] + [9] * 8 \
        + [5, 0, 0, 3] + [0] * 12 + [2, 2, 2, 2, 2, 2, 2, 2] + [10, 7, 4, 8, 0, 9, 6, 5]
    x = torch.cat([group(k) for k in order] + [torch.randn(100, generator=g)]).to(dtype)
    for mode in ("fast", "curand", "rtn"):
        check_case(x, bits, seed=5, rng_mode=mode)
    # the same groups in a tensor large enough for tiles of 8 groups (two rounds over the resident warps)
    if dtype != torch.float32 and bits in (2, 8):
        big = make_input("relu", 256 * 60000, dtype, seed=8)
        big[256 * 1000:256 * 1000 + x.numel()] = x
        big[256 * 59990:256 * 59990 + 256 * 8] = x[256 * 8:256 * 16]
        check_case(big, bits, seed=6, rng_mode="fast")


def test_random_cases_soak():
    """Sixty seeded random cases - dtype, width, noise mode, size (1 .. 3 M elements), distribution, storage offset -
    each compared bit for bit with the oracle."""
    import random
    rnd = random.Random(20240607)
    kinds = ["randn", "relu", "uniform", "tiny", "large", "special", "zeros_signed"]
    for case in range(60):
        dtype = rnd.choice(DTYPES)
        bits = rnd.choice(BITS)
        mode = rnd.choice(["fast", "fast", "curand", "rtn"])
        n = rnd.choice([rnd.randint(1, 5000), rnd.randint(5000, 300000), rnd.randint(300000, 3000000)])
        off = rnd.choice([0, 0, 1, 3, 8])
        x = make_input(rnd.choice(kinds), n + off, dtype, seed=case)
        xg = x.cuda()[off:]
        seed = rnd.getrandbits(40)
        pk, mn, sc = abi_quantize(xg, bits, seed, mode)
        opk, omn, osc = oracle.quantize(x[off:].contiguous(), bits, seed, mode)
        tag = f"case {case}: {dtype} b={bits} n={n} off={off} {mode}"
        assert_bits_equal(mn, omn, "qmin " + tag)
        assert_bits_equal(sc, osc, "qscale " + tag)
        assert_bits_equal(pk, opk, "packed " + tag)
        assert_bits_equal(abi_dequantize(pk, mn, sc, n, bits), oracle.dequantize(opk, omn, osc, n, bits), "dequantized " + tag)


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
    assert f(x.data_ptr() + 2, 0, 500, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 4  # not even element-aligned
    assert f(x.data_ptr(), 0, 512, 2, 0, 0, None, 1, pk.data_ptr() + 8, q.data_ptr(), q.data_ptr(), s) == 4  # packed output
    assert f(x.data_ptr(), 0, -1, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 5       # size
    assert f(x.data_ptr(), 0, 512, 2, 0, 3, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 6      # noise missing
    assert f(x.data_ptr(), 0, 0, 2, 0, 0, None, 1, pk.data_ptr(), q.data_ptr(), q.data_ptr(), s) == 0        # empty input
    torch.cuda.synchronize()


def test_more_than_2_to_31_elements():
    """64-bit indexing: a 4.3 GB fp16 tensor; the far end is checked against the oracle (round to nearest has no
    index-dependent noise, so a slice that starts on a row-block boundary can be checked on its own)."""
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


# ---- the sizes at which the 16-bit kernel changes what it does ------------------------------------------------------
TILE = 8 * 256                      # elements per warp tile
WARPS = 148 * 3 * 8                 # resident warps of a full launch on a B200


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", BITS)
def test_tile_and_wave_boundaries(dtype, bits):
    """Whole tiles only / one group more / a ragged end; fewer tiles than a block has warps; one tile fewer, as many
    and one more than the resident warps (where a warp's second stage comes into use), and twice that plus one
    (where the first stage is refilled); the group counts either side of the switch from 4- to 8-group tiles."""
    small = 2 * WARPS * 8                 # groups: below this many a tensor is cut into tiles of 4 groups, from here on of 8
    sizes = [TILE, TILE + 256, TILE - 1, 3 * TILE + 5 * 256 + 77, 8 * TILE, 9 * TILE + 1,
             (WARPS - 1) * TILE, WARPS * TILE + 100, (WARPS + 1) * TILE + 256 * 3, (2 * WARPS + 1) * TILE + 19,
             (small - 1) * 256 + 5, small * 256, (small + 1) * 256 - 3]
    for j, n in enumerate(sizes):
        check_case(make_input("relu" if j % 2 else "randn", n, dtype, seed=j), bits, 3 + j, "fast")
    check_case(make_input("randn", (2 * WARPS + 1) * TILE + 19, dtype, seed=5), bits, 1, "rtn")
    if bits in (1, 4):
        check_case(make_input("special", (WARPS + 2) * TILE + 300, dtype, seed=6), bits, 2, "curand")


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_mixed_list_sizes(bits):
    """2^20 ... 2^26 elements, the sizes of the sweep's mixed list."""
    for k in range(20, 27):
        check_case(make_input("randn", 1 << k, torch.float16, seed=k), bits, k, "fast")


# ---- the whole benchmark tensor --------------------------------------------------------------------------------------
_BIG = {}


def big_relu(dtype):
    if dtype not in _BIG:
        g = torch.Generator().manual_seed(0)
        _BIG[dtype] = torch.randn(128 * 64 * 112 * 112, generator=g).clamp_min_(0).to(dtype)
    return _BIG[dtype]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", BITS)
def test_whole_config2_tensor(dtype, bits):
    """128x64x112x112 post-ReLU activations: every packed byte, min, scale and dequantized value of the full tensor
    against the oracle - the default mode for both types, the reference's stream for fp16 (the reference has no bf16)."""
    x = big_relu(dtype)
    check_case(x, bits, 42, "fast")
    if dtype == torch.float16:
        check_case(x, bits, 42, "curand")
    if bits == 2:
        check_case(x, bits, 42, "rtn")


# ---- contiguous tensors that do not start on a 16-byte boundary ----------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("bits", [1, 4])
def test_inputs_at_odd_offsets(dtype, bits):
    """A contiguous view may start anywhere in its storage (t[1:] of a tensor with an odd row length); the reference
    takes any contiguous tensor.  Same bytes as for an aligned copy, and the output may sit at an odd offset too."""
    from gact import _native as nv
    for off, n in ((1, 256 * 21 + 3), (3, 5 * TILE + 77), (5, 300)):
        base = make_input("randn", n + off, dtype, seed=off)
        x_cpu = base[off:].clone()
        xg = base.cuda()[off:]
        assert xg.data_ptr() % 16 != 0 and xg.is_contiguous()
        for mode in ("fast", "curand", "rtn"):
            pk, mn, sc = abi_quantize(xg, bits, 9, mode)
            opk, omn, osc = oracle.quantize(x_cpu, bits, 9, mode)
            assert_bits_equal(pk, opk, "packed")
            assert_bits_equal(mn, omn, "min")
            assert_bits_equal(sc, osc, "scale")
        # dequantize into a view at an odd offset, with guard elements on both sides
        out = torch.full((n + off + 8,), -777.0, dtype=dtype, device="cuda")
        view = out[off:off + n]
        dpk, dmn, dsc = opk.cuda(), omn.cuda(), osc.cuda()
        st = nv.lib.gact_dequantize(dpk.data_ptr(), dmn.data_ptr(), dsc.data_ptr(), nv.DTYPE_CODE[dtype],
                                    n, bits, view.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()
        assert_bits_equal(view, oracle.dequantize(opk, omn, osc, n, bits), "dequantized")
        assert bool((out[:off] == -777.0).all()) and bool((out[off + n:] == -777.0).all())
        # min / max only
        G = (n + 255) // 256
        lo = torch.empty(G, dtype=dtype, device="cuda")
        hi = torch.empty(G, dtype=dtype, device="cuda")
        assert nv.lib.gact_minimax(xg.data_ptr(), nv.DTYPE_CODE[dtype], n, lo.data_ptr(), hi.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream) == 0
        wlo, whi = oracle.minimax(x_cpu)
        assert_bits_equal(lo, wlo, "min")
        assert_bits_equal(hi, whi, "max")


# ---- a wait of the bulk-copy pipeline that runs out ------------------------------------------------------------------
def test_bounded_wait_runs_out_and_the_library_recovers():
    """With one bulk copy withheld (a diagnostics switch) the waiting warp gives up after the wait limit, records the
    error and leaves; the launch ends by itself.  After a reset the next launch is bit-exact again.  Nothing faults
    and nothing spins: the wait is a bounded poll of an mbarrier that simply never completes."""
    from gact import _native as nv
    x_cpu = make_input("randn", 64 * TILE + 100, torch.float16, seed=1)
    x = x_cpu.cuda()
    assert nv.lib.gact_pipeline_error() == 0
    nv.lib.gact_pipeline_test_hook(2000, 1)
    try:
        n = x.numel()
        pk = torch.zeros(nv.lib.gact_packed_bytes(n, 4), dtype=torch.uint8, device="cuda")
        mn = torch.zeros((n + 255) // 256, dtype=torch.float16, device="cuda")
        sc = torch.zeros_like(mn)
        st = nv.lib.gact_quantize(x.data_ptr(), nv.F16, n, 4, 1, nv.RNG_FAST, None, 1, pk.data_ptr(), mn.data_ptr(), sc.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
        assert st == 0
        torch.cuda.synchronize()                                   # the launch finished on its own
        assert nv.lib.gact_pipeline_error() == 2
        with pytest.raises(nv.GactError):
            nv.check_pipeline("test")                              # what the Python layer does at its sync points
    finally:
        nv.lib.gact_pipeline_test_hook(0, 0)
        nv.lib.gact_pipeline_error_reset()
    assert nv.lib.gact_pipeline_error() == 0
    check_case(x_cpu, 4, 1, "fast")
