"""CPU tests that pin the oracle: golden vectors, known answers from the reference's own tests, an independent
numpy restatement, and the arithmetic identities the kernels rely on."""
import json
import struct

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle


# ---- golden vectors ----------------------------------------------------------------------------------------------
def test_philox_and_uniform_against_curand_header(golden_dir):
    """Vectors drawn by the CUDA toolkit's cuRAND header compiled for the host (gen_curand_vectors.cu)."""
    d = json.loads((golden_dir / "curand_philox_uniform.json").read_text())
    assert len(d["cases"]) == 63
    for c in d["cases"]:
        for i, bits in enumerate(c["bits"]):
            u = oracle.curand_uniform(c["seed"], c["subsequence"], i)
            assert struct.unpack("I", struct.pack("f", u))[0] == bits, (c["seed"], c["subsequence"], i)


def test_philox_known_answer():
    """Random123's published test vector for Philox4x32-10 with all-ones counter and key."""
    assert oracle.philox([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert oracle.philox([0] * 4, [0] * 2) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]


def test_philox_round_count():
    """The rounds-parameterised routine is the same round function: ten rounds give cuRAND's generator (pinned above),
    and the seven rounds of rng_mode 'fast' are its first seven (three more rounds, with the key advanced seven times,
    arrive at the ten-round output)."""
    ctr, key = [0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]
    assert oracle.philox(ctr, key, rounds=10) == oracle.philox(ctr, key)
    seven = oracle.philox(ctr, key, rounds=7)
    key7 = [(key[0] + 7 * 0x9E3779B9) & 0xffffffff, (key[1] + 7 * 0xBB67AE85) & 0xffffffff]
    assert oracle.philox(seven, key7, rounds=3) == oracle.philox(ctr, key)
    assert seven != oracle.philox(ctr, key, rounds=6) and seven != oracle.philox(ctr, key)
    # the fast noise takes byte e of block j from the seven-round output
    seed, elem = 12345 + (9 << 32), 256 * 7 + 19                       # group 7 (odd), position 19
    j, e = (7 >> 1) * 32 + (19 >> 3), 8 + (19 & 7)
    out = oracle.philox([j, 0, 0, 0x46415354], [seed & 0xffffffff, seed >> 32], rounds=7)
    byte = (out[e >> 2] >> ((e & 3) * 8)) & 0xff
    assert oracle.fast_noise(seed, elem) == (byte + 0.5) / 256


def test_calc_precision_against_reference_vectors(golden_dir):
    """Inputs/outputs recorded from the reference's calc_precision.cc built unmodified."""
    cases = json.loads((golden_dir / "calc_precision.json").read_text())["cases"]
    assert len(cases) >= 60
    for c in cases:
        C = torch.from_numpy(np.array(c["C_bits"], dtype=np.uint32).view(np.float32).copy())
        w = torch.tensor(c["w"], dtype=torch.int64)
        b = torch.full((len(c["w"]),), c["start"], dtype=torch.int32)
        out, st = oracle.calc_precision(b, C, w, c["target"])
        assert out.tolist() == c["bits"] and st == 0


def test_calc_precision_unreachable_budget_reports_status():
    b = torch.full((4,), 32, dtype=torch.int32)
    out, st = oracle.calc_precision(b, torch.ones(4), torch.full((4,), 256, dtype=torch.int64), 100.0)
    assert out.tolist() == [1, 1, 1, 1] and st == 1


def test_reference_gpu_vectors(golden_dir):
    """Outputs of the reference's own CUDA kernels, recorded on a B200 (gen_reference_gpu_vectors.py)."""
    path = golden_dir / "reference_gpu_vectors.npz"
    if not path.exists():
        pytest.skip("fixture not generated yet")
    z = np.load(path)
    n_cases = int(z["n_cases"])
    assert n_cases >= 16
    for i in range(n_cases):
        dtype = torch.float16 if int(z[f"c{i}_dtype"]) == 1 else torch.float32
        bits, seed = int(z[f"c{i}_bits"]), int(z[f"c{i}_seed"])
        x = torch.from_numpy(z[f"c{i}_x"].copy())
        x = x.view(torch.float16) if dtype == torch.float16 else x.view(torch.float32)
        pk, mn, sc = oracle.quantize(x, bits, seed)
        itype = torch.int16 if dtype == torch.float16 else torch.int32
        assert torch.equal(pk, torch.from_numpy(z[f"c{i}_packed"].copy())), i
        assert torch.equal(mn.view(itype), torch.from_numpy(z[f"c{i}_min"].copy()).view(itype)), i
        assert torch.equal(sc.view(itype), torch.from_numpy(z[f"c{i}_scale"].copy()).view(itype)), i
        out = oracle.dequantize(pk, mn, sc, x.numel(), bits)
        want = torch.from_numpy(z[f"c{i}_out"].copy()).view(itype)
        nan = torch.isnan(out)
        assert torch.equal(out.view(itype)[~nan], want[~nan]), i


# ---- 16-bit float formats -------------------------------------------------------------------------------------------
def test_half_to_float_all_patterns():
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    want = bits.view(torch.float16).float()
    L = oracle.lib()
    got = torch.tensor([L.oracle_half_to_float(int(b) & 0xffff) for b in bits.tolist()])
    both_nan = torch.isnan(want) & torch.isnan(got)
    assert torch.equal(got.view(torch.int32)[~both_nan], want.view(torch.int32)[~both_nan])


def test_float_to_half_and_bf16_rounding():
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(20000, generator=g) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 7e4)])
    # ties: midpoints between neighbouring halfs, plus specials
    h = torch.arange(0, 0x7c00, 7, dtype=torch.int32).to(torch.int16).view(torch.float16).float()
    nxt = (torch.arange(0, 0x7c00, 7, dtype=torch.int32) + 1).to(torch.int16).view(torch.float16).float()
    x = torch.cat([x, (h + nxt) / 2, -(h + nxt) / 2, torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 65504.0, 65520.0, 65519.9])])
    L = oracle.lib()
    got_h = torch.tensor([L.oracle_float_to_half(float(v)) for v in x.tolist()], dtype=torch.int32)
    assert torch.equal(got_h, x.half().view(torch.int16).to(torch.int32) & 0xffff)
    got_b = torch.tensor([L.oracle_float_to_bf16(float(v)) for v in x.tolist()], dtype=torch.int32)
    assert torch.equal(got_b, x.bfloat16().view(torch.int16).to(torch.int32) & 0xffff)


# ---- min / max ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_minimax_matches_torch(dtype):
    torch.manual_seed(1)
    x = torch.randn(300, 256).to(dtype)
    mn, mx = oracle.minimax(x)
    assert torch.equal(mn, x.min(dim=1).values) and torch.equal(mx, x.max(dim=1).values)
    # ragged: the tail is padded with zeros that take part
    y = (torch.rand(1000) + 1).to(dtype)
    mn, mx = oracle.minimax(y)
    assert float(mn[3]) == 0.0 and float(mx[3]) == float(y[768:].max())


def test_minimax_ignores_nan_and_keeps_start_values():
    x = torch.full((256,), float("nan"))
    mn, mx = oracle.minimax(x)
    assert float(mn) == float(np.float32(1e30)) == -float(mx)   # fp32 start values +-1e30
    mn, mx = oracle.minimax(x.half())
    assert float(mn) == float("inf") and float(mx) == -float("inf")
    x[17], x[200] = 3.0, -2.0
    mn, mx = oracle.minimax(x)
    assert (float(mn), float(mx)) == (-2.0, 3.0)


def test_zero_sign_follows_the_reference_reduction_order():
    """Among tied zeros the one with the smallest (bitrev5(d % 32), d // 32) wins (lane-strided scan, then a
    shuffle-down tree in which a lane keeps its own value on ties)."""
    def sign_of_min(pos_neg0, pos_pos0):
        x = torch.ones(256)
        for p in pos_neg0:
            x[p] = -0.0
        for p in pos_pos0:
            x[p] = 0.0
        mn, _ = oracle.minimax(x)
        return "-" if torch.signbit(mn)[0] else "+"
    assert sign_of_min([5], []) == "-" and sign_of_min([], [5]) == "+"
    assert sign_of_min([16], [8]) == "-"          # lane 16 (bitrev 1) beats lane 8 (bitrev 2)
    assert sign_of_min([8], [16]) == "+"
    assert sign_of_min([1], [2]) == "+"           # lane 2 (bitrev 8) beats lane 1 (bitrev 16)
    assert sign_of_min([32 + 4], [4]) == "+"      # same lane: the earlier element wins
    assert sign_of_min([4], [32 + 4]) == "-"
    assert sign_of_min([0], list(range(1, 256))) == "-"


# ---- known answers from the reference's own tests -----------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_one_hot_round_trips_exactly_at_1_bit(dtype):
    inp = F.one_hot(torch.arange(1000), 1000).to(dtype)
    d = oracle.op_dequantize(oracle.op_quantize(inp, 1, 0), inp.shape)
    assert float(((d.float() - inp.float()) ** 2).sum() / (inp.float() ** 2).sum()) < 1e-10
    inp = F.one_hot(torch.arange(0, 100) % 77).to(dtype)                       # (100, 77): ragged
    d = oracle.op_dequantize(oracle.op_quantize(inp, 1, 0), inp.shape)
    assert torch.equal(d.to(torch.uint8), inp.to(torch.uint8))


def test_exact_min_and_shapes():
    x = torch.rand(3000, 256)
    q_input, q_bit, q_scale, q_min = oracle.op_quantize(x, 4, 0)
    assert q_min.shape == (3000, 1, 1) and q_scale.shape == (3000, 1, 1) and q_input.dtype == torch.int8
    assert q_input.numel() == 3000 * 256 // 2 + 1
    assert torch.equal(q_min.reshape(-1), x.min(dim=1).values)


def test_32_bit_passthrough():
    x = torch.rand(64, 256)
    q = oracle.op_quantize(x, 32, 0)
    assert torch.equal(q[3].reshape(-1), x.min(dim=1).values)
    assert torch.equal(q[2].reshape(-1), x.max(dim=1).values - x.min(dim=1).values)
    assert torch.equal(oracle.op_dequantize(q, x.shape), x)


def test_mask_one_hot_round_trip_and_layout():
    inp = F.one_hot(torch.arange(1000), 1000).to(torch.uint8)
    words = oracle.mask_pack(inp)
    assert words.numel() == (10**6 + 511) // 512 * 16
    assert torch.equal(oracle.mask_unpack(words, 10**6).reshape(1000, 1000), inp)
    x = torch.zeros(1024, dtype=torch.uint8)
    x[0] = x[17] = x[512 + 33] = 1
    w = oracle.mask_pack(x)
    assert int(w[0]) == 1 and int(w[1]) == 2 and int(w[16 + 1]) == 4        # e -> word blk*16 + t%16, bit t//16
    assert int(w.to(torch.int64).abs().sum()) == 7


# ---- layout and arithmetic --------------------------------------------------------------------------------------
def test_packed_layout_interleaves_groups_not_elements():
    """2 bits, round to nearest: byte d of row-block r holds element d of groups 4r..4r+3 in bits [2i, 2i+2)."""
    G = 6                                                   # G % 4 != 0: the last row-block has two groups
    x = torch.zeros(G, 256)
    for g in range(G):
        x[g, 0], x[g, 1] = 0.0, 3.0                         # range 3 -> scale ~1: codes = values
        x[g, 2:] = float(g % 4)
    pk, mn, sc = oracle.quantize(x.reshape(-1), 2, 0, "rtn")
    assert pk.numel() == 2 * 256
    assert int(pk[0]) == 0 and int(pk[1]) == 0xff                             # codes 0,0,0,0 and 3,3,3,3
    assert int(pk[2]) == (0 | 1 << 2 | 2 << 4 | 3 << 6)
    assert int(pk[256 + 1]) == (3 | 3 << 2) and int(pk[256 + 2]) == (0 | 1 << 2)   # absent groups leave zero bits


def _numpy_quantize_fp32_unfused(x, bits, noise):
    """Independent vectorised restatement (fp32, product rounded before the add)."""
    n = x.size
    G = -(-n // 256)
    xp = np.zeros(G * 256, np.float32)
    xp[:n] = x
    g = xp.reshape(G, 256)
    mn, mx = g.min(1), g.max(1)
    scale = (np.float32(2 ** bits - 1).astype(np.float64) / ((mx - mn).astype(np.float32).astype(np.float64) + 2e-6)).astype(np.float32)
    t = (g - mn[:, None]).astype(np.float32)
    u = ((t * scale[:, None]).astype(np.float32) + noise.reshape(G, 256)).astype(np.float32)
    w = np.maximum(u.astype(np.float64) - 0.5, 0.0).astype(np.float32)
    codes = np.rint(w).astype(np.int64)
    wpt = 8 // bits
    R = -(-G // wpt)
    cp = np.zeros((R * wpt, 256), np.int64)
    cp[:G] = codes
    packed = np.zeros((R, 256), np.int64)
    for i in range(wpt):
        packed |= cp[i::wpt] << (i * bits)
    return (packed & 0xff).astype(np.uint8).reshape(-1), mn, scale


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_against_independent_numpy_restatement(bits):
    rng = np.random.default_rng(bits)
    n = 256 * 50 + 77
    x = rng.standard_normal(n).astype(np.float32)
    G = -(-n // 256)
    noise = rng.random(G * 256).astype(np.float32)
    noise[::53] = 1.0
    pk, mn, sc = oracle.quantize(torch.from_numpy(x), bits, 0, "external", noise=torch.from_numpy(noise), fma=False)
    npk, nmn, nsc = _numpy_quantize_fp32_unfused(x, bits, noise)
    assert np.array_equal(pk.numpy(), npk) and np.array_equal(mn.numpy(), nmn) and np.array_equal(sc.numpy(), nsc)
    out = oracle.dequantize(pk, mn, sc, n, bits).numpy()
    wpt = 8 // bits
    codes = np.stack([(npk.reshape(-1, 256) >> (i * bits)) & (2 ** bits - 1) for i in range(wpt)], 1).reshape(-1, 256)[:G]
    want = ((codes.astype(np.float32) / nsc[:, None]).astype(np.float32) + nmn[:, None]).astype(np.float32).reshape(-1)[:n]
    assert np.array_equal(out, want)


def test_no_upper_clamp_spills_like_the_reference():
    """noise == 1.0 on the group maximum gives code 2^b: it wraps at 8 bits and spills into the next slot below."""
    x = torch.zeros(2, 256)
    x[:, 1] = 1024.0                       # scale = fl32(255 / 1024.000002) = 255/1024 exactly, so t*scale = 255
    noise = torch.full((512,), 0.5)
    noise[1] = 1.0
    pk8, _, _ = oracle.quantize(x.reshape(-1), 8, 0, "external", noise=noise)
    assert int(pk8[1]) == 0 and int(pk8[256 + 1]) == 255              # 256 wrapped to 0; the other group is fine
    pk4, _, _ = oracle.quantize(x.reshape(-1), 4, 0, "external", noise=noise)
    assert int(pk4[1]) == ((16 | 15 << 4) & 0xff)                     # 16 spills into the neighbour's low bit
    xb = x.reshape(-1).bfloat16()                                     # bf16 (ours) clamps
    pkb, _, _ = oracle.quantize(xb, 8, 0, "external", noise=noise)
    assert int(pkb[1]) == 255


def test_fast_noise_is_uniform_and_reproducible():
    a = [oracle.fast_noise(7, i) for i in range(20000)]
    assert a == [oracle.fast_noise(7, i) for i in range(20000)]
    assert a != [oracle.fast_noise(8, i) for i in range(20000)]
    v = np.array(a)
    assert 0 < v.min() and v.max() < 1 and abs(v.mean() - 0.5) < 0.01 and abs(v.var() - 1 / 12) < 0.005
    assert len(set(np.round(v * 256 - 0.5).astype(int))) == 256       # 8 bits of noise per element


def test_stochastic_rounding_is_unbiased():
    x = torch.rand(256 * 400) * 3
    x[::256], x[1::256] = 0.0, 3.0
    acc = torch.zeros_like(x)
    for seed in range(40):
        for mode in ("curand", "fast"):
            pk, mn, sc = oracle.quantize(x, 2, seed, mode)
            acc += oracle.dequantize(pk, mn, sc, x.numel(), 2)
    assert float((acc / 80 - x).abs().mean()) < 0.05 and abs(float((acc / 80 - x).mean())) < 2e-3


# ---- identities behind the division-free dequantize kernel -----------------------------------------------------
def test_half_reciprocal_identity_exhaustive():
    assert oracle.lib().oracle_check_half_reciprocal() == 0


def test_markstein_quotient_identity():
    assert oracle.lib().oracle_check_markstein(1, 60) == 0            # every significand, binades 2^-60 and 2^0
    assert oracle.lib().oracle_check_markstein(97, 1) == 0            # every binade, sampled significands
