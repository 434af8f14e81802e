"""GPU parity of the auto-precision kernels: squared distances, sensitivity clamp, greedy allocation."""
import json

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def gpu_sq_diffs3(g0, g1, g2_or_segments):
    from gact import _native as nv
    scratch = torch.empty(nv.lib.gact_sq_diffs3_scratch_bytes(), dtype=torch.uint8, device="cuda")
    out = torch.zeros(3, dtype=torch.float64, device="cuda")
    if isinstance(g2_or_segments, torch.Tensor):
        st = nv.lib.gact_sq_diffs3(g0.data_ptr(), g1.data_ptr(), g2_or_segments.data_ptr(), g0.numel(), None, None, None, 0,
                                   scratch.data_ptr(), out.data_ptr(), _stream())
    else:
        segs = g2_or_segments
        lens = [s.numel() for s in segs]
        offs = np.cumsum([0] + lens[:-1]).tolist()
        table = torch.tensor([[s.data_ptr() for s in segs], offs, lens], dtype=torch.int64).cuda()
        st = nv.lib.gact_sq_diffs3(g0.data_ptr(), g1.data_ptr(), None, g0.numel(), table[0].data_ptr(), table[1].data_ptr(),
                                   table[2].data_ptr(), len(segs), scratch.data_ptr(), out.data_ptr(), _stream())
    assert st == 0
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("P", [1, 3, 1000, 4097, 1 << 20, (1 << 22) + 13])
def test_sq_diffs3_contiguous(P):
    g = torch.Generator().manual_seed(P)
    g0, g1, g2 = (torch.randn(P, generator=g) for _ in range(3))
    got = gpu_sq_diffs3(g0.cuda(), g1.cuda(), g2.cuda())
    want = oracle.sq_diffs3(g0, g1, g2)
    # both accumulate fp32 squares in double; only the grouping of the fp32 products differs
    torch.testing.assert_close(got, want, rtol=1e-6, atol=0)
    again = gpu_sq_diffs3(g0.cuda(), g1.cuda(), g2.cuda())
    assert torch.equal(got, again), "the reduction must be reproducible"


def test_sq_diffs3_segments_match_contiguous():
    g = torch.Generator().manual_seed(1)
    lens = [5, 1024, 1, 77, 300000, 4096, 3, 123457]
    segs = [torch.randn(n, generator=g).cuda() for n in lens]
    P = sum(lens)
    g0, g1 = torch.randn(P, generator=g).cuda(), torch.randn(P, generator=g).cuda()
    flat2 = torch.cat(segs)
    a = gpu_sq_diffs3(g0, g1, segs)
    b = oracle.sq_diffs3(g0.cpu(), g1.cpu(), flat2.cpu())
    torch.testing.assert_close(a, b, rtol=1e-6, atol=0)


def test_sensitivity_kernel():
    from gact import _native as nv
    rows = [[1.0, 2.0, 3.0], [10.0, 1.0, 2.0], [float("nan"), 1.0, 1.0], [1.0, float("nan"), 1.0], [1.0, 1.0, float("nan")],
            [float("inf"), 0.0, 0.0], [0.0, 6e9, 0.0], [0.0, 0.0, 0.0], [3e10, 1.0, 1.0]]
    d3 = torch.tensor(rows, dtype=torch.float64)
    C = torch.empty(len(rows), dtype=torch.float32, device="cuda")
    for scale in (1.0, 0.25):
        st = nv.lib.gact_sensitivity(d3.cuda().data_ptr(), scale, C.data_ptr(), len(rows), _stream())
        assert st == 0
        got = C.cpu().tolist()
        for r, c in zip(rows, got):
            want = oracle.sensitivity([np.float32(v * scale) for v in r])
            assert c == np.float32(want), (r, scale, c, want)


def gpu_calc_precision(b, C, w, target):
    from gact import _native as nv
    bd, Cd, wd = b.cuda(), C.cuda(), w.cuda()
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    st = nv.lib.gact_calc_precision(bd.data_ptr(), Cd.data_ptr(), wd.data_ptr(), b.numel(), float(target), status.data_ptr(), _stream())
    assert st == 0
    torch.cuda.synchronize()
    return bd.cpu(), int(status.item())


def test_calc_precision_against_reference_vectors(golden_dir):
    """Inputs and outputs recorded from the reference's calc_precision.cc (tests/golden/gen_calc_precision.py)."""
    cases = json.loads((golden_dir / "calc_precision.json").read_text())["cases"]
    for c in cases:
        C = torch.from_numpy(np.array(c["C_bits"], dtype=np.uint32).view(np.float32).copy())
        w = torch.tensor(c["w"], dtype=torch.int64)
        b = torch.full((len(c["w"]),), c["start"], dtype=torch.int32)
        got, status = gpu_calc_precision(b, C, w, c["target"])
        assert got.tolist() == c["bits"]
        assert status == 0


def test_calc_precision_large_and_unreachable():
    g = torch.Generator().manual_seed(0)
    L = 5000                                   # more candidates than threads, > 32 KB of shared memory
    C = torch.rand(L, generator=g).exp()
    w = torch.randint(256, 1 << 20, (L,), generator=g)
    b = torch.full((L,), 32, dtype=torch.int32)
    target = 3.0 * float(w.sum())
    got, status = gpu_calc_precision(b, C, w, target)
    want, ost = oracle.calc_precision(b.clone(), C, w, target)
    assert got.tolist() == want.tolist() and status == 0 and ost == 0
    # a budget below one bit per element cannot be met: every tensor ends at 1 bit and the status says so
    got, status = gpu_calc_precision(b, C, w, 0.5 * float(w.sum()))
    assert set(got.tolist()) == {1} and status == 8


def test_calc_precision_mixed_starting_widths():
    """Starting widths other than 32, entries already at 1 bit included (the reference leaves those out of the
    budget sum, calc_precision.cc:96-101), against the oracle and the host twin."""
    from gact.cpp_extension.calc_precision import calc_precision as host_calc_precision
    g = torch.Generator().manual_seed(11)
    for L in (5, 64, 1500):
        C = torch.rand(L, generator=g) * 50
        C[::9] = 2.0
        w = torch.randint(1, 1 << 18, (L,), generator=g, dtype=torch.int64)
        start = torch.tensor([32, 8, 4, 2, 1], dtype=torch.int32)[torch.randint(0, 5, (L,), generator=g)]
        for avg in (1.0, 2.5, 6.0):
            target = avg * float(w.sum())
            want, ost = oracle.calc_precision(start.clone(), C, w, target)
            got, status = gpu_calc_precision(start.clone(), C, w, target)
            assert got.tolist() == want.tolist() and (status != 0) == (ost != 0)
            if ost == 0:
                assert torch.equal(host_calc_precision(start.clone(), C, w, target), want)
