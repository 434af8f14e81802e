"""The allocation-free variant of the squared-distance reduction, through the C ABI.

gact_sq_diffs3_noalloc serves callers that cannot allocate device memory (code in a no-allocation section,
or a host binding without a device allocator): its scratch is a fixed array inside the library.  It must give
what gact_sq_diffs3 gives with caller-owned scratch, also on a second call that finds the first call's
leftovers in the shared array, and it must refuse more segments than its table holds.

Collected last on purpose (file name), so a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _existing(nv, g0, g1, g2, segs):
    scratch = torch.empty(nv.lib.gact_sq_diffs3_scratch_bytes(), dtype=torch.uint8, device="cuda")
    out = torch.zeros(3, dtype=torch.float64, device="cuda")
    if segs is None:
        st = nv.lib.gact_sq_diffs3(g0.data_ptr(), g1.data_ptr(), g2.data_ptr(), g0.numel(), None, None, None, 0,
                                   scratch.data_ptr(), out.data_ptr(), _stream())
    else:
        lens = [s.numel() for s in segs]
        offs = np.cumsum([0] + lens[:-1]).tolist()
        table = torch.tensor([[s.data_ptr() for s in segs], offs, lens], dtype=torch.int64).cuda()
        st = nv.lib.gact_sq_diffs3(g0.data_ptr(), g1.data_ptr(), None, g0.numel(), table[0].data_ptr(), table[1].data_ptr(),
                                   table[2].data_ptr(), len(segs), scratch.data_ptr(), out.data_ptr(), _stream())
    assert st == 0
    torch.cuda.synchronize()
    return out.cpu()


def _noalloc(nv, g0, g1, g2, segs):
    out = torch.zeros(3, dtype=torch.float64, device="cuda")      # an output the caller owns, as for any entry point
    if segs is None:
        st = nv.lib.gact_sq_diffs3_noalloc(g0.data_ptr(), g1.data_ptr(), g2.data_ptr(), g0.numel(), None, None, None, 0,
                                           out.data_ptr(), _stream())
    else:
        n = len(segs)
        lens = [s.numel() for s in segs]
        offs = np.cumsum([0] + lens[:-1]).tolist()
        ptrs = (ctypes.c_uint64 * n)(*[s.data_ptr() for s in segs])          # host tables
        offs_c = (ctypes.c_int64 * n)(*offs)
        lens_c = (ctypes.c_int64 * n)(*lens)
        st = nv.lib.gact_sq_diffs3_noalloc(g0.data_ptr(), g1.data_ptr(), None, g0.numel(), ctypes.addressof(ptrs),
                                           ctypes.addressof(offs_c), ctypes.addressof(lens_c), n, out.data_ptr(), _stream())
    assert st == 0, nv.lib.gact_error_string(st)
    torch.cuda.synchronize()
    return out.cpu()


def test_noalloc_matches_existing_entry_point_twice_in_a_row():
    from gact import _native as nv
    g = torch.Generator().manual_seed(7)
    # first call: segmented, second call: contiguous and a different size, so the second call meets a scratch
    # array full of the first one's partials and table
    lens = [3, 4096, 1, 250000, 77, 1 << 20]
    segs = [torch.randn(n, generator=g).cuda() for n in lens]
    P = sum(lens)
    g0, g1 = torch.randn(P, generator=g).cuda(), torch.randn(P, generator=g).cuda()
    want1 = _existing(nv, g0, g1, None, segs)
    got1 = _noalloc(nv, g0, g1, None, segs)
    torch.testing.assert_close(got1, want1, rtol=1e-6, atol=0)

    P2 = (1 << 21) + 5
    h0, h1, h2 = (torch.randn(P2, generator=g).cuda() * 3 for _ in range(3))
    want2 = _existing(nv, h0, h1, h2, None)
    got2 = _noalloc(nv, h0, h1, h2, None)
    torch.testing.assert_close(got2, want2, rtol=1e-6, atol=0)

    # and the first problem again: same answer as before
    got3 = _noalloc(nv, g0, g1, None, segs)
    torch.testing.assert_close(got3, want1, rtol=1e-6, atol=0)

    # both also agree with the CPU oracle (double accumulation of fp32 differences, summation order free)
    torch.testing.assert_close(got1, oracle.sq_diffs3(g0.cpu(), g1.cpu(), torch.cat([s.cpu() for s in segs])), rtol=1e-6, atol=0)
    torch.testing.assert_close(got2, oracle.sq_diffs3(h0.cpu(), h1.cpu(), h2.cpu()), rtol=1e-6, atol=0)


def test_noalloc_leaves_device_memory_as_it_found_it():
    """What the entry point is for: once the library's kernels are loaded (first call), a call changes neither the
    free memory the driver reports nor what torch's allocator holds."""
    from gact import _native as nv
    g = torch.Generator().manual_seed(3)
    segs = [torch.randn(n, generator=g).cuda() for n in (1000, 1 << 18, 5)]
    P = sum(s.numel() for s in segs)
    g0, g1 = torch.randn(P, generator=g).cuda(), torch.randn(P, generator=g).cuda()
    out = torch.zeros(3, dtype=torch.float64, device="cuda")
    n = len(segs)
    lens = [s.numel() for s in segs]
    ptrs = (ctypes.c_uint64 * n)(*[s.data_ptr() for s in segs])
    offs = (ctypes.c_int64 * n)(*np.cumsum([0] + lens[:-1]).tolist())
    lens_c = (ctypes.c_int64 * n)(*lens)

    def call():
        for args in ((None, ctypes.addressof(ptrs), ctypes.addressof(offs), ctypes.addressof(lens_c), n),
                     (segs[1].data_ptr(), None, None, None, 0)):
            Pk = P if args[4] else segs[1].numel()
            assert nv.lib.gact_sq_diffs3_noalloc(g0.data_ptr(), g1.data_ptr(), args[0], Pk, args[1], args[2], args[3], args[4],
                                                 out.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()

    call()                                              # loads the kernels, looks up the scratch address
    free0, _ = torch.cuda.mem_get_info()
    held0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"free device memory changed by {free0 - free1} bytes"
    assert torch.cuda.memory_allocated() == held0 and torch.cuda.memory_reserved() == reserved0


def test_noalloc_rejects_tables_that_do_not_tile_the_vector():
    from gact import _native as nv
    x = torch.zeros(64, device="cuda")
    out = torch.zeros(3, dtype=torch.float64, device="cuda")
    ptrs = (ctypes.c_uint64 * 2)(x.data_ptr(), x.data_ptr())
    lens = (ctypes.c_int64 * 2)(32, 32)
    for offs, want in (((0, 40), 5), ((0, 16), 5), ((8, 40), 5)):
        o = (ctypes.c_int64 * 2)(*offs)
        st = nv.lib.gact_sq_diffs3_noalloc(x.data_ptr(), x.data_ptr(), None, 64, ctypes.addressof(ptrs), ctypes.addressof(o),
                                           ctypes.addressof(lens), 2, out.data_ptr(), _stream())
        assert st == want
    torch.cuda.synchronize()


def test_noalloc_rejects_more_segments_than_its_table_holds():
    from gact import _native as nv
    n = 2048 + 1
    x = torch.zeros(n, device="cuda")
    out = torch.zeros(3, dtype=torch.float64, device="cuda")
    ptrs = (ctypes.c_uint64 * n)(*[x.data_ptr() + 4 * i for i in range(n)])
    offs = (ctypes.c_int64 * n)(*range(n))
    lens = (ctypes.c_int64 * n)(*([1] * n))
    st = nv.lib.gact_sq_diffs3_noalloc(x.data_ptr(), x.data_ptr(), None, n, ctypes.addressof(ptrs), ctypes.addressof(offs),
                                       ctypes.addressof(lens), n, out.data_ptr(), _stream())
    assert st == 9
    assert b"GACT_NOALLOC_MAX_SEGMENTS" in nv.lib.gact_error_string(st)
    torch.cuda.synchronize()
