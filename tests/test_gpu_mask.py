"""GPU parity of the 1-bit dropout-mask kernels against the oracle (bit-exact)."""
import pytest
import torch
import torch.nn.functional as F

import oracle

pytestmark = pytest.mark.gpu


def pack(x, flag=None, pad=16):
    from gact import _native as nv
    n = x.numel()
    nw = (n + 511) // 512 * 16
    words = torch.full((nw + 2 * pad,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    st = nv.lib.gact_mask_pack(x.data_ptr(), n, words.data_ptr() + 4 * pad, None if flag is None else flag.data_ptr(),
                               torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    w = words.cpu()
    assert bool((w[:pad] == 0x5A5A5A5A).all()) and bool((w[pad + nw:] == 0x5A5A5A5A).all()), "guard words overwritten"
    return w[pad:pad + nw].clone()


def unpack(words, n, pad=64):
    from gact import _native as nv
    out = torch.full((n + 2 * pad,), 7, dtype=torch.uint8, device="cuda")
    w = words.cuda()
    st = nv.lib.gact_mask_unpack(w.data_ptr(), n, out.data_ptr() + pad, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    o = out.cpu()
    assert bool((o[:pad] == 7).all()) and bool((o[pad + n:] == 7).all()), "guard bytes overwritten"
    return o[pad:pad + n].clone()


@pytest.mark.parametrize("n", [1, 31, 32, 33, 511, 512, 513, 7700, 1000 * 1000, 512 * 5000 + 17])
def test_mask_round_trip_and_layout(n):
    g = torch.Generator().manual_seed(n)
    x_cpu = (torch.rand(n, generator=g) < 0.3).to(torch.uint8)
    words = pack(x_cpu.cuda())
    assert torch.equal(words, oracle.mask_pack(x_cpu))
    out = unpack(words, n)
    assert torch.equal(out, x_cpu)
    assert torch.equal(out, oracle.mask_unpack(words, n))


def test_one_hot_mask_like_the_reference_test():
    """1000 x 1000 one-hot uint8 -> mask -> back, exact."""
    from gact.ops import op_quantize_mask, op_dequantize_mask
    inp = F.one_hot(torch.arange(1000), 1000).to(torch.uint8).cuda()
    q = op_quantize_mask(inp)
    assert q[0].dtype == torch.int32 and q[0].numel() == (1000 * 1000 + 511) // 512 * 16
    out = op_dequantize_mask(q)
    assert out.dtype == torch.uint8 and out.shape == inp.shape
    assert torch.equal(out, inp)


def test_bool_mask_and_non_binary_flag():
    from gact.ops import op_quantize_mask, op_dequantize_mask
    m = torch.rand(3, 77, 129, device="cuda") < 0.9
    q = op_quantize_mask(m)
    assert torch.equal(op_dequantize_mask(q, dtype=torch.bool), m)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = (torch.rand(5000, device="cuda") < 0.5).to(torch.uint8)
    pack(x, flag)
    assert int(flag.item()) == 0
    x[4321] = 2
    pack(x, flag)
    assert int(flag.item()) == 1
