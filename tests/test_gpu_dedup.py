"""config.check_dup without host round-trips: the fingerprint kernel against its restatement, the merges the
reference's key would make (gact/gact/quantizer.py:85-93: same address, same sampled values, same sum), and the
single read-back per step that verifies them."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _fp(t):
    from gact import _native as nv
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    x = t.contiguous()
    assert nv.lib.gact_fingerprint(x.data_ptr(), x.element_size(), x.numel(), out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    return tuple(v & (2**64 - 1) for v in out.tolist())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.uint8])
def test_fingerprint_kernel_matches_its_restatement(dtype):
    g = torch.Generator().manual_seed(0)
    for n in (1, 7, 99, 100, 101, 256 * 33 + 5, 1 << 21):
        x = torch.randn(n, generator=g).mul(50).to(dtype)
        assert _fp(x.cuda()) == oracle.fingerprint(x), (dtype, n)
    z = torch.zeros(5000, dtype=dtype)
    assert _fp(z.cuda())[1] == 0 and _fp(z.cuda()) == oracle.fingerprint(z)
    # one changed element that is not among the samples still changes the sum
    x = torch.randn(100000, generator=g).to(dtype)
    y = x.clone()
    y[12345] = y[12345] + 1
    a, b = _fp(x.cuda()), _fp(y.cuda())
    assert a[0] == b[0] and a[1] != b[1]
    assert _fp(x.cuda()[1:]) == oracle.fingerprint(x[1:])              # odd offset


def test_three_identical_and_two_near_identical_saves(monkeypatch):
    import gact
    from gact.quantizer import Quantizer
    gact.config.reset()
    gact.config.check_dup = True
    q = Quantizer(4, False, False)
    x = torch.randn(64, 512, device="cuda", requires_grad=True)
    alias = x.view_as(x)                                   # another object, the same bytes
    detached = x.detach().requires_grad_()                 # shares storage and version counter
    near_copy = x.detach().clone()
    near_copy[3, 3] += 1.0                                 # equal but for one element, at another address
    near_copy.requires_grad_()

    # nothing on the per-tensor path may read back from the device
    def forbidden(*a, **k):
        raise AssertionError("host read-back on the per-tensor path")
    with monkeypatch.context() as m:
        m.setattr(torch.Tensor, "item", forbidden)
        m.setattr(torch.Tensor, "tolist", forbidden)
        m.setattr(torch.Tensor, "cpu", forbidden)
        r = [q.quantize(t) for t in (x, alias, detached, near_copy)]
        with torch.no_grad():
            x.mul_(1.0000001).add_(1e-3)                   # modified in place: the version counter moves on
        r.append(q.quantize(x))
    keys = [t[2] for t in r]
    assert keys[0] == keys[1] == keys[2] and len({keys[0], keys[3], keys[4]}) == 3
    assert [t[4] for t in r] == [0, 1, 2, 3, 4]
    assert q.ptr_qtensor_map[keys[0]][1] == 3 and len(q.ptr_qtensor_map) == 3
    assert list(q.bits) == [0, 3, 4]                       # shared saves register no width of their own
    outs = [q.dequantize(t) for t in r]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]) and not q.ptr_qtensor_map
    q.iterate()                                            # the step's one read-back: verifies the merges
    assert q.dup_report == {"merged": 2, "missed": 0}
    # what the reference's key would have decided, from the same ingredients on the host
    fps = [oracle.fingerprint(t.detach().cpu()) for t in (alias, detached, near_copy)]
    assert fps[0] == fps[1] and fps[0] != fps[2]


def test_a_merge_that_was_not_value_identical_is_reported():
    import gact
    from gact.quantizer import Quantizer
    gact.config.reset()
    gact.config.check_dup = True
    q = Quantizer(4, False, False)
    x = torch.randn(32, 256, device="cuda", requires_grad=True)
    a = q.quantize(x)
    x.data.add_(1.0)                                       # changes the values behind the version counter's back
    b = q.quantize(x.view_as(x))
    assert a[2] == b[2]
    q.dequantize(a); q.dequantize(b)
    with pytest.raises(RuntimeError, match="values differ"):
        q.iterate()
