"""The native fast path of the saved-tensor hooks (gact/_hooks.so) against the Python implementation it mirrors:
same tuples, same dictionaries, same payload bytes, same training losses."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _quantizer(native, bit=4, swap=False):
    import gact
    from gact.quantizer import Quantizer
    gact.config.reset()
    gact.config.native_hooks = native
    return Quantizer(bit, swap, False)


def test_native_module_is_built_and_used():
    from gact import ops
    assert ops._hooks is not None, "gact/_hooks.so was not built (python gact-icml_b200/build.py)"
    q = _quantizer(True)
    before = ops._hooks.launches()
    x = torch.randn(8, 256, device="cuda", requires_grad=True)
    r = q.quantize(x)
    assert r[0] is True and ops._hooks.launches() == before + 1
    y = q.dequantize(r)
    assert ops._hooks.launches() == before + 2 and y.shape == x.shape and not q.ptr_qtensor_map


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_same_tuples_state_and_bytes(dtype):
    torch.manual_seed(0)
    base = torch.randn(6, 40, 33, device="cuda").to(dtype)
    cases = {
        "plain": base.clone().requires_grad_(),
        "odd_offset": base[1:].requires_grad_(),                                    # contiguous, not 16-byte aligned
        "permuted": torch.randn(4, 6, 32, 16, device="cuda").to(dtype).transpose(1, 2).requires_grad_(),   # dense
        "gappy": torch.randn(8, 64, 40, device="cuda").to(dtype)[:, :, :32].requires_grad_(),              # takes a copy
        "no_grad": base.clone(),
        "one_dim": base.reshape(-1).clone().requires_grad_(),
        "param": base.clone().requires_grad_(),
    }
    results = {}
    for native in (False, True):
        q = _quantizer(native)
        q.unrelated_tensors.add(cases["param"].data_ptr())
        q.seed_iter, q.seed_offset = 3, 5 << 32
        rec = {}
        for name, t in cases.items():
            r = q.quantize(t)
            if name in ("plain", "permuted"):
                r2 = q.quantize(t)                               # the same object again: shares the payload
                assert r2[2] == r[2] and r2[4] == r[4] + 1 and q.ptr_qtensor_map[r[2]][1] == 2
                rec[name + "_again"] = (r2, q.dequantize(r2))
            payload = q.ptr_qtensor_map[r[2]][0] if r[0] else None
            # codes without the spare last byte, scale, min (the alignment gaps of the buffer hold whatever was there)
            rec[name] = (r, None if payload is None else ((payload[0][:-1].clone(), payload[2].clone(), payload[3].clone()),
                                                          payload.bits, payload.dtype, payload.n, payload.strides))
        rec["state"] = (dict(q.bits), dict(q.dims), dict(q.seeds), q.tid, q.tids_registered, dict(q.layer_key_map))
        rec["out"] = {name: q.dequantize(rec[name][0]) for name in cases}
        assert not q.ptr_qtensor_map
        results[native] = rec
    py, nat = results[False], results[True]
    assert py["state"] == nat["state"]
    for name in cases:
        (rp, pp), (rn, pn) = py[name], nat[name]
        assert rp[0] == rn[0]
        if not rp[0]:
            assert rn[1] is cases[name] and pn is None
            continue
        assert rp[1:] == rn[1:] and type(rn[3]) is torch.Size
        assert all(torch.equal(u.view(torch.uint8), v.view(torch.uint8)) for u, v in zip(pp[0], pn[0])) and pp[1:] == pn[1:], name
        a, b = py["out"][name], nat["out"][name]
        assert a.stride() == b.stride() and a.dtype == b.dtype and torch.equal(a, b), name


def test_bool_masks_native_and_python_agree():
    """torch.bool dropout masks take the native path too; payload, tuple format and restored mask equal the Python
    path's, the quantizer's state is untouched, and the decisions of the filter are the same."""
    import gact
    from gact import ops
    from gact.quantizer import Quantizer
    gact.config.reset()
    q = Quantizer(4, False, False)

    def both(fn):                                   # the same call on the native and on the Python path
        gact.config.native_hooks = True
        a = fn()
        gact.config.native_hooks = False
        b = fn()
        gact.config.native_hooks = True
        return a, b

    for shape in ((100, 77), (64, 16, 128, 128), (5,), (3, 512)):
        m = torch.rand(*shape, device="cuda") < 0.3
        before = ops._hooks.launches()
        rn, rp = both(lambda: q.quantize(m))
        assert ops._hooks.launches() == before + 1
        assert rn[0] is True and rn[1] is True and rp[0] is True and rp[1] is True and len(rn) == len(rp) == 3
        assert torch.equal(rn[2][0], rp[2][0]) and rn[2][0].dtype == torch.int32
        assert tuple(rn[2][1]) == tuple(rp[2][1]) == shape and rn[2][2] is torch.bool and rp[2][2] is torch.bool
        assert q.tid == 0 and not q.ptr_qtensor_map
        for r in (rn, rp):                          # payloads are interchangeable
            on, op_ = both(lambda: q.dequantize(r))
            assert on.dtype == torch.bool and torch.equal(on, m) and torch.equal(op_, m)
        assert ops._hooks.launches() == before + 3
    # a transposed mask is packed in its logical order, like the Python path does
    m = (torch.rand(40, 600, device="cuda") < 0.5).t()
    rn, rp = both(lambda: q.quantize(m))
    assert torch.equal(rn[2][0], rp[2][0]) and torch.equal(q.dequantize(rn), m)
    # the filter: empty, CPU and unrelated masks pass through; pack_bool_masks off leaves masks alone
    for t in (torch.zeros(0, 4, dtype=torch.bool, device="cuda"), torch.ones(4, 4, dtype=torch.bool)):
        for r in both(lambda: q.quantize(t)):
            assert r[0] is False and r[1] is t
    m = torch.rand(64, 64, device="cuda") < 0.5
    q.unrelated_tensors.add(m.data_ptr())
    assert all(r[0] is False for r in both(lambda: q.quantize(m)))
    gact.config.pack_bool_masks = False
    try:
        m2 = torch.rand(64, 64, device="cuda") < 0.5
        assert all(r[0] is False for r in both(lambda: q.quantize(m2)))
    finally:
        gact.config.reset()


def test_cases_left_to_the_python_path():
    """uint8 masks, 32-bit passthrough, swapping and value fingerprints are handed back untouched."""
    import gact
    from gact import ops
    q = _quantizer(True)
    m = (torch.rand(100, 77, device="cuda") < 0.5).to(torch.uint8)
    before = ops._hooks.launches()
    r = q.quantize(m)
    assert r[0] and r[1] and torch.equal(q.dequantize(r), m) and ops._hooks.launches() == before
    q32 = _quantizer(True, bit=32)
    x = torch.randn(4, 300, device="cuda", requires_grad=True)
    r = q32.quantize(x)
    assert r[0] and torch.equal(q32.dequantize(r), x) and ops._hooks.launches() == before and q32.tid == 1
    qs = _quantizer(True, swap=True)
    r = qs.quantize(x)
    assert r[0] and not qs.ptr_qtensor_map[r[2]][0].buf.is_cuda
    assert float((qs.dequantize(r) - x).abs().max()) < 0.5 and ops._hooks.launches() == before
    qd = _quantizer(True)
    gact.config.check_dup = True
    a, b = qd.quantize(x), qd.quantize(x.view_as(x))
    assert a[2] == b[2] and ops._hooks.launches() == before       # another object, the same bytes: the fingerprint path
    qd.dequantize(a); qd.dequantize(b)
    # a tid that iteration 0 never saw stays an error
    q = _quantizer(True)
    q.quantize(x); q.iterate(); q.quantize(x)
    with pytest.raises(KeyError):
        q.quantize(x.detach().clone().requires_grad_())


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.c1 = nn.Conv2d(3, 16, 3, padding=1)
        self.bn = nn.BatchNorm2d(16)
        self.c2 = nn.Conv2d(16, 32, 3, padding=1)
        self.drop = nn.Dropout(0.1)
        self.fc = nn.Linear(32 * 8 * 8, 10)

    def forward(self, x):
        x = F.relu(self.bn(self.c1(x)))
        x = F.max_pool2d(F.relu(self.c2(x)), 4)
        return self.fc(self.drop(x.flatten(1)))


@pytest.mark.parametrize("level", ["L1", "L2"])
def test_training_is_identical_with_and_without_the_native_hooks(level):
    import gact

    def train(native):
        gact.config.reset()
        gact.set_optimization_level(level)
        gact.set_adapt_interval(2)
        gact.config.native_hooks = native
        torch.manual_seed(0)
        torch.cuda.manual_seed_all(0)
        model = Net().cuda()
        opt = torch.optim.SGD(model.parameters(), lr=0.05)
        x, y = torch.randn(32, 3, 32, 32, device="cuda"), torch.randint(0, 10, (32,), device="cuda")
        ctl = gact.Controller(model)
        ctl.install_hook()
        losses = []

        def backprop():
            opt.zero_grad()
            F.cross_entropy(model(x[:8]), y[:8]).backward()

        try:
            for _ in range(4):
                opt.zero_grad()
                loss = F.cross_entropy(model(x), y)
                loss.backward()
                opt.step()
                losses.append(loss.item())
                ctl.iterate(backprop)
        finally:
            ctl.uninstall_hook()
        return losses, dict(ctl.quantizer.bits), dict(ctl.quantizer.dims)

    det = torch.backends.cudnn.deterministic
    torch.backends.cudnn.deterministic = True          # so that two runs of the same code agree to begin with
    try:
        (l0, b0, d0), (l1, b1, d1) = train(False), train(True)
    finally:
        torch.backends.cudnn.deterministic = det
    assert d0 == d1 and set(b0) == set(b1)
    assert l0 == pytest.approx(l1, rel=1e-4)
    if l0 == l1:
        assert b0 == b1
