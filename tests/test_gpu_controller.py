"""End-to-end on the GPU through the public API: ops contract, hooks, fixed-bit training, swap, auto precision."""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import oracle
from helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def gact_mode():
    import gact
    return gact.config.rng_mode


def error_rate(q, x):
    return (((q - x) ** 2).sum() / (x ** 2).sum()).item()


# ---- the reference's own op tests (tests/test_act_quantized_ops.py), re-expressed ----
def test_quantize_1bit_one_hot():
    from gact.ops import op_quantize, op_dequantize
    inp = F.one_hot(torch.arange(1000), 1000).cuda()
    d = op_dequantize(op_quantize(inp.to(torch.float32), 1, 0), inp.shape)
    assert error_rate(d.to(torch.uint8).float(), inp.float()) < 1e-10


def test_quantize_mask_shape_100x77():
    from gact.ops import op_quantize, op_dequantize
    inp = F.one_hot(torch.arange(0, 100) % 77).to(torch.uint8).cuda()
    d = op_dequantize(op_quantize(inp.to(torch.float32), 1, 0), inp.shape)
    assert error_rate(d.to(torch.uint8).float(), inp.float()) < 1e-10


def test_quantize_big_min():
    """655 350 rows of 256: the reference needs several launches for this many row-blocks."""
    from gact.ops import op_quantize
    x = torch.rand((65535 * 10, 256), device="cuda")
    q_input, q_bit, q_scale, q_min = op_quantize(x, 4, 0)
    assert q_min.shape == (65535 * 10, 1, 1) and q_scale.shape == (65535 * 10, 1, 1)
    assert q_input.dtype == torch.int8 and q_input.numel() == 65535 * 10 * 256 // 2 + 1
    assert torch.equal(q_min.reshape(-1), x.min(dim=1).values)


def test_quantize_32bit_passthrough():
    from gact.ops import op_quantize, op_dequantize
    x = torch.rand((2048, 256), device="cuda")
    q = op_quantize(x, 32, 0)
    assert torch.equal(q[3].reshape(-1), x.min(dim=1).values)
    assert torch.equal(q[2].reshape(-1), x.max(dim=1).values - x.min(dim=1).values)
    assert torch.equal(op_dequantize(q, x.shape), x)
    y = torch.rand((3, 100), device="cuda")                 # ragged: padded with zeros inside the payload
    assert torch.equal(op_dequantize(op_quantize(y, 32, 0), y.shape), y)


@pytest.mark.parametrize("bits,bound", [(1, 0.9), (2, 0.2), (4, 0.01), (8, 1e-4)])
def test_quantize_error_rates(bits, bound):
    from gact.ops import op_quantize, op_dequantize
    torch.manual_seed(1)
    x = torch.rand((64, 3, 224, 224), device="cuda")
    e = error_rate(op_dequantize(op_quantize(x, bits, 3), x.shape), x)
    assert e < bound
    ones = torch.ones_like(x)
    assert error_rate(op_dequantize(op_quantize(ones, bits, 3), x.shape), ones) < 1e-10


def test_op_contract_matches_oracle_front_end():
    from gact.ops import op_quantize, op_dequantize
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        x_cpu = torch.randn(7, 33, 129).to(dtype)
        q = op_quantize(x_cpu.cuda(), 2, 5)
        oq = oracle.op_quantize(x_cpu, 2, 5, rng_mode=gact_mode())
        assert q[0].shape == oq[0].shape and q[0].dtype == torch.int8
        assert q[2].shape == oq[2].shape and q[3].shape == oq[3].shape and q[3].dtype == dtype
        assert q[2].dtype == (torch.float32 if dtype == torch.bfloat16 else dtype)
        assert torch.equal(q[0].cpu()[:-1], oq[0][:-1])
        assert_bits_equal(q[2], oq[2], "scale")
        assert_bits_equal(q[3], oq[3], "min")
        y = op_dequantize(q, x_cpu.shape)
        assert y.shape == x_cpu.shape and y.is_contiguous()
        assert_bits_equal(y, oracle.op_dequantize(oq, x_cpu.shape), "dequantized")
    with pytest.raises(RuntimeError):
        op_quantize(torch.randn(512), 2, 0)                 # CPU tensor: rejected like the reference does
    with pytest.raises(ValueError):
        op_quantize(torch.randn(512, device="cuda"), 3, 0)


def test_full_size_properties_config2():
    """128x64x112x112 post-ReLU fp16, every width: properties that need no oracle pass over 103 M elements:
    min is the true group min, scale follows from min/max, |x - dq(x)| <= one quantization step, same seed ->
    same bytes, different seed -> different bytes; and a bit-exact oracle check on a slice of groups."""
    from gact.ops import quantize_pack, dequantize_and_unpack
    torch.manual_seed(0)
    shape = (128, 64, 112, 112)
    x = torch.randn(shape, device="cuda").clamp_min(0).to(torch.float16)
    n = x.numel()
    groups = x.reshape(-1, 256)
    gmin, gmax = groups.amin(dim=1), groups.amax(dim=1)
    for bits in (1, 2, 4, 8):
        q, sc, mn = quantize_pack(x, bits, 42)
        assert torch.equal(mn.reshape(-1), gmin)
        step = (1.0 / sc.float().reshape(-1, 1)).expand(-1, 256).reshape(shape)
        tol = step * 1.01 + (x.float().abs() + gmax.float().reshape(-1, 1).expand(-1, 256).reshape(shape)) * 2e-3
        y = dequantize_and_unpack(q, shape, bits, sc, mn)
        err = (y.float() - x.float()).abs()
        # The reference has no upper clamp: when an fp16 scale rounds up, the largest element of a group can
        # reach code 2^bits with noise close to 1, and then wraps to 0 or spills into the neighbouring code
        # (about 6 elements in 10^5 at 8 bits, far fewer below).  Round-to-nearest cannot overflow, so there
        # the bound holds everywhere.
        assert float((err > tol).float().mean()) < 2e-4, f"b={bits}"
        qr, scr, mnr = quantize_pack(x, bits, 42, rng_mode="rtn")
        err = (dequantize_and_unpack(qr, shape, bits, scr, mnr).float() - x.float()).abs()
        assert bool((err <= tol * 0.51 + 1e-3).all()), f"rtn b={bits}: {float((err - tol * 0.51).max())}"
        q2, _, _ = quantize_pack(x, bits, 42)
        assert torch.equal(q[:-1], q2[:-1])
        q3, _, _ = quantize_pack(x, bits, 43)
        assert not torch.equal(q[:-1], q3[:-1])
        # oracle on the first 2048 groups (row-blocks are independent of what follows them)
        k = 2048 * 256
        opk, omn, osc = oracle.quantize(x.reshape(-1)[:k].cpu(), bits, 42, gact_mode())
        nb = opk.numel()
        assert torch.equal(q[:nb].cpu().view(torch.uint8), opk)
        assert_bits_equal(sc.reshape(-1)[:2048], osc, "scale")


# ---- controller ----
class SmallNet(nn.Module):
    def __init__(self, drop=0.0):
        super().__init__()
        self.c1 = nn.Conv2d(3, 16, 3, padding=1)
        self.bn = nn.BatchNorm2d(16)
        self.c2 = nn.Conv2d(16, 32, 3, padding=1)
        self.drop = nn.Dropout(drop)
        self.fc = nn.Linear(32 * 8 * 8, 10)

    def forward(self, x):
        x = F.relu(self.bn(self.c1(x)))
        x = F.max_pool2d(F.relu(self.c2(x)), 2)
        x = self.drop(x)
        return self.fc(torch.flatten(x, 1))


def run_steps(level, steps=4, swap=False, seed=0, drop=0.0, auto_interval=None):
    import gact
    gact.config.reset()
    gact.set_optimization_level(level)
    if swap:
        gact.config.swap = True
        gact.config.prefetch = True
    if auto_interval:
        gact.set_adapt_interval(auto_interval)
    torch.manual_seed(seed)
    model = SmallNet(drop).cuda()
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    x = torch.randn(64, 3, 16, 16, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda")
    ctl = gact.Controller(model)
    ctl.install_hook()
    losses = []

    def backprop():
        model.train()
        opt.zero_grad()
        F.cross_entropy(model(x), y).backward()

    for _ in range(steps):
        opt.zero_grad()
        loss = F.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
        ctl.iterate(backprop)
    ctl.uninstall_hook()
    return losses, ctl, model


def test_l0_is_exact_and_l1_is_close():
    base, _, _ = run_steps("L0")
    again, _, _ = run_steps("L0")
    assert base == again
    l11, ctl, _ = run_steps("L1.1")
    assert len(ctl.quantizer.bits) > 0 and set(ctl.quantizer.bits.values()) == {8}
    np.testing.assert_allclose(l11, base, rtol=2e-2)
    l1, ctl, _ = run_steps("L1")
    assert set(ctl.quantizer.bits.values()) == {4}
    np.testing.assert_allclose(l1, base, rtol=1e-1)
    assert not ctl.quantizer.ptr_qtensor_map, "every payload is released once backward has consumed it"


def test_swap_gives_identical_losses():
    """The reference's own integration assertion: losses with swap == losses without."""
    a, _, _ = run_steps("L1")
    b, _, _ = run_steps("L1", swap=True)
    np.testing.assert_allclose(a, b, rtol=0, atol=0)


def test_gradients_close_to_exact():
    import gact
    torch.manual_seed(0)
    model = SmallNet().cuda()
    x = torch.randn(64, 3, 16, 16, device="cuda")
    y = torch.randint(0, 10, (64,), device="cuda")

    def grads():
        model.zero_grad()
        F.cross_entropy(model(x), y).backward()
        return torch.cat([p.grad.reshape(-1) for p in model.parameters()]).clone()

    exact = grads()
    gact.config.reset()
    gact.set_optimization_level("L1.1")
    ctl = gact.Controller(model)
    ctl.install_hook()
    g8 = grads()
    ctl.uninstall_hook()
    rel = ((g8 - exact).norm() / exact.norm()).item()
    assert rel < 2e-2, rel


def test_dropout_mask_is_packed_and_restored():
    import gact
    gact.config.reset()
    gact.set_optimization_level("L1.1")
    model = nn.Sequential(nn.Linear(64, 64), nn.Dropout(0.5), nn.Linear(64, 4)).cuda()
    ctl = gact.Controller(model)
    kinds = []
    orig = ctl.quantizer.quantize

    def spy(t):
        r = orig(t)
        kinds.append((t.dtype, r[0], r[1] if r[0] else None))
        return r

    ctl.quantizer.quantize = spy
    ctl.install_hook()
    x = torch.randn(32, 64, device="cuda", requires_grad=True)
    model(x).sum().backward()
    ctl.uninstall_hook()
    assert any(dt == torch.bool and q and is_mask for dt, q, is_mask in kinds), kinds
    assert torch.isfinite(x.grad).all()


def test_auto_precision_runs_and_respects_the_budget():
    losses, ctl, _ = run_steps("L2", steps=3, auto_interval=2)
    ap = ctl.ap
    L = len(ctl.quantizer.bits)
    assert L > 0 and set(ap.C.keys()) == set(ctl.quantizer.bits.keys())
    assert all(b in (1, 2, 4, 8, 32) for b in ctl.quantizer.bits.values())
    total = sum(ctl.quantizer.bits[l] * ctl.quantizer.dims[l] for l in ctl.quantizer.bits)
    assert total <= ap.total_bits and ap.last_status == 0
    assert all(np.isfinite(v) and v >= 0 for v in ap.C.values())
    # the same decisions as the reference's greedy allocator on the same sensitivities
    l_list = list(ap.dims.keys())
    b0 = torch.full((L,), 32, dtype=torch.int32)
    want, _ = oracle.calc_precision(b0, torch.tensor([ap.C[l] for l in l_list], dtype=torch.float32),
                                    torch.tensor([ap.dims[l] for l in l_list], dtype=torch.int64), ap.total_bits)
    assert [ctl.quantizer.bits[l] for l in l_list] == want.tolist()
    assert all(np.isfinite(losses))


def test_state_dict_round_trip():
    _, ctl, model = run_steps("L2", steps=2, auto_interval=100)
    sd = ctl.state_dict()
    import gact
    ctl2 = gact.Controller(model)
    ctl2.load_state_dict(sd)
    assert ctl2.quantizer.bits == ctl.quantizer.bits and ctl2.ap.C == ctl.ap.C and ctl2.iter == ctl.iter


@pytest.mark.parametrize("rng_mode", ["fast", "curand"])
def test_training_converges_like_the_uncompressed_run(rng_mode):
    """60 steps of the small network at 2 bits: the loss falls as it does without compression, in both noise
    arrangements (the gradient estimate is unbiased either way; only its variance grows)."""
    import gact

    def train(level):
        gact.config.reset()
        gact.set_optimization_level(level)
        gact.config.rng_mode = rng_mode
        torch.manual_seed(0)
        model = SmallNet().cuda()
        opt = torch.optim.SGD(model.parameters(), lr=0.02)
        g = torch.Generator(device="cuda").manual_seed(1)
        x = torch.randn(256, 3, 16, 16, device="cuda", generator=g)
        w = torch.randn(3 * 16 * 16, 10, device="cuda", generator=g)
        y = (x.flatten(1) @ w).argmax(1)                      # labels a linear map can explain: learnable
        ctl = gact.Controller(model)
        ctl.install_hook()
        losses = []
        for _ in range(60):
            opt.zero_grad()
            loss = F.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
            ctl.iterate(lambda: None)
        ctl.uninstall_hook()
        return losses

    base = train("L0")
    comp = train("L1.2")                                       # fixed 2 bits on every saved tensor
    assert base[-1] < base[0] - 0.3                            # measured: 2.315 -> 1.80
    np.testing.assert_allclose(comp, base, atol=0.05, rtol=0)  # measured: the curves differ by less than 0.01


def test_saved_views_at_odd_offsets_are_compressed():
    """A contiguous view that does not start on a 16-byte boundary (t[1:] of a tensor with an odd row length) is
    compressed like any other tensor - the reference accepts every contiguous CUDA tensor
    (gact/gact/cpp_extension/ext_common.h:2-27) - both through the op and through the hooks."""
    import gact
    from gact.ops import op_quantize, op_dequantize, op_quantize_mask, op_dequantize_mask
    h = torch.randn(5, 33, 7).half()
    v = h.cuda()[1:]
    assert v.is_contiguous() and v.data_ptr() % 16 != 0
    for mode in ("fast", "curand"):
        gact.config.rng_mode = mode
        q = op_quantize(v, 4, 3)
        oq = oracle.op_quantize(h[1:].contiguous(), 4, 3, rng_mode=mode)
        assert torch.equal(q[0].cpu()[:-1], oq[0][:-1])
        assert_bits_equal(q[2], oq[2], "scale")
        assert_bits_equal(q[3], oq[3], "min")
        assert_bits_equal(op_dequantize(q, v.shape), oracle.op_dequantize(oq, v.shape), "dequantized")
    m = (torch.rand(5, 33, 7, device="cuda") < 0.5)[1:]
    assert m.data_ptr() % 16 != 0
    assert torch.equal(op_dequantize_mask(op_quantize_mask(m), dtype=torch.bool), m)

    gact.config.reset()
    gact.set_optimization_level("L1.1")           # fixed 8 bits
    w = torch.randn(33, 7, device="cuda")

    def run(hooked):
        base = torch.randn(5, 33, 7, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0)).requires_grad_()
        ctl = gact.Controller(nn.Linear(1, 1).cuda()) if hooked else None
        if hooked:
            ctl.install_hook()
        try:
            view = base[1:]                        # saved by the multiplication below, at an odd offset
            assert view.data_ptr() % 16 != 0
            ((view * view) * w).sum().backward()
            n = len(ctl.quantizer.bits) if hooked else 0
        finally:
            if hooked:
                ctl.uninstall_hook()
        return base.grad, n

    exact, _ = run(False)
    got, compressed = run(True)
    assert compressed >= 1
    # 8-bit codes: the saved values are off by up to one step (range / 255 ~ 0.03), the gradient 2 * v * w by |2 w| times that
    torch.testing.assert_close(got, exact, rtol=0.05, atol=0.3)
    assert float((got - exact).abs().mean()) < 0.03
