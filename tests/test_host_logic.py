"""CPU tests of the host-side logic (config presets, Quantizer bookkeeping, Controller, AutoPrecision) with the
native calls routed to a host-memory stand-in (tests/fake_native.py, backed by the CPU oracle)."""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import gact
import oracle
from gact.conf import config
from gact.quantizer import Quantizer
from gact.controller import Controller

import fake_native


@pytest.fixture
def fake(monkeypatch):
    fake_native.install(monkeypatch)
    yield


def test_level_presets_and_their_leaks():
    gact.set_optimization_level("L1")
    assert (config.auto_prec, config.bit) == (False, 4)
    gact.set_optimization_level("L1.1")
    assert config.bit == 8
    gact.set_optimization_level("L1.2")
    assert config.bit == 2
    gact.set_optimization_level("L2.1")
    assert (config.auto_prec, config.bit) == (True, 3)
    gact.set_optimization_level("L3")
    assert config.swap and config.prefetch and config.auto_prec and config.bit == 4
    gact.set_optimization_level("L1")            # presets only touch what they name (as in the reference)
    assert config.swap and not config.auto_prec
    config.reset()
    gact.set_optimization_level("L0")
    assert not config.compress_activation
    gact.set_optimization_level("L4bit-swap")
    assert config.swap and config.prefetch and not config.auto_prec
    with pytest.raises(ValueError):
        gact.set_optimization_level("L1.4")       # the reference's sweep script asks for this undefined level
    gact.set_adapt_interval(7)
    assert config.adapt_interval == 7


def test_default_bit_mapping(fake):
    model = nn.Linear(4, 4)
    for bit, want in ((2, 2), (3, 4), (4, 4), (5, 8), (8, 8), (16, 8)):
        config.reset()
        config.bit = bit
        config.auto_prec = False
        assert Controller(model).quantizer.default_bit == want
    config.bit = 1
    with pytest.raises(AssertionError):
        Controller(model)


def test_check_quantize_filter(fake):
    q = Quantizer(4, False, False)
    p = nn.Parameter(torch.randn(8, 256))
    q.filter_tensors([("w", p)])
    act = torch.randn(8, 256, requires_grad=True)
    assert q.check_quantize(p) == (False, False)                                   # parameter
    assert q.check_quantize(act) == (True, False)
    assert q.check_quantize(torch.randn(8, 256)) == (False, False)                 # no grad (e.g. BN statistics)
    assert q.check_quantize(torch.randn(256, requires_grad=True)) == (False, False)          # 1-D
    assert q.check_quantize(torch.randn(2, 2, 2, 2, 64, requires_grad=True)) == (False, False)  # 5-D
    assert q.check_quantize(torch.randn(8, 256, dtype=torch.float64, requires_grad=True)) == (False, False)
    assert q.check_quantize(torch.randn(8, 256, requires_grad=True).half()) == (True, False)
    assert q.check_quantize(torch.randn(8, 256, requires_grad=True).bfloat16()) == (True, False)
    config.quantize_bf16 = False                                                   # the reference's behaviour
    assert q.check_quantize(torch.randn(8, 256, requires_grad=True).bfloat16()) == (False, False)
    assert q.check_quantize(torch.ones(10, dtype=torch.bool)) == (True, True)
    assert q.check_quantize(torch.ones(10, dtype=torch.uint8)) == (True, True)
    assert q.check_quantize(torch.ones(10, dtype=torch.int32)) == (False, False)
    assert q.check_quantize(torch.empty(0, dtype=torch.uint8)) == (False, False)


def test_quantizer_tuples_tids_seeds_and_refcounts(fake):
    q = Quantizer(2, False, False)
    x0 = torch.randn(4, 300, requires_grad=True)
    x1 = torch.randn(2, 3, 128, requires_grad=True).half()
    r0, r1 = q.quantize(x0), q.quantize(x1)
    assert r0 == (True, False, 0, x0.shape, 0) and r1 == (True, False, 1, x1.shape, 1)
    assert q.bits == {0: 2, 1: 2} and q.dims == {0: 1200, 1: 768} and q.seeds == {0: 0, 1: 1}
    skipped = torch.randn(5)
    assert q.quantize(skipped)[0] is False and q.quantize(skipped)[1] is skipped          # no tid consumed
    assert q.tid == 2
    # payload matches the oracle with seed = seeds[tid] + seed_iter
    q_inputs, ref, tid = q.ptr_qtensor_map[1]
    want = oracle.op_quantize(x1.detach(), 2, 1 + 0, rng_mode=config.rng_mode)
    assert ref == 1 and tid == 1 and torch.equal(q_inputs[0][:-1], want[0][:-1])
    y1 = q.dequantize(r1)
    assert y1.shape == x1.shape and y1.dtype == torch.float16
    assert 1 not in q.ptr_qtensor_map and 0 in q.ptr_qtensor_map                           # released at ref-count 0
    q.dequantize(r0)
    with pytest.raises(KeyError):
        q.dequantize(r0)
    # next iteration: tids restart, bits come from the table, the seed moves with seed_iter
    q.iterate()
    q.seed_iter = 5
    q.bits[0] = 8
    r = q.quantize(x0)
    assert r[4] == 0 and q.ptr_qtensor_map[0][0][1] == 8
    want = oracle.op_quantize(x0.detach(), 8, 0 + 5, rng_mode=config.rng_mode)
    assert torch.equal(q.ptr_qtensor_map[0][0][0][:-1], want[0][:-1])
    # a tensor that was never registered in iteration 0 is an error, as in the reference (static graph)
    q.quantize(x1)
    with pytest.raises(KeyError):
        q.quantize(torch.randn(3, 3, requires_grad=True))


def test_check_dup_shares_one_payload(fake):
    config.check_dup = True
    q = Quantizer(4, False, False)
    x = torch.randn(16, 256, requires_grad=True)
    a, b = q.quantize(x), q.quantize(x)
    assert a[2] == b[2] and a[4] == 0 and b[4] == 1
    (payload, ref, tid), = q.ptr_qtensor_map.values()
    assert ref == 2
    ya, yb = q.dequantize(a), q.dequantize(b)
    assert torch.equal(ya, yb) and not q.ptr_qtensor_map


def test_masks(fake):
    q = Quantizer(4, False, False)
    m = torch.rand(7, 100) < 0.5
    r = q.quantize(m)
    assert r[0] and r[1] and r[2][0].dtype == torch.int32
    assert torch.equal(q.dequantize(r), m)
    u = m.to(torch.uint8)
    r = q.quantize(u)
    assert r[0] and r[1] and torch.equal(q.dequantize(r), u)
    u2 = u.clone()
    u2[0, 0] = 3                                                                    # not a mask: kept as it is
    r = q.quantize(u2)
    assert r[0] is False and r[1] is u2


class TinyNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(64, 128)
        self.b = nn.Linear(128, 128)
        self.c = nn.Linear(128, 8)

    def forward(self, x):
        return self.c(F.gelu(self.b(F.relu(self.a(x)))))


def _train(level, steps, interval=2, seed=0):
    config.reset()
    gact.set_optimization_level(level)
    gact.set_adapt_interval(interval)
    torch.manual_seed(seed)
    model = TinyNet()
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    x, y = torch.randn(32, 64), torch.randint(0, 8, (32,))
    ctl = Controller(model)
    ctl.install_hook()
    losses = []

    def backprop():
        opt.zero_grad()
        F.cross_entropy(model(x), y).backward()

    try:
        for _ in range(steps):
            opt.zero_grad()
            loss = F.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
            ctl.iterate(backprop)
    finally:
        ctl.uninstall_hook()
    return losses, ctl


def test_controller_hooks_fixed_bits(fake):
    base, _ = _train("L0", 3)
    l8, ctl = _train("L1.1", 3)
    assert set(ctl.quantizer.bits.values()) == {8} and len(ctl.quantizer.bits) >= 3
    np.testing.assert_allclose(l8, base, rtol=5e-2)
    assert ctl.iter == 3 and ctl.quantizer.seed_iter == 3 and not ctl.quantizer.ptr_qtensor_map
    ctl.uninstall_hook()            # second call is a no-op: only what install_hook pushed is popped
    ctl.install_hook(); ctl.install_hook(); ctl.uninstall_hook()
    x = torch.randn(4, 64, requires_grad=True)
    (x * 2).sum().backward()        # no hook left behind


def test_auto_precision_end_to_end_on_cpu(fake):
    losses, ctl = _train("L2", 3, interval=2)
    ap = ctl.ap
    L = len(ctl.quantizer.bits)
    assert L >= 3 and set(ap.C) == set(ctl.quantizer.bits) and ap.iter == 3
    assert all(b in (1, 2, 4, 8, 32) for b in ctl.quantizer.bits.values())
    assert sum(ctl.quantizer.bits[l] * ap.dims[l] for l in ap.dims) <= ap.total_bits
    l_list = list(ap.dims)
    want, _ = oracle.calc_precision(torch.full((L,), 32, dtype=torch.int32),
                                    torch.tensor([ap.C[l] for l in l_list], dtype=torch.float32),
                                    torch.tensor([ap.dims[l] for l in l_list], dtype=torch.int64), ap.total_bits)
    assert [ctl.quantizer.bits[l] for l in l_list] == want.tolist()
    assert all(np.isfinite(losses))
    # probing must leave the table of seeds untouched and the bits consistent with the allocation
    assert ctl.quantizer.seeds == {l: l for l in l_list}      # seeds[tid] = tid; duplicates register nothing


def test_probe_matches_reference_formula(fake):
    """One tensor probed by hand: C = max(|g0-g1|^2, 2*max(|g0-g2|^2, |g1-g2|^2)) with the probe's seeds/bits."""
    config.reset()
    gact.set_optimization_level("L2")
    torch.manual_seed(3)
    model = TinyNet()
    x, y = torch.randn(16, 64), torch.randint(0, 8, (16,))
    ctl = Controller(model)
    ctl.install_hook()

    def backprop():
        model.zero_grad()
        F.cross_entropy(model(x), y).backward()

    try:
        backprop()
        ctl.iterate(backprop)
        q = ctl.quantizer

        def grad_with(l, bits, seed_shift):
            old_b, old_s = q.bits[l], q.seeds[l]
            q.bits[l], q.seeds[l] = bits, old_s + seed_shift
            q.iterate()
            q.seed_iter = 0            # the probe ran before the controller advanced its seed
            torch.manual_seed(0)
            backprop()
            g = torch.cat([p.grad.reshape(-1) for p in model.parameters()]).clone()
            q.bits[l], q.seeds[l] = old_b, old_s
            return g

        saved_bits = dict(q.bits)
        q.bits = {l: q.default_bit for l in saved_bits}        # the probe ran with the default widths elsewhere
        l = list(saved_bits)[1]
        g0, g1, g2 = grad_with(l, 1, 0), grad_with(l, 1, 1), grad_with(l, 8, 0)
        want = max(float(((g0 - g1) ** 2).sum()), 2 * max(float(((g0 - g2) ** 2).sum()), float(((g1 - g2) ** 2).sum())))
        assert ctl.ap.C[l] == pytest.approx(want, rel=1e-4)
    finally:
        ctl.uninstall_hook()


def test_state_dict_round_trip(fake):
    _, ctl = _train("L2", 2, interval=100)
    sd = ctl.state_dict()
    ctl2 = Controller(TinyNet())
    ctl2.load_state_dict(sd)
    assert ctl2.quantizer.bits == ctl.quantizer.bits and ctl2.ap.C == ctl.ap.C and ctl2.iter == ctl.iter
    assert ctl2.ap.total_bits == ctl.ap.total_bits


def test_utils():
    from gact.utils import compute_tensor_bytes, uniform_sample, uniform_sample_ref, exp_recorder
    t = torch.arange(1000, dtype=torch.float32)
    assert uniform_sample(t, 10) == uniform_sample_ref(t, 10) and len(uniform_sample(t, 10)) == 11
    assert uniform_sample(t, 10) == uniform_sample(t, 10)
    assert compute_tensor_bytes([torch.zeros(3, 4), torch.zeros(5, dtype=torch.int8), 7, torch.zeros(2, dtype=torch.bfloat16)]) == 48 + 5 + 4 + 4
    exp_recorder.record("x", np.float32(1.23456789))
    assert exp_recorder.val_dict["x"] == 1.234568


def test_same_tensor_saved_twice_shares_one_payload_without_reading_it(fake):
    q = Quantizer(4, False, False)
    x = torch.randn(16, 256, requires_grad=True)
    a, b = q.quantize(x), q.quantize(x)
    assert a[2] == b[2] and (a[4], b[4]) == (0, 1) and len(q.ptr_qtensor_map) == 1
    assert q.ptr_qtensor_map[a[2]][1] == 2 and list(q.bits) == [0]           # the duplicate registers no width of its own
    y = x.detach().clone().requires_grad_()
    c = q.quantize(y)                                                        # equal values, other object: not shared
    assert c[2] != a[2]
    with torch.no_grad():
        x.add_(1.0)                                                          # modified in place: version moved on
    d = q.quantize(x)
    assert d[2] != a[2]
    for r in (a, b, c, d):
        q.dequantize(r)
    assert not q.ptr_qtensor_map
    config.dedup_saved = False
    q = Quantizer(4, False, False)
    a, b = q.quantize(x), q.quantize(x)
    assert a[2] != b[2]


def test_dense_permuted_views_are_compressed_in_memory_order(fake):
    q = Quantizer(8, False, False)
    base = torch.randn(4, 6, 32, 16)
    x = base.transpose(1, 2).requires_grad_()                 # dense, not contiguous
    assert not x.is_contiguous()
    r = q.quantize(x)
    payload = q.ptr_qtensor_map[r[2]][0]
    assert payload.strides == x.stride()
    want = oracle.quantize(base.reshape(-1), 8, 0, config.rng_mode)[0]          # memory order = the base tensor's order
    assert torch.equal(payload[0][:-1].view(torch.uint8), want)
    y = q.dequantize(r)
    assert y.shape == x.shape and y.stride() == x.stride()
    assert float((y - x).abs().max()) < 0.05
    # a view with gaps is not dense: it takes the copy
    z = torch.randn(8, 64, 40)[:, :, :32].requires_grad_()
    r = q.quantize(z)
    assert q.ptr_qtensor_map[r[2]][0].strides is None
    assert float((q.dequantize(r) - z).abs().max()) < 0.05
    config.keep_layout = False
    r = q.quantize(x)
    assert q.ptr_qtensor_map[r[2]][0].strides is None


def test_logging_and_debug_branches(fake, tmp_path, capsys):
    """log_interval > 0 and debug = True (reference: gact/gact/autoprec.py:131-183,211-234): autoprec.log gets one
    JSON record per logged iteration, the variance comparison is printed, and the too-large-variance warning is
    recorded when the quantization variance exceeds a tenth of the gradient variance."""
    import json
    config.reset()
    gact.set_optimization_level("L2")
    gact.set_adapt_interval(2)
    config.log_interval = 1
    config.debug = True
    config.work_dir = str(tmp_path) + "/"
    torch.manual_seed(0)
    model = TinyNet()
    x, y = torch.randn(32, 64), torch.randint(0, 8, (32,))
    ctl = Controller(model)
    ctl.ap.warmpup_iter = 0                      # the reference only warns after 100 iterations
    ctl.install_hook()

    def backprop():
        model.zero_grad()
        F.cross_entropy(model(x), y).backward()

    try:
        for _ in range(4):
            backprop()
            ctl.iterate(backprop)
    finally:
        ctl.uninstall_hook()
    out = capsys.readouterr().out
    assert "Exact Variance" in out and "use 4 bit to compare" in out and "GACT: Initializing AutoPrec" in out
    records = [json.loads(l) for l in (tmp_path / "autoprec.log").read_text().splitlines()]
    # one record per iteration, plus the warning's own record at the adaptation of iteration 2 (> warm-up 0; the
    # running gradient variance is still tiny then).  The recorder never forgets a key (its clear() is a no-op in
    # the reference too), so the later records carry the warning's fields along.
    assert [r["iter"] for r in records] == [0, 1, 2, 2, 3]
    L = len(ctl.quantizer.bits)
    for r in records:
        assert len(r["layer sensitivity"]) == L and len(r["bits"]) == L and len(r["dims"]) == L
    assert "warning" not in records[0] and "warning" not in records[1]
    warned = records[2]
    assert warned["warning"] is True and warned["quantization var"] > 0.1 * warned["overall var"]
    assert "Quantization variance is too large" in out
    assert ctl.ap.grad_var > 0 and 0 < ctl.ap.beta1 < 1
    # debug leaves the allocated widths in place
    assert ctl.quantizer.bits == ctl.ap.bits


def test_python_layer_raises_when_a_pipeline_wait_ran_out(fake, monkeypatch):
    import gact.controller
    monkeypatch.setattr(gact.controller, "_device_live", lambda: True)
    config.reset()
    gact.set_optimization_level("L1")
    ctl = Controller(TinyNet())
    ctl.install_hook()
    fake_native.FakeLib.pipeline_error = 2
    try:
        with pytest.raises(RuntimeError, match="pipeline"):
            ctl.uninstall_hook()
        assert fake_native.FakeLib.pipeline_error == 0 and not ctl._hook_installed      # reported once, then cleared
        ctl.install_hook()
        ctl.uninstall_hook()
    finally:
        fake_native.FakeLib.pipeline_error = 0
    # and at the probe's synchronisation point
    fake_native.FakeLib.pipeline_error = 1
    try:
        with pytest.raises(RuntimeError, match="pipeline"):
            _train("L2", 1, interval=1)
    finally:
        fake_native.FakeLib.pipeline_error = 0


def test_probe_refuses_gradients_of_different_size(fake):
    _, ctl = _train("L2", 1, interval=100)
    g = [torch.zeros(10), torch.zeros(5)]
    with pytest.raises(RuntimeError, match="different total size"):
        ctl.ap._distances(torch.zeros(15), torch.zeros(14), g, torch.zeros(3, dtype=torch.float64))
    with pytest.raises(RuntimeError, match="different total size"):
        ctl.ap._distances(torch.zeros(15), torch.zeros(15), g[:1], torch.zeros(3, dtype=torch.float64))


def test_a_tid_that_was_a_duplicate_at_registration_can_stand_alone_later(fake):
    q = Quantizer(4, False, False)
    x = torch.randn(16, 256, requires_grad=True)
    q.quantize(x); q.quantize(x)                 # iteration 0: tid 1 shares tid 0's payload and registers nothing
    assert list(q.bits) == [0]
    q.iterate()
    a = q.quantize(x)
    b = q.quantize(x.detach().clone().requires_grad_())      # tid 1 is its own tensor now
    assert b[4] == 1 and q.ptr_qtensor_map[b[2]][0].bits == q.default_bit
    q.dequantize(a); q.dequantize(b)


def test_short_payloads_are_refused(fake, monkeypatch):
    from gact import ops
    import gact.cpp_extension.quantization as shim
    monkeypatch.setattr(shim, "nv", fake_native.FakeNative)
    x = torch.randn(3, 300)
    q = ops.op_quantize(x, 4, 0)
    with pytest.raises(ValueError):
        ops.op_dequantize([q[0][:100], 4, q[2], q[3]], x.shape)
    with pytest.raises(ValueError):
        ops.op_dequantize([q[0], 4, q[2][:1], q[3]], x.shape)
    m = (torch.rand(700) < 0.5).to(torch.uint8)
    words, shape = ops.op_quantize_mask(m)
    assert words.numel() == 32                                    # two started blocks of 512
    with pytest.raises(ValueError):
        ops.op_dequantize_mask([words[:22], shape])               # ceil(700/32) words, what the reference allocates
    with pytest.raises(ValueError):
        shim.act_dequantize_dropout_mask(words[:22], 700)
    with pytest.raises(ValueError):
        shim.unpack_single_precision(q[0][:64], 4, q[2], q[3], 4, 1, 256)
    assert torch.equal(shim.act_dequantize_dropout_mask(words, 700), m)
