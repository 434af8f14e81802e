"""The synthetic-data training drivers (gact-icml_b200/workloads.py): graph generator and GCN on the CPU, the
activation-memory protocol and the batch ladder on the GPU."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import workloads


def test_barabasi_albert_generator():
    n, m = 5000, 7
    e = workloads.barabasi_albert_edges(n, m, seed=0)
    assert e.shape[0] == 2 and e.dtype == torch.long
    assert e.shape[1] == m * (n - m)                       # a star on the first m + 1 nodes, then m edges per new node
    assert int(e.min()) == 0 and int(e.max()) == n - 1
    assert bool((e[0] != e[1]).all())                      # no self loops
    assert torch.equal(e, workloads.barabasi_albert_edges(n, m, seed=0))
    deg = torch.bincount(e.reshape(-1), minlength=n).float()
    assert float(deg.mean()) == pytest.approx(2 * m * (n - m) / n)
    # preferential attachment: a heavy tail (a uniform random graph of this size has a maximum degree of about 30)
    assert float(deg.max()) > 10 * float(deg.mean()) and float(deg.median()) <= 2 * m


def test_gcn_forward_backward_on_a_small_graph():
    torch.manual_seed(0)
    n = 300
    e = workloads.barabasi_albert_edges(n, 3, seed=1)
    e = torch.cat([e, e.flip(0), torch.arange(n).repeat(2, 1)], dim=1)
    adj = torch.sparse_coo_tensor(e, torch.ones(e.shape[1]), (n, n)).coalesce()
    model = workloads.GCN(16, 32, 5)
    x = torch.randn(n, 16)
    out = model(adj, x)
    assert out.shape == (n, 5)
    F.cross_entropy(out, torch.randint(0, 5, (n,))).backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


def _tiny_workload(dev, batch, hidden=1024):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, hidden), nn.GELU(), nn.Linear(hidden, hidden), nn.ReLU(), nn.Linear(hidden, 10)).to(dev)
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    x = torch.randn(batch, 256, device=dev)
    y = torch.randint(0, 10, (batch,), device=dev)

    def forward():
        opt.zero_grad(set_to_none=True)
        out = model(x)
        return F.cross_entropy(out, y), [out]

    def finish(loss):
        loss.backward()
        opt.step()

    def step():
        loss, _ = forward()
        finish(loss)
        return loss.detach()

    def backprop():
        opt.zero_grad(set_to_none=True)
        F.cross_entropy(model(x[:8]), y[:8]).backward()

    return workloads.Workload("tiny", model, opt, step, backprop, batch, {}, forward, finish)


@pytest.mark.gpu
def test_activation_memory_protocol_and_batch_ladder():
    """Allocated bytes before backward minus the level before the forward pass minus loss and outputs
    (benchmark/vision/train.py:242-281): smaller with compression, linear in the batch; the ladder stops by prediction."""
    import gact
    dev = torch.device("cuda", 0)
    torch.cuda.empty_cache()
    base = torch.cuda.memory_reserved()                    # whatever earlier tests of this process still hold

    def measure(level, batch):
        gact.config.reset()
        gact.set_optimization_level(level)
        wl = _tiny_workload(dev, batch)
        ctl = gact.Controller(wl.model)
        ctl.install_hook()
        try:
            wl.step()
            ctl.iterate(wl.backprop)
            return workloads.activation_memory(wl, lambda: ctl.iterate(wl.backprop))
        finally:
            ctl.uninstall_hook()

    m0, m1 = measure("L0", 4096), measure("L1", 4096)
    saved = 4096 * 1024 * 3 * 4                            # what the forward pass leaves behind: the GELU's input and output and the ReLU's output, fp32
    assert m0["activation_bytes"] == pytest.approx(saved, rel=0.15)
    assert m1["activation_bytes"] < 0.25 * m0["activation_bytes"]          # 4-bit codes + min / scale
    assert m0["peak_bytes"] >= m0["before_backward_bytes"] >= m0["before_forward_bytes"]
    m0b = measure("L0", 8192)
    assert m0b["activation_bytes"] == pytest.approx(2 * m0["activation_bytes"], rel=0.1)

    gact.config.reset()
    gact.set_optimization_level("L0")

    def build(batch):
        wl = _tiny_workload(dev, batch)
        return wl, None, (lambda: None)

    limit = base + 3 * (m0b["peak_reserved_bytes"] - base)  # a small pretend device
    rungs = workloads.batch_ladder(build, 2048, limit)
    assert [r["batch"] for r in rungs][:2] == [2048, 4096] and len(rungs) <= 6
    assert all(r["peak_reserved_bytes"] <= limit for r in rungs)
    last = rungs[-1]
    assert last["batch"] <= last["predicted_max_batch"] < 4 * last["batch"]
