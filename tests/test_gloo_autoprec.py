"""World-size-2 CPU test (gloo) of the data-parallel part of auto precision: after the single all-reduce of the
L x 3 probe statistics every rank holds the same sensitivities and therefore the same bit widths, in both probe
modes; ranks draw different noise (seed offset rank << 32)."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, mode, out_dir):
    for p in (ROOT, ROOT / "gact-icml_b200", ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as F
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import gact
    import gact.ops, gact.autoprec, gact.quantizer
    import fake_native
    gact.ops.nv = fake_native.FakeNative
    gact.autoprec.nv = fake_native.FakeNative
    gact.quantizer.Quantizer._on_device = staticmethod(lambda t: True)
    gact.quantizer._hooks = None                           # the native hooks only take CUDA tensors
    import gact.controller
    gact.controller._nv = fake_native.FakeNative
    gact.config.reset()
    gact.set_optimization_level("L2")
    gact.config.dp_probe = mode
    torch.manual_seed(0)                                   # same initial weights on every rank
    net = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 64), nn.GELU(), nn.Linear(64, 4))
    model = nn.parallel.DistributedDataParallel(net)
    torch.manual_seed(100 + rank)                          # different data per rank
    x, y = torch.randn(16, 32), torch.randint(0, 4, (16,))
    ctl = gact.Controller(model)
    assert ctl.quantizer.seed_offset == rank << 32
    ctl.install_hook()

    def backprop():
        model.zero_grad()
        F.cross_entropy(model(x), y).backward()

    backprop()
    ctl.iterate(backprop)
    ctl.uninstall_hook()
    torch.save({"bits": dict(ctl.quantizer.bits), "C": dict(ctl.ap.C)}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["allreduce", "local", "shard"])
def test_ranks_agree_on_sensitivities_and_bits(tmp_path, mode):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=True)
    r0, r1 = torch.load(tmp_path / "r0.pt"), torch.load(tmp_path / "r1.pt")
    assert r0["bits"] == r1["bits"] and len(r0["bits"]) >= 3
    assert r0["C"] == r1["C"]
    assert all(v >= 0 for v in r0["C"].values())
