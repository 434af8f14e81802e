"""Two ranks on two GPUs over NCCL: DDP training with auto precision.  After the one all-reduce of the L x 3 probe
statistics every rank holds the same sensitivities and the same widths, in every probe mode; ranks draw different
noise.  Skipped unless two GPUs are visible.  NVLS is switched off: nothing here needs it, and a rank that ended
early while bound to an NVLink multicast object would disturb its peer."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
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
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import datetime

    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as F
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    import gact
    gact.config.reset()
    gact.set_optimization_level("L2")
    gact.config.dp_probe = mode
    torch.manual_seed(0)                                   # same initial weights on every rank
    net = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.Linear(512, 512), nn.GELU(), nn.Linear(512, 8)).to(dev)
    model = nn.parallel.DistributedDataParallel(net, device_ids=[rank])
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    torch.manual_seed(100 + rank)                          # different data per rank
    x, y = torch.randn(64, 256, device=dev), torch.randint(0, 8, (64,), device=dev)
    ctl = gact.Controller(model)
    assert ctl.quantizer.seed_offset == rank << 32
    ctl.install_hook()

    def backprop():
        opt.zero_grad()
        F.cross_entropy(model(x[:8]), y[:8]).backward()

    losses = []
    try:
        for _ in range(3):
            opt.zero_grad()
            loss = F.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            losses.append(float(loss))
            ctl.iterate(backprop)
    finally:
        ctl.uninstall_hook()
    w = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    torch.save({"bits": dict(ctl.quantizer.bits), "C": dict(ctl.ap.C), "losses": losses, "wsum": float(w.double().sum())},
               os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["allreduce", "local", "shard"])
def test_ranks_agree_over_nccl(tmp_path, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), mode, str(tmp_path)), nprocs=world, join=True)
    r0, r1 = torch.load(tmp_path / "r0.pt"), torch.load(tmp_path / "r1.pt")
    assert r0["bits"] == r1["bits"] and len(r0["bits"]) >= 3
    assert r0["C"] == r1["C"] and all(v >= 0 for v in r0["C"].values())
    assert r0["wsum"] == r1["wsum"]                         # DDP kept the replicas identical
    assert r0["losses"] != r1["losses"]                     # different data on each rank
