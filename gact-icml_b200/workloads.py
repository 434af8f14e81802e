"""End-to-end training workloads with synthetic data, for measuring compressed training throughput.

These stand in for the reference's dataset-driven benchmark drivers (GLUE fine-tuning, ImageNet, ogbn-arxiv): same
model shapes, random-init weights, seeded synthetic inputs of the same shapes and value distributions.  Each
workload follows the loop of the reference drivers: forward / backward / optimizer step, then
``controller.iterate(backprop)`` where ``backprop`` runs one forward + backward on the first 8 samples
(reference: benchmark/text_classification/run_glue.py:611-623, benchmark/vision/train.py:316-330).

    BUILDERS[name](device, batch=..., world=..., seed=...) -> Workload(model, step(), backprop(), forward(), finish(), ...)

``activation_memory`` and ``batch_ladder`` measure what the reference's drivers report with ``--get-mem`` and what
its ``exp_mem_speed.py`` sweeps search for (activation bytes per step, largest batch that fits).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class Workload:
    name: str
    model: nn.Module
    optimizer: torch.optim.Optimizer
    step: Callable[[], torch.Tensor]        # forward + backward + optimizer step on the full batch, returns the loss
    backprop: Callable[[], None]            # forward + backward on the probe batch (first 8 samples)
    samples_per_step: int
    describe: dict
    forward: Callable[[], tuple] = None      # forward pass on the full batch -> (loss, [outputs])
    finish: Callable[[torch.Tensor], None] = None   # backward + optimizer step for that loss


DDP_BUCKET_MB = 25          # torch's default; benchmarks may raise it (fewer, larger NVLink all-reduces)


def _wrap_ddp(model, device, world):
    if world > 1:
        return nn.parallel.DistributedDataParallel(model, device_ids=[device.index], gradient_as_bucket_view=True,
                                                   bucket_cap_mb=DDP_BUCKET_MB)
    return model


def bert_large(device, batch=64, seq_len=128, world=1, seed=0, layers=24, autocast=torch.bfloat16) -> Workload:
    """BERT-large sequence classification: 24 layers, hidden 1024, 16 heads, FFN 4096, vocab 30522; uniform random
    token ids, 2 uniform random labels, AdamW lr 2e-5, bf16 autocast."""
    from transformers import BertConfig, BertForSequenceClassification
    torch.manual_seed(seed)
    cfg = BertConfig(vocab_size=30522, hidden_size=1024, num_hidden_layers=layers, num_attention_heads=16,
                     intermediate_size=4096, max_position_embeddings=512, num_labels=2)
    model = BertForSequenceClassification(cfg).to(device)
    model.train()
    model = _wrap_ddp(model, device, world)
    opt = torch.optim.AdamW(model.parameters(), lr=2e-5)
    g = torch.Generator(device=device).manual_seed(1000 + seed)
    ids = torch.randint(0, 30522, (batch, seq_len), device=device, generator=g)
    labels = torch.randint(0, 2, (batch,), device=device, generator=g)
    mask = torch.ones_like(ids)

    def fwd(i, m, y):
        with torch.autocast("cuda", dtype=autocast, enabled=autocast is not None):
            out = model(input_ids=i, attention_mask=m, labels=y)
        return out.loss, [out.logits]

    def forward():
        opt.zero_grad(set_to_none=True)
        return fwd(ids, mask, labels)

    def finish(loss):
        loss.backward()
        opt.step()

    def step():
        loss, _ = forward()
        finish(loss)
        return loss.detach()

    def backprop():
        opt.zero_grad(set_to_none=True)
        fwd(ids[:8], mask[:8], labels[:8])[0].backward()

    return Workload("bert_large", model, opt, step, backprop, batch,
                    {"model": "BERT-large seq-cls (random init)", "layers": layers, "seq_len": seq_len, "batch_per_gpu": batch,
                     "optimizer": "AdamW lr 2e-5", "autocast": str(autocast).split(".")[-1] if autocast else "off"},
                    forward, finish)


def resnet50(device, batch=256, world=1, seed=0, autocast=None) -> Workload:
    """ResNet-50, 3x224x224 N(0,1) images, 1000 uniform random labels, SGD momentum 0.9."""
    import torchvision
    torch.manual_seed(seed)
    model = torchvision.models.resnet50(weights=None).to(device)
    model.train()
    model = _wrap_ddp(model, device, world)
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    g = torch.Generator(device=device).manual_seed(2000 + seed)
    x = torch.randn(batch, 3, 224, 224, device=device, generator=g)
    y = torch.randint(0, 1000, (batch,), device=device, generator=g)

    def fwd(a, b):
        with torch.autocast("cuda", dtype=autocast, enabled=autocast is not None):
            out = model(a)
            loss = F.cross_entropy(out, b)
        return loss, [out]

    def forward():
        opt.zero_grad(set_to_none=True)
        return fwd(x, y)

    def finish(loss):
        loss.backward()
        opt.step()

    def step():
        loss, _ = forward()
        finish(loss)
        return loss.detach()

    def backprop():
        opt.zero_grad(set_to_none=True)
        fwd(x[:8], y[:8])[0].backward()

    return Workload("resnet50", model, opt, step, backprop, batch,
                    {"model": "ResNet-50 (random init)", "batch_per_gpu": batch, "optimizer": "SGD momentum 0.9",
                     "autocast": str(autocast).split(".")[-1] if autocast else "off"},
                    forward, finish)


class GCN(nn.Module):
    """Three graph-convolution layers, H' = A_hat (H W) + b, ReLU and dropout between them."""

    def __init__(self, in_dim, hidden, classes, dropout=0.5):
        super().__init__()
        self.lins = nn.ModuleList([nn.Linear(in_dim, hidden), nn.Linear(hidden, hidden), nn.Linear(hidden, classes)])
        self.dropout = dropout

    def forward(self, adj, x):
        for i, lin in enumerate(self.lins):
            x = torch.sparse.mm(adj, lin(x))
            if i < len(self.lins) - 1:
                x = F.dropout(F.relu(x), self.dropout, self.training)
        return x


def barabasi_albert_edges(n, m, seed):
    """Preferential attachment (Barabasi-Albert): every new node links to m existing nodes drawn in proportion to
    their degree (sampling from the list of edge endpoints).  Returns undirected edges as a (2, E) tensor."""
    g = torch.Generator().manual_seed(seed)
    src = [torch.arange(1, m + 1), ]                     # a star on the first m+1 nodes to start from
    dst = [torch.zeros(m, dtype=torch.long)]
    endpoints = torch.cat([src[0], dst[0]])
    chunk = 4096                                         # nodes attached per vectorised round (degrees lag by one round)
    node = m + 1
    pool = [endpoints]
    pool_cat = endpoints
    while node < n:
        k = min(chunk, n - node, max(1, pool_cat.numel() // (4 * m)))
        new = torch.arange(node, node + k)
        pick = pool_cat[torch.randint(0, pool_cat.numel(), (k, m), generator=g)]
        s = new.repeat_interleave(m)
        d = pick.reshape(-1)
        src.append(s); dst.append(d)
        pool_cat = torch.cat([pool_cat, s, d])
        node += k
    return torch.stack([torch.cat(src), torch.cat(dst)])


def gcn(device, world=1, seed=0, nodes=169343, feat=128, hidden=256, classes=40, m=7, autocast=None) -> Workload:
    """Full-batch 3-layer GCN on a synthetic power-law graph: 169 343 nodes, ~1.17 M undirected edges (m = 7),
    128-d N(0,1) features, 40 uniform random classes, Adam lr 0.01."""
    torch.manual_seed(seed)
    e = barabasi_albert_edges(nodes, m, seed)
    e = torch.cat([e, e.flip(0), torch.arange(nodes).repeat(2, 1)], dim=1)          # symmetric + self loops
    adj = torch.sparse_coo_tensor(e, torch.ones(e.shape[1]), (nodes, nodes)).coalesce()
    deg = torch.sparse.sum(adj, dim=1).to_dense().clamp_min(1)
    idx = adj.indices()
    val = adj.values() / (deg[idx[0]].sqrt() * deg[idx[1]].sqrt())                  # D^-1/2 A D^-1/2
    adj = torch.sparse_coo_tensor(idx, val, (nodes, nodes)).coalesce().to(device).to_sparse_csr()
    g = torch.Generator().manual_seed(3000 + seed)
    x = torch.randn(nodes, feat, generator=g).to(device)
    y = torch.randint(0, classes, (nodes,), generator=g).to(device)
    model = GCN(feat, hidden, classes).to(device)
    model.train()
    opt = torch.optim.Adam(model.parameters(), lr=0.01)

    def forward():
        opt.zero_grad(set_to_none=True)
        out = model(adj, x)
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
        forward()[0].backward()

    return Workload("gcn", model, opt, step, backprop, 1,
                    {"model": "3-layer GCN, hidden 256", "nodes": nodes, "undirected_edges": int((e.shape[1] - nodes) // 2),
                     "optimizer": "Adam lr 0.01", "unit_note": "one sample = one full-batch epoch"},
                    forward, finish)


BUILDERS = {"bert_large": bert_large, "resnet50": resnet50, "gcn": gcn}


# ---------------------------------------------------------------------------------------------------------------
# Memory, measured the way the reference's drivers do with --get-mem (benchmark/vision/train.py:242-281,
# benchmark/text_classification/run_glue.py:508-559): allocated bytes right before backward, minus the level before
# the forward pass (weights, optimizer state, data, gradients of the previous step) and minus loss and outputs, is
# what the saved tensors of one step hold.
# ---------------------------------------------------------------------------------------------------------------
def _nbytes(ts):
    return sum(t.numel() * t.element_size() for t in ts)


def activation_memory(wl: Workload, iterate: Callable[[], None] = None) -> dict:
    """One training step with the three readings of the reference protocol.  ``iterate``: what follows the optimizer
    step in the training loop (``controller.iterate(backprop)``), or None."""
    torch.cuda.synchronize()
    init = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    loss, outs = wl.forward()
    torch.cuda.synchronize()
    before_backward = torch.cuda.memory_allocated()
    act = before_backward - init - _nbytes([loss] + list(outs))
    del outs
    wl.finish(loss)
    del loss
    if iterate is not None:
        iterate()
    torch.cuda.synchronize()
    after = torch.cuda.memory_allocated()
    return {"activation_bytes": int(act), "before_forward_bytes": int(init), "before_backward_bytes": int(before_backward),
            "after_step_bytes": int(after), "peak_bytes": int(torch.cuda.max_memory_allocated()),
            "peak_reserved_bytes": int(torch.cuda.max_memory_reserved())}


def batch_ladder(build: Callable[[int], tuple], start: int, limit_bytes: int, max_rungs: int = 12) -> list:
    """Doubles the batch while the NEXT rung is predicted to stay below ``limit_bytes`` (a linear fit of the peak of
    reserved memory over the rungs measured so far), instead of the reference's search by running out of memory
    (benchmark/vision/exp_mem_speed.py:42-54).  ``build(batch)`` -> (workload, iterate or None, cleanup); every rung
    runs two steps and reports the second.  Returns one record per rung; the last carries ``predicted_max_batch``."""
    rungs = []
    b = start
    for _ in range(max_rungs):
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        wl, iterate, cleanup = build(b)
        try:
            wl.step()
            if iterate is not None:
                iterate()
            m = activation_memory(wl, iterate)
        finally:
            cleanup()
            del wl
            torch.cuda.empty_cache()
        m["batch"] = b
        rungs.append(m)
        # what decides whether the next rung fits is what the caching allocator has to RESERVE (its blocks fragment:
        # reserved memory runs well ahead of allocated memory at large batches), so the prediction is made on that
        if len(rungs) >= 2:
            (b0, p0), (b1, p1) = [(r["batch"], r["peak_reserved_bytes"]) for r in rungs[-2:]]
            slope = max((p1 - p0) / (b1 - b0), 1.0)
        else:
            slope = max((m["activation_bytes"] * 1.5) / b, 1.0)          # first guess: activations dominate the growth
        fixed = m["peak_reserved_bytes"] - slope * b
        m["predicted_max_batch"] = int((limit_bytes - fixed) // slope)
        # the same fit on ALLOCATED memory: what a run with a defragmenting allocator could reach, and the figure
        # to compare between levels (fragmentation differs from level to level)
        if len(rungs) >= 2:
            (b0, p0), (b1, p1) = [(r["batch"], r["peak_bytes"]) for r in rungs[-2:]]
            aslope = max((p1 - p0) / (b1 - b0), 1.0)
        else:
            aslope = slope
        m["predicted_max_batch_by_allocated"] = int((limit_bytes - (m["peak_bytes"] - aslope * b)) // aslope)
        if fixed + slope * 2 * b > limit_bytes:
            break
        b *= 2
    return rungs
