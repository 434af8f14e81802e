"""End-to-end training workloads with synthetic data, for measuring compressed training throughput.

These stand in for the reference's dataset-driven benchmark drivers (GLUE fine-tuning, ImageNet, ogbn-arxiv): same
model shapes, random-init weights, seeded synthetic inputs of the same shapes and value distributions.  Each
workload follows the loop of the reference drivers: forward / backward / optimizer step, then
``controller.iterate(backprop)`` where ``backprop`` runs one forward + backward on the first 8 samples
(reference: benchmark/text_classification/run_glue.py:611-623, benchmark/vision/train.py:316-330).

    build(name, device, batch, dtype_autocast) -> Workload(model, step(), backprop(), samples_per_step)
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

    def fwd_bwd(i, m, y):
        with torch.autocast("cuda", dtype=autocast, enabled=autocast is not None):
            out = model(input_ids=i, attention_mask=m, labels=y)
        out.loss.backward()
        return out.loss

    def step():
        opt.zero_grad(set_to_none=True)
        loss = fwd_bwd(ids, mask, labels)
        opt.step()
        return loss.detach()

    def backprop():
        opt.zero_grad(set_to_none=True)
        fwd_bwd(ids[:8], mask[:8], labels[:8])

    return Workload("bert_large", model, opt, step, backprop, batch,
                    {"model": "BERT-large seq-cls (random init)", "layers": layers, "seq_len": seq_len, "batch_per_gpu": batch,
                     "optimizer": "AdamW lr 2e-5", "autocast": str(autocast).split(".")[-1] if autocast else "off"})


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

    def fwd_bwd(a, b):
        with torch.autocast("cuda", dtype=autocast, enabled=autocast is not None):
            loss = F.cross_entropy(model(a), b)
        loss.backward()
        return loss

    def step():
        opt.zero_grad(set_to_none=True)
        loss = fwd_bwd(x, y)
        opt.step()
        return loss.detach()

    def backprop():
        opt.zero_grad(set_to_none=True)
        fwd_bwd(x[:8], y[:8])

    return Workload("resnet50", model, opt, step, backprop, batch,
                    {"model": "ResNet-50 (random init)", "batch_per_gpu": batch, "optimizer": "SGD momentum 0.9"})


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

    def fwd_bwd():
        loss = F.cross_entropy(model(adj, x), y)
        loss.backward()
        return loss

    def step():
        opt.zero_grad(set_to_none=True)
        loss = fwd_bwd()
        opt.step()
        return loss.detach()

    def backprop():
        opt.zero_grad(set_to_none=True)
        fwd_bwd()

    return Workload("gcn", model, opt, step, backprop, 1,
                    {"model": "3-layer GCN, hidden 256", "nodes": nodes, "undirected_edges": int((e.shape[1] - nodes) // 2),
                     "optimizer": "Adam lr 0.01", "unit_note": "one sample = one full-batch epoch"})


BUILDERS = {"bert_large": bert_large, "resnet50": resnet50, "gcn": gcn}
