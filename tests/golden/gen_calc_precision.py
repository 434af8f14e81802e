"""Generates tests/golden/calc_precision.json from the reference's own greedy allocator.

The reference's ``gact/gact/cpp_extension/calc_precision.cc`` is host C++; ``oracle/build_ref.py`` compiles
it unmodified into ``oracle/_ref/ref_calc_precision.so``.  This script feeds it seeded inputs shaped like
``AutoPrecision.refresh_bits`` does (gact/gact/autoprec.py:188-209: all bits start at 32, target =
avg_bits * sum(dims)) and stores inputs + outputs, so the check travels to machines without the reference.

    python oracle/build_ref.py && python tests/golden/gen_calc_precision.py
"""
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402

ref = build_ref.load("ref_calc_precision")
assert ref is not None, "build oracle/_ref first"

rng = np.random.default_rng(20240607)
cases = []


def add(C, w, avg, start=32):
    C = np.asarray(C, dtype=np.float32)
    w = np.asarray(w, dtype=np.int64)
    b = torch.full((len(C),), start, dtype=torch.int32)
    target = float(avg) * float(w.sum())
    out = ref.calc_precision(b, torch.from_numpy(C.copy()), torch.from_numpy(w.copy()), target)
    cases.append({"C_bits": C.view(np.uint32).tolist(), "w": w.tolist(), "avg_bits": avg, "target": target,
                  "start": start, "bits": out.tolist()})


for L in [1, 2, 3, 7, 16, 33, 100, 257, 400]:
    for avg in [2, 3, 4, 8]:
        C = np.exp(rng.uniform(-12, 12, size=L))
        w = rng.choice([256, 1000, 4096, 65536, 802816, 3211264, 25690112], size=L)
        add(C, w, avg)
# ties: identical sensitivities and sizes -> popping order decided by the index
for L in [4, 9, 64]:
    for avg in [2, 3, 4]:
        add(np.ones(L), np.full(L, 4096), avg)
        add(np.full(L, 1e10), np.full(L, 1 << 20), avg)      # all clamped (autoprec.py:123-126)
# blocks of equal keys mixed with distinct ones, zero sensitivity
for avg in [2, 3, 4]:
    C = np.concatenate([np.zeros(5), np.ones(5), rng.uniform(0, 1, 10), np.ones(5)])
    w = np.concatenate([np.full(5, 512), np.full(5, 2048), rng.integers(256, 1 << 22, 10), np.full(5, 2048)])
    add(C, w, avg)
# fractional budgets (e.g. the controller passes avg_bits * sum(dims) as a double)
for avg in [1.5, 2.5, 5.0, 16.0, 31.9]:
    C = np.exp(rng.uniform(-5, 5, size=50))
    w = rng.integers(256, 1 << 24, size=50)
    add(C, w, avg)

out = Path(__file__).with_name("calc_precision.json")
out.write_text(json.dumps({"source": "reference calc_precision.cc built unmodified", "cases": cases}))
print("wrote", out, len(cases), "cases", out.stat().st_size, "bytes")
