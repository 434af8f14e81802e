"""Records outputs of the reference's own CUDA kernels (built unmodified by oracle/build_ref.py) on a GPU, so that
the CPU oracle can be checked against the reference on machines that have neither the reference nor a GPU.

    python tests/golden/gen_reference_gpu_vectors.py [out.npz]      # needs a CUDA device and oracle/_ref/*.so

Small seeded inputs (a few thousand elements each, incl. ragged sizes, zeros of both signs, NaN / inf):
for each case the input bits, the packed bytes, min, scale and the dequantized tensor are stored.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402


def make(kind, n, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g)
    if kind == "relu":
        x = x.clamp_min(0)
    elif kind == "special":
        idx = torch.randperm(n, generator=g)
        k = max(1, n // 40)
        x[idx[:k]] = float("nan"); x[idx[k:2 * k]] = float("inf"); x[idx[2 * k:3 * k]] = float("-inf")
        x[idx[3 * k:6 * k]] = 0.0; x[idx[6 * k:9 * k]] = -0.0
    elif kind == "zeros":
        x = x.abs()
        idx = torch.randperm(n, generator=g)
        x[idx[: n // 3]] = 0.0; x[idx[n // 3: n // 2]] = -0.0
    elif kind == "tiny":
        x = x * 1e-6
    return x.to(dtype)


def main():
    out = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).with_name("reference_gpu_vectors.npz")
    q, m = build_ref.load("ref_quantization"), build_ref.load("ref_minimax")
    assert q is not None and m is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    data, i = {}, 0
    for dtype, code in ((torch.float32, 0), (torch.float16, 1)):
        for bits in (1, 2, 4, 8):
            for kind, n, seed in (("randn", 256 * 6 + 19, 3), ("relu", 256 * 7, 11), ("special", 256 * 5 + 100, 5),
                                  ("zeros", 256 * 4 + 7, 2), ("tiny", 256 * 3, 9)):
                x = make(kind, n, dtype, seed + bits).cuda()
                G = (n + 255) // 256
                flat = torch.zeros(G * 256, dtype=dtype, device="cuda")
                flat[:n] = x
                groups = flat.reshape(G, 256)
                mn, mx = m.minimax(groups)
                packed, scale = q.pack_single_precision(groups.view(G, 1, 256), mn.view(G, 1, 1), mx.view(G, 1, 1), bits, True, seed)
                deq = q.unpack_single_precision(packed, bits, scale, mn.view(G, 1, 1), G, 1, 256).reshape(-1)[:n]
                torch.cuda.synchronize()
                it = np.int16 if dtype == torch.float16 else np.int32
                tv = torch.int16 if dtype == torch.float16 else torch.int32
                data[f"c{i}_dtype"] = code
                data[f"c{i}_bits"] = bits
                data[f"c{i}_seed"] = seed
                data[f"c{i}_x"] = x.cpu().view(tv).numpy().astype(it)
                data[f"c{i}_packed"] = packed.cpu().view(torch.uint8)[:-1].numpy()
                data[f"c{i}_min"] = mn.cpu().view(tv).numpy().astype(it)
                data[f"c{i}_scale"] = scale.reshape(-1).cpu().view(tv).numpy().astype(it)
                data[f"c{i}_out"] = deq.cpu().view(tv).numpy().astype(it)
                i += 1
    data["n_cases"] = i
    np.savez_compressed(out, **data)
    print("wrote", out, i, "cases", out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
