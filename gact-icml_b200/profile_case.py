"""Runs one quantize + dequantize case a few times, for use under a profiler.

    python gact-icml_b200/profile_case.py --dtype f16 --bits 2 --numel 134217728 --reps 3 [--rng curand] [--relu]
    python gact-icml_b200/profile_case.py --mask --numel 411041792 --reps 3        (dropout-mask pack + unpack)

The tensor should be larger than L2 (126 MB on B200) for DRAM counters to mean anything and small enough for a
multi-pass capture to finish quickly (a few hundred MB).  Prints the CUDA-event time of every launch.
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="f16", choices=["f32", "f16", "bf16"])
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--numel", type=int, default=1 << 27)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--rng", default="curand")
    ap.add_argument("--relu", action="store_true")
    ap.add_argument("--mask", action="store_true", help="run the 1-bit mask kernels on --numel bytes instead")
    a = ap.parse_args()
    from gact import _native as nv
    if a.mask:
        return run_mask(a, nv)
    dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[a.dtype]
    torch.manual_seed(0)
    x = torch.randn(a.numel, device="cuda")
    if a.relu:
        x.clamp_min_(0)
    x = x.to(dt)
    n = x.numel()
    G = (n + 255) // 256
    pk = torch.empty(nv.lib.gact_packed_bytes(n, a.bits), dtype=torch.uint8, device="cuda")
    mn = torch.empty(G, dtype=dt, device="cuda")
    sc = torch.empty(G, dtype=torch.float32 if dt == torch.bfloat16 else dt, device="cuda")
    out = torch.empty_like(x)
    s = torch.cuda.current_stream().cuda_stream
    es = x.element_size()
    by = n * es + pk.numel() + G * (es + sc.element_size())
    for r in range(a.reps):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        st = nv.lib.gact_quantize(x.data_ptr(), nv.DTYPE_CODE[dt], n, a.bits, r, nv.RNG_CODE[a.rng], None, 1, pk.data_ptr(),
                                  mn.data_ptr(), sc.data_ptr(), s)
        assert st == 0
        e[1].record()
        st = nv.lib.gact_dequantize(pk.data_ptr(), mn.data_ptr(), sc.data_ptr(), nv.DTYPE_CODE[dt], n, a.bits, out.data_ptr(), s)
        assert st == 0
        e[2].record()
        torch.cuda.synchronize()
        tq, td = e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])
        print(f"rep {r}: quantize {tq*1e3:.1f} us ({by/tq/1e6:.0f} GB/s)  dequantize {td*1e3:.1f} us ({by/td/1e6:.0f} GB/s)  "
              f"algorithmic bytes per launch {by}")


def run_mask(a, nv):
    torch.manual_seed(0)
    x = (torch.rand(a.numel, device="cuda") < 0.9).to(torch.uint8)
    n = x.numel()
    words = torch.empty(nv.lib.gact_mask_words(n), dtype=torch.int32, device="cuda")
    out = torch.empty_like(x)
    s = torch.cuda.current_stream().cuda_stream
    by = n + words.numel() * 4
    for r in range(a.reps):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        assert nv.lib.gact_mask_pack(x.data_ptr(), n, words.data_ptr(), None, s) == 0
        e[1].record()
        assert nv.lib.gact_mask_unpack(words.data_ptr(), n, out.data_ptr(), s) == 0
        e[2].record()
        torch.cuda.synchronize()
        tp, tu = e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])
        print(f"rep {r}: mask pack {tp*1e3:.1f} us ({by/tp/1e6:.0f} GB/s)  unpack {tu*1e3:.1f} us ({by/tu/1e6:.0f} GB/s)  "
              f"algorithmic bytes per launch {by}")
    assert torch.equal(out, x)


if __name__ == "__main__":
    main()
