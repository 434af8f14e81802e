#!/usr/bin/env python
"""Benchmark of the activation-compression hot path (quantize + dequantize GB/s) and of compressed training.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rng curand|fast|rtn] [--no-train]
    python bench.py --impl reference [--gpus N] [--steps K] [--warmup W]
    python bench.py --workload bert_large|resnet50|gcn [--level L2] [--batch B] [--get-mem] [--impl reference]
    python bench.py --case f16:2:fast --numel 102760448 --reps 3 [--relu]        (one kernel case, for profilers)
    python bench.py --case mask --numel 411041792 --reps 3

Default workload (the kernel sweep the metric is quoted on): post-ReLU activations of shape 128x64x112x112 in fp16 and
bf16 at 1/2/4/8 bits, plus a mixed list of 50 fp16 tensors of 2^20..2^26 elements with widths drawn from {2,4,8}.  One
pass = a "forward" phase that quantizes every tensor of the set followed by a "backward" phase that dequantizes them
in reverse order, so that nothing a kernel reads is still in L2 from the kernel that wrote it (the set moves ~10 GB
per pass; every big tensor is larger than L2).  One step = `passes_per_step` passes, chosen so that the timed
region lasts about a second.  `value` = algorithmic bytes (tensor + packed codes + per-group min and scale, each
counted once) of all launches of all ranks / max-over-ranks device time, inputs resident in HBM.  `e2e` = the same
bytes through the public ops (gact.ops.op_quantize / op_dequantize) starting from pinned host buffers and ending with
the reconstructed tensors back in host memory.  `train` = BERT-large sequence-classification training (batch 64 per
GPU, seq 128, bf16 autocast, AdamW; DDP over NCCL for N > 1) without compression (L0) and with auto-precision
compression (L2): samples/s over the steps after the adaptation step.

`--impl reference` times the CPU restatement of the reference quantizer (the oracle; the reference has no CPU
implementation of its own) on the host cores over a bounded sample of the same workload; with `--workload` it runs
the reference's own Python package on its own CUDA extensions (built unmodified into oracle/_ref) instead.

One process per GPU under torchrun for N > 1: every rank compresses its own tensors, no collective on the data
path (weak scaling).  Rank 0 prints exactly one JSON line on stdout.
"""
from __future__ import annotations

import argparse
import gc
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "gact-icml_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402

GROUP = 256
METRIC = "act quant+dequant GB/s"
# DRAM read + write of one quantize16 launch on the relu fp16 2-bit tensor (ncu dram__bytes_read.sum +
# dram__bytes_write.sum; the input is read once, part of the output is still in L2 when the kernel ends)
DOM_TRAFFIC_BYTES = 219258624
BIG_SHAPE = (128, 64, 112, 112)
DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def alg_bytes(n: int, bits: int, elem_size: int, scale_size: int) -> int:
    """Algorithmic bytes of ONE direction (quantize, or dequantize): the tensor, the packed codes, min + scale."""
    G = (n + GROUP - 1) // GROUP
    wpt = 8 // bits
    R = (G + wpt - 1) // wpt
    return n * elem_size + R * GROUP + G * (elem_size + scale_size)


def workload_spec():
    """[(name, dtype, numel, bits)] of the sweep.  Mixed list: numel = 2^k, k ~ U{20..26} (seed 1), bits ~ U{2,4,8}
    (seed 2)."""
    spec = []
    n_big = math.prod(BIG_SHAPE)
    for dt in (torch.float16, torch.bfloat16):
        for bits in (1, 2, 4, 8):
            spec.append((f"relu_{str(dt).split('.')[-1]}_b{bits}", dt, n_big, bits))
    g1 = torch.Generator().manual_seed(1)
    g2 = torch.Generator().manual_seed(2)
    ks = torch.randint(20, 27, (50,), generator=g1).tolist()
    bs = [(2, 4, 8)[i] for i in torch.randint(0, 3, (50,), generator=g2).tolist()]
    for i, (k, b) in enumerate(zip(ks, bs)):
        spec.append((f"mixed{i:02d}_2^{k}_b{b}", torch.float16, 1 << k, b))
    return spec


def spec_bytes(spec):
    total = 0
    for _, dt, n, bits in spec:
        es = 2 if dt != torch.float32 else 4
        ss = 4 if dt == torch.bfloat16 else es
        total += 2 * alg_bytes(n, bits, es, ss)
    return total


# ----------------------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, smax, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); smax.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def make_inputs(spec, device, seed):
    """Synthetic stand-ins with the sweep's shapes and value distributions: N(0,1) clamped at 0 (about half exact
    zeros) for the big tensors, N(0,1) for the mixed list.  Tensors that share dtype and size share storage."""
    cache = {}
    g = torch.Generator(device=device).manual_seed(seed)
    xs = []
    for name, dt, n, bits in spec:
        key = (dt, n, name.startswith("relu"))
        if key not in cache:
            x = torch.randn(n, device=device, generator=g)
            if name.startswith("relu"):
                x = x.clamp_min_(0)
            cache[key] = x.to(dt)
        xs.append(cache[key])
    return xs


def run_ours(args):
    import gact
    from gact import _native as nv
    from gact.ops import op_quantize, op_dequantize

    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    spec = workload_spec()
    xs = make_inputs(spec, dev, seed=1234 + rank)
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream
    mode = nv.RNG_CODE[args.rng]

    # ---- device-resident arm: straight through the C ABI, outputs preallocated -------------------------------
    bufs = []
    for (name, dt, n, bits), x in zip(spec, xs):
        G = (n + GROUP - 1) // GROUP
        nb = nv.lib.gact_packed_bytes(n, bits)
        sdt = torch.float32 if dt == torch.bfloat16 else dt
        bufs.append((torch.empty(nb, dtype=torch.uint8, device=dev), torch.empty(G, dtype=dt, device=dev),
                     torch.empty(G, dtype=sdt, device=dev)))
    out_big = {}
    for (name, dt, n, bits) in spec:
        if (dt, n) not in out_big:
            out_big[(dt, n)] = torch.empty(n, dtype=dt, device=dev)

    DOM = 1                                   # the launch the roofline is quoted on: relu fp16, 2 bit
    dom_events = []

    def forward_phase(seed, timed=False):
        for i, ((name, dt, n, bits), x) in enumerate(zip(spec, xs)):
            pk, mn, sc = bufs[i]
            if timed and i == DOM:
                e0 = torch.cuda.Event(enable_timing=True); e0.record(stream)
            st = nv.lib.gact_quantize(x.data_ptr(), nv.DTYPE_CODE[dt], n, bits, i + seed, mode, None, 1, pk.data_ptr(),
                                      mn.data_ptr(), sc.data_ptr(), sp)
            if timed and i == DOM:
                e1 = torch.cuda.Event(enable_timing=True); e1.record(stream)
                dom_events.append((e0, e1))
            if st:
                raise RuntimeError(nv.lib.gact_error_string(st).decode())

    def backward_phase():
        for i in range(len(spec) - 1, -1, -1):
            name, dt, n, bits = spec[i]
            pk, mn, sc = bufs[i]
            st = nv.lib.gact_dequantize(pk.data_ptr(), mn.data_ptr(), sc.data_ptr(), nv.DTYPE_CODE[dt], n, bits,
                                        out_big[(dt, n)].data_ptr(), sp)
            if st:
                raise RuntimeError(nv.lib.gact_error_string(st).decode())

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # warm-up passes, the last of them timed to size the steps: one step = R passes, R such that the K timed steps
    # last about a second (the same R on every rank)
    for w in range(args.warmup):
        forward_phase(w); backward_phase()
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record(stream); forward_phase(args.warmup); backward_phase(); c1.record(stream)
    torch.cuda.synchronize()
    est = torch.tensor([c0.elapsed_time(c1)], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(est, op=torch.distributed.ReduceOp.MAX)
    R = args.passes if args.passes > 0 else max(1, min(64, int(math.ceil(args.min_region_ms / (args.steps * float(est.item()))))))
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps * R + 1)]
    ev[0].record(stream)
    j = 0
    for k in range(args.steps):
        for r in range(R):
            forward_phase(args.warmup + 1 + k * R + r, timed=(r == 0))
            ev[2 * j + 1].record(stream)
            backward_phase()
            ev[2 * j + 2].record(stream)
            j += 1
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    q_ms = sum(ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(args.steps * R))
    d_ms = sum(ev[2 * k + 1].elapsed_time(ev[2 * k + 2]) for k in range(args.steps * R))
    clocks = sampler.stop() if rank == 0 else None
    passes = args.steps * R

    # ---- per-kernel table on rank 0 (stderr): every case timed alone with an L2 flush between launches ------
    # The flush writes 256 MB and then reads another 256 MB: the write alone would leave the L2 full of dirty lines
    # whose write-back runs into the timed launch (15-20 % for the kernels close to the DRAM limit); after the read
    # the cache is cold and clean.
    table = {}
    if rank == 0 and not args.no_table:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        flush_rd = torch.zeros(64 << 20, dtype=torch.int32, device=dev)
        for i, (name, dt, n, bits) in enumerate(spec[:8]):
            es = 2
            by = alg_bytes(n, bits, es, 4 if dt == torch.bfloat16 else 2)
            pk, mn, sc = bufs[i]

            def timed(fn):
                ts = []
                for rep in range(7):
                    flush.zero_()
                    flush_rd.max()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    fn(rep)
                    e1.record(stream)
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1))
                ts.sort()
                return ts[3]

            row = {}
            for mname in ("fast", "curand", "rtn"):
                m = nv.RNG_CODE[mname]
                t = timed(lambda rep: nv.lib.gact_quantize(xs[i].data_ptr(), nv.DTYPE_CODE[dt], n, bits, rep, m, None, 1,
                                                           pk.data_ptr(), mn.data_ptr(), sc.data_ptr(), sp))
                row[f"quantize_{mname}_GBps"] = round(by / t / 1e6, 1)
                row[f"quantize_{mname}_us"] = round(t * 1e3, 1)
            t = timed(lambda rep: nv.lib.gact_dequantize(pk.data_ptr(), mn.data_ptr(), sc.data_ptr(), nv.DTYPE_CODE[dt], n, bits,
                                                         out_big[(dt, n)].data_ptr(), sp))
            row["dequantize_GBps"] = round(by / t / 1e6, 1)
            row["dequantize_us"] = round(t * 1e3, 1)
            table[name] = row
            print(f"[bench] {name:20s} quantize fast {row['quantize_fast_GBps']:7.0f} curand {row['quantize_curand_GBps']:7.0f} "
                  f"rtn {row['quantize_rtn_GBps']:7.0f} | dequantize {row['dequantize_GBps']:7.0f} GB/s", file=sys.stderr)
        del flush, flush_rd

    # ---- end-to-end arm: pinned host -> op_quantize -> op_dequantize -> host ---------------------------------
    # (the big tensors only share two host buffers; every step copies each case's input in and its result out)
    e2e_spec = list(range(len(spec)))
    host_in, host_out = {}, {}
    for i in e2e_spec:
        name, dt, n, bits = spec[i]
        key = (dt, n, name.startswith("relu"))
        if key not in host_in:
            host_in[key] = xs[i].cpu().pin_memory()
            host_out[key] = torch.empty(n, dtype=dt).pin_memory()
    h2d = sum(spec[i][2] * 2 for i in e2e_spec)
    d2h = h2d

    # Three streams: inputs arrive on `s_in`, the library runs on torch's current stream, results leave on `s_out`;
    # PCIe is full duplex, so the results of one step drain while the inputs of the next arrive.  Nothing waits on
    # the host inside a step; the timed region ends with a device-wide synchronize.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    e2e_done = []

    def e2e_step(step):
        main = torch.cuda.current_stream()
        if len(e2e_done) >= 2:
            e2e_done[-2].synchronize()          # the host runs at most two steps ahead of the device
        saved = []
        for i in e2e_spec:
            name, dt, n, bits = spec[i]
            key = (dt, n, name.startswith("relu"))
            with torch.cuda.stream(s_in):
                x = host_in[key].to(dev, non_blocking=True)
            main.wait_stream(s_in)
            x.record_stream(main)
            saved.append((op_quantize(x, bits, i + step), x.shape, key))
            del x
        for q, shape, key in reversed(saved):
            y = op_dequantize(q, shape)
            s_out.wait_stream(main)
            with torch.cuda.stream(s_out):
                host_out[key].copy_(y, non_blocking=True)
            y.record_stream(s_out)
        ev = torch.cuda.Event()
        ev.record(s_out)
        e2e_done.append(ev)

    gact.config.rng_mode = args.rng
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    for w in range(min(args.warmup, 2)):
        e2e_step(w)
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for k in range(e2e_steps):
        e2e_step(100 + k)
    torch.cuda.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    # ---- reduce over ranks: max time, sum of bytes -----------------------------------------------------------
    times = torch.tensor([total_ms, q_ms, d_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    total_ms, q_ms, d_ms, e2e_ms = times.tolist()
    pass_bytes = spec_bytes(spec)
    value = world * pass_bytes * passes / (total_ms * 1e-3) / 1e9
    e2e_value = world * pass_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
    dom_us = sum(a.elapsed_time(b) for a, b in dom_events) / max(len(dom_events), 1) * 1e3
    n_dom = len(dom_events)

    # ---- training: BERT-large data parallel, L0 and L2 ----------------------------------------------------------
    del bufs, out_big, xs, host_in, host_out, e2e_done, dom_events
    gc.collect()
    torch.cuda.empty_cache()
    train = None
    if not args.no_train:
        train = {}
        for level in ("L0", "L2"):
            res = train_once(args, "bert_large", level, dev, rank, world, steps=args.train_steps, warmup=3)
            if rank == 0:
                train[level] = res
        if rank == 0:
            train["L2_over_L0"] = round(train["L2"]["samples_per_s"] / train["L0"]["samples_per_s"], 3)
            train["workload"] = "BERT-large seq-cls, seq 128, batch 64 per GPU, AdamW, bf16 autocast, synthetic tokens; DDP over NCCL for N > 1"

    if rank == 0:
        peaks = {}
        pk_path = ROOT / "MEASURED_PEAKS.json"
        if pk_path.exists():
            peaks = json.loads(pk_path.read_text())
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
        q_gbps = (pass_bytes / 2) * passes / (q_ms * 1e-3) / 1e9
        d_gbps = (pass_bytes / 2) * passes / (d_ms * 1e-3) / 1e9
        n_launch = len(spec)
        dom_bytes = alg_bytes(spec[DOM][2], spec[DOM][3], 2, 2)
        dom_gbps = dom_bytes / (dom_us * 1e-6) / 1e9 if dom_us > 0 else 0.0
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(total_ms / args.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16/bf16 in, u8 codes", "data": "synthetic",
            "config": {"workload": "kernel sweep: relu 128x64x112x112 fp16+bf16 x bits{1,2,4,8} + 50 mixed fp16 tensors 2^20..2^26 x bits{2,4,8}",
                       "group_size": GROUP, "rng": args.rng,
                       "rng_note": "fast = the library's default noise arrangement (Philox4x32-7, 8 bits per element), not the reference's stream; "
                                   "rng=curand reproduces the reference's bytes and is timed in `kernels` (quantize_curand_*)",
                       "l2": "inputs larger than L2; all quantizes of a pass run before its dequantizes",
                       "passes_per_step": R, "bytes_per_pass_per_gpu": pass_bytes, "bytes_per_step_per_gpu": pass_bytes * R},
            "pct_of_8TBps": round(100 * value / world / 8000.0, 1),
            "roofline": {"kernel": "quantize16_kernel<f16, 2 bit, %s> on relu 128x64x112x112 (%d launches timed inside the steps)" % (args.rng, n_dom),
                         "bound": "hbm", "achieved": round(dom_gbps, 1), "peak": peak, "unit": "GB/s", "frac": round(dom_gbps / peak, 3),
                         "traffic": DOM_TRAFFIC_BYTES, "algorithmic_bytes": dom_bytes, "avg_launch_us": round(dom_us, 2),
                         "peak_source": peak_src,
                         "all_quantize_launches": {"achieved": round(q_gbps, 1), "frac": round(q_gbps / peak, 3)},
                         "all_dequantize_launches": {"achieved": round(d_gbps, 1), "frac": round(d_gbps / peak, 3)}},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": "gact.ops.op_quantize/op_dequantize from pinned host buffers; copy-in, compute and copy-out on three streams"},
            "gpu_launches": 2 * n_launch * passes,
            "clocks": clocks,
            "kernels": table,
            "kernels_note": "every case launched alone, median of 7, L2 flushed before each launch by a 256 MB write followed by a 256 MB read (cold and clean)",
        }
        if train is not None:
            line["train"] = train
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(spec, sample_elems=1 << 24, reps=6)
        emit(line)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


# ----------------------------------------------------------------------------------------------------------------
def host_threads():
    """Host threads this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sample(spec, sample_elems):
    """Bounded sample of the workload for the CPU runs: the first `sample_elems` elements of the eight big cases
    and of the first eight mixed tensors (same dtypes, widths and distributions)."""
    g = torch.Generator().manual_seed(99)
    base = torch.randn(sample_elems, generator=g)
    cases = []
    for name, dt, n, bits in spec[:16]:
        m = min(n, sample_elems)
        x = base[:m].clamp_min(0) if name.startswith("relu") else base[:m]
        cases.append((name, x.to(dt).contiguous(), bits))
    return cases


def cpu_pass(cases, seed):
    import oracle
    by = 0
    t0 = time.perf_counter()
    for name, x, bits in cases:
        pk, mn, sc = oracle.quantize(x, bits, seed)
        oracle.dequantize(pk, mn, sc, x.numel(), bits)
        by += 2 * alg_bytes(x.numel(), bits, 2, 4 if x.dtype == torch.bfloat16 else 2)
    return by, time.perf_counter() - t0


def cpu_baseline(spec, sample_elems, reps):
    import oracle
    oracle.set_threads(host_threads())
    cases = cpu_sample(spec, sample_elems)
    cpu_pass(cases[:2], 0)
    by, dt = 0, 0.0
    for r in range(reps):
        b, t = cpu_pass(cases, r)
        by += b; dt += t
    return {"value": round(by / dt / 1e9, 3), "unit": "GB/s", "cores": oracle.threads(), "kind": "port",
            "sample": f"first {sample_elems} elements of the 8 big cases and of 8 mixed tensors, quantize+dequantize, "
                      f"CPU restatement of the reference kernels (oracle/gact_oracle.c, OpenMP), {reps} pass(es), {dt:.1f} s"}


def reference_cuda_rows():
    """Extra information for the reference arm: the reference's own CUDA kernels (built unmodified into
    oracle/_ref) timed on this GPU for the fp16 cases of the sweep (the reference does not take bf16):
    quantize = its minimax + scale + pack kernels, dequantize = its unpack kernel.  None without a GPU or binaries."""
    if not torch.cuda.is_available():
        return None
    try:
        from oracle import build_ref
        q, m = build_ref.load("ref_quantization"), build_ref.load("ref_minimax")
    except Exception:
        return None
    if q is None or m is None:
        return None
    dev = torch.device("cuda", 0)
    n = math.prod(BIG_SHAPE)
    G = n // GROUP
    x = torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(1234)).clamp_min_(0).half()
    groups = x.view(G, GROUP)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush_rd = torch.zeros(64 << 20, dtype=torch.int32, device=dev)      # read after the write: cold AND clean, as in the table above
    rows = {}
    for bits in (1, 2, 4, 8):
        by = alg_bytes(n, bits, 2, 2)

        def med(fn):
            ts = []
            for _ in range(5):
                flush.zero_()
                flush_rd.max()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); r = fn(); e1.record(); torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ts.sort()
            return ts[2], r

        def quant():
            mn, mx = m.minimax(groups)
            return q.pack_single_precision(groups.view(G, 1, GROUP), mn.view(G, 1, 1), mx.view(G, 1, 1), bits, True, 1) + (mn,)

        tq, (packed, scale, mn) = med(quant)
        td, _ = med(lambda: q.unpack_single_precision(packed, bits, scale, mn.view(G, 1, 1), G, 1, GROUP))
        rows[f"relu_float16_b{bits}"] = {"quantize_GBps": round(by / tq / 1e6, 1), "dequantize_GBps": round(by / td / 1e6, 1),
                                          "quantize_us": round(tq * 1e3, 1), "dequantize_us": round(td * 1e3, 1)}
        del packed, scale, mn
    return rows


def run_reference(args):
    """The reference has no CPU implementation of this path (every entry point demands CUDA tensors), so its
    arm is the CPU restatement of its kernels (the oracle) over a bounded sample.  Under torchrun every rank runs
    the sample on its share of the host cores and the bytes are summed over the ranks, as the GPU arm sums its
    ranks' bytes."""
    rank, world, local = dist_env()
    import oracle
    threads = max(1, host_threads() // world)
    oracle.set_threads(threads)
    if world > 1:
        torch.distributed.init_process_group("gloo")
    spec = workload_spec()
    sample = 1 << 22
    cases = cpu_sample(spec, sample)
    for w in range(args.warmup):
        cpu_pass(cases[:4], w)
    if world > 1:
        torch.distributed.barrier()
    by, dt = 0, 0.0
    for k in range(args.steps):
        b, t = cpu_pass(cases, k)
        by += b; dt += t
    red = torch.tensor([float(by), dt, float(oracle.threads())], dtype=torch.float64)
    if world > 1:
        mx = red.clone()
        torch.distributed.all_reduce(red, op=torch.distributed.ReduceOp.SUM)
        torch.distributed.all_reduce(mx, op=torch.distributed.ReduceOp.MAX)
        by, dt, cores = red[0].item(), mx[1].item(), int(red[2].item())
    else:
        cores = int(red[2].item())
    if rank == 0:
        v = round(by / dt / 1e9, 3)
        base = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port",
                "sample": f"per step and rank: first {sample} elements of the 8 big cases and of 8 mixed tensors, quantize+dequantize; "
                          f"{world} rank(s) x {threads} thread(s)"}
        line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f16/bf16 in, u8 codes", "data": "synthetic",
                "config": {"workload": "kernel sweep (bounded sample on host cores)", "group_size": GROUP, "rng": "curand"},
                "cpu_baseline": base,
                "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        extra = reference_cuda_rows()
        if extra is not None:
            line["reference_cuda_kernels_on_this_gpu"] = extra
        emit(line)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


# ----------------------------------------------------------------------------------------------------------------
def import_gact(reference: bool):
    """The product's `gact`, or - for the reference training arm - the reference's own Python package on its own CUDA
    extensions, as oracle/build_ref.py installed them (unmodified) under oracle/_ref/pkg.  Returns the module, or None
    when the reference package is not there."""
    if reference:
        pkg = ROOT / "oracle" / "_ref" / "pkg"
        if not (pkg / "gact" / "__init__.py").exists():
            return None
        sys.path.insert(0, str(pkg))
    import gact
    return gact


AUTOCAST = {"bf16": torch.bfloat16, "fp16": torch.float16, "off": None}


def train_once(args, workload, level, dev, rank, world, steps, warmup, reference=False, get_mem=False):
    """Builds the workload, runs the adaptation step, `warmup` steps and `steps` timed steps (CUDA events, barrier and
    synchronize on both sides, max over ranks), and tears everything down again.  The loop is the reference
    drivers': step, then controller.iterate(backprop) (benchmark/text_classification/run_glue.py:577-623,
    benchmark/vision/train.py:316-350).  Returns the result dict on every rank."""
    import workloads
    gact = import_gact(reference)
    if hasattr(gact.config, "reset"):
        gact.config.reset()
    else:                                      # the reference keeps whatever an earlier level left behind
        gact.config.swap = gact.config.prefetch = False
    gact.set_optimization_level(level)
    if not reference:
        gact.config.rng_mode = args.rng
        gact.config.dp_probe = args.dp_probe
    workloads.DDP_BUCKET_MB = args.bucket_mb
    kw = {"world": world, "seed": rank}
    if args.batch:
        kw["batch"] = args.batch
    if workload == "bert_large" and args.layers:
        kw["layers"] = args.layers
    if workload != "gcn" and args.autocast is not None:
        kw["autocast"] = AUTOCAST[args.autocast]
    wl = workloads.BUILDERS[workload](dev, **kw)
    from gact.controller import Controller
    ctl = Controller(wl.model)
    ctl.install_hook()
    launch_counter = None if reference else sys.modules["gact.ops"].launches

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def one_step():
        loss = wl.step()
        ctl.iterate(wl.backprop)
        return loss

    try:
        t_adapt0 = time.perf_counter()
        loss = one_step()                          # first iteration: the sensitivity probe + bit allocation
        barrier()
        adapt_s = time.perf_counter() - t_adapt0
        for _ in range(max(warmup - 1, 0)):
            loss = one_step()
        barrier()
        torch.cuda.reset_peak_memory_stats()
        sampler = ClockSampler(dev.index)
        if rank == 0:
            sampler.start()
        launches0 = launch_counter() if launch_counter else 0
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for k in range(steps):
            loss = one_step()
            ev[k + 1].record()
        barrier()
        total_ms = ev[0].elapsed_time(ev[-1])
        per_step = [ev[k].elapsed_time(ev[k + 1]) for k in range(steps)]
        clocks = sampler.stop() if rank == 0 else None
        launches = (launch_counter() - launches0) if launch_counter else None
        peak_mem = torch.cuda.max_memory_allocated()
        mem = workloads.activation_memory(wl, lambda: ctl.iterate(wl.backprop)) if get_mem or args.train_mem else None
        final_loss = float(loss)
    finally:
        ctl.uninstall_hook()
    t = torch.tensor([total_ms, statistics.median(per_step)], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    total_ms, med_ms = t.tolist()
    compress = getattr(gact.config, "compress_activation", False)
    bits = dict(ctl.quantizer.bits) if compress else {}
    hist = {}
    for b in bits.values():
        hist[str(b)] = hist.get(str(b), 0) + 1
    res = {"samples_per_s": round(world * wl.samples_per_step * steps / (total_ms * 1e-3), 2),
           "samples_per_s_median_step": round(world * wl.samples_per_step / (med_ms * 1e-3), 2),
           "ms_per_step": round(total_ms / steps, 3), "median_ms_per_step": round(med_ms, 3), "steps": steps,
           "adapt_seconds": round(adapt_s, 2), "compressed_tensors": len(bits), "bit_histogram": hist,
           "peak_mem_GB": round(peak_mem / 2**30, 2), "final_loss": final_loss, "gpu_launches": launches, "clocks": clocks,
           "describe": wl.describe, "name": wl.name}
    if mem is not None:
        res["memory"] = mem
    del wl, ctl
    gc.collect()
    torch.cuda.empty_cache()
    return res


def run_training(args):
    """`--workload X`: training throughput (samples/s) of one synthetic-data workload at one level; with `--get-mem`
    also the activation memory of a step and a batch ladder; with `--impl reference` on the reference's own code."""
    rank, world, local = dist_env()
    reference = args.impl == "reference"
    if reference and import_gact(True) is None:
        if rank == 0:
            emit({"impl": "reference", "unavailable": "oracle/_ref/pkg (the reference package installed by oracle/build_ref.py) is missing"})
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    res = train_once(args, args.workload, args.level, dev, rank, world, steps=args.steps, warmup=args.warmup,
                     reference=reference, get_mem=args.get_mem)
    ladder = None
    if args.get_mem and world == 1 and args.workload != "gcn":
        ladder = memory_ladder(args, dev, reference)
    if rank == 0:
        line = {"metric": f"GACT {res['name']} samples/s", "value": res["samples_per_s"], "unit": "samples/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
                "median_ms_per_step": res["median_ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": res["describe"].get("autocast", "fp32"), "data": "synthetic",
                "config": dict(res["describe"], workload=res["name"], level=args.level, rng=args.rng, dp_probe=args.dp_probe,
                               parallelism=f"dp{world}", ddp_bucket_mb=args.bucket_mb),
                "compressed_tensors": res["compressed_tensors"], "bit_histogram": res["bit_histogram"],
                "adapt_seconds": res["adapt_seconds"], "peak_mem_GB": res["peak_mem_GB"], "final_loss": res["final_loss"],
                "gpu_launches": res["gpu_launches"], "clocks": res["clocks"]}
        if reference:
            line["impl"] = "reference"
            line["config"]["code"] = "the reference's gact package and CUDA extensions, unmodified (oracle/_ref/pkg)"
        if "memory" in res:
            line["memory"] = res["memory"]
        if ladder is not None:
            line["batch_ladder"] = ladder
        emit(line)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


def memory_ladder(args, dev, reference):
    """Batch ladder of `workloads.batch_ladder` for the current level: doubles the batch while the next rung is
    predicted to stay below 80 % of the device memory (reserved by the caching allocator, which runs ahead of what is allocated)."""
    import workloads
    gact = import_gact(reference)
    from gact.controller import Controller
    total = torch.cuda.get_device_properties(dev).total_memory
    kw = {}
    if args.autocast is not None:
        kw["autocast"] = AUTOCAST[args.autocast]

    def build(batch):
        wl = workloads.BUILDERS[args.workload](dev, batch=batch, **kw)
        ctl = Controller(wl.model)
        ctl.install_hook()
        return wl, (lambda: ctl.iterate(wl.backprop)), ctl.uninstall_hook

    start = args.batch or {"bert_large": 64, "resnet50": 256}[args.workload]
    return workloads.batch_ladder(build, start, int(0.8 * total))


# ----------------------------------------------------------------------------------------------------------------
def run_case(args):
    """One quantize + dequantize case (or the mask kernels) a few times, for use under a profiler.  The tensor should be
    larger than L2 (126 MB on B200) for DRAM counters to mean anything and small enough for a multi-pass capture to
    finish quickly (a few hundred MB).  Prints the CUDA-event time of every launch."""
    from gact import _native as nv
    torch.manual_seed(0)
    s = torch.cuda.current_stream().cuda_stream
    if args.case == "mask":
        x = (torch.rand(args.numel, device="cuda") < 0.9).to(torch.uint8)
        n = x.numel()
        words = torch.empty(nv.lib.gact_mask_words(n), dtype=torch.int32, device="cuda")
        out = torch.empty_like(x)
        by = n + words.numel() * 4
        for r in range(args.reps):
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
        return
    dname, bits, rng = args.case.split(":")
    dt, bits = DTYPES[dname], int(bits)
    x = torch.randn(args.numel, device="cuda")
    if args.relu:
        x.clamp_min_(0)
    x = x.to(dt)
    n = x.numel()
    G = (n + 255) // 256
    pk = torch.empty(nv.lib.gact_packed_bytes(n, bits), dtype=torch.uint8, device="cuda")
    mn = torch.empty(G, dtype=dt, device="cuda")
    sc = torch.empty(G, dtype=torch.float32 if dt == torch.bfloat16 else dt, device="cuda")
    out = torch.empty_like(x)
    es = x.element_size()
    by = n * es + pk.numel() + G * (es + sc.element_size())
    for r in range(args.reps):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        st = nv.lib.gact_quantize(x.data_ptr(), nv.DTYPE_CODE[dt], n, bits, r, nv.RNG_CODE[rng], None, 1, pk.data_ptr(),
                                  mn.data_ptr(), sc.data_ptr(), s)
        assert st == 0
        e[1].record()
        st = nv.lib.gact_dequantize(pk.data_ptr(), mn.data_ptr(), sc.data_ptr(), nv.DTYPE_CODE[dt], n, bits, out.data_ptr(), s)
        assert st == 0
        e[2].record()
        torch.cuda.synchronize()
        tq, td = e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])
        print(f"rep {r}: quantize {tq*1e3:.1f} us ({by/tq/1e6:.0f} GB/s)  dequantize {td*1e3:.1f} us ({by/td/1e6:.0f} GB/s)  "
              f"algorithmic bytes per launch {by}")


_RESULT_FD = None


def claim_stdout():
    """Keep file descriptor 1 for the result line alone: libraries that write to stdout on their own (NCCL prints
    its version there on the first collective) are sent to stderr for the rest of the run."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 20 for the sweep and for training)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rng", default="fast", choices=["curand", "fast", "rtn"])
    ap.add_argument("--workload", default="sweep", choices=["sweep", "bert_large", "resnet50", "gcn"])
    ap.add_argument("--level", default="L2", help="optimisation level of the training workloads (L0 = uncompressed)")
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch of the training workloads (0 = the workload's own)")
    ap.add_argument("--layers", type=int, default=0, help="bert_large only: fewer encoder layers for quick runs")
    ap.add_argument("--autocast", default=None, choices=["bf16", "fp16", "off"], help="autocast type of the training workloads (default: the workload's own)")
    ap.add_argument("--dp-probe", default="allreduce", choices=["allreduce", "local", "shard"])
    ap.add_argument("--bucket-mb", type=int, default=100, help="DDP gradient bucket size of the training workloads")
    ap.add_argument("--get-mem", action="store_true", help="training workloads: activation memory of a step and a batch ladder")
    ap.add_argument("--e2e-steps", type=int, default=8)
    ap.add_argument("--passes", type=int, default=0, help="sweep passes per step (0 = as many as make the timed region last --min-region-ms)")
    ap.add_argument("--min-region-ms", type=float, default=1000.0)
    ap.add_argument("--no-train", action="store_true", help="sweep only: leave out the BERT-large training runs")
    ap.add_argument("--train-steps", type=int, default=20)
    ap.add_argument("--train-mem", action="store_true", help="add the activation-memory readings to the `train` object")
    ap.add_argument("--no-table", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", default=None, help="DTYPE:BITS:RNG (e.g. f16:2:fast) or `mask`: run one kernel case --reps times and print its times")
    ap.add_argument("--numel", type=int, default=1 << 27)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--relu", action="store_true")
    args = ap.parse_args()
    if args.case is not None:
        return run_case(args)
    claim_stdout()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.steps is None:
        args.steps = 5 if (args.impl == "reference" and args.workload == "sweep") else 20
    if args.workload != "sweep":
        if not torch.cuda.is_available():
            raise SystemExit("training workloads need a CUDA device")
        return run_training(args)
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU baseline")
    run_ours(args)


if __name__ == "__main__":
    main()
