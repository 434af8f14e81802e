"""Auto precision: per-tensor bit widths from a gradient-sensitivity probe (reference: gact/gact/autoprec.py).

Every ``adapt_interval`` iterations each saved tensor l is probed with three extra forward/backward passes
(1 bit with seed s, 1 bit with seed s+1, 8 bit) and its sensitivity is
``C_l = max(|g0-g1|^2, 2*max(|g0-g2|^2, |g1-g2|^2))`` over the concatenated parameter gradients; a greedy
allocation then spends the bit budget ``avg_bits * sum(dims)`` where it reduces the predicted variance most.

What differs from the reference is where the arithmetic runs: the gradients are never concatenated (two
flat snapshots + the live ``.grad`` tensors through a pointer table), the three distances come from one
deterministic reduction kernel, sensitivities stay on the device, the greedy allocation is a device kernel,
and the host synchronises once per adaptation instead of once per tensor.  With ``torch.distributed``
initialised, the per-tensor statistics are all-reduced once so that every rank derives the same widths.
"""
import os
import random

import numpy as np
import torch
import torch.nn as nn

from gact.conf import config
from gact.utils import exp_recorder
from gact import _native as nv


def _dist():
    d = torch.distributed
    return d if (d.is_available() and d.is_initialized()) else None


class AutoPrecision:
    def __init__(self, model, quantizer, bits, max_bits, work_dir, adapt_interval, log_interval,
                 momentum=0.99, warmup_iter=100, debug=False):
        self.model = model
        self.quantizer = quantizer
        self.debug = debug

        self.dims = None
        self.bits = {}   # bits of each tensor
        self.C = {}      # sensitivity of each tensor

        self.avg_bits = bits
        self.max_bits = max_bits

        # running batch gradient, used to warn about an overly large quantization variance
        self.momentum = momentum
        self.warmpup_iter = warmup_iter
        self.beta1 = 1e-7
        self.batch_grad = 0
        self.grad_var = 0
        self.adapt_interval = adapt_interval

        self.iter = 0
        self.log_iter = log_interval
        self.work_dir = work_dir

        self._flat = [None, None]     # gradient snapshots of the first two probe passes
        self._scratch = None
        self._device = None           # device of the parameter gradients (set by the first probe)
        self.last_status = 0          # status of the last greedy allocation (0 = budget met)

    def init_from_dims(self):
        self.dims = self.quantizer.dims
        total_ele = 0
        for l in self.dims:
            self.C[l] = 1.0
            self.bits[l] = self.avg_bits
            total_ele += self.dims[l]
        self.total_bits = self.avg_bits * total_ele

    def iterate_wrapper(self, backprop):
        if self.dims is None:
            self.init_from_dims()
        self.iterate(backprop)

    # ------------------------------------------------------------------------------------------------
    # probe passes
    # ------------------------------------------------------------------------------------------------
    def _grads(self):
        return [p.grad for p in self.model.parameters() if p.grad is not None]

    def sample_grad(self):
        """All parameter gradients as one vector (a copy; only the debug / logging branches use it)."""
        return torch.cat([g.ravel() for g in self._grads()], 0)

    @staticmethod
    def _setup_seed(seed):
        random.seed(seed)
        np.random.seed(seed)
        torch.manual_seed(seed)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed)

    def _run_backprop(self, backprop):
        """One probe pass: BN running statistics frozen, every generator seeded with the iteration number so
        that the passes share their dropout masks, CPU generator state restored afterwards."""
        bn_layers = [m for m in self.model.modules() if isinstance(m, nn.modules.batchnorm._BatchNorm)]
        saved = [bn.track_running_stats for bn in bn_layers]
        for bn in bn_layers:
            bn.track_running_stats = False
        org_state = torch.get_rng_state().clone()
        self._setup_seed(self.iter)
        no_sync = getattr(self.model, "no_sync", None)
        if config.dp_probe in ("local", "shard") and _dist() is not None and no_sync is not None:
            with no_sync():
                backprop()
        else:
            backprop()
        torch.set_rng_state(org_state)
        for bn, s in zip(bn_layers, saved):
            bn.track_running_stats = s

    def get_grad(self, backprop):
        self._run_backprop(backprop)
        grad = self.sample_grad()
        self.quantizer.iterate()
        return grad

    def _snapshot(self, slot, grads):
        P = sum(g.numel() for g in grads)
        dev = grads[0].device
        flat = self._flat[slot]
        if flat is None or flat.numel() != P or flat.device != dev:
            flat = self._flat[slot] = torch.empty(P, dtype=torch.float32, device=dev)
        views, off = [], 0
        for g in grads:
            views.append(flat[off:off + g.numel()].view(g.shape))
            off += g.numel()
        torch._foreach_copy_(views, grads)
        return flat

    def _distances(self, flat0, flat1, grads, out3):
        """out3 <- (|g0-g1|^2, |g0-g2|^2, |g1-g2|^2); g2 is read in place from the live gradients."""
        dev = flat0.device
        # The three passes must have produced gradients for the same parameters (a conditionally used parameter
        # breaks that); the kernel indexes all three vectors with one length.
        if not (flat0.numel() == flat1.numel() == sum(g.numel() for g in grads)):
            raise RuntimeError("auto precision: the probe passes produced gradients of different total size "
                               "(%d, %d, %d)" % (flat0.numel(), flat1.numel(), sum(g.numel() for g in grads)))
        if self._scratch is None or self._scratch.device != dev:
            self._scratch = torch.empty(nv.lib.gact_sq_diffs3_scratch_bytes(), dtype=torch.uint8, device=dev)
        direct = all(g.dtype == torch.float32 and g.is_contiguous() for g in grads)
        with nv.device_guard(flat0):
            if direct:
                offs = np.cumsum([0] + [g.numel() for g in grads[:-1]])
                table = torch.tensor([[g.data_ptr() for g in grads], offs.tolist(), [g.numel() for g in grads]],
                                     dtype=torch.int64)
                if dev.type == 'cuda':
                    table = table.pin_memory().to(dev, non_blocking=True)
                st = nv.lib.gact_sq_diffs3(flat0.data_ptr(), flat1.data_ptr(), None, flat0.numel(),
                                           table[0].data_ptr(), table[1].data_ptr(), table[2].data_ptr(), len(grads),
                                           self._scratch.data_ptr(), out3.data_ptr(), nv.stream_ptr())
                if dev.type == 'cuda':
                    table.record_stream(torch.cuda.current_stream())
            else:
                flat2 = torch.cat([g.reshape(-1).float() for g in grads])
                st = nv.lib.gact_sq_diffs3(flat0.data_ptr(), flat1.data_ptr(), flat2.data_ptr(), flat0.numel(),
                                           None, None, None, 0, self._scratch.data_ptr(), out3.data_ptr(),
                                           nv.stream_ptr())
        nv.check(st, "gact_sq_diffs3")

    def _probe_all(self, backprop):
        q = self.quantizer
        tids = list(q.bits.keys())
        L = len(tids)
        dev = None
        d3 = None
        dist = _dist()
        W = dist.get_world_size() if dist is not None else 1
        # 'shard': every rank probes its own share of the tensors (no gradient all-reduce during the probes), so
        # the 3L extra passes are split W ways instead of being repeated on every rank
        sharded = config.dp_probe == "shard" and W > 1
        rank = dist.get_rank() if sharded else 0
        for i, l in enumerate(tids):
            if sharded and i % W != rank:
                continue
            b = q.bits[l]
            q.bits[l] = 1
            self._run_backprop(backprop)
            grads = self._grads()
            if d3 is None:
                dev = self._device = grads[0].device
                d3 = torch.zeros((L, 3), dtype=torch.float64, device=dev)
            flat0 = self._snapshot(0, grads)
            q.iterate()
            q.seeds[l] += 1
            self._run_backprop(backprop)
            flat1 = self._snapshot(1, self._grads())
            q.iterate()
            q.seeds[l] -= 1
            q.bits[l] = 8
            self._run_backprop(backprop)
            self._distances(flat0, flat1, self._grads(), d3[i])
            q.iterate()
            q.bits[l] = b
        if L == 0:
            return
        if d3 is None:                                    # a rank without a share (more ranks than tensors)
            dev = self._device = next(self.model.parameters()).device
            d3 = torch.zeros((L, 3), dtype=torch.float64, device=dev)
        # one exchange of L x 3 statistics keeps every rank's decisions identical
        scale = 1.0
        if W > 1:
            dist.all_reduce(d3, op=dist.ReduceOp.SUM)
            # 'allreduce': every rank measured the averaged gradient -> mean of identical numbers.
            # 'local': ranks measured their own gradients; the noise terms are independent across ranks, so
            # the squared distance of the averaged gradient is the sum of the local ones over W^2.
            # 'shard': one rank's local measurement stands for all W ranks' (equal in expectation), W * d / W^2.
            scale = {"local": 1.0 / (W * W), "shard": 1.0 / W}.get(config.dp_probe, 1.0 / W)
        C_dev = torch.empty(L, dtype=torch.float32, device=dev)
        with nv.device_guard(C_dev):
            st = nv.lib.gact_sensitivity(d3.data_ptr(), scale, C_dev.data_ptr(), L, nv.stream_ptr())
        nv.check(st, "gact_sensitivity")
        for l, c in zip(tids, C_dev.tolist()):            # the only host synchronisation of the probe
            self.C[l] = c
        with nv.device_guard(C_dev):
            nv.check_pipeline("auto precision probe")     # the host has just waited for the device anyway
        self._flat = [None, None]

    # ------------------------------------------------------------------------------------------------
    def iterate(self, backprop):
        if self.iter % self.adapt_interval == 0:
            dist = _dist()
            if dist is None or dist.get_rank() == 0:
                print('GACT: Initializing AutoPrec..., run extra %d iters' % (len(self.quantizer.bits)))
            self._probe_all(backprop)
            self.refresh_bits()

        if self.debug and self.iter % self.adapt_interval == 0:
            # compare the predicted quantization variance with the measured one
            grad = self.get_grad(backprop)
            for l in self.quantizer.bits:
                self.quantizer.bits[l] = 32
            det_grad = self.get_grad(backprop)         # exact gradient: 32-bit passthrough
            ap_var = ((grad - det_grad) ** 2).sum()
            C_arr = np.array([self.C[l] for l in self.C])
            b_arr = np.array([self.bits[l] for l in self.C])
            predicted_var = (C_arr * 2 ** (-2.0 * (b_arr - 1))).sum()
            print('Exact Variance %f, Predicted Variance %f' % (ap_var.item(), predicted_var.item()))
            for b in [4]:
                self.quantizer.bits = {l: b for l in self.bits}
                grad = self.get_grad(backprop)
                quant_var = ((grad - det_grad) ** 2).sum()
                predicted_var = (C_arr * 2 ** (-2.0 * (b - 1))).sum()
                print('use %d bit to compare, exact variance %f, predicted variance %f' % (
                    b, quant_var.item(), predicted_var.item()))
            self.quantizer.bits = self.bits.copy()

        if self.log_iter > 0 and self.iter % self.log_iter == 0:
            det_grad = self.get_grad(backprop)
            momentum = self.momentum
            self.beta1 = self.beta1 * momentum + 1 - momentum
            self.batch_grad = self.batch_grad * momentum + (1 - momentum) * det_grad
            bgrad = self.batch_grad / self.beta1
            gvar = ((bgrad - det_grad) ** 2).sum()
            self.grad_var = self.grad_var * momentum + (1 - momentum) * gvar
            exp_recorder.record("iter", self.iter)
            exp_recorder.record("layer sensitivity", self.C)
            exp_recorder.record("bits", self.bits)
            exp_recorder.record("dims", self.dims)
            os.makedirs(self.work_dir, exist_ok=True)
            exp_recorder.dump(self.work_dir + "autoprec.log")

        self.iter += 1

    def refresh_bits(self):
        """Greedy allocation on the device from the current sensitivities (reference: autoprec.py:188-209)."""
        l_list = list(self.dims.keys())
        L = len(l_list)
        if L == 0:
            return
        dev = self._device if self._device is not None else next(self.model.parameters()).device
        dims_dev = torch.tensor([self.dims[l] for l in l_list], dtype=torch.int64).to(dev)
        C_dev = torch.tensor([self.C[l] for l in l_list], dtype=torch.float32).to(dev)
        bits_dev = torch.full((L + 1,), self.max_bits, dtype=torch.int32, device=dev)   # [L] = status
        with nv.device_guard(bits_dev):
            st = nv.lib.gact_calc_precision(bits_dev.data_ptr(), C_dev.data_ptr(), dims_dev.data_ptr(), L,
                                            float(self.total_bits), bits_dev[L:].data_ptr(), nv.stream_ptr())
        nv.check(st, "gact_calc_precision")
        out = bits_dev.tolist()
        self.last_status = out[L]
        for i, l in enumerate(l_list):
            self.bits[l] = out[i]
        self.quantizer.bits = self.bits.copy()

        # warn when the predicted quantization variance is large against the gradient variance
        if self.log_iter > 0 and self.iter > self.warmpup_iter:
            overall_var = self.grad_var / self.beta1
            C_arr = np.array([self.C[l] for l in self.C])
            b_arr = np.array([self.bits[l] for l in self.C])
            quantization_var = (C_arr * 2 ** (-2.0 * b_arr)).sum()
            if quantization_var > overall_var * 0.1:
                print("========================================")
                print('GACT Warning: Quantization variance is too large. Consider increasing number of bits.',
                      quantization_var, overall_var)
                exp_recorder.record("iter", self.iter)
                exp_recorder.record("layer sensitivity", self.C)
                exp_recorder.record("bits", self.bits)
                exp_recorder.record("dims", self.dims)
                exp_recorder.record("warning", True)
                exp_recorder.record("quantization var", float(quantization_var))
                exp_recorder.record("overall var", float(overall_var))
                exp_recorder.dump(self.work_dir + "autoprec.log")
                print("========================================")
