"""Per-step bookkeeping of the saved-tensor compression (reference: gact/gact/quantizer.py).

Decides which saved tensors are compressed, numbers them in forward order (``tid``), looks up their bit
width and seed, and keeps the compressed payloads in a ref-counted map until backward asks for them.
The tuples handed to autograd keep the reference's formats:
``(False, tensor)`` | ``(True, True, [mask_words, shape])`` | ``(True, False, key, shape, tid)``.
"""
import weakref

import torch

from gact.conf import config
from gact.ops import op_quantize, op_dequantize, op_quantize_mask, op_dequantize_mask
from gact import ops as _ops
from gact.ops import _hooks
from gact.utils import uniform_sample


class Quantizer:
    """
    default_bit: bits per element until auto precision decides otherwise
    swap: move compressed payloads to pinned host memory after the forward pass
    prefetch: while tensor ``tid`` is dequantized, bring tensor ``tid - 1`` back on a side stream
              (only meaningful with swap)
    """

    def __init__(self, default_bit, swap, prefetch):
        self.unrelated_tensors = set()      # data_ptr of tensors never to be compressed (parameters)
        self.default_bit = default_bit
        self.swap = swap
        if swap:
            self.swap_out_stream = torch.cuda.Stream()
            self.swap_in_stream = torch.cuda.Stream()
        self.compute_stream = torch.cuda.current_stream() if torch.cuda.is_available() else None
        self.ptr_qtensor_map = {}
        self.prefetch = prefetch
        if prefetch:
            self.start_prefetch_event = torch.cuda.Event(blocking=True)
            self.end_prefetch_event = torch.cuda.Event(blocking=True)
        self.layer_key_map = {}
        self.tid = 0
        self.tids_registered = 0    # tids handed out during iteration 0, shared payloads included
        self.start_bwd = True
        # collected for auto precision
        self.seeds = {}
        self.bits = {}
        self.dims = {}
        self.iter = 0        # iterations seen, the extra probe passes of auto precision included
        self.seed_iter = 0   # seed component shared by all passes of one optimizer step
        # added to every seed so that data-parallel ranks draw independent noise (0 on a single process)
        self.seed_offset = 0
        self._mask_flag = None
        # tensors compressed in this forward pass, by object identity: id -> (weak reference, version, key)
        self._live = {}
        # config.check_dup: saves of this step by (address, dtype, shape, strides), merges made, device fingerprints
        self._live_ptr, self._merged, self._fp_meta = {}, [], {}
        self._fp_table = None
        self.dup_report = {"merged": 0, "missed": 0}

    def filter_tensors(self, pairs):
        for _, v in pairs:
            self.unrelated_tensors.add(v.data_ptr())

    @staticmethod
    def _on_device(t):
        """Only tensors that live on a GPU are compressed; anything else passes through untouched."""
        return t.is_cuda

    # returns (should_be_quantized, is_dropout_mask)
    def check_quantize(self, input_tensor):
        # parameters are not compressed
        if input_tensor.layout != torch.strided:            # sparse tensors are left alone
            return False, False
        if input_tensor.data_ptr() in self.unrelated_tensors:
            return False, False
        # 0/1 byte tensors (dropout masks) take the 1-bit path
        if input_tensor.numel() > 0:
            if input_tensor.dtype == torch.bool and config.pack_bool_masks:
                return self._on_device(input_tensor), True
            if input_tensor.dtype == torch.uint8:
                # decided after packing, from the flag the pack kernel raises (see quantize)
                return self._on_device(input_tensor), True
        dtypes = (torch.float32, torch.float16, torch.bfloat16) if config.quantize_bf16 \
            else (torch.float32, torch.float16)
        if input_tensor.dtype not in dtypes:
            return False, False
        # only activations that take part in the gradient (e.g. not BN running statistics)
        if input_tensor.requires_grad is False:
            return False, False
        # 2-D, 3-D and 4-D tensors only, as in the reference
        if input_tensor.dim() not in (2, 3, 4):
            return False, False
        if not self._on_device(input_tensor):
            return False, False
        return True, False

    def __del__(self):
        self.ptr_qtensor_map = None
        self.layer_key_map = None
        self.unrelated_tensors = None

    def iterate(self):
        if self._fp_meta:
            self._check_fingerprints()
        self._live_ptr, self._merged, self._fp_meta = {}, [], {}
        self.ptr_qtensor_map = {}
        self.layer_key_map = {}
        self._live = {}
        self.tid = 0
        self.start_bwd = True
        self.iter += 1

    def generate_tensor_key(self, t, tid):
        """Key under which the payload of this save is stored; equal keys share one payload.

        The reference (config.check_dup) builds the key from the data pointer, 100 evenly spaced values and the sum
        of the tensor, reading both back to the host: a synchronisation per saved tensor.  Two saves can only get
        the same key there if they sit at the same address, so for tensors on the GPU the same merges are decided
        here without reading anything back: an earlier save of this step at the same address, with the same
        dtype, shape and strides, whose tensor is still alive (so the address cannot have been reused) and whose
        version counter has not moved (so the bytes cannot have changed) holds the same values.  The value
        fingerprint itself is still taken - by a kernel, into a device table - and all fingerprints of a step come
        back in ONE copy at iterate(), where every merge is verified and saves that had equal fingerprints but
        could not be proven equal on the host are counted (dup_report)."""
        if config.check_dup:
            if not t.is_cuda:
                # host tensors: nothing to synchronise with; the reference's key as it is
                sample_cnt = min(100, t.numel())
                key = uniform_sample(t, sample_cnt, add_dataptr=True)
                key.append(t.sum().item())
                return tuple(key)
            ident = (t.data_ptr(), t.dtype, tuple(t.shape), t.stride())
            self._fingerprint(t, tid, ident)
            seen = self._live_ptr.get(ident)
            if seen is not None and seen[0]() is not None and seen[1] == t._version and seen[2] in self.ptr_qtensor_map:
                self._merged.append((tid, seen[2]))
                return seen[2]
            self._live_ptr[ident] = (weakref.ref(t), t._version, tid)
            return tid
        return tid

    def _fingerprint(self, t, tid, ident):
        """Enqueue the fingerprint of save `tid` into row `tid` of the device table (no read-back here)."""
        from gact import _native as nv
        if self._fp_table is None or self._fp_table.device != t.device or tid >= self._fp_table.shape[0]:
            rows = max(1024, 2 * (tid + 1))
            new = torch.zeros((rows, 2), dtype=torch.int64, device=t.device)
            if self._fp_table is not None and self._fp_table.device == t.device:
                new[:self._fp_table.shape[0]] = self._fp_table
            self._fp_table = new
        x = t if t.is_contiguous() else t.contiguous()
        with nv.device_guard(x):
            st = nv.lib.gact_fingerprint(x.data_ptr(), x.element_size(), x.numel(), self._fp_table[tid].data_ptr(), nv.stream_ptr())
        nv.check(st, "gact_fingerprint")
        self._fp_meta[tid] = ident

    def _check_fingerprints(self):
        """One read-back for the whole step: every merge made on the strength of address + version must also agree
        in value, and saves with equal address and fingerprint that were kept apart are counted."""
        meta, merges = self._fp_meta, self._merged
        self._fp_meta, self._merged = {}, []                    # a failed check is reported once
        if not meta:
            return
        n = max(meta) + 1
        rows = self._fp_table[:n].tolist()                      # the step's only synchronisation for deduplication
        self._fp_table.zero_()
        for tid, first in merges:
            if rows[tid] != rows[first]:
                raise RuntimeError("check_dup: saves %d and %d shared a payload but their values differ "
                                   "(a tensor was modified without its version counter moving)" % (first, tid))
        groups = {}
        for tid, ident in meta.items():
            groups.setdefault((ident, tuple(rows[tid])), []).append(tid)
        merged = {t for t, _ in merges}
        missed = sum(len([t for t in g[1:] if t not in merged]) for g in groups.values())
        self.dup_report = {"merged": len(merges), "missed": missed}

    def _quantize_mask(self, input):
        if input.dtype == torch.bool:
            return True, True, op_quantize_mask(input) + [torch.bool]
        # uint8: the reference compresses only tensors whose max is 1 and min is 0, found with two
        # synchronising reductions; here the pack kernel reports non-binary content through a flag and the
        # tensor is kept as it is in that case.  One small read-back instead of two reductions.
        if self._mask_flag is None or self._mask_flag.device != input.device:
            self._mask_flag = torch.zeros(1, dtype=torch.int32, device=input.device)
        q_inputs = op_quantize_mask(input, flag=self._mask_flag)
        if int(self._mask_flag.item()) != 0:
            self._mask_flag.zero_()
            return False, input
        return True, True, q_inputs

    def quantize(self, input):
        # The plain case (a floating-point activation, no swapping, no value fingerprints) is handled by the native
        # module when it is there; it answers NotImplemented, before changing anything, for everything else.
        if _hooks is not None and config.native_hooks:
            r = _hooks.quantize(self, config, input)
            if r is not NotImplemented:
                return r
        # Same decisions as check_quantize, cheapest tests first: this runs for every saved tensor of every step.
        dt = input.dtype
        if dt is torch.float32 or dt is torch.float16 or (dt is torch.bfloat16 and config.quantize_bf16):
            if (not input.requires_grad) or input.layout is not torch.strided or not (2 <= input.dim() <= 4) \
                    or not self._on_device(input) or input.data_ptr() in self.unrelated_tensors:
                return False, input
            is_dropout_mask = False
        else:
            quantize, is_dropout_mask = self.check_quantize(input)
            if not quantize:
                return False, input
            if is_dropout_mask:
                return self._quantize_mask(input)

        tid = self.tid
        self.tid += 1
        if self.iter == 0:
            self.tids_registered = self.tid
        input_shape = input.shape

        # The same tensor object saved again, unmodified (e.g. one activation feeding three linear layers): share
        # the payload of its first save.  Identity + version counter decide it, so nothing is read back from the
        # device (the reference's check_dup fingerprints the values and synchronises for it).
        seen = self._live.get(id(input)) if config.dedup_saved else None
        if seen is not None and seen[0]() is input and seen[1] == input._version and seen[2] in self.ptr_qtensor_map:
            key = seen[2]
        else:
            key = self.generate_tensor_key(input, tid)
            if config.dedup_saved:
                self._live[id(input)] = (weakref.ref(input), input._version, key)
        self.layer_key_map[tid] = key
        entry = self.ptr_qtensor_map.get(key)
        if entry is None:
            if self.iter == 0:
                bit = self.default_bit
                self.bits[tid] = bit
                self.dims[tid] = input.numel()
                self.seeds[tid] = tid
            else:
                bit = self.bits.get(tid)
                if bit is None:
                    # A tid that shared another save's payload while the widths were registered (iteration 0) has
                    # no entry of its own; should a later step save it on its own after all, it takes the default
                    # width.  A tid iteration 0 never saw is an error, as in the reference (static graph).
                    if tid >= self.tids_registered:
                        raise KeyError(tid)
                    bit = self.default_bit
            seed = self.seeds.get(tid, tid) + self.seed_iter + self.seed_offset
            if bit == 32:
                q_inputs = op_quantize(input, bit, seed)
            else:
                q_inputs = _ops.quantize_compact(input, bit, seed)
            if self.swap:
                self._swap_out(q_inputs)
            self.ptr_qtensor_map[key] = [q_inputs, 1, tid]
        else:
            entry[1] += 1       # same tensor saved again: share the payload
        return True, is_dropout_mask, key, input_shape, tid

    @staticmethod
    def _payload(q):
        return q.buf if type(q) is _ops.Packed else q[0]

    @staticmethod
    def _set_payload(q, t):
        if type(q) is _ops.Packed:
            q.buf = t
        else:
            q[0] = t

    def _swap_out(self, q_inputs):
        # device -> pinned host copy of the packed bytes on the side stream, ordered after the kernel that
        # produced them; the device buffer is handed back to the allocator once the copy has been queued.
        q_gpu = self._payload(q_inputs)
        self.swap_out_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.swap_out_stream):
            q_cpu = torch.empty(q_gpu.shape, dtype=q_gpu.dtype, device="cpu", pin_memory=True)
            q_cpu.copy_(q_gpu, non_blocking=True)
        q_gpu.record_stream(self.swap_out_stream)
        self._set_payload(q_inputs, q_cpu)

    def dequantize(self, input):
        if _hooks is not None and config.native_hooks:
            r = _hooks.dequantize(self, input)
            if r is not NotImplemented:
                return r
        quantized = input[0]
        if not quantized:
            return input[1]
        is_dropout_mask = input[1]
        if is_dropout_mask:
            q_inputs = input[2]
            if len(q_inputs) == 3:
                return op_dequantize_mask(q_inputs[:2], dtype=q_inputs[2])
            return op_dequantize_mask(q_inputs)

        _, _, key, input_shape, tid = input
        q_inputs, ref_cnt, key_tid = self.ptr_qtensor_map[key]

        if self.swap:
            cur = torch.cuda.current_stream()
            if self.start_bwd:
                cur.wait_stream(self.swap_out_stream)      # all swap-outs of the forward pass have landed
                self.start_bwd = False
            if self.prefetch:
                cur.wait_stream(self.swap_in_stream)       # a prefetch of this tensor may be in flight
            if not self._payload(q_inputs).is_cuda:
                self._set_payload(q_inputs, self._payload(q_inputs).cuda(non_blocking=True))
            if self.prefetch and tid > 0:
                previous_key = self.layer_key_map.get(tid - 1)
                prev = self.ptr_qtensor_map.get(previous_key) if previous_key is not None else None
                if prev is not None and not self._payload(prev[0]).is_cuda:
                    self.swap_in_stream.wait_stream(cur)
                    with torch.cuda.stream(self.swap_in_stream):
                        self._set_payload(prev[0], self._payload(prev[0]).cuda(non_blocking=True))
                    self._payload(prev[0]).record_stream(cur)

        if type(q_inputs) is _ops.Packed:
            ret = _ops.dequantize_compact(q_inputs, input_shape)
        else:
            ret = op_dequantize(q_inputs, input_shape)

        ref_cnt -= 1
        if ref_cnt < 0:
            raise RuntimeError("[Error] Ref count < 0 %s %d" % (str(key), ref_cnt))
        elif ref_cnt == 0:
            del self.ptr_qtensor_map[key]
        else:
            self.ptr_qtensor_map[key] = [q_inputs, ref_cnt, key_tid]
        return ret
