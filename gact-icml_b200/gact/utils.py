"""Small helpers the reference's training scripts import (reference: gact/gact/utils.py)."""
from collections import OrderedDict
import json

import numpy as np
import torch


def uniform_sample_ref(input, sample_cnt, add_dataptr=True):
    """Element-by-element version of ``uniform_sample`` (reference: gact/gact/utils.py:6-14)."""
    step = max(torch.numel(input) // sample_cnt, 1)
    key = [input.data_ptr()] if add_dataptr else []
    flat = input.view(-1)
    for i in range(min(sample_cnt, torch.numel(input))):
        key.append(flat[i * step].item())
    return key


def uniform_sample(input, sample_cnt, add_dataptr=True):
    """``sample_cnt`` evenly spaced values (plus the data pointer) as a hashable fingerprint
    (reference: gact/gact/utils.py:16-24).  One gather, one device-to-host copy."""
    num_elem = input.numel()
    sample_cnt = min(num_elem, sample_cnt)
    key = [input.data_ptr()] if add_dataptr else []
    idx = torch.arange(0, sample_cnt, device=input.device, dtype=torch.long) * (num_elem // sample_cnt)
    key += input.reshape(-1)[idx].tolist()
    return key


def random_sample(input, sample_cnt, add_dataptr=True):
    """Fingerprint from pseudo-random positions; the CPU generator state is preserved
    (reference: gact/gact/utils.py:26-38)."""
    num_elem = input.numel()
    rng_state = torch.get_rng_state()
    torch.manual_seed(input.dim())
    key = [input.data_ptr()] if add_dataptr else []
    key += input.reshape(-1)[torch.randint(0, num_elem, (sample_cnt,)).to(input.device)].tolist()
    torch.set_rng_state(rng_state)
    return key


def get_memory_usage(print_info=False):
    """Bytes currently allocated by torch on the GPU (reference: gact/gact/utils.py:40-47)."""
    allocated = torch.cuda.memory_allocated()
    reserved = torch.cuda.memory_reserved()
    if print_info:
        print("allocated: %.2f MB" % (allocated / 1024 / 1024), flush=True)
        print("reserved:  %.2f MB" % (reserved / 1024 / 1024), flush=True)
    return allocated


_ITEMSIZE = {
    torch.long: 8, torch.float64: 8,
    torch.float32: 4, torch.int: 4,
    torch.bfloat16: 2, torch.float16: 2, torch.int16: 2,
    torch.int8: 1, torch.uint8: 1, torch.bool: 1,
}


def compute_tensor_bytes(tensors):
    """Bytes held by a tensor or a list of tensors / ints (reference: gact/gact/utils.py:49-70)."""
    if not isinstance(tensors, (list, tuple)):
        tensors = [tensors]
    total = 0
    for x in tensors:
        if type(x) == int:
            total += 4
        elif x.dtype in _ITEMSIZE:
            total += int(np.prod(x.size())) * _ITEMSIZE[x.dtype]
        else:
            raise TypeError("[Error] unsupport datatype %s" % x.dtype)
    return total


def empty_cache(ratio):
    if ratio is None:
        return
    allocated = torch.cuda.memory_allocated(0)
    reserved = torch.cuda.memory_reserved(0)
    if reserved > 0 and allocated / reserved < ratio:
        torch.cuda.empty_cache()


class GlobalExpRecorder:
    """Key/value recorder appended to a JSON-lines file (reference: gact/gact/utils.py:80-101)."""

    def __init__(self):
        self.val_dict = OrderedDict()

    def record(self, key, value, float_round=6):
        if isinstance(value, (np.int32, np.int64)):
            value = int(value)
        if isinstance(value, (float, np.float32, np.float64)):
            value = round(float(value), float_round)
        self.val_dict[key] = value

    def dump(self, filename):
        with open(filename, "a") as fout:
            fout.write(json.dumps(self.val_dict) + '\n')
        print("Save exp results to %s" % filename)

    def clear(self):
        pass


exp_recorder = GlobalExpRecorder()
