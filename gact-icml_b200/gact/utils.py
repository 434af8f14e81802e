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


_MB = float(1 << 20)


def get_memory_usage(print_info=False):
    """Bytes torch currently holds allocated on the GPU; with ``print_info`` also prints that figure and the bytes
    its caching allocator has reserved, in the two-line format the reference's drivers print
    (reference: gact/gact/utils.py:40-47)."""
    in_use = torch.cuda.memory_allocated()
    if print_info:
        for label, nbytes in (("allocated: ", in_use), ("reserved:  ", torch.cuda.memory_reserved())):
            print("%s%.2f MB" % (label, nbytes / _MB), flush=True)
    return in_use


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
    """Hand the caching allocator's unused blocks back to the driver when less than ``ratio`` of what it has
    reserved on device 0 is in use (reference: gact/gact/utils.py:72-78); ``None`` switches the check off."""
    if ratio is None:
        return
    reserved = torch.cuda.memory_reserved(0)
    if reserved > 0 and torch.cuda.memory_allocated(0) < ratio * reserved:
        torch.cuda.empty_cache()


class GlobalExpRecorder:
    """Key/value recorder whose current contents are appended to a file as one JSON line per ``dump``
    (reference: gact/gact/utils.py:80-101).  Keys stay until they are overwritten: ``clear`` does nothing, as in the
    reference, whose drivers rely on earlier keys still being there at the next dump."""

    _INT_TYPES = (np.int32, np.int64)
    _FLOAT_TYPES = (float, np.float32, np.float64)

    def __init__(self):
        self.val_dict = OrderedDict()

    def record(self, key, value, float_round=6):
        # numpy scalars are not JSON-serialisable; floats are rounded so that the log stays readable
        if isinstance(value, self._INT_TYPES):
            value = int(value)
        elif isinstance(value, self._FLOAT_TYPES):
            value = round(float(value), float_round)
        self.val_dict[key] = value

    def dump(self, filename):
        line = json.dumps(self.val_dict)
        with open(filename, "a") as fout:
            fout.write(line + "\n")
        print("Save exp results to %s" % filename)

    def clear(self):
        return None


exp_recorder = GlobalExpRecorder()
