"""``calc_precision(b, C, w, target) -> b`` on CPU tensors (reference binding:
gact/gact/cpp_extension/calc_precision.cc:66-122)."""
import torch

from gact import _native as nv


def calc_precision(b, C, w, target):
    """Greedy bit allocation in place: b int32[L], C float32[L], w int64[L], all contiguous CPU tensors.
    Where the reference fails an ``assert`` (budget below one bit per element) this raises RuntimeError."""
    for name, t, dt in (("b", b, torch.int32), ("C", C, torch.float32), ("w", w, torch.int64)):
        if t.is_cuda:
            raise RuntimeError(f"{name} must be a CPU tensor")
        if t.dtype != dt:
            raise RuntimeError(f"{name} must have dtype {dt}")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    L = b.numel()
    if C.numel() != L or w.numel() != L:
        raise RuntimeError("b, C and w must have the same length")
    st = nv.lib.gact_calc_precision_host(b.data_ptr(), C.data_ptr(), w.data_ptr(), L, float(target))
    nv.check(st, "gact_calc_precision_host")
    return b
