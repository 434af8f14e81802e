"""``minimax(data) -> (min, max)`` (reference binding: gact/gact/cpp_extension/minimax.cc:7-14)."""
import torch

from gact import _native as nv

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def minimax(data):
    """Per-row minimum and maximum of a contiguous CUDA tensor of shape (N, 256)."""
    nv.require_cuda(data, "data")
    if not data.is_contiguous():
        raise RuntimeError("data must be contiguous")
    if data.dim() != 2 or data.shape[1] != 256:
        raise ValueError("minimax expects a (N, 256) tensor")
    if data.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {data.dtype}")
    n_rows = data.shape[0]
    mn = torch.empty(n_rows, dtype=data.dtype, device=data.device)
    mx = torch.empty(n_rows, dtype=data.dtype, device=data.device)
    with nv.device_guard(data):
        st = nv.lib.gact_minimax(data.data_ptr(), _DTYPES[data.dtype], data.numel(), mn.data_ptr(), mx.data_ptr(),
                                 nv.stream_ptr())
    nv.check(st, "gact_minimax")
    return mn, mx
