"""``pack_single_precision`` / ``unpack_single_precision`` / dropout-mask packing with the signatures of the
reference binding (gact/gact/cpp_extension/quantization.cc:26-61)."""
import torch

from gact import _native as nv

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_CURAND = 0


def _check(t, name):
    nv.require_cuda(t, name)
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def pack_single_precision(data, mn, mx, bits, stochastic, seed):
    """data (N, 1, 256), mn / mx (N, 1, 1) as ``minimax`` returned them -> (packed int8[R*256 + 1], scale (N, 1, 1)).

    The library finds the group extrema itself while it reads the data, so ``mn`` and ``mx`` are only checked
    for shape: they must be the extrema of ``data`` (they are at the reference's one call site, ops.py:26-31).
    ``stochastic`` is ignored, as in the reference (quantization_cuda_kernel.cu:80-146 never reads it)."""
    _check(data, "data")
    _check(mn, "min")
    _check(mx, "max")
    if data.dim() != 3 or data.shape[1] != 1 or data.shape[2] != 256:
        raise ValueError("pack_single_precision expects data of shape (N, 1, 256)")
    if data.dtype not in (torch.float32, torch.float16):
        raise ValueError(f"unsupported dtype {data.dtype}")
    if bits not in (1, 2, 4, 8):
        raise ValueError("bits must be 1, 2, 4 or 8")
    G = data.shape[0]
    if mn.numel() != G or mx.numel() != G:
        raise ValueError("min / max must hold one value per group")
    n = data.numel()
    nbytes = nv.lib.gact_packed_bytes(n, bits)
    packed = torch.empty(nbytes + 1, dtype=torch.int8, device=data.device)
    scale = torch.empty((G, 1, 1), dtype=data.dtype, device=data.device)
    qmin = torch.empty(G, dtype=data.dtype, device=data.device)
    with nv.device_guard(data):
        st = nv.lib.gact_quantize(data.data_ptr(), _DTYPES[data.dtype], n, bits, int(seed) & (2**64 - 1), _CURAND, None, 1,
                                  packed.data_ptr(), qmin.data_ptr(), scale.data_ptr(), nv.stream_ptr())
    nv.check(st, "gact_quantize")
    return packed, scale


def unpack_single_precision(data, bits, scale, mn, N, num_groups, group_size):
    """-> tensor (N, num_groups, group_size) in scale.dtype; num_groups must be 1 and group_size 256 (the only
    values the reference passes, ops.py:41-46)."""
    _check(data, "data")
    _check(scale, "scale")
    _check(mn, "min")
    if num_groups != 1 or group_size != 256:
        raise ValueError("only num_groups = 1 and group_size = 256 are supported")
    if bits not in (1, 2, 4, 8):
        raise ValueError("bits must be 1, 2, 4 or 8")
    n = int(N) * 256
    # every extent the kernel reads follows from N: refuse tensors that are shorter than that
    if data.numel() * data.element_size() < nv.lib.gact_packed_bytes(n, bits) or scale.numel() < int(N) or mn.numel() < int(N):
        raise ValueError("data / scale / min are too small for N = %d groups at %d bits" % (int(N), bits))
    if mn.dtype != scale.dtype:
        raise ValueError("scale and min must have the same dtype")
    out = torch.empty((int(N), 1, 256), dtype=scale.dtype, device=data.device)
    with nv.device_guard(data):
        st = nv.lib.gact_dequantize(data.data_ptr(), mn.data_ptr(), scale.data_ptr(), _DTYPES[scale.dtype], n, bits,
                                    out.data_ptr(), nv.stream_ptr())
    nv.check(st, "gact_dequantize")
    return out


def act_quantize_dropout_mask(data):
    """uint8 0/1 tensor -> int32 words, bit t/16 of word blk*16 + t%16 for element blk*512 + t."""
    _check(data, "data")
    if data.dtype not in (torch.uint8, torch.bool):
        raise ValueError("the mask must be uint8 or bool")
    n = data.numel()
    words = torch.empty(nv.lib.gact_mask_words(n), dtype=torch.int32, device=data.device)
    with nv.device_guard(data):
        st = nv.lib.gact_mask_pack(data.data_ptr(), n, words.data_ptr(), None, nv.stream_ptr())
    nv.check(st, "gact_mask_pack")
    return words


def act_dequantize_dropout_mask(mask, N):
    _check(mask, "mask")
    n = int(N)
    # a partial last block of 512 elements spreads over all of its 16 words: a mask of ceil(n/32) words, as the
    # reference allocates, is too short unless n is a multiple of 512
    if mask.numel() < nv.lib.gact_mask_words(n):
        raise ValueError("mask holds %d words, N = %d needs %d" % (mask.numel(), n, nv.lib.gact_mask_words(n)))
    out = torch.empty(n, dtype=torch.uint8, device=mask.device)
    with nv.device_guard(mask):
        st = nv.lib.gact_mask_unpack(mask.data_ptr(), n, out.data_ptr(), nv.stream_ptr())
    nv.check(st, "gact_mask_unpack")
    return out
