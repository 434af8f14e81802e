"""The op contract of the compression path (reference: gact/gact/ops.py:11-69).

``op_quantize(input, q_bit, seed) -> [q_input, q_bit, q_scale, q_min]`` and
``op_dequantize([q_input, q_bit, q_scale, q_min], shape) -> Tensor`` keep the reference's return shapes
and dtypes: ``q_input`` is a 1-D int8 tensor of R*256 + 1 bytes (the reference allocates one spare byte),
``q_scale`` / ``q_min`` have shape (G, 1, 1) in the input dtype.  Unlike the reference there is no padding
copy, no separate min/max pass and no scale kernel: one fused kernel reads the tensor once.
"""
import numpy as np
import torch

from gact.conf import config
from gact import _native as nv


# number of library kernels enqueued by this module (benchmarks report it)
launch_count = 0


def _numel(shape):
    n = 1
    for s in shape:
        n *= int(s)
    return n


def quantize_pack(input, q_bit, seed, rng_mode=None, noise=None, fma=None):
    """Fused minimax + scale + stochastic rounding + packing.  Returns (q_input, q_scale, q_min)."""
    nv.require_cuda(input, "input")
    if input.dtype not in nv.DTYPE_CODE:
        raise RuntimeError("The type of input is not correct!")
    x = input if input.is_contiguous() else input.contiguous()
    n = x.numel()
    G = (n + nv.GROUP - 1) // nv.GROUP
    nbytes = nv.lib.gact_packed_bytes(n, q_bit)
    if nbytes < 0:
        raise ValueError("bits must be 1, 2, 4, 8 or 32, got %r" % (q_bit,))
    q_input = torch.empty(nbytes + 1, dtype=torch.int8, device=x.device)
    # bf16 (not a reference type) keeps its scale in fp32; q_min always carries the tensor's dtype
    q_scale = torch.empty((G, 1, 1), dtype=torch.float32 if x.dtype == torch.bfloat16 else x.dtype, device=x.device)
    q_min = torch.empty((G, 1, 1), dtype=x.dtype, device=x.device)
    mode = nv.RNG_CODE[rng_mode if rng_mode is not None else config.rng_mode]
    noise_ptr = None
    if mode == nv.RNG_EXTERNAL:
        noise = noise.to(device=x.device, dtype=torch.float32).contiguous()
        if noise.numel() != G * nv.GROUP:
            raise ValueError("noise must have G*256 elements")
        noise_ptr = noise.data_ptr()
    with nv.device_guard(x):
        st = nv.lib.gact_quantize(x.data_ptr(), nv.DTYPE_CODE[x.dtype], n, q_bit, int(seed) & 0xFFFFFFFFFFFFFFFF, mode,
                                  noise_ptr, int(config.fma if fma is None else fma), q_input.data_ptr(),
                                  q_min.data_ptr(), q_scale.data_ptr(), nv.stream_ptr())
    global launch_count
    launch_count += 1
    nv.check(st, "gact_quantize")
    return q_input, q_scale, q_min


def no_scheme_quantize_pack(input, q_bit, seed):
    """Reference: gact/gact/ops.py:11-32."""
    if q_bit == 32:
        # uncompressed passthrough used by the debug path: the payload is the zero-padded (G, 256) view
        nv.require_cuda(input, "input")
        n = input.numel()
        G = (n + config.group_size - 1) // config.group_size
        if G * config.group_size != n:
            flat = input.new_zeros(G * config.group_size)
            flat[:n] = input.reshape(-1)
        else:
            flat = input.reshape(-1)
        groups = flat.reshape(G, config.group_size)
        q_min = groups.min(dim=-1, keepdim=True).values
        q_scale = groups.max(dim=-1, keepdim=True).values - q_min
        return groups, q_scale, q_min
    return quantize_pack(input, q_bit, seed)


def dequantize_and_unpack(data, shape, q_bit, scale, mn):
    """Reference: gact/gact/ops.py:34-47.  Returns the tensor already in ``shape`` (n elements, no padding)."""
    if not isinstance(q_bit, int):
        print("bits must be intergers, now bits ", q_bit)
        assert False
    if q_bit == 32:
        return data
    nv.require_cuda(data, "data")
    n = _numel(shape)
    # the kernel derives every extent from n: refuse payloads that are shorter than that
    G = (n + nv.GROUP - 1) // nv.GROUP
    need = nv.lib.gact_packed_bytes(n, q_bit)
    if need < 0:
        raise ValueError("bits must be 1, 2, 4, 8 or 32, got %r" % (q_bit,))
    if data.numel() * data.element_size() < need or scale.numel() < G or mn.numel() < G:
        raise ValueError("compressed payload is too small for a tensor of shape %s at %d bits" % (tuple(shape), q_bit))
    out = torch.empty(tuple(int(s) for s in shape), dtype=mn.dtype, device=data.device)
    with nv.device_guard(data):
        st = nv.lib.gact_dequantize(data.data_ptr(), mn.data_ptr(), scale.data_ptr(), nv.DTYPE_CODE[mn.dtype], n, q_bit,
                                    out.data_ptr(), nv.stream_ptr())
    global launch_count
    launch_count += 1
    nv.check(st, "gact_dequantize")
    return out


def op_quantize_mask(input, flag=None):
    """1 bit per element for a 0/1 uint8 (or bool) tensor; returns [int32 words, shape]
    (reference: gact/gact/ops.py:49-50).  ``flag``: optional int32 device scalar, pre-zeroed, set to 1 by the
    kernel when some element is neither 0 nor 1."""
    nv.require_cuda(input, "input")
    if input.dtype not in (torch.uint8, torch.bool):
        raise RuntimeError("The type of data is not correct!")
    x = input.contiguous()
    n = x.numel()
    words = torch.empty(nv.lib.gact_mask_words(n), dtype=torch.int32, device=x.device)
    with nv.device_guard(x):
        st = nv.lib.gact_mask_pack(x.data_ptr(), n, words.data_ptr(), None if flag is None else flag.data_ptr(),
                                   nv.stream_ptr())
    global launch_count
    launch_count += 1
    nv.check(st, "gact_mask_pack")
    return [words, input.shape]


def op_dequantize_mask(input, dtype=torch.uint8):
    """Reference: gact/gact/ops.py:52-55."""
    q_mask, input_shape = input
    n = _numel(input_shape)
    # a partial last block of 512 elements still spreads over all of its 16 words
    if q_mask.numel() < nv.lib.gact_mask_words(n):
        raise ValueError("packed mask holds %d words, %d elements need %d" % (q_mask.numel(), n, nv.lib.gact_mask_words(n)))
    out = torch.empty(tuple(int(s) for s in input_shape), dtype=torch.uint8, device=q_mask.device)
    with nv.device_guard(q_mask):
        st = nv.lib.gact_mask_unpack(q_mask.data_ptr(), n, out.data_ptr(), nv.stream_ptr())
    global launch_count
    launch_count += 1
    nv.check(st, "gact_mask_unpack")
    return out if dtype == torch.uint8 else out.view(dtype)


def op_quantize(input, q_bit, seed):
    """Reference: gact/gact/ops.py:57-59."""
    q_input, q_scale, q_min = no_scheme_quantize_pack(input, q_bit, seed)
    return [q_input, q_bit, q_scale, q_min]


def op_dequantize(input, input_shape):
    """Reference: gact/gact/ops.py:61-69."""
    q_input, q_bit, q_scale, q_min = input
    out = dequantize_and_unpack(q_input, input_shape, q_bit, q_scale, q_min)
    if q_bit == 32:
        num_features = int(np.prod(input_shape))
        out = out.ravel()[:num_features].reshape(*input_shape).contiguous()
    return out


def minimax(data):
    """Per-row min and max of a (N, 256) tensor (reference binding: gact/gact/cpp_extension/minimax.cc:7-14)."""
    nv.require_cuda(data, "data")
    if data.dim() != 2 or data.shape[1] != nv.GROUP:
        raise RuntimeError("minimax expects rows of 256 elements")
    x = data.contiguous()
    mn = torch.empty(x.shape[0], dtype=x.dtype, device=x.device)
    mx = torch.empty_like(mn)
    with nv.device_guard(x):
        st = nv.lib.gact_minimax(x.data_ptr(), nv.DTYPE_CODE[x.dtype], x.numel(), mn.data_ptr(), mx.data_ptr(), nv.stream_ptr())
    nv.check(st, "gact_minimax")
    return mn, mx


# ---------------------------------------------------------------------------------------------------------------
# Compact payload used by the saved-tensor hooks: ONE allocation holds packed codes, per-group min and scale, and
# the library is called with offsets into it.  A training step runs hundreds of hooks, each of them a few
# microseconds of kernel time, so host overhead per call matters as much as the kernels.
# ---------------------------------------------------------------------------------------------------------------
_ELEM_SIZE = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2}
_layout_cache = {}


def _layout(n, bits, dtype):
    key = (n, bits, dtype)
    lay = _layout_cache.get(key)
    if lay is None:
        G = (n + nv.GROUP - 1) // nv.GROUP
        nbytes = nv.lib.gact_packed_bytes(n, bits)
        if nbytes < 0:
            raise ValueError("bits must be 1, 2, 4, 8 or 32, got %r" % (bits,))
        es = _ELEM_SIZE[dtype]
        ss = 4 if dtype == torch.bfloat16 else es
        off_min = (nbytes + 15) // 16 * 16
        off_scale = (off_min + G * es + 15) // 16 * 16
        lay = _layout_cache[key] = (G, nbytes, off_min, off_scale, off_scale + G * ss, nv.DTYPE_CODE[dtype])
    return lay


class Packed:
    """Compressed tensor in one buffer.  Indexing gives the reference's list view
    ``[q_input, q_bit, q_scale, q_min]`` (gact/gact/ops.py:57-59) for code that wants to look inside.
    ``strides`` is None for a contiguous source, else the strides of the dense, permuted source whose memory
    order was compressed (the reconstruction is laid out the same way)."""
    __slots__ = ("buf", "bits", "dtype", "n", "strides")

    def __init__(self, buf, bits, dtype, n, strides=None):
        self.buf, self.bits, self.dtype, self.n, self.strides = buf, bits, dtype, n, strides

    def __getitem__(self, i):
        G, nbytes, off_min, off_scale, total, _ = _layout(self.n, self.bits, self.dtype)
        if i == 0:
            return self.buf[:nbytes + 1].view(torch.int8)       # R*256 + 1 bytes, the last one unspecified, as in the reference
        if i == 1:
            return self.bits
        sdt = torch.float32 if self.dtype == torch.bfloat16 else self.dtype
        if i == 2:
            return self.buf[off_scale:total].view(sdt).reshape(G, 1, 1)
        if i == 3:
            return self.buf[off_min:off_min + G * _ELEM_SIZE[self.dtype]].view(self.dtype).reshape(G, 1, 1)
        raise IndexError(i)

    def __len__(self):
        return 4


# The native fast path of the hooks (csrc/hooks.cpp, optional) builds the same payload objects.
try:
    from gact import _hooks
    _hooks.bind(Packed)
except ImportError:
    _hooks = None


def launches():
    """Library kernels enqueued so far by this module and by the native hooks."""
    return launch_count + (_hooks.launches() if _hooks is not None else 0)


_dense_cache = {}


def _is_dense_permutation(shape, strides):
    """True when the strides describe a permutation of a contiguous block (no gaps, no overlap)."""
    key = (shape, strides)
    r = _dense_cache.get(key)
    if r is None:
        dims = sorted((st, sz) for st, sz in zip(strides, shape) if sz != 1)
        expect, r = 1, True
        for st, sz in dims:
            if st != expect:
                r = False
                break
            expect *= sz
        _dense_cache[key] = r
    return r


def quantize_compact(input, q_bit, seed):
    """Fused quantize into a single-buffer payload (the hooks' fast path).

    A non-contiguous but dense tensor (a transposed / permuted view, as attention layers save them) is compressed
    in MEMORY order, without the contiguous copy that the reference's ``reshape(-1, 256)`` makes: the groups are
    256 neighbouring elements of memory instead of 256 neighbouring elements of the logical order, and the
    reconstruction comes back with the source's strides.  ``config.keep_layout = False`` restores the copy."""
    strides = None
    if input.is_contiguous():
        x = input
    elif config.keep_layout and _is_dense_permutation(tuple(input.shape), input.stride()):
        x, strides = input, input.stride()
    else:
        x = input.contiguous()
    n = x.numel()
    G, nbytes, off_min, off_scale, total, code = _layout(n, q_bit, x.dtype)
    buf = torch.empty(total, dtype=torch.uint8, device=x.device)
    base = buf.data_ptr()
    guard, stream = nv.guard_and_stream(x)
    with guard:
        st = nv.quantize_call(x.data_ptr(), code, n, q_bit, int(seed) & 0xFFFFFFFFFFFFFFFF, nv.RNG_CODE[config.rng_mode],
                              None, int(config.fma), base, base + off_min, base + off_scale, stream)
    global launch_count
    launch_count += 1
    if st:
        nv.check(st, "gact_quantize")
    return Packed(buf, q_bit, x.dtype, n, strides)


def dequantize_compact(p, shape):
    G, nbytes, off_min, off_scale, total, code = _layout(p.n, p.bits, p.dtype)
    if p.strides is None:
        out = torch.empty(shape, dtype=p.dtype, device=p.buf.device)
    else:
        out = torch.empty_strided(shape, p.strides, dtype=p.dtype, device=p.buf.device)
    base = p.buf.data_ptr()
    guard, stream = nv.guard_and_stream(out)
    with guard:
        st = nv.dequantize_call(base, base + off_min, base + off_scale, code, p.n, p.bits, out.data_ptr(), stream)
    global launch_count
    launch_count += 1
    if st:
        nv.check(st, "gact_dequantize")
    return out
