/*
 * gact_b200.h -- C ABI of libgact_b200.so: GACT's saved-tensor compression path for NVIDIA B200 (sm_100a).
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes, returns an int status
 * (0 = GACT_OK, see gact_error_string) and never throws.  The caller owns every buffer.  Kernels are
 * enqueued on the stream passed in (a cudaStream_t, 0 = the legacy default stream) of the CURRENT device;
 * nothing synchronises with the host and nothing is allocated unless a comment says otherwise.
 * The library keeps no mutable global state (the one exception is documented at gact_sq_diffs3_noalloc), so
 * calls may come from any thread (PyTorch runs the backward-side calls on its autograd worker threads).
 *
 * Each declaration names the interface of the reference implementation (paths inside the GACT
 * repository) that it replaces.
 *
 * Layout shared by quantize and dequantize.  A tensor of n elements is cut into G = ceil(n/256) groups of
 * 256 consecutive elements; elements past n count as zeros (gact/gact/ops.py:12-19) and are never read.
 * With b bits per code, wpt = 8/b groups share one row-block of 256 bytes: byte r*256 + d holds element d
 * of groups r*wpt .. r*wpt+wpt-1, group r*wpt+i in bits [i*b, i*b+b).  R = ceil(G/wpt) row-blocks.
 */
#ifndef GACT_B200_H
#define GACT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GACT_GROUP_SIZE 256

/* element types */
enum { GACT_F32 = 0, GACT_F16 = 1, GACT_BF16 = 2 };

/* where the rounding noise comes from */
enum {
    GACT_RNG_CURAND = 0,   /* the reference's stream: curand_init(seed, byte index, 0) + curand_uniform per slot */
    GACT_RNG_FAST = 1,     /* Philox4x32-10 as well, but one call feeds 16 elements with 8 bits each */
    GACT_RNG_RTN = 2,      /* noise = 0.5 everywhere: round to nearest */
    GACT_RNG_EXTERNAL = 3  /* noise read from a caller-supplied fp32 array (G*256 values in [0,1]) */
};

/* status codes */
enum {
    GACT_OK = 0,
    GACT_ERR_BITS = 1,       /* bits not in {1,2,4,8} */
    GACT_ERR_DTYPE = 2,      /* unknown element type */
    GACT_ERR_NULL = 3,       /* a required pointer is null */
    GACT_ERR_ALIGN = 4,      /* a base pointer is not aligned as documented */
    GACT_ERR_SIZE = 5,       /* negative or unsupported size */
    GACT_ERR_MODE = 6,       /* unknown rng mode / missing noise array */
    GACT_ERR_LAUNCH = 7,     /* the CUDA runtime refused the launch (cudaGetLastError) */
    GACT_ERR_BUDGET = 8,     /* greedy allocation: budget cannot be met even at 1 bit everywhere */
    GACT_ERR_NOALLOC_LIMIT = 9 /* gact_sq_diffs3_noalloc: more segments than GACT_NOALLOC_MAX_SEGMENTS */
};

int gact_version(void);
const char* gact_error_string(int status);

/* Number of bytes of packed codes for n elements at `bits` bits (R*256), or -1 for invalid bits. */
int64_t gact_packed_bytes(int64_t n, int bits);

/*
 * Fused per-group min/max + scale + stochastic rounding + bit packing, one pass over x.
 * Replaces minimax() (gact/gact/cpp_extension/minimax.cc:7-10, minimax_cuda_kernel.cu:23-89) followed by
 * pack_single_precision() (gact/gact/cpp_extension/quantization.cc:51-61,
 * quantization_cuda_kernel.cu:23-146) as called from gact/gact/ops.py:11-32.
 *   x       n elements of `dtype`, 16-byte aligned
 *   packed  R*256 bytes (gact_packed_bytes), 16-byte aligned
 *   qmin    G elements of `dtype`
 *   qscale  G elements of `dtype`; for GACT_BF16 (a type the reference does not compress) G floats: bf16
 *           inputs run the fp32 arithmetic on widened values, keep an fp32 scale and clamp codes at 2^bits-1
 *   seed    the reference passes seeds[tid] + seed_iter (gact/gact/quantizer.py:123-124)
 *   noise   GACT_RNG_EXTERNAL only: G*256 floats indexed like the zero-padded input; else ignored
 *   fma_mode  fp32 only: 1 = (x-min)*scale+noise as one fused multiply-add (what nvcc's default makes of
 *             the reference expression), 0 = product rounded first
 */
int gact_quantize(const void* x, int dtype, int64_t n, int bits, uint64_t seed, int rng_mode,
                  const float* noise, int fma_mode, void* packed, void* qmin, void* qscale, void* stream);

/*
 * 0 while every bounded wait inside the bulk-copy pipeline of gact_quantize has been satisfied; non-zero once a
 * wait ran out (the kernel then winds down instead of spinning).  Synchronises with the device; for tests and
 * diagnostics.  -1 if the value could not be read.
 */
int gact_pipeline_error(void);

/*
 * Tuning knob without a reference counterpart: gact_quantize runs 16-bit inputs with generated noise through
 * its bulk-copy ring kernel when the tensor holds at least `min_chunks` whole 32 KB chunks (default 1536, i.e.
 * 48 MB), and through the direct-load kernel otherwise; both give the same bytes.  Returns the previous value;
 * min_chunks < 1 only reads it.  Process-wide; tests lower it to push small cases through the ring.
 */
int64_t gact_set_ring_min_chunks(int64_t min_chunks);

/*
 * Unpack + dequantize: out[i] = T(T(code)/scale) + min for the first n elements (bf16, not a reference type:
 * bf16(fma(code, fl32(1/scale), min)) with the fp32 qscale written by gact_quantize).
 * Replaces unpack_single_precision() (gact/gact/cpp_extension/quantization.cc:36-49,
 * quantization_cuda_kernel.cu:149-221) and the slice in gact/gact/ops.py:61-69.
 *   out     n elements of `dtype`, 16-byte aligned (no padded tail is written)
 */
int gact_dequantize(const void* packed, const void* qmin, const void* qscale, int dtype, int64_t n,
                    int bits, void* out, void* stream);

/*
 * Per-group min and max only (G values each, in `dtype`).
 * Replaces minimax() (gact/gact/cpp_extension/minimax.cc:7-14).
 */
int gact_minimax(const void* x, int dtype, int64_t n, void* mn, void* mx, void* stream);

/*
 * 1-bit packing of a 0/1 byte tensor (uint8 or bool dropout mask): element e goes to bit (t/16) of word
 * (e/512)*16 + t%16, t = e%512.  words: gact_mask_words(n) = ceil(n/512)*16 uint32 (a partial last block
 * still uses all of its 16 words; the reference allocates ceil(n/32) and runs past it), 4-byte aligned;
 * x: 16-byte aligned.
 * Replaces act_quantize_dropout_mask() (gact/gact/cpp_extension/quantization.cc:26-29,
 * quantization_cuda_kernel.cu:229-274), without its out-of-bounds tail write.
 * not_binary (optional device int, caller zeroes it): set to 1 when some byte is neither 0 nor 1; this
 * replaces the two synchronising reductions of gact/gact/quantizer.py:52-55.
 */
int64_t gact_mask_words(int64_t n);
int gact_mask_pack(const uint8_t* x, int64_t n, uint32_t* words, int* not_binary, void* stream);

/*
 * Inverse of gact_mask_pack: n bytes of 0/1.
 * Replaces act_dequantize_dropout_mask() (gact/gact/cpp_extension/quantization.cc:31-33,
 * quantization_cuda_kernel.cu:276-303).
 */
int gact_mask_unpack(const uint32_t* words, int64_t n, uint8_t* out, void* stream);

/*
 * The three squared distances of the sensitivity probe, out3 = { |g0-g1|^2, |g0-g2|^2, |g1-g2|^2 } in
 * double.  Replaces the three `((ga - gb) ** 2).sum()` of gact/gact/autoprec.py:116-118.
 *   g0, g1  P floats each (contiguous snapshots)
 *   g2      either P contiguous floats (nseg = 0) or nseg segments: seg_ptr[k] points at seg_len[k] floats
 *           (the live .grad tensors, in parameter order); seg_off[k] is the segment's offset in g0 / g1
 *   scratch gact_sq_diffs3_scratch_bytes() bytes of device memory, 16-byte aligned, owned by the caller;
 *           calls that overlap on the GPU must not share it
 * Deterministic: block partials are combined in a fixed order.
 */
int64_t gact_sq_diffs3_scratch_bytes(void);
int gact_sq_diffs3(const float* g0, const float* g1, const float* g2, int64_t P,
                   const float* const* seg_ptr, const int64_t* seg_off, const int64_t* seg_len, int nseg,
                   void* scratch, double* out3, void* stream);

/*
 * gact_sq_diffs3 for callers that cannot allocate device memory.  (No counterpart in the reference, which
 * concatenates the gradients and lets PyTorch allocate every temporary.)
 *
 * Some callers only hold the pointers they were handed: code inside a section where the device allocator
 * must stay untouched (cudaMalloc synchronises the whole device, which a latency-bound loop cannot afford), or
 * a binding from a host language that has no device allocator to ask.  For them the scratch of
 * gact_sq_diffs3 - the block partials and the segment table - sits in a fixed array inside the library image,
 * about 62 KB that every GPU using the library holds until the process exits.  This entry point calls no
 * cudaMalloc / cudaFree and no allocating library routine.
 *
 * Differences from gact_sq_diffs3: no `scratch` argument; the three segment tables are HOST arrays
 * (seg_ptr_host[k] is still a device pointer), copied by the call itself, in stream order, into the library's
 * table, so they may be reused as soon as the call returns.  Limit: nseg <= GACT_NOALLOC_MAX_SEGMENTS, else
 * GACT_ERR_NOALLOC_LIMIT and nothing is launched; P is not limited.  nseg = 0 selects the contiguous g2.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current) and caches it; make that first call outside of any stream capture.  All calls on a device share the
 * one array, which simply keeps what the last call left in it; nothing in it has to start at zero, because
 * every call rewrites the partials and the table entries it reads before reading them.  For the same reason
 * two calls that overlap on the GPU (different streams, or different threads on different streams) race on it:
 * issue them on one stream, or order them with events.
 */
#define GACT_NOALLOC_MAX_SEGMENTS 2048
int gact_sq_diffs3_noalloc(const float* g0, const float* g1, const float* g2, int64_t P,
                           const float* const* seg_ptr_host, const int64_t* seg_off_host,
                           const int64_t* seg_len_host, int nseg, double* out3, void* stream);

/*
 * Sensitivities from the distances, on the device, for L tensors at once: with (d01, d02, d12) =
 * scale * d3[3*l .. 3*l+2] rounded to float, C[l] = max(d01, 2*max(d02, d12)), and NaN / inf / > 1e10
 * -> 1e10 (gact/gact/autoprec.py:119-126).  `scale` folds the data-parallel averaging of the statistics.
 */
int gact_sensitivity(const double* d3, double scale, float* C, int L, void* stream);

/*
 * Greedy bit allocation on the device (one thread block): starting from b[i], repeatedly lower the tensor
 * with the largest key to the next width (32->8->4->2->1) until sum(b[i]*w[i]) <= target.
 * Replaces calc_precision() (gact/gact/cpp_extension/calc_precision.cc:66-118), including its tie-break
 * (equal keys: larger index first).  b: int32[L] in/out, C: float[L], w: int64[L], all device memory.
 * status (device int): GACT_OK or GACT_ERR_BUDGET, where the reference only asserts.
 */
int gact_calc_precision(int32_t* b, const float* C, const int64_t* w, int L, double target, int* status,
                        void* stream);

/*
 * The same allocation on host arrays (no GPU involved), for callers that keep b, C and w in host memory as
 * the reference's calc_precision() does (calc_precision.cc:66 takes CPU tensors).  Returns GACT_OK or
 * GACT_ERR_BUDGET.
 */
int gact_calc_precision_host(int32_t* b, const float* C, const int64_t* w, int L, double target);

#ifdef __cplusplus
}
#endif
#endif /* GACT_B200_H */
