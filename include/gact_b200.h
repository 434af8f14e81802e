/*
 * gact_b200.h -- C ABI of libgact_b200.so: GACT's saved-tensor compression path for NVIDIA B200 (sm_100a).
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes, returns an int status
 * (0 = GACT_OK, see gact_error_string) and never throws.  The caller owns every buffer.  Kernels are
 * enqueued on the stream passed in (a cudaStream_t, 0 = the legacy default stream) of the CURRENT device;
 * nothing synchronises with the host and nothing is allocated unless a comment says otherwise.
 * Calls may come from any thread (PyTorch runs the backward-side calls on its autograd worker threads).
 * Process-wide state the library does keep, all of it safe to touch from several threads:
 *   - per-device caches filled on first use: the SM count, each kernel's resident-block count and
 *     shared-memory opt-in, the device address of the gact_sq_diffs3_noalloc scratch array (none of them
 *     survives cudaDeviceReset: do not reset a device the library has been used on and then go on using it);
 *   - the sticky error word of the bulk-copy pipeline (gact_pipeline_error / gact_pipeline_error_reset);
 *   - the diagnostics knobs of gact_pipeline_test_hook;
 *   - the scratch array of gact_sq_diffs3_noalloc (documented there).
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
    GACT_RNG_FAST = 1,     /* Philox4x32 with 7 rounds, one call feeds 16 elements with 8 bits each */
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
 *   x       n elements of `dtype`, aligned to the element size.  Any contiguous tensor is accepted, as by the
 *           reference (gact/gact/cpp_extension/ext_common.h:2-27); 16-byte alignment (what an allocator returns)
 *           selects the vectorised loads, anything else - a contiguous view that starts at an odd offset of its
 *           storage - is read element by element, same result, several times slower
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
 * The fp16 / bf16 kernel of gact_quantize stages its input through shared memory with bulk copies and waits for
 * them on mbarriers.  Every such wait is bounded; a wait that runs out makes the warp record an error and leave
 * (the tiles it had not written keep whatever the output buffers held), so a launch can never spin forever.
 * gact_pipeline_error: 0 while no wait has ever run out on the current device, non-zero afterwards (sticky);
 * -1 if the word could not be read.  gact_pipeline_error_reset: clears it.  Both synchronise with the device,
 * so call them where the host waits anyway (the Python layer does so once per adaptation and when the hooks
 * are removed, and raises).  No counterpart in the reference, whose kernels never wait.
 */
int gact_pipeline_error(void);
int gact_pipeline_error_reset(void);

/*
 * Diagnostics, no counterpart in the reference.  wait_limit: polls after which a wait of the pipeline above gives
 * up (0 restores the default, 2^20).  withhold_one_copy != 0: warp 0 of block 0 leaves its first bulk copy
 * unissued, so that its wait runs out after wait_limit polls - the only way to see the give-up path work without
 * a broken GPU.  Process-wide, read at launch; meant for the test-suite.
 */
void gact_pipeline_test_hook(uint32_t wait_limit, int withhold_one_copy);

/*
 * Unpack + dequantize: out[i] = T(T(code)/scale) + min for the first n elements (bf16, not a reference type:
 * bf16(fma(code, fl32(1/scale), min)) with the fp32 qscale written by gact_quantize).
 * Replaces unpack_single_precision() (gact/gact/cpp_extension/quantization.cc:36-49,
 * quantization_cuda_kernel.cu:149-221) and the slice in gact/gact/ops.py:61-69.
 *   out     n elements of `dtype`, aligned to the element size (16-byte alignment selects vector stores);
 *           no padded tail is written
 *   packed  16-byte aligned
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
 * x: any address (16-byte alignment selects vector loads).
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
 * Fingerprint of a tensor for value-based deduplication, kept on the device: adds to out2[0] a hash of the
 * min(n, 100) evenly spaced elements i * (n div count) and to out2[1] the sum of all elements' raw bit patterns,
 * both as wrapping 64-bit integers (the caller zeroes out2 first; several tensors' fingerprints go to one table
 * and come back to the host in one copy).  Replaces the per-tensor read-backs of the reference's dedup key
 * (gact/gact/quantizer.py:85-93: uniform_sample(...).tolist() and t.sum().item(); gact/gact/utils.py:16-24).
 *   x  n elements of elem_bytes (1, 2 or 4) bytes, aligned to the element size;  out2  two uint64, 8-byte aligned
 */
int gact_fingerprint(const void* x, int elem_bytes, int64_t n, uint64_t* out2, void* stream);

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
 * (seg_ptr_host[k] is still a device pointer), copied by the call itself, in stream order (cudaMemcpyAsync),
 * into the library's table.  Tables in PAGEABLE host memory are staged by the runtime before the call returns
 * and may be reused at once; tables in PINNED host memory are read by the copy engine when the stream gets
 * there, so keep them unchanged until then (an event after the call, or any later synchronisation of the
 * stream).  Because the tables are on the host they are checked before anything is launched: the segments must
 * tile [0, P) in order (seg_off_host[0] = 0, each offset = the previous offset + length, lengths summing to P,
 * no null pointer), else GACT_ERR_SIZE / GACT_ERR_NULL.  Limit: nseg <= GACT_NOALLOC_MAX_SEGMENTS, else
 * GACT_ERR_NOALLOC_LIMIT and nothing is launched; P is not limited.  nseg = 0 selects the contiguous g2.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current) and caches it; make that first call outside of any stream capture.  The cached address belongs to the
 * device's current context: it does not survive cudaDeviceReset.  All calls on a device share the
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
