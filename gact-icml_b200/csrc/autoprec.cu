// Device side of the auto-precision controller: squared distances between gradient vectors, the
// sensitivity clamp, and the greedy bit allocation.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include "gact_common.cuh"

namespace gact {

// ---------------------------------------------------------------------------------------------------
// Squared distances.  Stage 1: a fixed grid, each block leaves three double partials in scratch.
// Stage 2: one block adds the partials in a fixed order.  No atomics, so the result is reproducible.
// ---------------------------------------------------------------------------------------------------
constexpr int kSThreads = 256;
constexpr int kSBlocks = 592;             // fixed reduction grid (4 blocks for each of a B200's 148 SMs): it sizes the scratch

__device__ __forceinline__ void block_sum3(double& a, double& b, double& c, double* out3) {
    __shared__ double sh[3][kSThreads / 32];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        a += __shfl_xor_sync(kFull, a, o);
        b += __shfl_xor_sync(kFull, b, o);
        c += __shfl_xor_sync(kFull, c, o);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sh[0][warp] = a; sh[1][warp] = b; sh[2][warp] = c; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
        for (int w = 0; w < kSThreads / 32; w++) { s0 += sh[0][w]; s1 += sh[1][w]; s2 += sh[2][w]; }
        out3[0] = s0; out3[1] = s1; out3[2] = s2;
    }
}

__device__ __forceinline__ void acc3(float x0, float x1, float x2, float& p01, float& p02, float& p12) {
    const float a = x0 - x1, b = x0 - x2, c = x1 - x2;
    p01 = fmaf(a, a, p01); p02 = fmaf(b, b, p02); p12 = fmaf(c, c, p12);
}

// contiguous g2
__global__ void __launch_bounds__(kSThreads) sq_diffs3_partial_kernel(const float* __restrict__ g0, const float* __restrict__ g1,
                                                                      const float* __restrict__ g2, int64_t P, double* scratch) {
    double d01 = 0, d02 = 0, d12 = 0;
    const int64_t nvec = ((((uintptr_t)g0 | (uintptr_t)g1 | (uintptr_t)g2) & 15) == 0) ? P / 4 : 0;
    const int64_t stride = (int64_t)gridDim.x * kSThreads;
    for (int64_t i = (int64_t)blockIdx.x * kSThreads + threadIdx.x; i < nvec; i += stride) {
        const uint4 a = ld_stream_u4(g0 + i * 4), b = ld_stream_u4(g1 + i * 4), c = ld_stream_u4(g2 + i * 4);
        float p01 = 0, p02 = 0, p12 = 0;
        acc3(__uint_as_float(a.x), __uint_as_float(b.x), __uint_as_float(c.x), p01, p02, p12);
        acc3(__uint_as_float(a.y), __uint_as_float(b.y), __uint_as_float(c.y), p01, p02, p12);
        acc3(__uint_as_float(a.z), __uint_as_float(b.z), __uint_as_float(c.z), p01, p02, p12);
        acc3(__uint_as_float(a.w), __uint_as_float(b.w), __uint_as_float(c.w), p01, p02, p12);
        d01 += (double)p01; d02 += (double)p02; d12 += (double)p12;
    }
    for (int64_t i = nvec * 4 + (int64_t)blockIdx.x * kSThreads + threadIdx.x; i < P; i += stride) {
        float p01 = 0, p02 = 0, p12 = 0;
        acc3(g0[i], g1[i], g2[i], p01, p02, p12);
        d01 += (double)p01; d02 += (double)p02; d12 += (double)p12;
    }
    block_sum3(d01, d02, d12, scratch + 3 * blockIdx.x);
}

// g2 given as segments (the live .grad tensors): flat position i belongs to the segment s with
// seg_off[s] <= i < seg_off[s] + seg_len[s]; segments are sorted by offset and tile [0, P).
__global__ void __launch_bounds__(kSThreads) sq_diffs3_partial_seg_kernel(const float* __restrict__ g0, const float* __restrict__ g1, int64_t P,
                                                                          const float* const* __restrict__ seg_ptr,
                                                                          const int64_t* __restrict__ seg_off,
                                                                          const int64_t* __restrict__ seg_len, int nseg, double* scratch) {
    double d01 = 0, d02 = 0, d12 = 0;
    const int64_t stride = (int64_t)gridDim.x * kSThreads;
    int64_t i = (int64_t)blockIdx.x * kSThreads + threadIdx.x;
    if (i < P) {
        int lo = 0, hi = nseg - 1;                        // last segment whose offset is <= i
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (seg_off[mid] <= i) lo = mid; else hi = mid - 1;
        }
        int s = lo;
        int64_t s_off = seg_off[s], s_end = s_off + seg_len[s];
        const float* s_ptr = seg_ptr[s];
        for (; i < P; i += stride) {
            while (i >= s_end && s + 1 < nseg) {
                s++;
                s_off = seg_off[s]; s_end = s_off + seg_len[s]; s_ptr = seg_ptr[s];
            }
            float p01 = 0, p02 = 0, p12 = 0;
            acc3(g0[i], g1[i], s_ptr[i - s_off], p01, p02, p12);
            d01 += (double)p01; d02 += (double)p02; d12 += (double)p12;
        }
    }
    block_sum3(d01, d02, d12, scratch + 3 * blockIdx.x);
}

__global__ void __launch_bounds__(kSThreads) sq_diffs3_final_kernel(const double* scratch, int nblocks, double* out3) {
    double a = 0, b = 0, c = 0;
    for (int i = threadIdx.x; i < nblocks; i += kSThreads) {
        a += scratch[3 * i]; b += scratch[3 * i + 1]; c += scratch[3 * i + 2];
    }
    block_sum3(a, b, c, out3);
}

// C = max(d01, 2*max(d02, d12)); NaN, inf and values above 1e10 become 1e10 (autoprec.py:119-126)
__global__ void sensitivity_kernel(const double* d3, double scale, float* C, int L) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l >= L) return;
    const float d01 = (float)(d3[3 * l] * scale), d02 = (float)(d3[3 * l + 1] * scale), d12 = (float)(d3[3 * l + 2] * scale);
    // python's max(a, b) keeps a unless b > a
    const float m = (d12 > d02) ? d12 : d02;
    const float m2 = m * 2.0f;
    float sens = (m2 > d01) ? m2 : d01;
    if (isnan(sens) || isinf(sens) || sens > 1e10f) sens = 1e10f;
    C[l] = sens;
}

// ---------------------------------------------------------------------------------------------------
// Greedy bit allocation in one thread block.  The reference keeps (float key, int64 index) pairs in a
// std::priority_queue; the pop order of that queue is "largest key, then largest index".  Here every
// candidate is one 64-bit word (order-preserving image of the key in the high half, index in the low
// half, 0 = absent) in shared memory and a pop is a block-wide max.
// ---------------------------------------------------------------------------------------------------
constexpr int kPThreads = 1024;

__host__ __device__ __forceinline__ int next_bits(int b) { return b == 32 ? 8 : b == 8 ? 4 : b == 4 ? 2 : b == 2 ? 1 : 0; }

__host__ __device__ __forceinline__ double step_gain(float C, int b) {
    const int nb = next_bits(b);
    const int c2 = ((1 << nb) - 1) * ((1 << nb) - 1);
    if (b == 32) return -(double)C / c2;
    const int c1 = ((1 << b) - 1) * ((1 << b) - 1);
    return C * (1.0 / c1 - 1.0 / c2);
}

__host__ __device__ __forceinline__ uint64_t make_candidate(float C, int b, int64_t w, int idx) {
    const int db = b - next_bits(b);
    float key = (float)(step_gain(C, b) / (double)(w * db));
    if (key == 0.0f) key = 0.0f;                                  // -0 and +0 compare equal in the reference
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(key);
#else
    uint32_t u;
    memcpy(&u, &key, sizeof u);
#endif
    u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;                   // order-preserving map to unsigned
    return ((uint64_t)u << 32) | (uint32_t)idx;
}

__global__ void __launch_bounds__(kPThreads) calc_precision_kernel(int32_t* __restrict__ b, const float* __restrict__ C,
                                                                   const int64_t* __restrict__ w, int L, double target, int* status) {
    extern __shared__ uint64_t cand[];                            // L candidates
    __shared__ uint64_t warp_best[kPThreads / 32];
    __shared__ double sh_sum[kPThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    double part = 0;
    for (int i = tid; i < L; i += kPThreads) {
        const int bi = b[i];
        if (bi > 1) {                                             // entries already at 1 bit are not counted (as in the reference)
            cand[i] = make_candidate(C[i], bi, w[i], i);
            part += (double)((int64_t)bi * w[i]);                 // integer-valued: the order of the sum is immaterial
        } else {
            cand[i] = 0;
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) part += __shfl_xor_sync(kFull, part, o);
    if (lane == 0) sh_sum[warp] = part;
    __syncthreads();
    double b_sum = 0;                                             // every thread keeps the same copy
    for (int k = 0; k < kPThreads / 32; k++) b_sum += sh_sum[k];

    int st = GACT_OK;
    for (int pops = 0; pops <= 4 * L && b_sum > target; pops++) {
        uint64_t best = 0;
        for (int i = tid; i < L; i += kPThreads) best = max(best, cand[i]);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const uint64_t other = __shfl_xor_sync(kFull, best, o);
            best = max(best, other);
        }
        if (lane == 0) warp_best[warp] = best;
        __syncthreads();
        best = warp_best[lane];                                   // kPThreads / 32 == 32 entries
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const uint64_t other = __shfl_xor_sync(kFull, best, o);
            best = max(best, other);
        }
        if (best == 0) { st = GACT_ERR_BUDGET; break; }           // queue empty, budget not met
        const int i = (int)(uint32_t)best;
        const int bi = b[i];
        const int nb = next_bits(bi);
        const int64_t wi = w[i];
        b_sum -= (double)(wi * (bi - nb));
        __syncthreads();                                          // everyone has read b[i] and warp_best
        if (tid == 0) {
            b[i] = nb;
            cand[i] = (nb > 1) ? make_candidate(C[i], nb, wi, i) : 0;
        }
        __syncthreads();
    }
    if (tid == 0 && status != nullptr) *status = st;
}


// ---------------------------------------------------------------------------------------------------
// gact_sq_diffs3_noalloc: the same reduction for callers that cannot allocate device memory.
//
// Who that is: code running inside a region where the CUDA allocator must not be touched (a framework's
// allocator-free section, a real-time loop that forbids cudaMalloc because it synchronises the device), or a
// host language binding that has no device allocator at hand and only holds the pointers it was given.  The
// scratch that gact_sq_diffs3 takes from its caller lives here in a fixed array inside the library image: the
// block partials plus a table for up to GACT_NOALLOC_MAX_SEGMENTS gradient segments.  Every GPU that loads the
// library carries these ~62 KB until the process exits.
//
// In host code the array's name is only a handle for the runtime, not a device address, so the address the
// kernels get is looked up with cudaGetSymbolAddress once per device (with that device current) and cached.
// ---------------------------------------------------------------------------------------------------
constexpr int kNoAllocPartialBytes = ((kSBlocks * 3 * (int)sizeof(double) + 255) / 256) * 256;
constexpr int kNoAllocTableBytes = GACT_NOALLOC_MAX_SEGMENTS * 8;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocPartialBytes + 3 * kNoAllocTableBytes];

static void* g_noalloc_addr[kMaxDevices];          // device address of g_noalloc_scratch, per device ordinal
static std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device; looked up on the first call per device.
static int noalloc_scratch_address(unsigned char** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return GACT_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return GACT_ERR_LAUNCH;
        g_noalloc_addr[dev] = p;
    }
    *out = (unsigned char*)g_noalloc_addr[dev];
    return GACT_OK;
}

}  // namespace gact

using namespace gact;

extern "C" int64_t gact_sq_diffs3_scratch_bytes(void) { return (int64_t)kSBlocks * 3 * sizeof(double); }

extern "C" int gact_sq_diffs3(const float* g0, const float* g1, const float* g2, int64_t P, const float* const* seg_ptr,
                              const int64_t* seg_off, const int64_t* seg_len, int nseg, void* scratch, double* out3,
                              void* stream) {
    if (P < 0 || nseg < 0) return GACT_ERR_SIZE;
    if (!g0 || !g1 || !scratch || !out3) return GACT_ERR_NULL;
    if (nseg == 0 && !g2) return GACT_ERR_NULL;
    if (nseg > 0 && (!seg_ptr || !seg_off || !seg_len)) return GACT_ERR_NULL;
    if (((uintptr_t)scratch & 15) || ((uintptr_t)out3 & 7)) return GACT_ERR_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    if (nseg == 0)
        sq_diffs3_partial_kernel<<<kSBlocks, kSThreads, 0, s>>>(g0, g1, g2, P, (double*)scratch);
    else
        sq_diffs3_partial_seg_kernel<<<kSBlocks, kSThreads, 0, s>>>(g0, g1, P, seg_ptr, seg_off, seg_len, nseg, (double*)scratch);
    sq_diffs3_final_kernel<<<1, kSThreads, 0, s>>>((const double*)scratch, kSBlocks, out3);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

extern "C" int gact_sq_diffs3_noalloc(const float* g0, const float* g1, const float* g2, int64_t P,
                                      const float* const* seg_ptr_host, const int64_t* seg_off_host,
                                      const int64_t* seg_len_host, int nseg, double* out3, void* stream) {
    if (P < 0 || nseg < 0) return GACT_ERR_SIZE;
    if (nseg > GACT_NOALLOC_MAX_SEGMENTS) return GACT_ERR_NOALLOC_LIMIT;
    if (!g0 || !g1 || !out3) return GACT_ERR_NULL;
    if (nseg == 0 && !g2) return GACT_ERR_NULL;
    if (nseg > 0 && (!seg_ptr_host || !seg_off_host || !seg_len_host)) return GACT_ERR_NULL;
    if ((uintptr_t)out3 & 7) return GACT_ERR_ALIGN;
    // the tables are host memory here, so they can be checked before anything is launched: the segments must
    // tile [0, P) in order, without gaps or overlap (the kernel indexes them without further bounds tests)
    if (nseg > 0) {
        int64_t expect = 0;
        for (int k = 0; k < nseg; k++) {
            if (seg_ptr_host[k] == nullptr) return GACT_ERR_NULL;
            if (seg_len_host[k] < 0 || seg_off_host[k] != expect) return GACT_ERR_SIZE;
            expect += seg_len_host[k];
        }
        if (expect != P) return GACT_ERR_SIZE;
    }
    unsigned char* base = nullptr;
    const int rc = noalloc_scratch_address(&base);
    if (rc != GACT_OK) return rc;
    double* partials = (double*)base;               // fully rewritten by stage 1 before stage 2 reads it
    cudaStream_t s = (cudaStream_t)stream;
    if (nseg == 0) {
        sq_diffs3_partial_kernel<<<kSBlocks, kSThreads, 0, s>>>(g0, g1, g2, P, partials);
    } else {
        unsigned char* t_ptr = base + kNoAllocPartialBytes;
        unsigned char* t_off = t_ptr + kNoAllocTableBytes;
        unsigned char* t_len = t_off + kNoAllocTableBytes;
        const size_t bytes = (size_t)nseg * 8;
        // stream-ordered copies of the caller's host tables into the library's own table
        if (cudaMemcpyAsync(t_ptr, seg_ptr_host, bytes, cudaMemcpyHostToDevice, s) != cudaSuccess ||
            cudaMemcpyAsync(t_off, seg_off_host, bytes, cudaMemcpyHostToDevice, s) != cudaSuccess ||
            cudaMemcpyAsync(t_len, seg_len_host, bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
            return GACT_ERR_LAUNCH;
        sq_diffs3_partial_seg_kernel<<<kSBlocks, kSThreads, 0, s>>>(g0, g1, P, (const float* const*)t_ptr, (const int64_t*)t_off,
                                                                   (const int64_t*)t_len, nseg, partials);
    }
    sq_diffs3_final_kernel<<<1, kSThreads, 0, s>>>(partials, kSBlocks, out3);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

extern "C" int gact_sensitivity(const double* d3, double scale, float* C, int L, void* stream) {
    if (L < 0) return GACT_ERR_SIZE;
    if (L == 0) return GACT_OK;
    if (!d3 || !C) return GACT_ERR_NULL;
    sensitivity_kernel<<<(L + 127) / 128, 128, 0, (cudaStream_t)stream>>>(d3, scale, C, L);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

extern "C" int gact_calc_precision(int32_t* b, const float* C, const int64_t* w, int L, double target, int* status,
                                   void* stream) {
    if (L < 0) return GACT_ERR_SIZE;
    if (L == 0) return GACT_OK;
    if (!b || !C || !w) return GACT_ERR_NULL;
    const size_t smem = (size_t)L * sizeof(uint64_t);
    if (smem > 200 * 1024) return GACT_ERR_SIZE;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(calc_precision_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return GACT_ERR_LAUNCH;
    }
    calc_precision_kernel<<<1, kPThreads, smem, (cudaStream_t)stream>>>(b, C, w, L, target, status);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

// Host twin of the kernel above for callers that hold b, C and w in host memory (the reference's calc_precision
// takes CPU tensors): same keys, same pop order (a max-heap of the 64-bit candidates), same stopping rule.
extern "C" int gact_calc_precision_host(int32_t* b, const float* C, const int64_t* w, int L, double target) {
    if (L < 0) return GACT_ERR_SIZE;
    if (L == 0) return GACT_OK;
    if (!b || !C || !w) return GACT_ERR_NULL;
    std::vector<uint64_t> heap;
    heap.reserve((size_t)L);
    double b_sum = 0;
    for (int i = 0; i < L; i++) {
        if (b[i] > 1) {                                           // entries already at 1 bit are not counted (as in the reference)
            b_sum += (double)((int64_t)b[i] * w[i]);
            heap.push_back(make_candidate(C[i], b[i], w[i], i));
        }
    }
    std::make_heap(heap.begin(), heap.end());
    while (b_sum > target) {
        if (heap.empty()) return GACT_ERR_BUDGET;
        std::pop_heap(heap.begin(), heap.end());
        const int i = (int)(uint32_t)heap.back();
        heap.pop_back();
        const int nb = next_bits(b[i]);
        b_sum -= (double)(w[i] * (b[i] - nb));
        b[i] = nb;
        if (nb > 1) {
            heap.push_back(make_candidate(C[i], nb, w[i], i));
            std::push_heap(heap.begin(), heap.end());
        }
    }
    return GACT_OK;
}

extern "C" int gact_version(void) { return 100; }

extern "C" const char* gact_error_string(int status) {
    switch (status) {
    case GACT_OK: return "ok";
    case GACT_ERR_BITS: return "bits must be 1, 2, 4 or 8";
    case GACT_ERR_DTYPE: return "element type must be fp32, fp16 or bf16";
    case GACT_ERR_NULL: return "a required pointer is null";
    case GACT_ERR_ALIGN: return "a base pointer is not aligned as required";
    case GACT_ERR_SIZE: return "size is negative or not supported";
    case GACT_ERR_MODE: return "unknown rng mode, or the noise array is missing";
    case GACT_ERR_LAUNCH: return "the CUDA runtime refused the launch";
    case GACT_ERR_BUDGET: return "bit budget cannot be met";
    case GACT_ERR_NOALLOC_LIMIT: return "more gradient segments than the allocation-free entry point holds (GACT_NOALLOC_MAX_SEGMENTS)";
    default: return "unknown status";
    }
}
