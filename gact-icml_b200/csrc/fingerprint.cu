// Device-side fingerprint of a saved tensor, for the value-based deduplication of the reference
// (config.check_dup; gact/gact/quantizer.py:85-93 builds its key from 100 evenly spaced values and the sum of the
// tensor, each read back to the host: one synchronisation per saved tensor).  Here the same two ingredients stay
// on the device: out2[0] += hash of the sampled elements, out2[1] += sum of all elements' raw bits, both as
// wrapping 64-bit integers, so that the host can fetch the fingerprints of a whole step in one copy.
#include "gact_common.cuh"

namespace gact {

constexpr int kFThreads = 256;
constexpr int kFSamples = 100;          // the reference's sample count

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {      // splitmix64 finaliser
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <int ES> __device__ __forceinline__ uint64_t raw_at(const void* x, int64_t i) {
    if (ES == 4) return ((const uint32_t*)x)[i];
    if (ES == 2) return ((const uint16_t*)x)[i];
    return ((const uint8_t*)x)[i];
}

template <int ES>
__global__ void __launch_bounds__(kFThreads) fingerprint_kernel(const void* __restrict__ x, int64_t n, unsigned long long* out2) {
    unsigned long long sum = 0;
    const int64_t stride = (int64_t)gridDim.x * kFThreads;
    for (int64_t i = (int64_t)blockIdx.x * kFThreads + threadIdx.x; i < n; i += stride) sum += raw_at<ES>(x, i);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
    if ((threadIdx.x & 31) == 0 && sum != 0) atomicAdd(out2 + 1, sum);
    if (blockIdx.x == 0) {
        // sample i sits at i * (n div cnt), cnt = min(n, 100) (gact/gact/utils.py:16-24)
        const int64_t cnt = n < kFSamples ? n : kFSamples;
        const int64_t step = n / cnt;
        unsigned long long h = 0;
        for (int64_t i = threadIdx.x; i < cnt; i += kFThreads) h += mix64(raw_at<ES>(x, i * step) + 0x9E3779B97F4A7C15ull * (uint64_t)(i + 1));
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) h += __shfl_xor_sync(kFull, h, o);
        if ((threadIdx.x & 31) == 0 && h != 0) atomicAdd(out2, h);
    }
}

}  // namespace gact

using namespace gact;

extern "C" int gact_fingerprint(const void* x, int elem_bytes, int64_t n, uint64_t* out2, void* stream) {
    if (n < 0) return GACT_ERR_SIZE;
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return GACT_ERR_DTYPE;
    if (n == 0) return GACT_OK;
    if (!x || !out2) return GACT_ERR_NULL;
    if (((uintptr_t)x & (uintptr_t)(elem_bytes - 1)) || ((uintptr_t)out2 & 7)) return GACT_ERR_ALIGN;
    const int64_t want = (n + kFThreads * 8 - 1) / (kFThreads * 8);
    const int64_t cap = (int64_t)sm_count() * 8;
    const int blocks = (int)(want < cap ? want : cap);
    cudaStream_t s = (cudaStream_t)stream;
    unsigned long long* o = (unsigned long long*)out2;
    if (elem_bytes == 4) fingerprint_kernel<4><<<blocks, kFThreads, 0, s>>>(x, n, o);
    else if (elem_bytes == 2) fingerprint_kernel<2><<<blocks, kFThreads, 0, s>>>(x, n, o);
    else fingerprint_kernel<1><<<blocks, kFThreads, 0, s>>>(x, n, o);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}
