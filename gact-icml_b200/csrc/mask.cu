// 1-bit packing of dropout masks (uint8 or bool, one byte per element) and its inverse.
//
// Layout (kept from the reference so packed masks are interchangeable): element e of 512-element block
// blk sits in bit (t / 16) of word blk*16 + (t % 16), t = e % 512.  Seen from a warp that owns one block
// with lane k holding the 16 consecutive bytes t = 16k .. 16k+15, word w is exactly the ballot of "my byte
// number w is non-zero": 16 ballots per block, no shared memory, no atomics.
// The packed mask has 16 words per started block, ceil(n/512)*16 in all: a partial last block still spreads
// its elements over all 16 words.  (The reference allocates ceil(n/32) words and lets its last block store
// and load past that allocation; for n a multiple of 512 the two sizes agree.)
#include "gact_common.cuh"

namespace gact {

constexpr int kMThreads = 256;

__global__ void __launch_bounds__(kMThreads) mask_pack_kernel(const uint8_t* __restrict__ x, int64_t n, uint32_t* __restrict__ words,
                                                              int64_t nwords, int* not_binary) {
    const int lane = threadIdx.x & 31;
    const int64_t nblk = (n + 511) / 512;
    const int64_t nwarps = (int64_t)gridDim.x * (kMThreads / 32);
    bool odd = false;
    for (int64_t blk = (int64_t)blockIdx.x * (kMThreads / 32) + (threadIdx.x >> 5); blk < nblk; blk += nwarps) {
        const int64_t base = blk * 512 + lane * 16;
        uint32_t q[4];
        if (blk * 512 + 512 <= n) {
            const uint4 v = ld_stream_u4(x + base);
            q[0] = v.x; q[1] = v.y; q[2] = v.z; q[3] = v.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                q[i] = 0;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const int64_t e = base + i * 4 + b;
                    if (e < n) q[i] |= (uint32_t)x[e] << (8 * b);
                }
            }
        }
        odd |= ((q[0] | q[1] | q[2] | q[3]) & 0xfefefefeu) != 0u;
        uint32_t mine = 0;
#pragma unroll
        for (int w = 0; w < 16; w++) {
            const uint32_t byte = (q[w >> 2] >> ((w & 3) * 8)) & 0xffu;
            const uint32_t bal = __ballot_sync(kFull, byte != 0u);
            if (lane == w) mine = bal;
        }
        const int64_t wi = blk * 16 + lane;
        if (lane < 16 && wi < nwords) words[wi] = mine;
    }
    if (not_binary != nullptr && odd) *not_binary = 1;
}

__global__ void __launch_bounds__(kMThreads) mask_unpack_kernel(const uint32_t* __restrict__ words, int64_t n, int64_t nwords,
                                                                uint8_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t nblk = (n + 511) / 512;
    const int64_t nwarps = (int64_t)gridDim.x * (kMThreads / 32);
    for (int64_t blk = (int64_t)blockIdx.x * (kMThreads / 32) + (threadIdx.x >> 5); blk < nblk; blk += nwarps) {
        const int64_t wi = blk * 16 + (lane & 15);
        const uint32_t mine = (wi < nwords) ? words[wi] : 0u;
        uint32_t q[4] = {0, 0, 0, 0};
#pragma unroll
        for (int w = 0; w < 16; w++) {
            const uint32_t word = __shfl_sync(kFull, mine, w);
            q[w >> 2] |= ((word >> lane) & 1u) << ((w & 3) * 8);
        }
        const int64_t base = blk * 512 + lane * 16;
        if (blk * 512 + 512 <= n) {
            st_stream_u4(out + base, make_uint4(q[0], q[1], q[2], q[3]));
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int64_t e = base + i;
                if (e < n) out[e] = (uint8_t)((q[i >> 2] >> ((i & 3) * 8)) & 0xffu);
            }
        }
    }
}

}  // namespace gact

using namespace gact;

static int mask_blocks(int64_t n) {
    const int64_t nblk = (n + 511) / 512;
    const int64_t want = (nblk + kMThreads / 32 - 1) / (kMThreads / 32);
    const int64_t cap = (int64_t)kSMs * 8;
    return (int)(want < cap ? want : cap);
}

extern "C" int64_t gact_mask_words(int64_t n) { return n < 0 ? -1 : (n + 511) / 512 * 16; }

extern "C" int gact_mask_pack(const uint8_t* x, int64_t n, uint32_t* words, int* not_binary, void* stream) {
    if (n < 0) return GACT_ERR_SIZE;
    if (n == 0) return GACT_OK;
    if (!x || !words) return GACT_ERR_NULL;
    if (((uintptr_t)x & 15) || ((uintptr_t)words & 3)) return GACT_ERR_ALIGN;
    mask_pack_kernel<<<mask_blocks(n), kMThreads, 0, (cudaStream_t)stream>>>(x, n, words, (n + 511) / 512 * 16, not_binary);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

extern "C" int gact_mask_unpack(const uint32_t* words, int64_t n, uint8_t* out, void* stream) {
    if (n < 0) return GACT_ERR_SIZE;
    if (n == 0) return GACT_OK;
    if (!words || !out) return GACT_ERR_NULL;
    if (((uintptr_t)out & 15) || ((uintptr_t)words & 3)) return GACT_ERR_ALIGN;
    mask_unpack_kernel<<<mask_blocks(n), kMThreads, 0, (cudaStream_t)stream>>>(words, n, (n + 511) / 512 * 16, out);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}
