// 1-bit packing of dropout masks (uint8 or bool, one byte per element) and its inverse.
//
// Layout (kept from the reference so packed masks are interchangeable): element e of 512-element block
// blk sits in bit (t / 16) of word blk*16 + (t % 16), t = e % 512.  Seen from a warp that owns the block
// with lane k holding the 16 consecutive bytes t = 16k .. 16k+15, the block is a 32 x 16 bit matrix (row k =
// lane k's 16 "non-zero" bits) and its 16 words are the columns: a bit-matrix transpose across the warp, done
// for two blocks at once (32 x 32) with five shuffle stages.  No shared memory, no atomics, no votes.
// The packed mask has 16 words per started block, ceil(n/512)*16 in all: a partial last block still spreads
// its elements over all 16 words.  (The reference allocates ceil(n/32) words and lets its last block store
// and load past that allocation; for n a multiple of 512 the two sizes agree.)
#include "gact_common.cuh"

namespace gact {

constexpr int kMThreads = 256;

// Transpose of a 32 x 32 bit matrix held one row per lane (bit j of lane i  ->  bit i of lane j): five butterfly
// stages; in each, lanes whose index has bit s clear keep their low half-blocks and take the partner's low
// half-blocks shifted up, the others keep their high half-blocks and take the partner's high ones shifted down.
// Both shifts are one rotation (the bits that wrap around fall outside the selected mask).
__device__ __forceinline__ uint32_t transpose_bits32(uint32_t x, int lane) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const uint32_t m = (s == 16) ? 0x0000FFFFu : (s == 8) ? 0x00FF00FFu : (s == 4) ? 0x0F0F0F0Fu : (s == 2) ? 0x33333333u : 0x55555555u;
        const bool up = (lane & s) == 0;
        const uint32_t y = __shfl_xor_sync(kFull, x, s);
        const uint32_t t = __funnelshift_l(y, y, up ? s : 32 - s);
        const uint32_t keep = up ? m : ~m;
        x = (x & keep) | (t & ~keep);
    }
    return x;
}

// 16 bytes (four words) -> 16 bits, bit j set when byte j is non-zero
__device__ __forceinline__ uint32_t nonzero_bits16(const uint32_t (&q)[4]) {
    uint32_t m = 0;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        const uint32_t r = (((q[w] & 0x7f7f7f7fu) + 0x7f7f7f7fu) | q[w]) & 0x80808080u;   // bit 7 of every non-zero byte
        m |= ((r * 0x00204081u) >> 28) << (4 * w);                                       // bits 7, 15, 23, 31 -> one nibble
    }
    return m;
}

// the 16 bytes of one lane in block blk (zero past the end of the tensor); `vec`: x is 16-byte aligned
__device__ __forceinline__ void load_mask16(const uint8_t* __restrict__ x, int64_t n, int64_t blk, int lane, bool vec, uint32_t (&q)[4]) {
    const int64_t base = blk * 512 + lane * 16;
    if (vec && blk * 512 + 512 <= n) {
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
}

// A warp takes two 512-element blocks per step: lane k reads its 16 consecutive bytes of each, reduces them to
// 16 + 16 bits, and one bit-matrix transpose across the warp turns the 32 rows into the 32 words of the two
// blocks (lane j < 16: word j of the first block, lane 16 + j: word j of the second), written as one 128-byte row.
__global__ void __launch_bounds__(kMThreads) mask_pack_kernel(const uint8_t* __restrict__ x, int64_t n, bool vec, uint32_t* __restrict__ words,
                                                              int64_t nwords, int* not_binary) {
    const int lane = threadIdx.x & 31;
    const int64_t nblk = (n + 511) / 512;
    const int64_t npair = (nblk + 1) / 2;
    const int64_t nwarps = (int64_t)gridDim.x * (kMThreads / 32);
    uint32_t seen = 0;
    // two pairs (four blocks, 64 bytes per lane) per step, all loads first
    const int64_t nstep = (npair + 1) / 2;
    for (int64_t step = (int64_t)blockIdx.x * (kMThreads / 32) + (threadIdx.x >> 5); step < nstep; step += nwarps) {
        uint32_t q[4][4];
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int64_t blk = 4 * step + b;
            if (blk < nblk) {
                load_mask16(x, n, blk, lane, vec, q[b]);
            } else {
                q[b][0] = q[b][1] = q[b][2] = q[b][3] = 0;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t (&qa)[4] = q[2 * h];
            const uint32_t (&qb)[4] = q[2 * h + 1];
            seen |= qa[0] | qa[1] | qa[2] | qa[3] | qb[0] | qb[1] | qb[2] | qb[3];
            const uint32_t row = nonzero_bits16(qa) | (nonzero_bits16(qb) << 16);
            const uint32_t col = transpose_bits32(row, lane);
            const int64_t wi = (2 * step + h) * 32 + lane;
            if (wi < nwords) words[wi] = col;
        }
    }
    if (not_binary != nullptr && (seen & 0xfefefefeu) != 0u) *not_binary = 1;
}

__global__ void __launch_bounds__(kMThreads) mask_unpack_kernel(const uint32_t* __restrict__ words, int64_t n, int64_t nwords,
                                                                uint8_t* __restrict__ out, bool vec) {
    const int lane = threadIdx.x & 31;
    const int64_t nblk = (n + 511) / 512;
    const int64_t npair = (nblk + 1) / 2;
    const int64_t nwarps = (int64_t)gridDim.x * (kMThreads / 32);
    // two pairs (four blocks) per step: both word loads first, then 64 bytes of stores per lane
    const int64_t nstep = (npair + 1) / 2;
    for (int64_t step = (int64_t)blockIdx.x * (kMThreads / 32) + (threadIdx.x >> 5); step < nstep; step += nwarps) {
        uint32_t col[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t wi = (2 * step + h) * 32 + lane;
            col[h] = (wi < nwords) ? words[wi] : 0u;
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t row = transpose_bits32(col[h], lane);   // low half: my 16 elements of the pair's first block, high half: second
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int64_t blk = 4 * step + 2 * h + k;
                if (blk >= nblk) break;
                const uint32_t m = (row >> (16 * k)) & 0xffffu;
                uint32_t q[4];
#pragma unroll
                for (int w = 0; w < 4; w++) q[w] = (((m >> (4 * w)) & 0xfu) * 0x00204081u) & 0x01010101u;   // bit i -> byte i
                const int64_t base = blk * 512 + lane * 16;
                if (vec && blk * 512 + 512 <= n) {
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
    }
}

}  // namespace gact

using namespace gact;

static int mask_blocks(int64_t n, int blocks_per_step) {
    const int64_t nstep = ((n + 511) / 512 + blocks_per_step - 1) / blocks_per_step;   // warp steps in all
    const int64_t want = (nstep + kMThreads / 32 - 1) / (kMThreads / 32);
    const int64_t cap = (int64_t)sm_count() * 8;
    return (int)(want < cap ? want : cap);
}

extern "C" int64_t gact_mask_words(int64_t n) { return n < 0 ? -1 : (n + 511) / 512 * 16; }

extern "C" int gact_mask_pack(const uint8_t* x, int64_t n, uint32_t* words, int* not_binary, void* stream) {
    if (n < 0) return GACT_ERR_SIZE;
    if (n == 0) return GACT_OK;
    if (!x || !words) return GACT_ERR_NULL;
    if ((uintptr_t)words & 3) return GACT_ERR_ALIGN;
    const bool vec = ((uintptr_t)x & 15) == 0;          // a byte tensor may start anywhere; 16-byte loads where it allows
    mask_pack_kernel<<<mask_blocks(n, 4), kMThreads, 0, (cudaStream_t)stream>>>(x, n, vec, words, (n + 511) / 512 * 16, not_binary);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

extern "C" int gact_mask_unpack(const uint32_t* words, int64_t n, uint8_t* out, void* stream) {
    if (n < 0) return GACT_ERR_SIZE;
    if (n == 0) return GACT_OK;
    if (!words || !out) return GACT_ERR_NULL;
    if ((uintptr_t)words & 3) return GACT_ERR_ALIGN;
    const bool vec = ((uintptr_t)out & 15) == 0;
    mask_unpack_kernel<<<mask_blocks(n, 4), kMThreads, 0, (cudaStream_t)stream>>>(words, n, (n + 511) / 512 * 16, out, vec);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}
