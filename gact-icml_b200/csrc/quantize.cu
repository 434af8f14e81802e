// Fused quantize: per-group min/max -> scale -> stochastic rounding -> bit packing, one pass over the input.
//
// Work decomposition.  A warp owns a tile of GPW = max(4, 8/bits) consecutive groups, i.e. U = GPW/wpt
// whole row-blocks of the packed layout.  Each lane keeps 8 values of every group of the tile in registers
// (all loads of a tile are issued before anything is reduced: 2-8 KB in flight per warp), reduces min/max
// with shuffles, lanes 0..GPW-1 each work out one group's scale (the double-precision divide is done once
// per group, GPW of them in parallel), and every lane then rounds its values and assembles 8 packed bytes
// per row-block, stored as one 8-byte (16-bit inputs) or two 4-byte (fp32) coalesced stores.
#include "gact_common.cuh"

namespace gact {

constexpr int kQThreads = 256;

struct QuantArgs {
    const void* x;
    int64_t n, G, R;
    uint64_t seed;
    const float* noise;
    uint8_t* packed;
    void* qmin;
    void* qscale;
};

template <int DT, int BITS, int RNG, bool FMA>
__global__ void __launch_bounds__(kQThreads) quantize_kernel(const QuantArgs a) {
    using E = Elem<DT>;
    using T = typename E::T;
    constexpr int WPT = 8 / BITS;                    // groups per row-block
    constexpr int U = (WPT >= 4) ? 1 : 4 / WPT;      // row-blocks per tile
    constexpr int GPW = WPT * U;                     // groups per tile
    constexpr int CALLS = (WPT + 3) / 4;             // Philox calls per packed byte (reference stream)

    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kQThreads / 32);
    const int64_t tiles = (a.R + U - 1) / U;
    const uint32_t key0 = (uint32_t)a.seed, key1 = (uint32_t)(a.seed >> 32);

    for (int64_t tile = (int64_t)blockIdx.x * (kQThreads / 32) + (threadIdx.x >> 5); tile < tiles; tile += nwarps) {
        const int64_t g0 = tile * GPW;

        float v[GPW][8];
#pragma unroll
        for (int k = 0; k < GPW; k++) {
            if (g0 + k < a.G) {
                load_group8<DT>(a.x, a.n, g0 + k, lane, v[k]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) v[k][j] = 0.0f;
            }
        }

        float mn[GPW], sc[GPW];
        float my_mn = 0.0f, my_mx = 0.0f;
#pragma unroll
        for (int k = 0; k < GPW; k++) {
            float lo, hi;
            group_minmax<DT>(v[k], lane, lo, hi);
            mn[k] = lo;
            if (lane == k) { my_mn = lo; my_mx = hi; }
        }
        const float my_sc = compute_scale<DT>(my_mn, my_mx, BITS);
        if (lane < GPW && g0 + lane < a.G) {
            ((T*)a.qmin)[g0 + lane] = E::from_float(my_mn);
            store_scale<DT>(a.qscale, g0 + lane, my_sc);
        }
#pragma unroll
        for (int k = 0; k < GPW; k++) sc[k] = __shfl_sync(kFull, my_sc, k);

#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t r = tile * U + u;
            if (r >= a.R) break;
            uint32_t bytes[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int d = elem_pos<DT>(lane, j);
                const uint64_t gid = (uint64_t)r * kGroup + d;     // packed byte index = Philox subsequence
                uint32_t acc = 0;
#pragma unroll
                for (int c = 0; c < CALLS; c++) {
                    uint4 rnd = make_uint4(0, 0, 0, 0);
                    if (RNG == GACT_RNG_CURAND)
                        rnd = philox4x32_10((uint32_t)c, 0u, (uint32_t)gid, (uint32_t)(gid >> 32), key0, key1);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int ni = c * 4 + q;
                        if (ni >= WPT) break;
                        const int k = u * WPT + ni;
                        if (g0 + k >= a.G) break;                  // tail row-block: absent groups leave zero bits
                        float nz;
                        if (RNG == GACT_RNG_CURAND) nz = uniform_from_word(word_of(rnd, q));
                        else if (RNG == GACT_RNG_RTN) nz = 0.5f;
                        else nz = a.noise[(g0 + k) * kGroup + d];
                        float t, uu;
                        if (DT != GACT_F16) {
                            t = __fsub_rn(v[k][j], mn[k]);
                            uu = (FMA || DT == GACT_BF16) ? __fmaf_rn(t, sc[k], nz) : __fadd_rn(__fmul_rn(t, sc[k]), nz);
                        } else {
                            t = E::round(__fsub_rn(v[k][j], mn[k]));
                            uu = __fadd_rn(E::round(__fmul_rn(t, sc[k])), nz);
                        }
                        // max(u - 0.5, 0): NaN and negatives give 0.  fp32 / fp16 have no upper clamp, as in the
                        // reference: a code of 2^bits (noise == 1.0, or an fp16 scale that rounded up) spills into
                        // the next slot / wraps.  bf16 is not a reference type and clamps.
                        float w = fmaxf(__fadd_rn(uu, -0.5f), 0.0f);
                        if (DT == GACT_BF16) w = fminf(w, (float)((1 << BITS) - 1));
                        acc |= (uint32_t)__float2int_rn(w) << (ni * BITS);
                    }
                }
                bytes[j] = acc & 0xffu;
            }
            const uint32_t lo = bytes[0] | (bytes[1] << 8) | (bytes[2] << 16) | (bytes[3] << 24);
            const uint32_t hi = bytes[4] | (bytes[5] << 8) | (bytes[6] << 16) | (bytes[7] << 24);
            uint8_t* row = a.packed + r * kGroup;
            if (DT == GACT_F32) {
                st_stream_u1(row + lane * 4, lo);
                st_stream_u1(row + 128 + lane * 4, hi);
            } else {
                st_stream_u2(row + lane * 8, make_uint2(lo, hi));
            }
        }
    }
}

template <int DT, int BITS, int RNG, bool FMA>
static int launch_quantize(const QuantArgs& a, cudaStream_t s) {
    constexpr int WPT = 8 / BITS;
    constexpr int U = (WPT >= 4) ? 1 : 4 / WPT;
    const int64_t tiles = (a.R + U - 1) / U;
    const int64_t want = (tiles + kQThreads / 32 - 1) / (kQThreads / 32);
    const int64_t cap = (int64_t)kSMs * 8;
    const int blocks = (int)(want < cap ? want : cap);
    quantize_kernel<DT, BITS, RNG, FMA><<<blocks, kQThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

template <int DT, int BITS>
static int dispatch_rng(const QuantArgs& a, int rng, int fma, cudaStream_t s) {
    switch (rng) {
    case GACT_RNG_CURAND:
        if (DT == GACT_F32 && !fma) return launch_quantize<DT, BITS, GACT_RNG_CURAND, false>(a, s);
        return launch_quantize<DT, BITS, GACT_RNG_CURAND, true>(a, s);
    case GACT_RNG_RTN:
        if (DT == GACT_F32 && !fma) return launch_quantize<DT, BITS, GACT_RNG_RTN, false>(a, s);
        return launch_quantize<DT, BITS, GACT_RNG_RTN, true>(a, s);
    case GACT_RNG_EXTERNAL:
        if (DT == GACT_F32 && !fma) return launch_quantize<DT, BITS, GACT_RNG_EXTERNAL, false>(a, s);
        return launch_quantize<DT, BITS, GACT_RNG_EXTERNAL, true>(a, s);
    default:
        return GACT_ERR_MODE;
    }
}

template <int DT>
static int dispatch_bits(const QuantArgs& a, int bits, int rng, int fma, cudaStream_t s) {
    switch (bits) {
    case 1: return dispatch_rng<DT, 1>(a, rng, fma, s);
    case 2: return dispatch_rng<DT, 2>(a, rng, fma, s);
    case 4: return dispatch_rng<DT, 4>(a, rng, fma, s);
    case 8: return dispatch_rng<DT, 8>(a, rng, fma, s);
    default: return GACT_ERR_BITS;
    }
}

// ---------------------------------------------------------------------------------------------------
// min / max only (the reference's separate minimax op)
// ---------------------------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kQThreads) minimax_kernel(const void* x, int64_t n, int64_t G, void* mn_out, void* mx_out) {
    using E = Elem<DT>;
    using T = typename E::T;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kQThreads / 32);
    for (int64_t g = (int64_t)blockIdx.x * (kQThreads / 32) + (threadIdx.x >> 5); g < G; g += nwarps) {
        float v[8], lo, hi;
        load_group8<DT>(x, n, g, lane, v);
        group_minmax<DT>(v, lane, lo, hi);
        if (lane == 0) {
            ((T*)mn_out)[g] = E::from_float(lo);
            ((T*)mx_out)[g] = E::from_float(hi);
        }
    }
}

}  // namespace gact

using namespace gact;

static inline bool misaligned(const void* p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) != 0; }

extern "C" int64_t gact_packed_bytes(int64_t n, int bits) {
    if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8) || n < 0) return -1;
    const int64_t G = (n + kGroup - 1) / kGroup;
    const int wpt = 8 / bits;
    return (G + wpt - 1) / wpt * kGroup;
}

extern "C" int gact_quantize(const void* x, int dtype, int64_t n, int bits, uint64_t seed, int rng_mode,
                             const float* noise, int fma_mode, void* packed, void* qmin, void* qscale,
                             void* stream) {
    if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8)) return GACT_ERR_BITS;
    if (dtype < GACT_F32 || dtype > GACT_BF16) return GACT_ERR_DTYPE;
    if (n < 0) return GACT_ERR_SIZE;
    if (rng_mode < GACT_RNG_CURAND || rng_mode > GACT_RNG_EXTERNAL) return GACT_ERR_MODE;
    if (n == 0) return GACT_OK;
    if (!x || !packed || !qmin || !qscale) return GACT_ERR_NULL;
    if (rng_mode == GACT_RNG_EXTERNAL && !noise) return GACT_ERR_MODE;
    if (misaligned(x, 16) || misaligned(packed, 16) || misaligned(qmin, dtype == GACT_F32 ? 4 : 2) ||
        misaligned(qscale, dtype == GACT_F16 ? 2 : 4))
        return GACT_ERR_ALIGN;
    QuantArgs a;
    a.x = x; a.n = n; a.G = (n + kGroup - 1) / kGroup;
    a.R = (a.G + 8 / bits - 1) / (8 / bits);
    a.seed = seed; a.noise = noise; a.packed = (uint8_t*)packed; a.qmin = qmin; a.qscale = qscale;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case GACT_F32: return dispatch_bits<GACT_F32>(a, bits, rng_mode, fma_mode, s);
    case GACT_F16: return dispatch_bits<GACT_F16>(a, bits, rng_mode, fma_mode, s);
    default: return dispatch_bits<GACT_BF16>(a, bits, rng_mode, fma_mode, s);
    }
}

extern "C" int gact_minimax(const void* x, int dtype, int64_t n, void* mn, void* mx, void* stream) {
    if (dtype < GACT_F32 || dtype > GACT_BF16) return GACT_ERR_DTYPE;
    if (n < 0) return GACT_ERR_SIZE;
    if (n == 0) return GACT_OK;
    if (!x || !mn || !mx) return GACT_ERR_NULL;
    if (misaligned(x, 16)) return GACT_ERR_ALIGN;
    const int64_t G = (n + kGroup - 1) / kGroup;
    const int64_t want = (G + kQThreads / 32 - 1) / (kQThreads / 32);
    const int blocks = (int)(want < (int64_t)kSMs * 8 ? want : (int64_t)kSMs * 8);
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case GACT_F32: minimax_kernel<GACT_F32><<<blocks, kQThreads, 0, s>>>(x, n, G, mn, mx); break;
    case GACT_F16: minimax_kernel<GACT_F16><<<blocks, kQThreads, 0, s>>>(x, n, G, mn, mx); break;
    default: minimax_kernel<GACT_BF16><<<blocks, kQThreads, 0, s>>>(x, n, G, mn, mx); break;
    }
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}
