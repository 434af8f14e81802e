// Fused quantize: per-group min/max -> scale -> stochastic rounding -> bit packing, one pass over the input.
//
// Work decomposition.  A warp owns a tile of GPW consecutive groups (8 for the 16-bit types, max(4, wpt) for
// fp32), i.e. U = GPW/wpt whole row-blocks of the packed layout.  Each lane keeps its 8 consecutive values of
// every group of the tile in registers, in storage format; all loads of a tile are issued before anything is
// reduced (4-8 KB in flight per warp).  min/max: two-wide min/max on the packed pairs inside the lane, then one
// warp-reduction instruction each (redux.sync.min/max.f32).  Lane k works out the scale of group k (the
// double-precision divide of the reference is evaluated once per group, GPW of them side by side) and the
// results are broadcast.  Every lane then rounds its values and assembles 8 packed bytes per row-block, written
// with one coalesced 8-byte store.
//
// Rounding without conversions: w + 1.5*2^23 leaves rint(w) (ties to even, like __float2int_rn) in the low
// mantissa bits; the bits above it fall off when the byte is cut out.  fp16 follows the reference's
// half-precision arithmetic with two-wide subtract / multiply; NaN products become 0 with a two-wide max, which
// is what the reference's `max(., 0)` does to them.
#include "gact_common.cuh"

namespace gact {

constexpr int kQThreads = 256;
constexpr float kMagic = 12582912.0f;   // 1.5 * 2^23

struct QuantArgs {
    const void* x;
    int64_t n, G, R;
    uint64_t seed;
    const float* noise;
    uint8_t* packed;
    void* qmin;
    void* qscale;
    int aligned32;
};

template <int DT, int BITS> struct Tile {
    static constexpr int WPT = 8 / BITS;
    static constexpr int GPW = (DT == GACT_F32) ? (WPT > 4 ? WPT : 4) : 8;
    static constexpr int U = GPW / WPT;
};

// rint(max(u - 0.5, 0)) as magic bits (code in the low bits).  `u` must not be NaN unless NANSAFE.
template <bool NANSAFE> __device__ __forceinline__ uint32_t round_code(float u) {
    float w = __fadd_rn(u, -0.5f);
    if (NANSAFE) w = fmaxf(w, 0.0f);                 // NaN -> 0; negatives round to (-)0 anyway
    return __float_as_uint(__fadd_rn(w, kMagic));
}

// noise of the FAST arrangement for the 8 elements [8*block, 8*block+8): one Philox4x32-10 call, counter
// (block_lo, block_hi, 0, "FAST"), 16 bits per element, noise = (h + 0.5) * 2^-16
__device__ __forceinline__ void fast_noise8(uint64_t block, uint32_t key0, uint32_t key1, float (&nz)[8]) {
    const uint4 r = philox4x32_10((uint32_t)block, (uint32_t)(block >> 32), 0u, 0x46415354u, key0, key1);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        // 2^23 + h as a float, then (2^23 + h) * 2^-16 - (2^7 - 2^-17) = (h + 0.5) * 2^-16, exact
        const float lo = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7410u));
        const float hi = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7432u));
        nz[2 * i] = __fmaf_rn(lo, 1.52587890625e-05f, -127.99999237060546875f);
        nz[2 * i + 1] = __fmaf_rn(hi, 1.52587890625e-05f, -127.99999237060546875f);
    }
}

// magic bits of the 8 codes of one group held by this lane
template <int DT, int BITS, bool FMA>
__device__ __forceinline__ void codes8(const uint32_t (&raw)[RawRegs<DT>::N], float mn, float sc, const float (&nz)[8],
                                       uint32_t (&cb)[8]) {
    if constexpr (DT == GACT_F16) {
        if (isinf(sc)) {
            // A half-precision scale overflows to +inf when the group's range is below (2^b-1)/65504.  The
            // reference then computes t*inf: +inf for every element above the minimum, which __float2int_rn
            // saturates to 0x7fffffff (all ones from the slot upwards), and NaN -> 0 for the minimum itself.
            float v[8];
            raw_to_float<DT>(raw, v);
#pragma unroll
            for (int j = 0; j < 8; j++) cb[j] = (Elem<DT>::round(__fsub_rn(v[j], mn)) > 0.0f) ? 0x7fffffffu : 0u;
            return;
        }
        const __half2 mn2 = __float2half2_rn(mn), sc2 = __float2half2_rn(sc);     // exact: both are half values
        const __half2 zero2 = __float2half2_rn(0.0f);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 t = __hsub2(*(const __half2*)&raw[i], mn2);
            const __half2 p = __hmax2(__hmul2(t, sc2), zero2);                    // NaN -> 0
            const float2 f = __half22float2(p);
            cb[2 * i] = round_code<false>(__fadd_rn(f.x, nz[2 * i]));
            cb[2 * i + 1] = round_code<false>(__fadd_rn(f.y, nz[2 * i + 1]));
        }
    } else {
        float v[8];
        raw_to_float<DT>(raw, v);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float t = __fsub_rn(v[j], mn);
            const float u = (FMA || DT == GACT_BF16) ? __fmaf_rn(t, sc, nz[j]) : __fadd_rn(__fmul_rn(t, sc), nz[j]);
            if (DT == GACT_BF16) {
                // ours: clamp at 2^bits - 1 (fp32 / fp16 keep the reference's missing clamp)
                const float w = fminf(fmaxf(__fadd_rn(u, -0.5f), 0.0f), (float)((1 << BITS) - 1));
                cb[j] = __float_as_uint(__fadd_rn(w, kMagic));
            } else {
                cb[j] = round_code<true>(u);
            }
        }
    }
}

template <int DT, int BITS, int RNG, bool FMA>
__global__ void __launch_bounds__(kQThreads) quantize_kernel(const QuantArgs a) {
    using E = Elem<DT>;
    using T = typename E::T;
    constexpr int WPT = Tile<DT, BITS>::WPT, GPW = Tile<DT, BITS>::GPW, U = Tile<DT, BITS>::U;
    constexpr int NR = RawRegs<DT>::N;

    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kQThreads / 32);
    const int64_t tiles = (a.G + GPW - 1) / GPW;
    const uint32_t key0 = (uint32_t)a.seed, key1 = (uint32_t)(a.seed >> 32);

    for (int64_t tile = (int64_t)blockIdx.x * (kQThreads / 32) + (threadIdx.x >> 5); tile < tiles; tile += nwarps) {
        const int64_t g0 = tile * GPW;

        uint32_t raw[GPW][NR];
#pragma unroll
        for (int k = 0; k < GPW; k++) {
            if (g0 + k < a.G) {
                load_raw<DT>(a.x, a.n, g0 + k, lane, a.aligned32 != 0, raw[k]);
            } else {
#pragma unroll
                for (int i = 0; i < NR; i++) raw[k][i] = 0;
            }
        }

        // min / max of every group; lane k keeps group k's pair and computes its scale
        float mn[GPW], sc[GPW];
        float my_mn = 0.0f, my_mx = 0.0f;
#pragma unroll
        for (int k = 0; k < GPW; k++) {
            float lo, hi;
            group_minmax_raw<DT>(raw[k], lane, lo, hi);
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

        // codes: acc[u][j] collects byte (row-block u, position lane*8 + j)
        uint32_t acc[U][8];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[u][j] = 0;

        if (RNG == GACT_RNG_CURAND) {
            // the reference stream: one generator per packed byte (subsequence = byte index), slot ni = draw ni
#pragma unroll
            for (int u = 0; u < U; u++) {
                const uint64_t gid0 = (uint64_t)(tile * U + u) * kGroup + lane * 8;
#pragma unroll
                for (int c = 0; c < (WPT + 3) / 4; c++) {
                    float nz[4][8];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint64_t gid = gid0 + j;
                        const uint4 r = philox4x32_10((uint32_t)c, 0u, (uint32_t)gid, (uint32_t)(gid >> 32), key0, key1);
                        nz[0][j] = uniform_from_word(r.x);
                        if (WPT > 1) nz[1][j] = uniform_from_word(r.y);
                        if (WPT > 2) { nz[2][j] = uniform_from_word(r.z); nz[3][j] = uniform_from_word(r.w); }
                    }
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int ni = c * 4 + q;
                        if (ni >= WPT) break;
                        const int k = u * WPT + ni;
                        if (g0 + k >= a.G) break;                  // tail row-block: absent groups leave zero bits
                        uint32_t cb[8];
                        codes8<DT, BITS, FMA>(raw[k], mn[k], sc[k], nz[q], cb);
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[u][j] |= cb[j] << (ni * BITS);
                    }
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < GPW; k++) {
                if (g0 + k >= a.G) break;
                const int u = k / WPT, ni = k % WPT;
                float nz[8];
                if (RNG == GACT_RNG_FAST) {
                    fast_noise8((uint64_t)(g0 + k) * (kGroup / 8) + lane, key0, key1, nz);
                } else if (RNG == GACT_RNG_RTN) {
#pragma unroll
                    for (int j = 0; j < 8; j++) nz[j] = 0.5f;
                } else {
                    const float* p = a.noise + (g0 + k) * kGroup + lane * 8;
#pragma unroll
                    for (int j = 0; j < 8; j++) nz[j] = p[j];
                }
                uint32_t cb[8];
                codes8<DT, BITS, FMA>(raw[k], mn[k], sc[k], nz, cb);
#pragma unroll
                for (int j = 0; j < 8; j++) acc[u][j] |= cb[j] << (ni * BITS);
            }
        }

#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t r = tile * U + u;
            if (r >= a.R) break;
            // low bytes of the eight accumulators -> two words
            const uint32_t lo = __byte_perm(__byte_perm(acc[u][0], acc[u][1], 0x0040u), __byte_perm(acc[u][2], acc[u][3], 0x0040u), 0x5410u);
            const uint32_t hi = __byte_perm(__byte_perm(acc[u][4], acc[u][5], 0x0040u), __byte_perm(acc[u][6], acc[u][7], 0x0040u), 0x5410u);
            st_stream_u2(a.packed + r * kGroup + lane * 8, make_uint2(lo, hi));
        }
    }
}

template <int DT, int BITS, int RNG, bool FMA>
static int launch_quantize(const QuantArgs& a, cudaStream_t s) {
    const int64_t tiles = (a.G + Tile<DT, BITS>::GPW - 1) / Tile<DT, BITS>::GPW;
    const int64_t want = (tiles + kQThreads / 32 - 1) / (kQThreads / 32);
    const int64_t cap = (int64_t)kSMs * 16;
    const int blocks = (int)(want < cap ? want : cap);
    quantize_kernel<DT, BITS, RNG, FMA><<<blocks, kQThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

template <int DT, int BITS>
static int dispatch_rng(const QuantArgs& a, int rng, int fma, cudaStream_t s) {
    const bool unfused = (DT == GACT_F32 && !fma);
    switch (rng) {
    case GACT_RNG_CURAND:
        return unfused ? launch_quantize<DT, BITS, GACT_RNG_CURAND, false>(a, s) : launch_quantize<DT, BITS, GACT_RNG_CURAND, true>(a, s);
    case GACT_RNG_FAST:
        return unfused ? launch_quantize<DT, BITS, GACT_RNG_FAST, false>(a, s) : launch_quantize<DT, BITS, GACT_RNG_FAST, true>(a, s);
    case GACT_RNG_RTN:
        return unfused ? launch_quantize<DT, BITS, GACT_RNG_RTN, false>(a, s) : launch_quantize<DT, BITS, GACT_RNG_RTN, true>(a, s);
    case GACT_RNG_EXTERNAL:
        return unfused ? launch_quantize<DT, BITS, GACT_RNG_EXTERNAL, false>(a, s) : launch_quantize<DT, BITS, GACT_RNG_EXTERNAL, true>(a, s);
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
        uint32_t raw[RawRegs<DT>::N];
        float lo, hi;
        load_raw<DT>(x, n, g, lane, false, raw);
        group_minmax_raw<DT>(raw, lane, lo, hi);
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
    a.aligned32 = misaligned(x, 32) ? 0 : 1;
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
