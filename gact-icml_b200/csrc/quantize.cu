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
    PhiloxKeys rk;
};

#ifndef GACT_GPW16
#define GACT_GPW16 8
#endif
template <int DT, int BITS> struct Tile {
    static constexpr int WPT = 8 / BITS;
    static constexpr int GPW = (DT == GACT_F32) ? (WPT > 4 ? WPT : 4) : (WPT > GACT_GPW16 ? WPT : GACT_GPW16);
    static constexpr int U = GPW / WPT;
};

// noise of the FAST arrangement for the 8 elements [8*block, 8*block+8): one Philox4x32-10 call, counter
// (block_lo, block_hi, 0, "FAST"), 16 bits per element, noise = (h + 0.5) * 2^-16
__device__ __forceinline__ void fast_noise8(uint64_t block, const PhiloxKeys& rk, float2 (&nz)[4]) {
    const uint4 r = philox4x32_10((uint32_t)block, (uint32_t)(block >> 32), 0u, 0x46415354u, rk);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        // both halfwords to float on the conversion unit (no shift / mask), then (h + 0.5) * 2^-16, exact
        float lo, hi;
        asm("{ .reg .b16 l, h; mov.b32 {l, h}, %2; cvt.rn.f32.u16 %0, l; cvt.rn.f32.u16 %1, h; }" : "=f"(lo), "=f"(hi) : "r"(w[i]));
        nz[i] = fma2(make_float2(lo, hi), splat2(1.52587890625e-05f), splat2(7.62939453125e-06f));
    }
}

// magic bits (code in the low mantissa bits of 1.5*2^23 + code) of the 8 codes of one group held by this
// lane; nz[i] = noise of elements 2i, 2i+1
template <int DT, int BITS, bool FMA>
__device__ __forceinline__ void codes8(const uint32_t (&raw)[RawRegs<DT>::N], float mn, float sc, const float2 (&nz)[4],
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
            const __half2 p = __hmax2(__hmul2(t, sc2), zero2);                    // NaN -> 0, as max(., 0) does
            // u = p + noise; w = u - 0.5 (> -0.5, so no clamp needed: it rounds to 0); w + magic
            const float2 r = add2(add2(add2(__half22float2(p), nz[i]), splat2(-0.5f)), splat2(kMagic));
            cb[2 * i] = __float_as_uint(r.x);
            cb[2 * i + 1] = __float_as_uint(r.y);
        }
    } else {
        float v[8];
        raw_to_float<DT>(raw, v);
        const float2 nmn = splat2(-mn), sc2 = splat2(sc);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 t = add2(make_float2(v[2 * i], v[2 * i + 1]), nmn);          // x - mn
            const float2 u = (FMA || DT == GACT_BF16) ? fma2(t, sc2, nz[i]) : add2(mul2(t, sc2), nz[i]);
            float2 w = add2(u, splat2(-0.5f));
            w.x = fmaxf(w.x, 0.0f); w.y = fmaxf(w.y, 0.0f);                           // NaN -> 0
            if (DT == GACT_BF16) {
                // ours: clamp at 2^bits - 1 (fp32 / fp16 keep the reference's missing clamp)
                w.x = fminf(w.x, (float)((1 << BITS) - 1)); w.y = fminf(w.y, (float)((1 << BITS) - 1));
            }
            const float2 r = add2(w, splat2(kMagic));
            cb[2 * i] = __float_as_uint(r.x);
            cb[2 * i + 1] = __float_as_uint(r.y);
        }
    }
}

// All loads of one tile (issued back to back, nothing waits on them here).  FULL: every group of the tile
// exists and is complete, so no bounds are tested.
template <int DT, int BITS, bool FULL>
__device__ __forceinline__ void load_tile(const QuantArgs& a, int64_t tile, int lane,
                                          uint32_t (&raw)[Tile<DT, BITS>::GPW][RawRegs<DT>::N]) {
    constexpr int GPW = Tile<DT, BITS>::GPW, NR = RawRegs<DT>::N;
    const int64_t g0 = tile * GPW;
#pragma unroll
    for (int k = 0; k < GPW; k++) {
        if (FULL) {
            load_raw<DT>(a.x, (g0 + GPW) * kGroup, g0 + k, lane, a.aligned32 != 0, raw[k]);
        } else if (g0 + k < a.G) {
            load_raw<DT>(a.x, a.n, g0 + k, lane, a.aligned32 != 0, raw[k]);
        } else {
#pragma unroll
            for (int i = 0; i < NR; i++) raw[k][i] = 0;
        }
    }
}

// min/max, scale, codes and stores of one tile whose values are already in registers
template <int DT, int BITS, int RNG, bool FMA, bool FULL>
__device__ __forceinline__ void process_tile(const QuantArgs& a, int64_t tile, int lane,
                                             const uint32_t (&raw)[Tile<DT, BITS>::GPW][RawRegs<DT>::N]) {
    using E = Elem<DT>;
    using T = typename E::T;
    constexpr int WPT = Tile<DT, BITS>::WPT, GPW = Tile<DT, BITS>::GPW, U = Tile<DT, BITS>::U;
    const int64_t g0 = tile * GPW;

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
    if (lane < GPW && (FULL || g0 + lane < a.G)) {
        ((T*)a.qmin)[g0 + lane] = E::from_float(my_mn);
        store_scale<DT>(a.qscale, g0 + lane, my_sc);
    }
#pragma unroll
    for (int k = 0; k < GPW; k++) sc[k] = __shfl_sync(kFull, my_sc, k);

    // codes, one row-block at a time: acc[j] collects byte (row-block, position lane*8 + j)
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int64_t r = tile * U + u;
        if (!FULL && r >= a.R) break;
        uint32_t acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0;

        if (RNG == GACT_RNG_CURAND) {
            // the reference stream: one generator per packed byte (subsequence = byte index), slot ni = draw ni
            const uint64_t gid0 = (uint64_t)r * kGroup + lane * 8;
#pragma unroll
            for (int c = 0; c < (WPT + 3) / 4; c++) {
                float2 nz[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint64_t gid = gid0 + 2 * i;
                    const uint4 ra = philox4x32_10((uint32_t)c, 0u, (uint32_t)gid, (uint32_t)(gid >> 32), a.rk);
                    const uint4 rb = philox4x32_10((uint32_t)c, 0u, (uint32_t)(gid + 1), (uint32_t)((gid + 1) >> 32), a.rk);
                    // cuRAND's uniform: float(word) * 2^-32 + 2^-33
                    const float2 s2 = splat2(2.3283064365386963e-10f), o2 = splat2(1.1641532182693481e-10f);
                    nz[0][i] = fma2(make_float2(__uint2float_rn(ra.x), __uint2float_rn(rb.x)), s2, o2);
                    if (WPT > 1) nz[1][i] = fma2(make_float2(__uint2float_rn(ra.y), __uint2float_rn(rb.y)), s2, o2);
                    if (WPT > 2) {
                        nz[2][i] = fma2(make_float2(__uint2float_rn(ra.z), __uint2float_rn(rb.z)), s2, o2);
                        nz[3][i] = fma2(make_float2(__uint2float_rn(ra.w), __uint2float_rn(rb.w)), s2, o2);
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int ni = c * 4 + q;
                    if (ni >= WPT) break;
                    const int k = u * WPT + ni;
                    if (!FULL && g0 + k >= a.G) break;         // tail row-block: absent groups leave zero bits
                    uint32_t cb[8];
                    codes8<DT, BITS, FMA>(raw[k], mn[k], sc[k], nz[q], cb);
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[j] |= cb[j] << (ni * BITS);
                }
            }
        } else {
#pragma unroll
            for (int ni = 0; ni < WPT; ni++) {
                const int k = u * WPT + ni;
                if (!FULL && g0 + k >= a.G) break;
                float2 nz[4];
                if (RNG == GACT_RNG_FAST) {
                    fast_noise8((uint64_t)(g0 + k) * (kGroup / 8) + lane, a.rk, nz);
                } else if (RNG == GACT_RNG_RTN) {
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = splat2(0.5f);
                } else {
                    const float2* p = (const float2*)(a.noise + (g0 + k) * kGroup + lane * 8);
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = p[i];
                }
                uint32_t cb[8];
                codes8<DT, BITS, FMA>(raw[k], mn[k], sc[k], nz, cb);
#pragma unroll
                for (int j = 0; j < 8; j++) acc[j] |= cb[j] << (ni * BITS);
            }
        }
        // low bytes of the eight accumulators -> two words -> one 8-byte store
        const uint32_t lo = __byte_perm(__byte_perm(acc[0], acc[1], 0x0040u), __byte_perm(acc[2], acc[3], 0x0040u), 0x5410u);
        const uint32_t hi = __byte_perm(__byte_perm(acc[4], acc[5], 0x0040u), __byte_perm(acc[6], acc[7], 0x0040u), 0x5410u);
        st_stream_u2(a.packed + r * kGroup + lane * 8, make_uint2(lo, hi));
    }
}

#ifndef GACT_QMINB
#define GACT_QMINB 3
#endif

template <int DT, int BITS, int RNG, bool FMA>
__global__ void __launch_bounds__(kQThreads, GACT_QMINB) quantize_kernel(const __grid_constant__ QuantArgs a) {
    constexpr int GPW = Tile<DT, BITS>::GPW, NR = RawRegs<DT>::N;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kQThreads / 32);
    const int64_t tiles = (a.G + GPW - 1) / GPW;
    const int64_t full_tiles = a.n / (GPW * kGroup);            // tiles whose groups all exist and are complete
    for (int64_t tile = (int64_t)blockIdx.x * (kQThreads / 32) + (threadIdx.x >> 5); tile < tiles; tile += nwarps) {
        uint32_t raw[GPW][NR];
        if (tile < full_tiles) {
            load_tile<DT, BITS, true>(a, tile, lane, raw);
            process_tile<DT, BITS, RNG, FMA, true>(a, tile, lane, raw);
        } else {
            load_tile<DT, BITS, false>(a, tile, lane, raw);
            process_tile<DT, BITS, RNG, FMA, false>(a, tile, lane, raw);
        }
    }
}

template <int DT, int BITS, int RNG, bool FMA>
static int launch_quantize(const QuantArgs& a, cudaStream_t s) {
    // one resident wave: as many CTAs as fit on the 148 SMs (the kernel strides over the tiles)
    static int resident = 0;
    if (resident == 0) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_kernel<DT, BITS, RNG, FMA>, kQThreads, 0) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        resident = per_sm * kSMs;
    }
    const int64_t tiles = (a.G + Tile<DT, BITS>::GPW - 1) / Tile<DT, BITS>::GPW;
    const int64_t want = (tiles + kQThreads / 32 - 1) / (kQThreads / 32);
    const int blocks = (int)(want < resident ? want : resident);
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
    if (rng_mode == GACT_RNG_EXTERNAL && (!noise || misaligned(noise, 8))) return GACT_ERR_MODE;
    if (misaligned(x, 16) || misaligned(packed, 16) || misaligned(qmin, dtype == GACT_F32 ? 4 : 2) ||
        misaligned(qscale, dtype == GACT_F16 ? 2 : 4))
        return GACT_ERR_ALIGN;
    QuantArgs a;
    a.x = x; a.n = n; a.G = (n + kGroup - 1) / kGroup;
    a.R = (a.G + 8 / bits - 1) / (8 / bits);
    a.seed = seed; a.noise = noise; a.packed = (uint8_t*)packed; a.qmin = qmin; a.qscale = qscale;
    a.aligned32 = misaligned(x, 32) ? 0 : 1;
    a.rk = philox_round_keys(seed);
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
