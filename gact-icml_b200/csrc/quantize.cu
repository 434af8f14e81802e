// Fused quantize: per-group min/max -> scale -> stochastic rounding -> bit packing, one pass over the input.
// This file holds the entry points, the fp32 kernel and the stand-alone min/max kernel; fp16 and bf16 inputs are
// in quantize16.cu.
//
// fp32 work decomposition.  A warp owns a tile of GPW = max(4, wpt) consecutive groups, i.e. U = GPW/wpt whole
// row-blocks of the packed layout.  Each lane keeps its 8 consecutive values of every group of the tile in
// registers (one 256-bit load per group); all loads of a tile are issued before anything is reduced (4-8 KB in
// flight per warp).  min/max: in-lane, then one warp-reduction instruction each (redux.sync.min/max.f32).  Lane k
// works out the scale of group k (the double-precision divide of the reference is evaluated once per group, GPW
// of them side by side) and the results are broadcast.  Every lane then rounds its values and assembles 8 packed
// bytes per row-block, written with one coalesced 8-byte store.
//
// Rounding without conversions: w + 1.5*2^23 leaves rint(w) (ties to even, like __float2int_rn) in the low
// mantissa bits; the bits above it fall off when the byte is cut out.
#include <atomic>

#include "quantize_common.cuh"

namespace gact {

// Tile of one warp: at least one row-block (8 / BITS groups), at least 4 groups.
template <int BITS> struct Tile32 {
    static constexpr int WPT = 8 / BITS;
    static constexpr int GPW = WPT > 4 ? WPT : 4;
    static constexpr int U = GPW / WPT;
};

// magic bits (code in the low mantissa bits of 1.5*2^23 + code) of the 8 codes of one group held by this
// lane; nz[i] = noise of elements 2i, 2i+1.  The reference's order of operations: (x - mn) * scale + noise as one
// fused multiply-add (FMA) or product first, then - 0.5, max(., 0) (which also turns NaN into 0), no upper clamp.
template <bool FMA>
__device__ __forceinline__ void codes8_f32(const uint32_t (&raw)[8], float mn, float sc, const float2 (&nz)[4], uint32_t (&cb)[8]) {
    const float2 nmn = splat2(-mn), sc2 = splat2(sc);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = add2(make_float2(__uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1])), nmn);
        const float2 u = FMA ? fma2(t, sc2, nz[i]) : add2(mul2(t, sc2), nz[i]);
        float2 w = add2(u, splat2(-0.5f));
        w.x = fmaxf(w.x, 0.0f); w.y = fmaxf(w.y, 0.0f);
        const float2 r = add2(w, splat2(kMagic));
        cb[2 * i] = __float_as_uint(r.x);
        cb[2 * i + 1] = __float_as_uint(r.y);
    }
}

// FULL: every group of the tile exists and is complete, so no bounds are tested.
template <int BITS, int RNG, bool FMA, bool FULL>
__device__ __forceinline__ void tile32(const QuantArgs& a, int64_t tile, int lane) {
    constexpr int DT = GACT_F32;
    constexpr int WPT = Tile32<BITS>::WPT, GPW = Tile32<BITS>::GPW, U = Tile32<BITS>::U;
    const int64_t g0 = tile * GPW;

    uint32_t raw[GPW][8];
#pragma unroll
    for (int k = 0; k < GPW; k++) {
        if (FULL) {
            load_raw<DT>(a.x, (g0 + GPW) * kGroup, g0 + k, lane, a.align, raw[k]);
        } else if (g0 + k < a.G) {
            load_raw<DT>(a.x, a.n, g0 + k, lane, a.align, raw[k]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) raw[k][i] = 0;
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
    if (lane < GPW && (FULL || g0 + lane < a.G)) {
        ((float*)a.qmin)[g0 + lane] = my_mn;
        ((float*)a.qscale)[g0 + lane] = my_sc;
    }
#pragma unroll
    for (int k = 0; k < GPW; k++) sc[k] = __shfl_sync(kFull, my_sc, k);

    // codes, one row-block at a time: acc[j] collects byte (row-block, position lane*8 + j)
    float2 nz_odd[4];            // FAST: noise of an odd group, produced together with the even group before it
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
                    nz[0][i] = curand_uniform2<false>(ra.x, rb.x);
                    if (WPT > 1) nz[1][i] = curand_uniform2<false>(ra.y, rb.y);
                    if (WPT > 2) {
                        nz[2][i] = curand_uniform2<false>(ra.z, rb.z);
                        nz[3][i] = curand_uniform2<false>(ra.w, rb.w);
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int ni = c * 4 + q;
                    if (ni >= WPT) break;
                    const int k = u * WPT + ni;
                    if (!FULL && g0 + k >= a.G) break;         // tail row-block: absent groups leave zero bits
                    uint32_t cb[8];
                    codes8_f32<FMA>(raw[k], mn[k], sc[k], nz[q], cb);
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
                    if ((k & 1) == 0) {
                        fast_noise16<false>((uint64_t)((g0 + k) >> 1) * (kGroup / 8) + lane, a.rk, nz, nz_odd);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++) nz[i] = nz_odd[i];
                    }
                } else if (RNG == GACT_RNG_RTN) {
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = splat2(0.5f);
                } else {
                    const float2* p = (const float2*)(a.noise + (g0 + k) * kGroup + lane * 8);
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = p[i];
                }
                uint32_t cb[8];
                codes8_f32<FMA>(raw[k], mn[k], sc[k], nz, cb);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (NoOverflow<RNG>::value) acc[j] += cb[j] << (ni * BITS);      // disjoint slots: a sum is an OR
                    else acc[j] |= cb[j] << (ni * BITS);
                }
            }
        }
        st_stream_u2(a.packed + r * kGroup + lane * 8, gather_bytes8(acc));
    }
}

template <int BITS, int RNG, bool FMA>
__global__ void __launch_bounds__(kQThreads, 3) quantize32_kernel(const __grid_constant__ QuantArgs a) {
    constexpr int GPW = Tile32<BITS>::GPW;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kQThreads / 32);
    const int64_t tiles = (a.G + GPW - 1) / GPW;
    const int64_t full_tiles = a.n / (GPW * kGroup);            // tiles whose groups all exist and are complete
    for (int64_t tile = (int64_t)blockIdx.x * (kQThreads / 32) + (threadIdx.x >> 5); tile < tiles; tile += nwarps) {
        if (tile < full_tiles) tile32<BITS, RNG, FMA, true>(a, tile, lane);
        else tile32<BITS, RNG, FMA, false>(a, tile, lane);
    }
}

template <int BITS, int RNG, bool FMA>
static int launch_quantize32(const QuantArgs& a, cudaStream_t s) {
    constexpr int GPW = Tile32<BITS>::GPW;
    const int64_t tiles = (a.G + GPW - 1) / GPW;
    // resident blocks per SM of this instantiation, asked once (the same on every device of a process)
    static std::atomic<int> per_sm_cached{0};
    int per_sm = per_sm_cached.load(std::memory_order_relaxed);
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize32_kernel<BITS, RNG, FMA>, kQThreads, 0) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        per_sm_cached.store(per_sm, std::memory_order_relaxed);
    }
    const int64_t resident = (int64_t)per_sm * sm_count();
    const int64_t want = (tiles + kQThreads / 32 - 1) / (kQThreads / 32);
    const int blocks = (int)(want < resident ? want : resident);
    quantize32_kernel<BITS, RNG, FMA><<<blocks, kQThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

template <int BITS>
static int dispatch_rng32(const QuantArgs& a, int rng, int fma, cudaStream_t s) {
    switch (rng) {
    case GACT_RNG_CURAND:
        return fma ? launch_quantize32<BITS, GACT_RNG_CURAND, true>(a, s) : launch_quantize32<BITS, GACT_RNG_CURAND, false>(a, s);
    case GACT_RNG_FAST:
        return fma ? launch_quantize32<BITS, GACT_RNG_FAST, true>(a, s) : launch_quantize32<BITS, GACT_RNG_FAST, false>(a, s);
    case GACT_RNG_RTN:
        return fma ? launch_quantize32<BITS, GACT_RNG_RTN, true>(a, s) : launch_quantize32<BITS, GACT_RNG_RTN, false>(a, s);
    case GACT_RNG_EXTERNAL:
        return fma ? launch_quantize32<BITS, GACT_RNG_EXTERNAL, true>(a, s) : launch_quantize32<BITS, GACT_RNG_EXTERNAL, false>(a, s);
    default:
        return GACT_ERR_MODE;
    }
}

static int dispatch_bits32(const QuantArgs& a, int bits, int rng, int fma, cudaStream_t s) {
    switch (bits) {
    case 1: return dispatch_rng32<1>(a, rng, fma, s);
    case 2: return dispatch_rng32<2>(a, rng, fma, s);
    case 4: return dispatch_rng32<4>(a, rng, fma, s);
    case 8: return dispatch_rng32<8>(a, rng, fma, s);
    default: return GACT_ERR_BITS;
    }
}

// ---------------------------------------------------------------------------------------------------
// min / max only (the reference's separate minimax op)
// ---------------------------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kQThreads) minimax_kernel(const void* x, int64_t n, int64_t G, int align, void* mn_out, void* mx_out) {
    using E = Elem<DT>;
    using T = typename E::T;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kQThreads / 32);
    for (int64_t g = (int64_t)blockIdx.x * (kQThreads / 32) + (threadIdx.x >> 5); g < G; g += nwarps) {
        uint32_t raw[RawRegs<DT>::N];
        float lo, hi;
        load_raw<DT>(x, n, g, lane, align, raw);
        group_minmax_raw<DT>(raw, lane, lo, hi);
        if (lane == 0) {
            ((T*)mn_out)[g] = E::from_float(lo);
            ((T*)mx_out)[g] = E::from_float(hi);
        }
    }
}

// process-wide diagnostics knobs of the bulk-copy pipeline (gact_pipeline_test_hook)
static std::atomic<uint32_t> g_wait_limit{1u << 20};
static std::atomic<int> g_withhold_copy{0};

}  // namespace gact

using namespace gact;

static inline bool misaligned(const void* p, uintptr_t a) { return ((uintptr_t)p & (a - 1)) != 0; }
static inline int elem_bytes(int dtype) { return dtype == GACT_F32 ? 4 : 2; }

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
    // x only has to be aligned to its element size (any contiguous tensor, as for the reference); the outputs,
    // which the caller allocates for this call, keep their vector alignment
    if (misaligned(x, elem_bytes(dtype)) || misaligned(packed, 16) || misaligned(qmin, elem_bytes(dtype)) ||
        misaligned(qscale, dtype == GACT_F16 ? 2 : 4))
        return GACT_ERR_ALIGN;
    QuantArgs a;
    a.x = x; a.n = n; a.G = (n + kGroup - 1) / kGroup;
    a.R = (a.G + 8 / bits - 1) / (8 / bits);
    a.seed = seed; a.noise = noise; a.packed = (uint8_t*)packed; a.qmin = qmin; a.qscale = qscale;
    a.align = misaligned(x, 16) ? 0 : (misaligned(x, 32) ? 16 : 32);
    a.wait_limit = g_wait_limit.load(std::memory_order_relaxed);
    a.withhold_copy = g_withhold_copy.load(std::memory_order_relaxed);
    a.rk = philox_round_keys(seed);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == GACT_F32) return dispatch_bits32(a, bits, rng_mode, fma_mode, s);
    return launch_quantize16(a, dtype, bits, rng_mode, s);
}

extern "C" void gact_pipeline_test_hook(uint32_t wait_limit, int withhold_one_copy) {
    g_wait_limit.store(wait_limit == 0 ? (1u << 20) : wait_limit, std::memory_order_relaxed);
    g_withhold_copy.store(withhold_one_copy ? 1 : 0, std::memory_order_relaxed);
}

extern "C" int gact_minimax(const void* x, int dtype, int64_t n, void* mn, void* mx, void* stream) {
    if (dtype < GACT_F32 || dtype > GACT_BF16) return GACT_ERR_DTYPE;
    if (n < 0) return GACT_ERR_SIZE;
    if (n == 0) return GACT_OK;
    if (!x || !mn || !mx) return GACT_ERR_NULL;
    if (misaligned(x, elem_bytes(dtype)) || misaligned(mn, elem_bytes(dtype)) || misaligned(mx, elem_bytes(dtype))) return GACT_ERR_ALIGN;
    const int align = misaligned(x, 16) ? 0 : 16;
    const int64_t G = (n + kGroup - 1) / kGroup;
    const int64_t want = (G + kQThreads / 32 - 1) / (kQThreads / 32);
    const int64_t cap = (int64_t)sm_count() * 8;
    const int blocks = (int)(want < cap ? want : cap);
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case GACT_F32: minimax_kernel<GACT_F32><<<blocks, kQThreads, 0, s>>>(x, n, G, align, mn, mx); break;
    case GACT_F16: minimax_kernel<GACT_F16><<<blocks, kQThreads, 0, s>>>(x, n, G, align, mn, mx); break;
    default: minimax_kernel<GACT_BF16><<<blocks, kQThreads, 0, s>>>(x, n, G, align, mn, mx); break;
    }
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}
