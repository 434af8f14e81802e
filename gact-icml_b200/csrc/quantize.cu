// Fused quantize: per-group min/max -> scale -> stochastic rounding -> bit packing, one pass over the input.
//
// Work decomposition.  A warp owns a tile of GPW consecutive groups (8 for the 16-bit types - 4 for small
// tensors -, max(4, wpt) for fp32), i.e. U = GPW/wpt whole row-blocks of the packed layout.  Each lane keeps its 8 consecutive values of
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
#include <atomic>

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
    int64_t tile_begin;      // first tile of the plain kernel (tiles before it belong to the bulk-copy kernel)
    PhiloxKeys rk;
};

// Tile of one warp: TG groups (at least one row-block, i.e. 8 / BITS groups).  16-bit inputs use 8 groups per
// tile for large tensors and 4 for small ones (shorter per-tile latency, finer spread over the SMs); fp32 uses 4.
template <int DT, int BITS, int TG> struct Tile {
    static constexpr int WPT = 8 / BITS;
    static constexpr int GPW = WPT > TG ? WPT : TG;
    static constexpr int U = GPW / WPT;
};
template <int DT> struct BigTile { static constexpr int value = (DT == GACT_F32) ? 4 : 8; };

// Which noise values reach codes8 "centred" (noise - 0.5 instead of noise).  With the 8-bit noise of FAST and the
// constant noise of RTN, and p a half-precision value, p + noise is exact in fp32, so (p + noise) - 0.5 equals
// p + (noise - 0.5) bit for bit and one addition is saved; bf16 (not a reference type) is defined on centred
// noise in every mode.  fp32 keeps the reference's order of operations.
template <int DT, int RNG> struct Centred {
    static constexpr bool value = (DT == GACT_BF16) || (DT == GACT_F16 && (RNG == GACT_RNG_FAST || RNG == GACT_RNG_RTN));
};
// FAST and RTN never produce a code above 2^bits - 1 (fp16: clamped, see codes8; fp32 / bf16: the noise stays
// below 1), so slots cannot collide and the packed byte may be summed instead of OR-ed.
template <int RNG> struct NoOverflow { static constexpr bool value = (RNG == GACT_RNG_FAST || RNG == GACT_RNG_RTN); };

// noise of the FAST arrangement: one Philox4x32-10 call, counter (block_lo, block_hi, 0, "FAST"), gives 16
// bytes = 8 bits for each of this lane's 8 elements of an even group (bytes 0..7) and of the following odd group
// (bytes 8..15); noise = (byte + 0.5) / 256 (minus 0.5 when CENTRED).  The bytes go to float on the conversion unit.
template <bool CENTRED>
__device__ __forceinline__ void fast_noise16(uint64_t block, const PhiloxKeys& rk, float2 (&even)[4], float2 (&odd)[4]) {
    const uint4 r = philox4x32_10((uint32_t)block, (uint32_t)(block >> 32), 0u, 0x46415354u, rk);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    // byte -> float without a conversion: a byte permute drops it into bits 8..15 of the mantissa of 2^23, giving
    // 2^23 + 256*b; times 2^-16 that is 128 + b/256, and the offset below brings (b + 0.5)/256 (- 0.5), all exact
    const float2 s2 = splat2(1.52587890625e-05f), o2 = splat2((CENTRED ? -0.498046875f : 0.001953125f) - 128.0f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float b0 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7504u)), b1 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7514u));
        const float b2 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7524u)), b3 = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7534u));
        float2 (&dst)[4] = (i < 2) ? even : odd;
        dst[(2 * i) & 3] = fma2(make_float2(b0, b1), s2, o2);
        dst[(2 * i + 1) & 3] = fma2(make_float2(b2, b3), s2, o2);
    }
}

// float(h) + c for both halves of a pair, one instruction each (sm_100 mixed-precision add: the half operand is
// widened exactly, so the result equals the conversion followed by an fp32 add)
__device__ __forceinline__ float2 mixed_add2(__half2 h, float2 c) {
    float2 d;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; add.rn.f32.f16 %0, lo, %3; add.rn.f32.f16 %1, hi, %4; }"
        : "=f"(d.x), "=f"(d.y) : "r"(*(const uint32_t*)&h), "f"(c.x), "f"(c.y));
    return d;
}

// the same for a pair of bf16 values
__device__ __forceinline__ float2 mixed_add2_bf16(uint32_t pair, float2 c) {
    float2 d;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; add.rn.f32.bf16 %0, lo, %3; add.rn.f32.bf16 %1, hi, %4; }"
        : "=f"(d.x), "=f"(d.y) : "r"(pair), "f"(c.x), "f"(c.y));
    return d;
}

// magic bits (code in the low mantissa bits of 1.5*2^23 + code) of the 8 codes of one group held by this
// lane; nz[i] = noise of elements 2i, 2i+1 (centred where Centred<DT, RNG> says so)
template <int DT, int BITS, int RNG, bool FMA>
__device__ __forceinline__ void codes8(const uint32_t (&raw)[RawRegs<DT>::N], float mn, float sc, const float2 (&nz)[4],
                                       uint32_t (&cb)[8]) {
    constexpr bool CENTRED = Centred<DT, RNG>::value;
    constexpr float MAXC = (float)((1 << BITS) - 1);
    if constexpr (DT == GACT_F16) {
        if (isinf(sc)) {
            // A half-precision scale overflows to +inf when the group's range is below (2^b-1)/65504.  The
            // reference then computes t*inf: +inf for every element above the minimum, which __float2int_rn
            // saturates to 0x7fffffff (all ones from the slot upwards), and NaN -> 0 for the minimum itself.
            // FAST / RTN clamp codes at 2^b - 1 instead.
            float v[8];
            raw_to_float<DT>(raw, v);
#pragma unroll
            for (int j = 0; j < 8; j++)
                cb[j] = (Elem<DT>::round(__fsub_rn(v[j], mn)) > 0.0f) ? (NoOverflow<RNG>::value ? (uint32_t)MAXC : 0x7fffffffu) : 0u;
            return;
        }
        const __half2 mn2 = __float2half2_rn(mn), sc2 = __float2half2_rn(sc);     // exact: both are half values
        const __half2 zero2 = __float2half2_rn(0.0f), maxc2 = __float2half2_rn(MAXC);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 t = __hsub2(*(const __half2*)&raw[i], mn2);
            __half2 p = __hmax2(__hmul2(t, sc2), zero2);                          // NaN -> 0, as max(., 0) does
            // The reference has no upper clamp: when the half-precision scale rounded up, the group maximum can
            // reach code 2^b and wrap / spill.  The reference stream (CURAND) and EXTERNAL reproduce that; FAST
            // and RTN clamp p at 2^b - 1, which caps the code as well.
            if (NoOverflow<RNG>::value) p = __hmin2(p, maxc2);
            float2 r;
            // float(p) + noise is one mixed-precision add per element (measured +5 % over convert, then packed add)
            if (RNG == GACT_RNG_RTN) r = add2(__half22float2(p), splat2(kMagic));                 // (p + 0.5) - 0.5 = p
            else if (CENTRED) r = add2(mixed_add2(p, nz[i]), splat2(kMagic));                     // p + (noise - 0.5)
            else r = add2(add2(mixed_add2(p, nz[i]), splat2(-0.5f)), splat2(kMagic));             // u - 0.5 > -0.5 rounds to 0
            cb[2 * i] = __float_as_uint(r.x);
            cb[2 * i + 1] = __float_as_uint(r.y);
        }
    } else {
        float v[8];
        raw_to_float<DT>(raw, v);
        const float2 nmn = splat2(-mn), sc2 = splat2(sc);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // x - mn; bf16 widens inside the add (one mixed-precision add per element, measured +2-4 %)
            const float2 t = (DT == GACT_BF16) ? mixed_add2_bf16(raw[DT == GACT_BF16 ? i : 0], nmn) : add2(make_float2(v[2 * i], v[2 * i + 1]), nmn);
            float2 w;
            if (DT == GACT_BF16) {
                // ours: u = fma(t, scale, noise - 0.5), clamped to [0, 2^bits - 1]
                w = fma2(t, sc2, nz[i]);
                w.x = fmaxf(w.x, 0.0f); w.y = fmaxf(w.y, 0.0f);                       // NaN -> 0
                if (!NoOverflow<RNG>::value) { w.x = fminf(w.x, MAXC); w.y = fminf(w.y, MAXC); }
            } else {
                const float2 u = FMA ? fma2(t, sc2, nz[i]) : add2(mul2(t, sc2), nz[i]);
                w = add2(u, splat2(-0.5f));
                w.x = fmaxf(w.x, 0.0f); w.y = fmaxf(w.y, 0.0f);                       // NaN -> 0; no upper clamp (reference)
            }
            const float2 r = add2(w, splat2(kMagic));
            cb[2 * i] = __float_as_uint(r.x);
            cb[2 * i + 1] = __float_as_uint(r.y);
        }
    }
}

// All loads of one tile (issued back to back, nothing waits on them here).  FULL: every group of the tile
// exists and is complete, so no bounds are tested.
template <int DT, int BITS, int TG, bool FULL>
__device__ __forceinline__ void load_tile(const QuantArgs& a, int64_t tile, int lane,
                                          uint32_t (&raw)[Tile<DT, BITS, TG>::GPW][RawRegs<DT>::N]) {
    constexpr int GPW = Tile<DT, BITS, TG>::GPW, NR = RawRegs<DT>::N;
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
template <int DT, int BITS, int RNG, bool FMA, int TG, bool FULL>
__device__ __forceinline__ void process_tile(const QuantArgs& a, int64_t tile, int lane,
                                             const uint32_t (&raw)[Tile<DT, BITS, TG>::GPW][RawRegs<DT>::N]) {
    using E = Elem<DT>;
    using T = typename E::T;
    constexpr int WPT = Tile<DT, BITS, TG>::WPT, GPW = Tile<DT, BITS, TG>::GPW, U = Tile<DT, BITS, TG>::U;
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
                    // cuRAND's uniform: float(word) * 2^-32 + 2^-33
                    const float2 s2 = splat2(2.3283064365386963e-10f), o2 = splat2(1.1641532182693481e-10f);
                    nz[0][i] = fma2(make_float2(__uint2float_rn(ra.x), __uint2float_rn(rb.x)), s2, o2);
                    if (WPT > 1) nz[1][i] = fma2(make_float2(__uint2float_rn(ra.y), __uint2float_rn(rb.y)), s2, o2);
                    if (WPT > 2) {
                        nz[2][i] = fma2(make_float2(__uint2float_rn(ra.z), __uint2float_rn(rb.z)), s2, o2);
                        nz[3][i] = fma2(make_float2(__uint2float_rn(ra.w), __uint2float_rn(rb.w)), s2, o2);
                    }
                }
                if (Centred<DT, RNG>::value) {
#pragma unroll
                    for (int q = 0; q < 4; q++)
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            if (q < WPT) nz[q][i] = add2(nz[q][i], splat2(-0.5f));
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int ni = c * 4 + q;
                    if (ni >= WPT) break;
                    const int k = u * WPT + ni;
                    if (!FULL && g0 + k >= a.G) break;         // tail row-block: absent groups leave zero bits
                    uint32_t cb[8];
                    codes8<DT, BITS, RNG, FMA>(raw[k], mn[k], sc[k], nz[q], cb);
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[j] |= cb[j] << (ni * BITS);
                }
            }
        } else {
#pragma unroll
#pragma unroll
            for (int ni = 0; ni < WPT; ni++) {
                const int k = u * WPT + ni;
                if (!FULL && g0 + k >= a.G) break;
                float2 nz[4];
                if (RNG == GACT_RNG_FAST) {
                    if ((k & 1) == 0) {
                        fast_noise16<Centred<DT, RNG>::value>((uint64_t)((g0 + k) >> 1) * (kGroup / 8) + lane, a.rk, nz, nz_odd);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++) nz[i] = nz_odd[i];
                    }
                } else if (RNG == GACT_RNG_RTN) {
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = splat2(Centred<DT, RNG>::value ? 0.0f : 0.5f);
                } else {
                    const float2* p = (const float2*)(a.noise + (g0 + k) * kGroup + lane * 8);
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = Centred<DT, RNG>::value ? add2(p[i], splat2(-0.5f)) : p[i];
                }
                uint32_t cb[8];
                codes8<DT, BITS, RNG, FMA>(raw[k], mn[k], sc[k], nz, cb);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (NoOverflow<RNG>::value) acc[j] += cb[j] << (ni * BITS);      // disjoint slots: a sum is an OR
                    else acc[j] |= cb[j] << (ni * BITS);
                }
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

template <int DT, int BITS, int RNG, bool FMA, int TG>
__global__ void __launch_bounds__(kQThreads, GACT_QMINB) quantize_kernel(const __grid_constant__ QuantArgs a) {
    constexpr int GPW = Tile<DT, BITS, TG>::GPW, NR = RawRegs<DT>::N;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kQThreads / 32);
    const int64_t tiles = (a.G + GPW - 1) / GPW;
    const int64_t full_tiles = a.n / (GPW * kGroup);            // tiles whose groups all exist and are complete
    for (int64_t tile = a.tile_begin + (int64_t)blockIdx.x * (kQThreads / 32) + (threadIdx.x >> 5); tile < tiles; tile += nwarps) {
        uint32_t raw[GPW][NR];
        if (tile < full_tiles) {
            load_tile<DT, BITS, TG, true>(a, tile, lane, raw);
            process_tile<DT, BITS, RNG, FMA, TG, true>(a, tile, lane, raw);
        } else {
            load_tile<DT, BITS, TG, false>(a, tile, lane, raw);
            process_tile<DT, BITS, RNG, FMA, TG, false>(a, tile, lane, raw);
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Bulk-copy pipeline (large 16-bit tensors with generated noise, see launch_quantize).  Persistent CTAs of 8 consumer warps + 1 producer warp.  The producer's
// elected lane streams chunks of the input (one tile per consumer warp: 32 KB, or 64 KB for 1-bit fp32) into a
// 3-stage (2 for the 64 KB chunks) shared-memory ring with cp.async.bulk (the TMA
// engine, plain 1-D copies of this GPU's own memory, no multicast); an mbarrier per stage counts the bytes in.
// Each consumer warp takes its tile of the chunk out of shared memory (16- or 32-byte reads, conflict free),
// releases the stage, and runs the same tile routine as the plain kernel.  64 KB per CTA are in flight
// whatever the warps are doing, so HBM latency is hidden without holding loads in registers.
// Every wait is bounded: a wait that runs out sets g_pipeline_error and the CTA winds down.
// ---------------------------------------------------------------------------------------------------
constexpr int kPipeWarps = 8;                         // consumer warps
constexpr int kPipeThreads = (kPipeWarps + 1) * 32;
constexpr uint32_t kWaitLimit = 1u << 20;
#ifndef GACT_PIPE_STAGES
#define GACT_PIPE_STAGES 3
#endif
#ifndef GACT_PIPE_MINB
#define GACT_PIPE_MINB 2
#endif
template <int DT, int BITS> struct Pipe {
    static constexpr int kChunkBytes = kPipeWarps * Tile<DT, BITS, BigTile<DT>::value>::GPW * kGroup * Elem<DT>::kBytes;
    static constexpr int kStages = kChunkBytes <= 32 * 1024 ? GACT_PIPE_STAGES : 2;
};

__device__ int g_pipeline_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// true once the phase with the given parity has completed; gives up after kWaitLimit polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int DT, int BITS, int RNG, bool FMA>
__global__ void __launch_bounds__(kPipeThreads, GACT_PIPE_MINB) quantize_pipe_kernel(const __grid_constant__ QuantArgs a, int64_t nchunks) {
    constexpr int TG = BigTile<DT>::value;
    constexpr int GPW = Tile<DT, BITS, TG>::GPW, NR = RawRegs<DT>::N;
    constexpr int kChunkBytes = Pipe<DT, BITS>::kChunkBytes, kPipeStages = Pipe<DT, BITS>::kStages;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t bars[2 * kPipeStages];       // [0..S) full, [S..2S) empty
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars), ring = smem_u32(smem);

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < kPipeStages; s++) {
            mbar_init(bar0 + 8 * s, 1);                           // full: the producer's expect_tx arrival
            mbar_init(bar0 + 8 * (kPipeStages + s), kPipeWarps);  // empty: one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kPipeWarps) {
        // ---- producer ----
        if (lane == 0) {
            int64_t issued = 0;
            bool ok = true;
            for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x, ++issued) {
                const int s = (int)(issued % kPipeStages);
                if (issued >= kPipeStages && !mbar_wait(bar0 + 8 * (kPipeStages + s), (uint32_t)((issued / kPipeStages - 1) & 1))) {
                    ok = false;
                    break;
                }
                mbar_expect_tx(bar0 + 8 * s, kChunkBytes);
                bulk_load(ring + s * kChunkBytes, (const unsigned char*)a.x + c * kChunkBytes, kChunkBytes, bar0 + 8 * s);
            }
            if (!ok) {
                atomicExch(&g_pipeline_error, 1);
                // do not leave while copies into this CTA's shared memory may still be in flight
                const int64_t first = issued > kPipeStages ? issued - kPipeStages : 0;
                for (int64_t i = first; i < issued; ++i)
                    mbar_wait(bar0 + 8 * (int)(i % kPipeStages), (uint32_t)((i / kPipeStages) & 1));
            }
        }
        return;
    }

    // ---- consumers ----
    int64_t done = 0;
    for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x, ++done) {
        const int s = (int)(done % kPipeStages);
        // all lanes poll; the verdict is taken jointly so that the warp never splits
        if (!__all_sync(kFull, mbar_wait(bar0 + 8 * s, (uint32_t)((done / kPipeStages) & 1)))) {
            if (lane == 0) atomicExch(&g_pipeline_error, 2);
            return;
        }
        uint32_t raw[GPW][NR];
        const unsigned char* src = smem + s * kChunkBytes + warp * (GPW * kGroup * Elem<DT>::kBytes) + lane * (8 * Elem<DT>::kBytes);
#pragma unroll
        for (int k = 0; k < GPW; k++) {
            const uint4* p = (const uint4*)(src + k * (kGroup * Elem<DT>::kBytes));
            if constexpr (DT == GACT_F32) {
                const uint4 v0 = p[0], v1 = p[1];
                raw[k][0] = v0.x; raw[k][1] = v0.y; raw[k][2] = v0.z; raw[k][3] = v0.w;
                raw[k][4] = v1.x; raw[k][5] = v1.y; raw[k][6] = v1.z; raw[k][7] = v1.w;
            } else {
                const uint4 v0 = p[0];
                raw[k][0] = v0.x; raw[k][1] = v0.y; raw[k][2] = v0.z; raw[k][3] = v0.w;
            }
        }
        __threadfence_block();                                       // this lane's reads of the stage are done
        __syncwarp();
        if (lane == 0) mbar_arrive(bar0 + 8 * (kPipeStages + s));    // the stage may be refilled
        process_tile<DT, BITS, RNG, FMA, TG, true>(a, c * kPipeWarps + warp, lane, raw);
    }
}

// smallest number of whole chunks for which the ring kernel is used (see launch_quantize); gact_set_ring_min_chunks
static std::atomic<int64_t> g_ring_min_chunks{1536};
constexpr int kMaxDevices = 64;
constexpr int64_t kSmallTileMaxGroups = 40960;      // 16-bit tensors of up to 20 MB take tiles of 4 groups

// direct-load kernel over the tiles from a.tile_begin on (in tiles of TG groups)
template <int DT, int BITS, int RNG, bool FMA, int TG>
static int launch_plain(const QuantArgs& a, cudaStream_t s) {
    constexpr int GPW = Tile<DT, BITS, TG>::GPW;
    const int64_t tiles = (a.G + GPW - 1) / GPW - a.tile_begin;
    if (tiles <= 0) return GACT_OK;
    static int resident = 0;
    if (resident == 0) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_kernel<DT, BITS, RNG, FMA, TG>, kQThreads, 0) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        resident = per_sm * kSMs;
    }
    const int64_t want = (tiles + kQThreads / 32 - 1) / (kQThreads / 32);
    const int blocks = (int)(want < resident ? want : resident);
    quantize_kernel<DT, BITS, RNG, FMA, TG><<<blocks, kQThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

template <int DT, int BITS, int RNG, bool FMA>
static int launch_quantize(const QuantArgs& args, cudaStream_t s) {
    constexpr int kBig = BigTile<DT>::value;
    constexpr int kChunkBytes = Pipe<DT, BITS>::kChunkBytes, kPipeStages = Pipe<DT, BITS>::kStages;
    QuantArgs a = args;
    a.tile_begin = 0;
    // Which kernel (all measured).  The bulk-copy ring pays off where the tile routine is long (16-bit inputs with
    // generated noise) and the tensor is large: with only a few chunks per CTA its whole-chunk granularity leaves
    // SMs unevenly loaded (33 MB bf16: 18.4 us direct vs 20.5 us ring; 67 MB: 30.7 vs 28.7).  fp32 inputs,
    // round-to-nearest and everything below ~48 MB run from direct loads, 16-bit tensors of up to 20 MB with tiles
    // of 4 groups instead of 8: the shorter tile brings a 16 MB launch from 8.9 to 7.7 us and a 1 MB one from 3.5 to 2.8.
    constexpr bool kUsePipe = (DT != GACT_F32) && (RNG != GACT_RNG_RTN);
    if constexpr (kUsePipe) {
        const int64_t nchunks = a.n / (kChunkBytes / Elem<DT>::kBytes);
        // the shared-memory opt-in is a per-device attribute of the kernel: 0 = not set up, 1 = usable, -1 = refused
        static int ready_on[kMaxDevices] = {0};
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = kMaxDevices - 1;
        int& pipe_ready = ready_on[dev];
        if (pipe_ready == 0) {
            pipe_ready = cudaFuncSetAttribute(quantize_pipe_kernel<DT, BITS, RNG, FMA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              kPipeStages * kChunkBytes) == cudaSuccess ? 1 : -1;
        }
        if (nchunks >= g_ring_min_chunks.load(std::memory_order_relaxed) && pipe_ready == 1) {
            static int pipe_resident = 0;
            if (pipe_resident == 0) {
                int per_sm = 0;
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_pipe_kernel<DT, BITS, RNG, FMA>, kPipeThreads,
                                                                  kPipeStages * kChunkBytes) != cudaSuccess || per_sm < 1)
                    per_sm = 1;
                pipe_resident = per_sm * kSMs;
            }
            // one resident wave, with the chunks spread evenly: every CTA gets the same number of chunks (+-1)
            const int64_t cap = pipe_resident;
            const int64_t rounds = (nchunks + cap - 1) / cap;
            const int blocks = (int)((nchunks + rounds - 1) / rounds);
            quantize_pipe_kernel<DT, BITS, RNG, FMA><<<blocks, kPipeThreads, kPipeStages * kChunkBytes, s>>>(a, nchunks);
            if (cudaGetLastError() != cudaSuccess) return GACT_ERR_LAUNCH;
            a.tile_begin = nchunks * kPipeWarps;
            return launch_plain<DT, BITS, RNG, FMA, kBig>(a, s);         // what is left: less than one chunk
        }
    }
    if constexpr (DT != GACT_F32 && BITS > 1) {
        if (a.G <= kSmallTileMaxGroups) return launch_plain<DT, BITS, RNG, FMA, 4>(a, s);
    }
    return launch_plain<DT, BITS, RNG, FMA, kBig>(a, s);
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
    a.tile_begin = 0;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case GACT_F32: return dispatch_bits<GACT_F32>(a, bits, rng_mode, fma_mode, s);
    case GACT_F16: return dispatch_bits<GACT_F16>(a, bits, rng_mode, fma_mode, s);
    default: return dispatch_bits<GACT_BF16>(a, bits, rng_mode, fma_mode, s);
    }
}

extern "C" int gact_pipeline_error(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_pipeline_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

extern "C" int64_t gact_set_ring_min_chunks(int64_t min_chunks) {
    if (min_chunks < 1) return g_ring_min_chunks.load(std::memory_order_relaxed);
    return g_ring_min_chunks.exchange(min_chunks, std::memory_order_relaxed);
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
