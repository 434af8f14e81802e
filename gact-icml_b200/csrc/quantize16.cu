// Fused quantize for fp16 / bf16 inputs: per-group min/max -> scale -> stochastic rounding -> bit packing, one
// pass over the input in HBM.
//
// Work decomposition.  A warp owns a tile of 8 consecutive groups (4 KB of input); each lane owns 8 consecutive
// values (16 bytes) of every group, so a group is one fully coalesced 512-byte row and a lane's 8 packed bytes of a
// row-block are contiguous (one 8-byte store).
//
// Input staging.  Every warp runs its own two-stage ring in shared memory: its elected lane brings the warp's next
// tile in with one cp.async.bulk (the TMA engine; a plain 1-D copy of this GPU's own memory, no multicast, no
// cluster) that completes on the stage's mbarrier, while the warp works on the current tile.  Nothing is shared
// between warps, so there is no producer warp and no block-wide barrier; 24 warps per SM keep up to 192 KB of
// loads in flight without holding them in registers.  The tile is read from shared memory twice (min/max pass,
// code pass), which keeps the routine below 80 registers.  Every wait is bounded: a wait that runs out records an
// error (gact_pipeline_error), the warp waits - bounded again - for its other copy in flight, and leaves.
// Tiles the bulk copies cannot take (the ragged last tile, and the whole tensor when x is not 16-byte aligned)
// are read straight from global memory, element by element where they must be.
//
// Tile routine.
//   pass 1  for the reduction a lane takes one contiguous 32nd of the tile (eight 16-byte chunks of ONE group,
//           visited in a lane-dependent rotation to stay off bank conflicts), runs one two-wide min / max chain
//           over them, folds the result into one word (min, -max) and finishes with two exchanges between the four
//           lanes of the group; lanes 4k..4k+3 end up with group k's pair, compute its scale and write min / scale.
//           The chain propagates NaN, which tells pass 2 whether a group holds one; a tile that does is reduced
//           again with NaN ignored, as the reference does.  (Tiles read from global memory keep per-group chains
//           and a butterfly over the eight words.)
//           fp16 scale: the reference's double-precision quotient rounded to float and then to half is taken from
//           an fp32 reciprocal whenever that cannot change the result (quotient further than 16 fp32 ulps from
//           every half-precision rounding boundary, checked on the bit pattern); the double-precision path
//           remains for the other ~0.4 % of the groups.
//   pass 2  (x - min) * scale in two-wide half arithmetic with the reference's roundings (fp16), or one
//           mixed-precision subtract and a packed fma in fp32 (bf16); noise added in fp32; w + 1.5*2^23 leaves
//           rint(w) in the low mantissa bits (no conversion instruction); slots are summed with multiply-adds and
//           the bytes cut out with byte permutes.  fp16 round-to-nearest never leaves half precision: p + 1024
//           rounds to the integer in the low mantissa bits of each half and two codes travel per instruction.
//           Groups come in three kinds - plain, guarded (a NaN, an infinity, an overflowing range: the lower clamp
//           matters), special (scale +inf / not positive); a tile of plain groups only, which is almost every
//           tile, runs a copy of the pass compiled without any per-group test.
#include <atomic>

#include "quantize_common.cuh"

namespace gact {

constexpr int kTGMax = 8;                            // groups per warp tile: 8, or 4 for tensors of few tiles
constexpr int kTileBytesMax = kTGMax * kGroup * 2;   // 4096: a stage of a warp's ring
#ifndef GACT_Q16_STAGES
#define GACT_Q16_STAGES 2
#endif
#ifndef GACT_Q16_MINB
#define GACT_Q16_MINB 3
#endif
constexpr int kStages = GACT_Q16_STAGES;
#ifndef GACT_Q16_WARPS
#define GACT_Q16_WARPS 8
#endif
constexpr int kWarps = GACT_Q16_WARPS;               // warps per block, each with its own ring
constexpr int kThreads16 = kWarps * 32;
constexpr int kSmemBytes = kWarps * kStages * kTileBytesMax;   // 64 KB per block, 3 blocks per SM

__device__ int g_pipeline_error = 0;

// ---- two-wide helpers on the bit patterns of half2 / bfloat162 --------------------------------------------------
// NP: NaN-propagating (a NaN operand gives NaN) instead of NaN-ignoring
template <int DT, bool NP = false> __device__ __forceinline__ uint32_t pmin2(uint32_t a, uint32_t b) {
    if constexpr (DT == GACT_F16) {
        const __half2 x = *(const __half2*)&a, y = *(const __half2*)&b;
        const __half2 r = NP ? __hmin2_nan(x, y) : __hmin2(x, y);
        return *(const uint32_t*)&r;
    } else {
        const __nv_bfloat162 x = *(const __nv_bfloat162*)&a, y = *(const __nv_bfloat162*)&b;
        const __nv_bfloat162 r = NP ? __hmin2_nan(x, y) : __hmin2(x, y);
        return *(const uint32_t*)&r;
    }
}
template <int DT, bool NP = false> __device__ __forceinline__ uint32_t pmax2(uint32_t a, uint32_t b) {
    if constexpr (DT == GACT_F16) {
        const __half2 x = *(const __half2*)&a, y = *(const __half2*)&b;
        const __half2 r = NP ? __hmax2_nan(x, y) : __hmax2(x, y);
        return *(const uint32_t*)&r;
    } else {
        const __nv_bfloat162 x = *(const __nv_bfloat162*)&a, y = *(const __nv_bfloat162*)&b;
        const __nv_bfloat162 r = NP ? __hmax2_nan(x, y) : __hmax2(x, y);
        return *(const uint32_t*)&r;
    }
}
__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *(const __half2*)&v; }
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *(const uint32_t*)&v; }
template <int DT> __device__ __forceinline__ float pair_lo(uint32_t v) {
    if constexpr (DT == GACT_F16) return __half2float(__ushort_as_half((unsigned short)(v & 0xffffu)));
    else return __uint_as_float(v << 16);
}
template <int DT> __device__ __forceinline__ float pair_hi(uint32_t v) {
    if constexpr (DT == GACT_F16) return __half2float(__ushort_as_half((unsigned short)(v >> 16)));
    else return __uint_as_float(v & 0xffff0000u);
}
// (hi, hi) with hi = the reference's start value 1e30 in T (half: +inf)
template <int DT> __device__ __forceinline__ uint32_t start_pair() { return DT == GACT_F16 ? 0x7c007c00u : 0x714a714au; }

// (min, -max) of the lane's 8 values.  NP = false: NaN values are ignored (an all-NaN lane yields NaN, ignored
// further on), which is the reference's min / max.  NP = true: any NaN makes both halves NaN - the same instruction
// count, and the result doubles as the test for "this group holds a NaN".
template <int DT, bool NP> __device__ __forceinline__ uint32_t lane_min_negmax(const uint32_t (&raw)[4]) {
    const uint32_t lo = pmin2<DT, NP>(pmin2<DT, NP>(raw[0], raw[1]), pmin2<DT, NP>(raw[2], raw[3]));
    const uint32_t hi = pmax2<DT, NP>(pmax2<DT, NP>(raw[0], raw[1]), pmax2<DT, NP>(raw[2], raw[3]));
    const uint32_t nh = hi ^ 0x80008000u;
    return pmin2<DT, NP>(__byte_perm(lo, nh, 0x5410u), __byte_perm(lo, nh, 0x7632u));
}

// Warp reduction of the tile's TG (min, -max) words at once.  The first log2(TG) exchanges (distance 16, 8, ...)
// each halve the number of words a lane still carries (a lane keeps the groups whose index bit matches its lane bit
// and hands the others over); the remaining distances finish the one word left.  With L = 32 / TG, lanes
// L*k .. L*k + L-1 return group k's word.
template <int DT, int TG, bool NP> __device__ __forceinline__ uint32_t tile_reduce(uint32_t (&v)[TG], int lane) {
    static_assert(TG == 4 || TG == 8, "tile of 4 or 8 groups");
    int dist = 16;
#pragma unroll
    for (int half = TG / 2; half >= 1; half >>= 1, dist >>= 1) {
        const bool up = (lane & dist) != 0;
#pragma unroll
        for (int i = 0; i < half; i++) {
            const uint32_t keep = up ? v[i + half] : v[i], send = up ? v[i] : v[i + half];
            v[i] = pmin2<DT, NP>(keep, __shfl_xor_sync(kFull, send, dist));
        }
    }
#pragma unroll
    for (; dist >= 1; dist >>= 1) v[0] = pmin2<DT, NP>(v[0], __shfl_xor_sync(kFull, v[0], dist));
    return v[0];
}

// scale of an fp16 group, T(double(T(2^b - 1)) / (double(T(mx - mn)) + 2e-6)) with T reached through float
// (quantization_cuda_kernel.cu:33), from an fp32 reciprocal where the two roundings cannot tell the difference.
template <int BITS> __device__ __forceinline__ float scale_f16(float mn, float mx) {
    constexpr float MAXC = (float)((1 << BITS) - 1);
    const float r = Elem<GACT_F16>::round(__fsub_rn(mx, mn));
    float rcp;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"(__fadd_rn(r, 2e-6f)));
    float q = MAXC * rcp;                                  // within 4 fp32 ulps of the double-precision quotient
    // The result is half(float(quotient)).  Half-precision rounding boundaries are the fp32 values whose low 13
    // mantissa bits read 0x1000; an estimate at least 16 ulps away from all of them rounds like the exact quotient
    // (this holds for results in the normal half range and above it, where everything becomes +inf).
    const uint32_t low = __float_as_uint(q) & 0x1fffu;
    if ((low - (0x1000u - 16u)) < 32u || !(q >= 6.2e-5f))  // near a boundary, subnormal, zero, negative or NaN
        q = __double2float_rn((double)MAXC / ((double)r + 2e-6));
    return Elem<GACT_F16>::round(q);
}

// ---- sources of a tile's values ----------------------------------------------------------------------------------
// the warp's stage in shared memory; `base` already points at this lane's 16 bytes of group 0
struct SmemSrc {
    const unsigned char* base;
    __device__ __forceinline__ void load(int k, uint32_t (&raw)[4]) const {
        const uint4 v = *(const uint4*)(base + k * (kGroup * 2));
        raw[0] = v.x; raw[1] = v.y; raw[2] = v.z; raw[3] = v.w;
    }
    __device__ __forceinline__ uint32_t load_pair(int k, int i) const { return *(const uint32_t*)(base + k * (kGroup * 2) + i * 4); }
};
// global memory, bounds-checked; elements at or past n (and whole groups at or past G) read as +0
template <int DT> struct GlobalSrc {
    const void* x;
    int64_t n, g0;
    int lane, align;
    __device__ __forceinline__ void load(int k, uint32_t (&raw)[4]) const { load_raw<DT>(x, n, g0 + k, lane, align, raw); }
    __device__ __forceinline__ uint32_t load_pair(int k, int i) const {
        uint32_t raw[4];
        load(k, raw);
        return raw[i];
    }
};

// (min, -max) of every group of the tile; lanes L*k .. L*k + L-1 return group k's word
template <int DT, int TG, bool NP, class Src> __device__ __forceinline__ uint32_t tile_min_negmax(const Src& src, int lane) {
    uint32_t v[TG];
#pragma unroll
    for (int k = 0; k < TG; k++) {
        uint32_t raw[4];
        src.load(k, raw);
        v[k] = lane_min_negmax<DT, NP>(raw);
    }
    // the reference starts from +-1e30 in T, which is what remains of a group of NaNs
    return pmin2<DT, NP>(tile_reduce<DT, TG, NP>(v, lane), start_pair<DT>());
}

// The same for a tile that lies in shared memory.  A reduction does not care which lane looks at which element, so
// here a lane takes one contiguous 32nd of the tile - 8 (TG = 8) or 4 chunks of 16 bytes, all of ONE group - instead
// of 16 bytes of every group: one long min / max chain per lane and L-1 exchanges between the L = 32 / TG lanes of a
// group, 70 instructions per lane and tile of 8 groups instead of 112 for per-group chains, the fold of each and the
// butterfly.  The chunks are visited in a lane-dependent rotation, which keeps the 16-byte reads of a quarter-warp
// on different banks.
template <int DT, int TG, bool NP> __device__ __forceinline__ uint32_t tile_min_negmax(const SmemSrc& src, int lane) {
    constexpr int CH = TG * kGroup * 2 / 32 / 16, LPG = 32 / TG;
    const unsigned char* mine = src.base + lane * ((CH - 1) * 16);          // base already holds lane * 16
    const int rot = lane * CH / 8;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < CH; j++) {
        const uint4 v = *(const uint4*)(mine + ((j + rot) & (CH - 1)) * 16);
        const uint32_t a = pmin2<DT, NP>(pmin2<DT, NP>(v.x, v.y), pmin2<DT, NP>(v.z, v.w));
        const uint32_t b = pmax2<DT, NP>(pmax2<DT, NP>(v.x, v.y), pmax2<DT, NP>(v.z, v.w));
        lo = j == 0 ? a : pmin2<DT, NP>(lo, a);
        hi = j == 0 ? b : pmax2<DT, NP>(hi, b);
    }
    const uint32_t nh = hi ^ 0x80008000u;
    uint32_t v = pmin2<DT, NP>(__byte_perm(lo, nh, 0x5410u), __byte_perm(lo, nh, 0x7632u));
#pragma unroll
    for (int dist = 1; dist < LPG; dist <<= 1) v = pmin2<DT, NP>(v, __shfl_xor_sync(kFull, v, dist));
    return pmin2<DT, NP>(v, start_pair<DT>());
}

// ---- codes of one pair of elements, as magic bits (1.5*2^23 + code) ------------------------------------------------
// fp16: the reference's half-precision arithmetic, p = round_h(round_h(x - mn) * scale), max(p, 0) (NaN -> 0), no
// upper clamp in the reference's modes (CURAND, EXTERNAL), clamp at 2^b - 1 in FAST / RTN.
// GUARD = false: a group of finite values only, with a finite scale > 0.  There x - mn >= 0 (or +inf, by overflow),
// the product is never NaN or negative, and max(p, 0) is the identity: it is left out.
template <int BITS, int RNG, bool GUARD>
__device__ __forceinline__ void code_pair_f16(uint32_t rawp, uint32_t mn2, uint32_t sc2, float2 nz, uint32_t& c0, uint32_t& c1) {
    constexpr float MAXC = (float)((1 << BITS) - 1);
    const __half2 zero2 = __float2half2_rn(0.0f), maxc2 = __float2half2_rn(MAXC);
    const __half2 t = __hsub2(as_h2(rawp), as_h2(mn2));
    __half2 p = __hmul2(t, as_h2(sc2));
    if (GUARD) p = __hmax2(p, zero2);
    if (NoOverflow<RNG>::value) p = __hmin2(p, maxc2);
    float2 r;
    if (RNG == GACT_RNG_RTN) r = add2(__half22float2(p), splat2(kMagic));                        // (p + 0.5) - 0.5 = p
    else if (Centred<GACT_F16, RNG>::value) r = add2(mixed_add2(p, nz), splat2(kMagic));         // p + (noise - 0.5)
    else r = add2(add2(mixed_add2(p, nz), splat2(-0.5f)), splat2(kMagic));                       // u - 0.5 >= -0.5 rounds to 0
    c0 = __float_as_uint(r.x);
    c1 = __float_as_uint(r.y);
}
// fp16 group whose scale overflowed to +inf (range below (2^b-1)/65504): the reference computes t*inf, +inf for
// every element above the minimum, which __float2int_rn saturates to 0x7fffffff (all ones from the slot upwards),
// and NaN -> 0 for the minimum itself.  FAST / RTN clamp at 2^b - 1 instead.
template <int BITS, int RNG>
__device__ __forceinline__ void code_pair_f16_inf(uint32_t rawp, uint32_t mn2, uint32_t& c0, uint32_t& c1) {
    const float2 t = __half22float2(__hsub2(as_h2(rawp), as_h2(mn2)));
    const uint32_t top = NoOverflow<RNG>::value ? (uint32_t)((1 << BITS) - 1) : 0x7fffffffu;
    c0 = t.x > 0.0f ? top : 0u;
    c1 = t.y > 0.0f ? top : 0u;
}
// fp16, round to nearest, staying in half precision: returns (0x6400 + code) in each half
// (KIND: 0 plain, 1 guarded, 2 scale +inf - see GroupConst)
template <int BITS, int KIND> __device__ __forceinline__ uint32_t code_pair_f16_rtn(uint32_t rawp, uint32_t mn2, uint32_t sc2) {
    constexpr float MAXC = (float)((1 << BITS) - 1);
    const __half2 zero2 = __float2half2_rn(0.0f), maxc2 = __float2half2_rn(MAXC);
    const __half2 t = __hsub2(as_h2(rawp), as_h2(mn2));
    __half2 p;
    if (KIND == 2) p = __hmul2(__hgt2(t, zero2), maxc2);                                         // t > 0 ? 2^b - 1 : 0
    else if (KIND == 1) p = __hmin2(__hmax2(__hmul2(t, as_h2(sc2)), zero2), maxc2);
    else p = __hmin2(__hmul2(t, as_h2(sc2)), maxc2);
    return h2_bits(__hadd2(p, __float2half2_rn(1024.0f)));
}
// bf16 (our semantics): u = fma(x - mn, scale, noise - 0.5) in fp32, clamped to [0, 2^b - 1], NaN -> 0.
// KIND 0: finite values only and scale > 0: u >= -0.5 and never NaN, both lower clamp and NaN rule are implied.
// KIND 1: scale > 0 but the group holds a NaN: max(x, mn) - a two-wide instruction that ignores NaN - sends it to
// the minimum, i.e. to code 0, like the clamp does.  KIND 2: anything else (an infinity in the group): clamped in fp32.
template <int BITS, int RNG, int KIND>
__device__ __forceinline__ void code_pair_bf16(uint32_t rawp, uint32_t mn2, float nmn, float sc, float2 nz, uint32_t& c0, uint32_t& c1) {
    constexpr float MAXC = (float)((1 << BITS) - 1);
    constexpr bool PLAIN = KIND != 2;
    if (KIND == 1) rawp = pmax2<GACT_BF16>(rawp, mn2);
    const float2 t = mixed_add2_bf16(rawp, splat2(nmn));
    float2 w = fma2(t, splat2(sc), nz);
    if (!PLAIN) { w.x = fmaxf(w.x, 0.0f); w.y = fmaxf(w.y, 0.0f); }
    if (!NoOverflow<RNG>::value) { w.x = fminf(w.x, MAXC); w.y = fminf(w.y, MAXC); }
    const float2 r = add2(w, splat2(kMagic));
    c0 = __float_as_uint(r.x);
    c1 = __float_as_uint(r.y);
}

// what every lane needs to know about one group in pass 2.  Kinds of group: 0 = plain (finite values only, a
// finite scale > 0), 1 = guarded (it holds a NaN or, fp16, its scale is 0 or NaN because of an infinity or an
// overflowing range: the reference's max(., 0) matters), 2 = special (fp16: scale +inf; bf16: not (scale > 0)).
// Which groups are special / guarded travels as two ballot masks (bit L*k = group k): warp-uniform values.
template <int DT> struct GroupConst;
// fp16: lane L*k publishes min and scale, each already doubled into both halves of a word, so that pass 2 gets its
// two-wide operands with two shuffles and no further instruction.
template <> struct GroupConst<GACT_F16> {
    uint32_t mn2, sc2;
    int kind;
    __device__ __forceinline__ void fetch(uint32_t w0, uint32_t w1, int src, unsigned smask, unsigned gmask) {
        mn2 = __shfl_sync(kFull, w0, src);
        sc2 = __shfl_sync(kFull, w1, src);
        kind = ((smask >> src) & 1u) ? 2 : ((gmask >> src) & 1u) ? 1 : 0;
    }
};
template <> struct GroupConst<GACT_BF16> {
    uint32_t mn2;
    float nmn, sc;
    int kind;
    __device__ __forceinline__ void fetch(uint32_t w0, uint32_t w1, int src, unsigned smask, unsigned gmask) {
        const uint32_t m = __shfl_sync(kFull, w0, src);
        sc = __uint_as_float(__shfl_sync(kFull, w1, src));
        const __nv_bfloat162 hi = __high2bfloat162(*(const __nv_bfloat162*)&m);
        mn2 = *(const uint32_t*)&hi;
        nmn = -__uint_as_float(m);
        kind = ((smask >> src) & 1u) ? 2 : ((gmask >> src) & 1u) ? 1 : 0;
    }
};

template <int DT, int BITS, int RNG, int KIND>
__device__ __forceinline__ void code_pair_as(uint32_t rawp, const GroupConst<DT>& gc, float2 nz, uint32_t& c0, uint32_t& c1) {
    if constexpr (DT == GACT_F16) {
        if (KIND == 2) code_pair_f16_inf<BITS, RNG>(rawp, gc.mn2, c0, c1);
        else code_pair_f16<BITS, RNG, KIND == 1>(rawp, gc.mn2, gc.sc2, nz, c0, c1);
    } else {
        code_pair_bf16<BITS, RNG, KIND>(rawp, gc.mn2, gc.nmn, gc.sc, nz, c0, c1);
    }
}
// one pair, kind decided here (the reference-stream arrangement works pair by pair)
template <int DT, int BITS, int RNG>
__device__ __forceinline__ void code_pair(uint32_t rawp, const GroupConst<DT>& gc, float2 nz, uint32_t& c0, uint32_t& c1) {
    if (gc.kind == 0) code_pair_as<DT, BITS, RNG, 0>(rawp, gc, nz, c0, c1);
    else if (gc.kind == 1) code_pair_as<DT, BITS, RNG, 1>(rawp, gc, nz, c0, c1);
    else code_pair_as<DT, BITS, RNG, 2>(rawp, gc, nz, c0, c1);
}
// the eight codes of a group; the kind is decided once for the group (it is the same for the whole warp)
template <int DT, int BITS, int RNG>
__device__ __forceinline__ void codes8(const uint32_t (&raw)[4], const GroupConst<DT>& gc, const float2 (&nz)[4], uint32_t (&cb)[8]) {
    if (gc.kind == 0) {
#pragma unroll
        for (int i = 0; i < 4; i++) code_pair_as<DT, BITS, RNG, 0>(raw[i], gc, nz[i], cb[2 * i], cb[2 * i + 1]);
    } else if (gc.kind == 1) {
#pragma unroll
        for (int i = 0; i < 4; i++) code_pair_as<DT, BITS, RNG, 1>(raw[i], gc, nz[i], cb[2 * i], cb[2 * i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) code_pair_as<DT, BITS, RNG, 2>(raw[i], gc, nz[i], cb[2 * i], cb[2 * i + 1]);
    }
}
// acc + (v << SHIFT) as a multiply-add: on the FMA pipe, which this kernel leaves idle, rather than the ALU
__device__ __forceinline__ uint32_t shl_add(uint32_t v, int shift, uint32_t acc) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(v), "r"(1u << shift), "r"(acc));      // shift is a constant once unrolled
    return d;
}

// The code pass of a tile: w0 / w1 are the words lanes L*k publish for group k (see GroupConst), smask / gmask the
// ballots of special and guarded groups.
template <int DT, int BITS, int RNG, int TG, bool FULL, class Src>
__device__ __forceinline__ void tile16_codes(const QuantArgs& a, int64_t tile, int lane, const Src& src, uint32_t w0, uint32_t w1,
                                             unsigned smask, unsigned gmask) {
    constexpr int kTG = TG;
    constexpr int WPT = 8 / BITS, U = kTG / WPT;
    constexpr int LPG = 32 / kTG;
    const int64_t g0 = tile * kTG;
    // FAST: Philox counter of this lane for the tile's first pair of groups (g0 is even); a pair further on adds 32
    const uint64_t blk0 = (uint64_t)(g0 >> 1) * (kGroup / 8) + lane;
    float2 nz_odd[4];            // FAST: noise of an odd group, produced together with the even group before it
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int64_t r = tile * U + u;
        if (!FULL && r >= a.R) break;
        uint8_t* dst = a.packed + r * kGroup + lane * 8;

        if constexpr (DT == GACT_F16 && RNG == GACT_RNG_FAST && BITS == 1) {
            // One-bit codes never leave half precision either.  code = rint(clamp(p, 0, 1) + noise - 0.5) is 1 exactly
            // when p > 1 - noise =: thr (p + noise - 0.5 is exact in fp32, a tie at 0.5 rounds to the even 0, and
            // neither clamp nor a NaN - for which the comparison is false, like NaN -> 0 - changes the outcome).
            // thr = (255.5 - b) / 256 comes exact out of one two-wide fma on the halves 1024 + (255 - b), which a
            // byte permute builds from the inverted noise word; the bits are summed into 1024 + byte by a second one.
            const __half2 c2m8 = __float2half2_rn(0.00390625f), off = __float2half2_rn(-3.998046875f), zero2 = __float2half2_rn(0.0f);
            uint32_t acc2[4] = {0x64006400u, 0x64006400u, 0x64006400u, 0x64006400u};
            uint32_t nb[4];                                 // inverted noise bytes of an even group and the odd one after it
#pragma unroll
            for (int ni = 0; ni < WPT; ni++) {
                const int k = u * WPT + ni;
                if (!FULL && g0 + k >= a.G) break;
                if ((k & 1) == 0) {
                    fast_bytes16(blk0 + (uint64_t)(k >> 1) * (kGroup / 8), a.rk, nb);
#pragma unroll
                    for (int i = 0; i < 4; i++) nb[i] = ~nb[i];
                }
                GroupConst<DT> gc;
                gc.fetch(w0, w1, LPG * k, smask, gmask);
                uint32_t raw[4];
                src.load(k, raw);
                const __half2 weight = __float2half2_rn((float)(1 << ni));
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const __half2 t = __hsub2(as_h2(raw[i]), as_h2(gc.mn2));
                    __half2 bit;
                    if (gc.kind == 2) {
                        bit = __hgt2(t, zero2);             // scale +inf: every element above the minimum gets the top code
                    } else {
                        const uint32_t hb = __byte_perm(nb[2 * (k & 1) + (i >> 1)], 0x64646464u, (i & 1) ? 0x4342u : 0x4140u);
                        bit = __hgt2(__hmul2(t, as_h2(gc.sc2)), __hfma2(as_h2(hb), c2m8, off));
                    }
                    acc2[i] = h2_bits(__hfma2(bit, weight, as_h2(acc2[i])));
                }
            }
            st_stream_u2(dst, make_uint2(__byte_perm(acc2[0], acc2[1], 0x6420u), __byte_perm(acc2[2], acc2[3], 0x6420u)));
        } else if constexpr (DT == GACT_F16 && RNG == GACT_RNG_RTN) {
            // two codes per register: every slot adds (0x6400 + code) << shift; the 0x6400s are taken out again by the
            // start value, and what they carry across the halves cancels with it (arithmetic modulo 2^32)
            uint32_t init = 0;
#pragma unroll
            for (int ni = 0; ni < WPT; ni++) init -= 0x64006400u << (ni * BITS);
            uint32_t acc2[4] = {init, init, init, init};
#pragma unroll
            for (int ni = 0; ni < WPT; ni++) {
                const int k = u * WPT + ni;
                GroupConst<DT> gc;
                gc.fetch(w0, w1, LPG * k, smask, gmask);
                uint32_t raw[4];
                src.load(k, raw);
                const bool present = FULL || g0 + k < a.G;
                uint32_t c[4];
                if (!present) {
#pragma unroll
                    for (int i = 0; i < 4; i++) c[i] = 0x64006400u;
                } else if (gc.kind == 0) {
#pragma unroll
                    for (int i = 0; i < 4; i++) c[i] = code_pair_f16_rtn<BITS, 0>(raw[i], gc.mn2, gc.sc2);
                } else if (gc.kind == 1) {
#pragma unroll
                    for (int i = 0; i < 4; i++) c[i] = code_pair_f16_rtn<BITS, 1>(raw[i], gc.mn2, gc.sc2);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; i++) c[i] = code_pair_f16_rtn<BITS, 2>(raw[i], gc.mn2, gc.sc2);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) acc2[i] = shl_add(c[i], ni * BITS, acc2[i]);
            }
            st_stream_u2(dst, make_uint2(__byte_perm(acc2[0], acc2[1], 0x6420u), __byte_perm(acc2[2], acc2[3], 0x6420u)));
        } else if constexpr (RNG == GACT_RNG_CURAND) {
            // the reference stream: one generator per packed byte (subsequence = byte index), slot ni = draw ni, so
            // the work goes byte pair by byte pair: two Philox calls serve up to four slots of two bytes
            uint32_t acc[8];
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = 0;
            GroupConst<DT> gc[WPT];
#pragma unroll
            for (int ni = 0; ni < WPT; ni++) gc[ni].fetch(w0, w1, LPG * (u * WPT + ni), smask, gmask);
            const uint64_t gid0 = (uint64_t)r * kGroup + lane * 8;
#pragma unroll
            for (int c = 0; c < (WPT + 3) / 4; c++) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint64_t gid = gid0 + 2 * i;
                    const uint4 ra = philox4x32_10((uint32_t)c, 0u, (uint32_t)gid, (uint32_t)(gid >> 32), a.rk);
                    const uint4 rb = philox4x32_10((uint32_t)c, 0u, (uint32_t)(gid + 1), (uint32_t)((gid + 1) >> 32), a.rk);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int ni = c * 4 + q;
                        if (ni >= WPT) break;
                        const int k = u * WPT + ni;
                        if (!FULL && g0 + k >= a.G) break;     // tail row-block: absent groups leave zero bits
                        const float2 nz = curand_uniform2<Centred<DT, RNG>::value>(word_of(ra, q), word_of(rb, q));
                        uint32_t c0, c1;
                        code_pair<DT, BITS, RNG>(src.load_pair(k, i), gc[ni], nz, c0, c1);
                        acc[2 * i] |= c0 << (ni * BITS);
                        acc[2 * i + 1] |= c1 << (ni * BITS);
                    }
                }
            }
            st_stream_u2(dst, gather_bytes8(acc));
        } else {
            uint32_t acc[8];
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = 0;
#pragma unroll
            for (int ni = 0; ni < WPT; ni++) {
                const int k = u * WPT + ni;
                if (!FULL && g0 + k >= a.G) break;
                float2 nz[4];
                if (RNG == GACT_RNG_FAST) {
                    if ((k & 1) == 0) {
                        fast_noise16<true>(blk0 + (uint64_t)(k >> 1) * (kGroup / 8), a.rk, nz, nz_odd);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++) nz[i] = nz_odd[i];
                    }
                } else if (RNG == GACT_RNG_RTN) {
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = splat2(0.0f);
                } else {
                    const float2* p = (const float2*)(a.noise + (g0 + k) * kGroup + lane * 8);
#pragma unroll
                    for (int i = 0; i < 4; i++) nz[i] = Centred<DT, RNG>::value ? add2(p[i], splat2(-0.5f)) : p[i];
                }
                GroupConst<DT> gc;
                gc.fetch(w0, w1, LPG * k, smask, gmask);
                uint32_t raw[4];
                src.load(k, raw);
                uint32_t cb[8];
                codes8<DT, BITS, RNG>(raw, gc, nz, cb);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (NoOverflow<RNG>::value) acc[j] = shl_add(cb[j], ni * BITS, acc[j]);      // disjoint slots: a sum is an OR
                    else acc[j] |= cb[j] << (ni * BITS);
                }
            }
            st_stream_u2(dst, gather_bytes8(acc));
        }
    }
}

// ---- one tile ---------------------------------------------------------------------------------------------------------
// TG groups per tile (at least one row-block).  FULL: all of them exist and are complete.
template <int DT, int BITS, int RNG, int TG, bool FULL, class Src>
__device__ __forceinline__ void tile16(const QuantArgs& a, int64_t tile, int lane, const Src& src) {
    constexpr int kTG = TG;
    constexpr int WPT = 8 / BITS, U = kTG / WPT;
    constexpr int LPG = 32 / kTG;                           // lanes that end up with the same group's result
    static_assert(U >= 1, "a tile holds whole row-blocks");
    const int64_t g0 = tile * kTG;
    const int myk = lane / LPG;                             // the group whose min / max / scale this lane ends up with

    // ---- pass 1: min, max, scale ----
    // First with NaN-propagating min / max: the result then also says whether the group holds a NaN (which the code
    // pass wants to know).  The few tiles that do are reduced again the reference's way, NaN ignored.
    uint32_t mnx = tile_min_negmax<DT, kTG, true>(src, lane);
    float mn = pair_lo<DT>(mnx), mx = -pair_hi<DT>(mnx);
    const unsigned nanmask = __ballot_sync(kFull, mn != mn || mx != mx);
    if (nanmask) {
        mnx = tile_min_negmax<DT, kTG, false>(src, lane);
        mn = pair_lo<DT>(mnx);
        mx = -pair_hi<DT>(mnx);
    }
    // a zero extreme takes the sign the reference's reduction order gives it (rare; decided per group by the whole warp)
    const unsigned amb = __ballot_sync(kFull, zero_sign_ambiguous(mn, mx));
    if (amb) {
#pragma unroll
        for (int k = 0; k < kTG; k++) {
            if (amb & ((0xffffffffu >> (32 - LPG)) << (LPG * k))) {
                uint32_t raw[4];
                float vals[8];
                src.load(k, raw);
                raw_to_float<DT>(raw, vals);
                const float z = zero_sign_like_reference<DT>(vals, lane);
                if (myk == k) {
                    if (mn == 0.0f) mn = z;
                    if (mx == 0.0f) mx = z;
                }
            }
        }
    }
    float sc;
    uint32_t w0, w1;                                        // what pass 2 fetches from lane L*k
    bool special, guard = (nanmask >> lane) & 1u;
    if constexpr (DT == GACT_F16) {
        sc = scale_f16<BITS>(mn, mx);
        w0 = h2_bits(__float2half2_rn(mn));                 // both are half-precision values already
        w1 = h2_bits(__float2half2_rn(sc));
        special = (w1 & 0x7fffu) == 0x7c00u;
        guard = guard || !(sc > 0.0f);                      // scale 0 or NaN: an infinity in the group, or a range that overflows
    } else {
        sc = compute_scale<DT>(mn, mx, BITS);
        w0 = __float_as_uint(mn);
        w1 = __float_as_uint(sc);
        special = !(sc > 0.0f);
    }
    if ((lane & (LPG - 1)) == 0 && (FULL || g0 + myk < a.G)) {
        if constexpr (DT == GACT_F16) {
            ((unsigned short*)a.qmin)[g0 + myk] = (unsigned short)(w0 & 0xffffu);
            ((unsigned short*)a.qscale)[g0 + myk] = (unsigned short)(w1 & 0xffffu);
        } else {
            ((unsigned short*)a.qmin)[g0 + myk] = (unsigned short)(w0 >> 16);
            ((float*)a.qscale)[g0 + myk] = sc;
        }
    }
    const unsigned smask = __ballot_sync(kFull, special), gmask = __ballot_sync(kFull, guard);

    // ---- pass 2: codes ----
    // Almost every tile holds plain groups only; its code pass is compiled with both masks known to be zero, which
    // removes every per-group test and branch from it.
    if ((smask | gmask) == 0u) tile16_codes<DT, BITS, RNG, TG, FULL>(a, tile, lane, src, w0, w1, 0u, 0u);
    else tile16_codes<DT, BITS, RNG, TG, FULL>(a, tile, lane, src, w0, w1, smask, gmask);
}

// ---- the warp-private bulk-copy ring -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// true once the phase with the given parity has completed; gives up after `limit` polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// plain 1-D bulk copy global -> this block's shared memory (no multicast), completing on `bar`
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// TG: groups per warp tile.  bulk_tiles: the leading tiles that come through the rings (0 when x is not 16-byte aligned)
template <int DT, int BITS, int RNG, int TG>
__global__ void __launch_bounds__(kThreads16, GACT_Q16_MINB) quantize16_kernel(const __grid_constant__ QuantArgs a, int64_t bulk_tiles) {
    constexpr int kTileBytes = TG * kGroup * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t bars[kWarps][kStages];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t nw = (int64_t)gridDim.x * kWarps, gw = (int64_t)blockIdx.x * kWarps + warp;
    const int64_t tiles = (a.G + TG - 1) / TG;

    if (gw < bulk_tiles) {
        unsigned char* buf = smem + warp * (kStages * kTileBytes);
        const uint32_t bar0 = smem_u32(&bars[warp][0]), buf0 = smem_u32(buf);
        const unsigned char* x = (const unsigned char*)a.x;
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < kStages; s++) mbar_init(bar0 + 8 * s, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
#pragma unroll
            for (int s = 0; s < kStages; s++) {
                const int64_t t = gw + s * nw;
                if (t < bulk_tiles && !(a.withhold_copy && gw == 0 && s == 0)) {
                    mbar_expect_tx(bar0 + 8 * s, kTileBytes);
                    bulk_load(buf0 + s * kTileBytes, x + t * kTileBytes, kTileBytes, bar0 + 8 * s);
                }
            }
        }
        __syncwarp();
        int64_t i = 0;
        for (int64_t t = gw; t < bulk_tiles; t += nw, ++i) {
            const int s = (int)(i % kStages);
            // all lanes poll; the outcome is decided jointly so that the warp never splits
            if (!__all_sync(kFull, mbar_wait(bar0 + 8 * s, (uint32_t)((i / kStages) & 1), a.wait_limit))) {
                if (lane == 0) atomicExch(&g_pipeline_error, 2);
                // do not leave while copies into the other stages may still be in flight
#pragma unroll
                for (int d = 1; d < kStages; d++)
                    if (t + d * nw < bulk_tiles)
                        mbar_wait(bar0 + 8 * (int)((i + d) % kStages), (uint32_t)(((i + d) / kStages) & 1), a.wait_limit);
                return;
            }
            const SmemSrc src{buf + s * kTileBytes + lane * 16};
            tile16<DT, BITS, RNG, TG, true>(a, t, lane, src);
            __syncwarp();                                        // every lane is done reading the stage
            const int64_t tn = t + kStages * nw;
            if (lane == 0 && tn < bulk_tiles) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(bar0 + 8 * s, kTileBytes);
                bulk_load(buf0 + s * kTileBytes, x + tn * kTileBytes, kTileBytes, bar0 + 8 * s);
            }
        }
    }
    // what the rings do not take: the ragged end, or everything when x is not 16-byte aligned
    for (int64_t t = bulk_tiles + gw; t < tiles; t += nw) {
        const GlobalSrc<DT> src{a.x, a.n, t * TG, lane, a.align};
        tile16<DT, BITS, RNG, TG, false>(a, t, lane, src);
    }
}

#ifndef GACT_Q16_SMALL_ROUNDS
#define GACT_Q16_SMALL_ROUNDS 2
#endif

template <int DT, int BITS, int RNG, int TG>
static int launch16_tg(const QuantArgs& a, cudaStream_t s) {
    // the shared-memory opt-in is a per-device attribute of the kernel: 0 = not set up, 1 = usable, -1 = refused
    static std::atomic<int> ready_on[kMaxDevices];
    static std::atomic<int> per_sm_cached{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return GACT_ERR_LAUNCH;
    int ready = ready_on[dev].load(std::memory_order_relaxed);
    if (ready == 0) {
        ready = cudaFuncSetAttribute(quantize16_kernel<DT, BITS, RNG, TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess ? 1 : -1;
        ready_on[dev].store(ready, std::memory_order_relaxed);
    }
    if (ready != 1) return GACT_ERR_LAUNCH;
    int per_sm = per_sm_cached.load(std::memory_order_relaxed);
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize16_kernel<DT, BITS, RNG, TG>, kThreads16, kSmemBytes) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        per_sm_cached.store(per_sm, std::memory_order_relaxed);
    }
    const int64_t tiles = (a.G + TG - 1) / TG;
    const int64_t bulk_tiles = a.align >= 16 ? a.n / (TG * kGroup) : 0;
    const int64_t resident = (int64_t)per_sm * sm_count();
    const int64_t want = (tiles + kWarps - 1) / kWarps;
    const int blocks = (int)(want < resident ? want : resident);
    quantize16_kernel<DT, BITS, RNG, TG><<<blocks, kThreads16, kSmemBytes, s>>>(a, bulk_tiles);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

// Tile size by tensor size: tiles of 8 groups amortise the per-tile work best, but a tensor of only a few tiles per
// resident warp (3552 warps on a B200) leaves the last round mostly idle; below GACT_Q16_SMALL_ROUNDS (two) rounds of
// 8-group tiles the tensor is cut into tiles of 4 groups instead (1-bit codes need 8 groups for one row-block).
template <int DT, int BITS, int RNG>
static int launch16(const QuantArgs& a, cudaStream_t s) {
    if constexpr (BITS > 1) {
        const int64_t warps = (int64_t)sm_count() * GACT_Q16_MINB * kWarps;
        if (a.G < (int64_t)GACT_Q16_SMALL_ROUNDS * warps * 8) return launch16_tg<DT, BITS, RNG, 4>(a, s);
    }
    return launch16_tg<DT, BITS, RNG, 8>(a, s);
}

template <int DT, int BITS>
static int dispatch_rng16(const QuantArgs& a, int rng, cudaStream_t s) {
    switch (rng) {
    case GACT_RNG_CURAND: return launch16<DT, BITS, GACT_RNG_CURAND>(a, s);
    case GACT_RNG_FAST: return launch16<DT, BITS, GACT_RNG_FAST>(a, s);
    case GACT_RNG_RTN: return launch16<DT, BITS, GACT_RNG_RTN>(a, s);
    case GACT_RNG_EXTERNAL: return launch16<DT, BITS, GACT_RNG_EXTERNAL>(a, s);
    default: return GACT_ERR_MODE;
    }
}

template <int DT>
static int dispatch_bits16(const QuantArgs& a, int bits, int rng, cudaStream_t s) {
    switch (bits) {
    case 1: return dispatch_rng16<DT, 1>(a, rng, s);
    case 2: return dispatch_rng16<DT, 2>(a, rng, s);
    case 4: return dispatch_rng16<DT, 4>(a, rng, s);
    case 8: return dispatch_rng16<DT, 8>(a, rng, s);
    default: return GACT_ERR_BITS;
    }
}

int launch_quantize16(const QuantArgs& a, int dtype, int bits, int rng, cudaStream_t s) {
    return dtype == GACT_F16 ? dispatch_bits16<GACT_F16>(a, bits, rng, s) : dispatch_bits16<GACT_BF16>(a, bits, rng, s);
}

}  // namespace gact

using namespace gact;

extern "C" int gact_pipeline_error(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_pipeline_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

extern "C" int gact_pipeline_error_reset(void) {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_pipeline_error, &zero, sizeof(int)) == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}
