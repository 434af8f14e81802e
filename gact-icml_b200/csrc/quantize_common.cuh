// Shared by the two translation units of the fused quantize kernels (quantize.cu: fp32 inputs and the entry
// points; quantize16.cu: fp16 / bf16 inputs): launch arguments, noise arrangements, rounding helpers.
#pragma once

#include "gact_common.cuh"

namespace gact {

constexpr int kQThreads = 256;
constexpr float kMagic = 12582912.0f;   // 1.5 * 2^23: w + kMagic leaves rint(w) in the low mantissa bits

struct QuantArgs {
    const void* x;
    int64_t n, G, R;
    uint64_t seed;
    const float* noise;
    uint8_t* packed;
    void* qmin;
    void* qscale;
    int align;               // guaranteed alignment of x in bytes: 32, 16, or 0 (element-aligned only)
    uint32_t wait_limit;     // polls after which a wait on a bulk copy gives up
    int withhold_copy;       // diagnostics: warp 0 of block 0 leaves its first bulk copy unissued
    PhiloxKeys rk;
};

// fp16 / bf16 inputs (quantize16.cu); dtype is GACT_F16 or GACT_BF16
int launch_quantize16(const QuantArgs& a, int dtype, int bits, int rng, cudaStream_t s);

// Which noise values reach the code routines "centred" (noise - 0.5 instead of noise).  With the 8-bit noise of
// FAST and the constant noise of RTN, and p a half-precision value, p + noise is exact in fp32, so
// (p + noise) - 0.5 equals p + (noise - 0.5) bit for bit and one addition is saved; bf16 (not a reference type)
// is defined on centred noise in every mode.  fp32 keeps the reference's order of operations.
template <int DT, int RNG> struct Centred {
    static constexpr bool value = (DT == GACT_BF16) || (DT == GACT_F16 && (RNG == GACT_RNG_FAST || RNG == GACT_RNG_RTN));
};
// FAST and RTN never produce a code above 2^bits - 1 (fp16: clamped; fp32 / bf16: the noise stays below 1), so
// slots cannot collide and the packed byte may be summed instead of OR-ed.
template <int RNG> struct NoOverflow { static constexpr bool value = (RNG == GACT_RNG_FAST || RNG == GACT_RNG_RTN); };

// noise of the FAST arrangement: one Philox4x32-7 call, counter (block_lo, block_hi, 0, "FAST"), gives 16
// bytes = 8 bits for each of this lane's 8 elements of an even group (bytes 0..7) and of the following odd group
// (bytes 8..15); noise = (byte + 0.5) / 256 (minus 0.5 when CENTRED).  Seven rounds: the member of the Philox4x32
// family with the fewest rounds that passes BigCrush (Salmon et al., SC'11); the ten rounds of cuRAND's generator
// (which the CURAND mode uses) add a safety margin that rounding noise does not need, at 6-7 % of the kernel's time.
#ifndef GACT_FAST_ROUNDS
#define GACT_FAST_ROUNDS 7
#endif
// the 16 noise bytes themselves: words 0, 1 = the even group's elements 0..3, 4..7; words 2, 3 = the odd group's
__device__ __forceinline__ void fast_bytes16(uint64_t block, const PhiloxKeys& rk, uint32_t (&w)[4]) {
    const uint4 r = philox4x32<GACT_FAST_ROUNDS>((uint32_t)block, (uint32_t)(block >> 32), 0u, 0x46415354u, rk);
    w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
}
template <bool CENTRED>
__device__ __forceinline__ void fast_noise16(uint64_t block, const PhiloxKeys& rk, float2 (&even)[4], float2 (&odd)[4]) {
    uint32_t w[4];
    fast_bytes16(block, rk, w);
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


// cuRAND's uniform of two words: float(word) * 2^-32 + 2^-33 (minus 0.5 when CENTRED)
template <bool CENTRED>
__device__ __forceinline__ float2 curand_uniform2(uint32_t wa, uint32_t wb) {
    const float2 u = fma2(make_float2(__uint2float_rn(wa), __uint2float_rn(wb)), splat2(2.3283064365386963e-10f),
                          splat2(1.1641532182693481e-10f));
    return CENTRED ? add2(u, splat2(-0.5f)) : u;
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

// low bytes of eight 32-bit accumulators -> two words (bytes in element order)
__device__ __forceinline__ uint2 gather_bytes8(const uint32_t (&acc)[8]) {
    const uint32_t lo = __byte_perm(__byte_perm(acc[0], acc[1], 0x0040u), __byte_perm(acc[2], acc[3], 0x0040u), 0x5410u);
    const uint32_t hi = __byte_perm(__byte_perm(acc[4], acc[5], 0x0040u), __byte_perm(acc[6], acc[7], 0x0040u), 0x5410u);
    return make_uint2(lo, hi);
}

}  // namespace gact
