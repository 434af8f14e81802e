// Shared device helpers for libgact_b200: element-type traits, Philox4x32-10, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gact_b200.h"

namespace gact {

constexpr int kGroup = GACT_GROUP_SIZE;   // elements per quantization group
constexpr int kSMs = 148;                 // B200
constexpr unsigned kFull = 0xffffffffu;

// ---------------------------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., SC'11).  Ten rounds, key bumped by the Weyl constants every round.
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                               uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        c1 = (uint32_t)p1;
        c3 = (uint32_t)p0;
        c0 = n0;
        c2 = n2;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
}

// cuRAND's curand_uniform mapping of one 32-bit word to (0, 1]: float(w) * 2^-32 + 2^-33 in fp32.
__device__ __forceinline__ float uniform_from_word(uint32_t w) {
    return __fmaf_rn(__uint2float_rn(w), 2.3283064365386963e-10f, 1.1641532182693481e-10f);
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// ---------------------------------------------------------------------------------------------------
// Element types.  `T` is the storage type, arithmetic on single values goes through float with an
// explicit rounding back to T, which is what the reference's c10::Half operators do.
// ---------------------------------------------------------------------------------------------------
template <int DT> struct Elem;

template <> struct Elem<GACT_F32> {
    using T = float;
    static constexpr int kBytes = 4;
    static __device__ __forceinline__ float to_float(T v) { return v; }
    static __device__ __forceinline__ T from_float(float v) { return v; }
    static __device__ __forceinline__ float round(float v) { return v; }
    static __device__ __forceinline__ float init_hi() { return 1e30f; }
};
template <> struct Elem<GACT_F16> {
    using T = __half;
    static constexpr int kBytes = 2;
    static __device__ __forceinline__ float to_float(T v) { return __half2float(v); }
    static __device__ __forceinline__ T from_float(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ float init_hi() { return __int_as_float(0x7f800000); }   // half(1e30) = inf
};
template <> struct Elem<GACT_BF16> {
    using T = __nv_bfloat16;
    static constexpr int kBytes = 2;
    static __device__ __forceinline__ float to_float(T v) { return __bfloat162float(v); }
    static __device__ __forceinline__ T from_float(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ float init_hi() { return __bfloat162float(__float2bfloat16_rn(1e30f)); }
};

// Position inside a 256-element group of the j-th (0..7) value a lane holds.
//   16-bit types: one 16-byte load per lane, d = lane*8 + j.
//   fp32: two 16-byte loads per lane, each fully coalesced across the warp:
//         d = lane*4 + j (j < 4) and 128 + lane*4 + (j-4).
template <int DT> __device__ __forceinline__ int elem_pos(int lane, int j) {
    if (DT == GACT_F32) return (j < 4) ? lane * 4 + j : 128 + lane * 4 + (j - 4);
    return lane * 8 + j;
}

// Streaming 128-bit accesses: the data is touched once, keep it out of L1.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u1(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream_u4(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream_u2(void* p, uint2 v) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream_u1(void* p, uint32_t v) {
    asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Load the 8 values of group `g` that belong to `lane`, as floats (exact widening for 16-bit types).
// Elements at or past n read as +0 (the reference pads with real zeros, gact/gact/ops.py:12-19).
template <int DT>
__device__ __forceinline__ void load_group8(const void* x, int64_t n, int64_t g, int lane, float (&v)[8]) {
    using E = Elem<DT>;
    const int64_t base = g * kGroup;
    if (base + kGroup <= n) {
        if (DT == GACT_F32) {
            const float* p = (const float*)x + base + lane * 4;
            const uint4 a = ld_stream_u4(p), b = ld_stream_u4(p + 128);
            v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
            v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
        } else {
            const uint4 a = ld_stream_u4((const uint16_t*)x + base + lane * 8);
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (DT == GACT_F16) {
                    const float2 f = __half22float2(*(const __half2*)&w[i]);
                    v[2 * i] = f.x; v[2 * i + 1] = f.y;
                } else {
                    v[2 * i] = __uint_as_float(w[i] << 16);
                    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
                }
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int64_t i = base + elem_pos<DT>(lane, j);
            v[j] = (i < n) ? E::to_float(((const typename E::T*)x)[i]) : 0.0f;
        }
    }
}

// Warp-wide min and max of per-lane candidates.  Hardware min/max ignore NaN operands and order
// -0 below +0, so the result is the numeric extreme with a deterministic zero sign.
__device__ __forceinline__ void warp_minmax(float& mn, float& mx) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(kFull, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, o));
    }
}

// Which zero (+0 or -0) the reference's reduction order reports when the extreme of a group is zero.
// minimax_cuda_kernel.cu:29-66 scans element k*32 + l on lane l in increasing k, keeping the running value
// on ties, then folds lanes with a shuffle-down tree (offsets 16, 8, 4, 2, 1) in which a lane keeps its own
// value on ties, so lane 0 prefers lanes in bit-reversed order (0, 16, 8, 24, 4, ...): among the
// zero-valued elements the one with the smallest (bitrev5(d mod 32), d div 32) wins.  Returns the float
// zero with that element's sign.  Call with all 32 lanes; v = this lane's 8 values.
template <int DT>
__device__ __forceinline__ float zero_sign_like_reference(const float (&v)[8], int lane) {
    uint32_t best = 0xffffffffu;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int d = elem_pos<DT>(lane, j);
        const uint32_t rank = ((__brev((uint32_t)d & 31u) >> 27) << 3) | ((uint32_t)d >> 5);
        const uint32_t key = (rank << 1) | (__float_as_uint(v[j]) >> 31);
        if (v[j] == 0.0f) best = min(best, key);
    }
    best = __reduce_min_sync(kFull, best);
    return __uint_as_float((best & 1u) << 31);
}

// Per-group min and max exactly as the reference reports them (including the start values +-1e30 in T,
// NaN elements ignored, and the sign of a zero extreme).
template <int DT>
__device__ __forceinline__ void group_minmax(const float (&v)[8], int lane, float& mn, float& mx) {
    const float hi = Elem<DT>::init_hi();
    mn = hi;
    mx = -hi;
#pragma unroll
    for (int j = 0; j < 8; j++) { mn = fminf(mn, v[j]); mx = fmaxf(mx, v[j]); }
    warp_minmax(mn, mx);
    const uint32_t bmn = __float_as_uint(mn), bmx = __float_as_uint(mx);
    // ambiguous only when a zero extreme could be either sign: a -0 is present in a group whose min is 0,
    // or the max is 0 and the group is not all +0.
    if (bmn == 0x80000000u || (bmx == 0u && bmn != 0u)) {
        const float z = zero_sign_like_reference<DT>(v, lane);
        if (mn == 0.0f) mn = z;
        if (mx == 0.0f) mx = z;
    }
}

// scale = T( double(T(2^b - 1)) / (double(T(mx - mn)) + 2e-6) ), quantization_cuda_kernel.cu:33.
// fp16 reaches T through float, as c10::Half only constructs from float.  bf16 inputs (which the reference
// does not handle) run the fp32 pipeline on widened values and keep their scale in fp32.
template <int DT> __device__ __forceinline__ float compute_scale(float mn, float mx, int bits) {
    const float d = __fsub_rn(mx, mn);
    const float r = (DT == GACT_F16) ? Elem<DT>::round(d) : d;
    const double q = (double)(float)((1 << bits) - 1) / ((double)r + 2e-6);
    const float s = __double2float_rn(q);
    return (DT == GACT_F16) ? Elem<DT>::round(s) : s;
}

// storage of the per-group scale: the element type, except fp32 for bf16
template <int DT> __device__ __forceinline__ void store_scale(void* qscale, int64_t g, float s) {
    if (DT == GACT_F16) ((__half*)qscale)[g] = __float2half_rn(s);
    else ((float*)qscale)[g] = s;
}
template <int DT> __device__ __forceinline__ float load_scale(const void* qscale, int64_t g) {
    if (DT == GACT_F16) return __half2float(((const __half*)qscale)[g]);
    return ((const float*)qscale)[g];
}

}  // namespace gact
