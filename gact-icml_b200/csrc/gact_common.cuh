// Shared device helpers for libgact_b200: element-type traits, Philox4x32-10, warp reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "gact_b200.h"

namespace gact {

constexpr int kGroup = GACT_GROUP_SIZE;   // elements per quantization group
constexpr unsigned kFull = 0xffffffffu;
constexpr int kMaxDevices = 64;

// Number of SMs of the current device (148 on a B200), asked of the runtime once per device and cached.
static inline int sm_count() {
    static std::atomic<int> cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// ---------------------------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., SC'11).  Ten rounds; round r uses the key bumped r times by the Weyl
// constants.  The 20 round keys depend only on the seed, so the host computes them once per launch and they
// reach the kernel as parameters (constant bank operands: no instruction, no register per round key).
// ---------------------------------------------------------------------------------------------------
struct PhiloxKeys { uint32_t k[20]; };

static inline PhiloxKeys philox_round_keys(uint64_t seed) {
    PhiloxKeys rk;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (int r = 0; r < 10; r++) {
        rk.k[2 * r] = k0; rk.k[2 * r + 1] = k1;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return rk;
}

template <int ROUNDS>
__device__ __forceinline__ uint4 philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const PhiloxKeys& rk) {
#pragma unroll
    for (int r = 0; r < ROUNDS; r++) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ rk.k[2 * r];
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ rk.k[2 * r + 1];
        c1 = (uint32_t)p1;
        c3 = (uint32_t)p0;
        c0 = n0;
        c2 = n2;
    }
    return make_uint4(c0, c1, c2, c3);
}
__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const PhiloxKeys& rk) {
    return philox4x32<10>(c0, c1, c2, c3, rk);
}

// Two fp32 operations per instruction (sm_100 add/fma .f32x2): each half is an ordinary IEEE
// round-to-nearest operation, so results are bit-identical to the scalar forms.
#ifdef GACT_NO_F32X2
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return make_float2(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y)); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return make_float2(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y)); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return make_float2(__fmaf_rn(a.x, b.x, c.x), __fmaf_rn(a.y, b.y, c.y)); }
#else
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{ .reg .b64 ra, rb, rd; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; add.rn.f32x2 rd, ra, rb; mov.b64 {%0,%1}, rd; }"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("{ .reg .b64 ra, rb, rd; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; mul.rn.f32x2 rd, ra, rb; mov.b64 {%0,%1}, rd; }"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{ .reg .b64 ra, rb, rc, rd; mov.b64 ra, {%2,%3}; mov.b64 rb, {%4,%5}; mov.b64 rc, {%6,%7}; fma.rn.f32x2 rd, ra, rb, rc; "
        "mov.b64 {%0,%1}, rd; }"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
#endif
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }

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

// Every lane of a warp holds 8 consecutive values of a 256-element group: position d = lane*8 + j.
// That is one 16-byte access per lane for the 16-bit types and one 32-byte (256-bit) access for fp32, both
// fully coalesced, and it makes a lane's 8 packed bytes of a row-block contiguous as well.
template <int DT> __device__ __forceinline__ int elem_pos(int lane, int j) { return lane * 8 + j; }

// Streaming accesses: the data is touched once, keep it out of L1.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// 256-bit load (sm_100): 8 consecutive 32-bit words, 32-byte aligned
__device__ __forceinline__ void ld_stream_u8(const void* p, uint32_t (&v)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(p));
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
__device__ __forceinline__ void st_stream_u8(void* p, const uint32_t (&v)[8]) {
    asm volatile("st.global.cs.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                 "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void st_stream_u2(void* p, uint2 v) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream_u1(void* p, uint32_t v) {
    asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Number of 32-bit registers holding a lane's 8 values in storage format.
template <int DT> struct RawRegs { static constexpr int N = (DT == GACT_F32) ? 8 : 4; };

// The 8 values of group `g` that belong to `lane`, in storage format (fp32: 8 words; 16-bit: 4 packed pairs).
// Elements at or past n read as +0 (the reference pads with real zeros, gact/gact/ops.py:12-19).
// `align`: what the base pointer is known to be aligned to: 32 (the 256-bit fp32 load), 16 (128-bit loads), or
// anything less (element by element, for contiguous views that start at an odd offset of their storage).
template <int DT>
__device__ __forceinline__ void load_raw(const void* x, int64_t n, int64_t g, int lane, int align,
                                         uint32_t (&raw)[RawRegs<DT>::N]) {
    const int64_t base = g * kGroup;
    if (base + kGroup <= n && align >= 16) {
        if constexpr (DT == GACT_F32) {
            const float* p = (const float*)x + base + lane * 8;
            if (align >= 32) {
                ld_stream_u8(p, raw);
            } else {
                const uint4 a = ld_stream_u4(p), b = ld_stream_u4(p + 4);
                raw[0] = a.x; raw[1] = a.y; raw[2] = a.z; raw[3] = a.w; raw[4] = b.x; raw[5] = b.y; raw[6] = b.z; raw[7] = b.w;
            }
        } else {
            const uint4 a = ld_stream_u4((const uint16_t*)x + base + lane * 8);
            raw[0] = a.x; raw[1] = a.y; raw[2] = a.z; raw[3] = a.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < RawRegs<DT>::N; i++) raw[i] = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int64_t i = base + lane * 8 + j;
            if (i < n) {
                if constexpr (DT == GACT_F32) raw[j] = ((const uint32_t*)x)[i];
                else raw[j >> 1] |= (uint32_t)((const uint16_t*)x)[i] << ((j & 1) * 16);
            }
        }
    }
}

// storage format -> 8 floats (exact widening)
template <int DT>
__device__ __forceinline__ void raw_to_float(const uint32_t (&raw)[RawRegs<DT>::N], float (&v)[8]) {
#pragma unroll
    for (int i = 0; i < RawRegs<DT>::N; i++) {
        if constexpr (DT == GACT_F32) {
            v[i] = __uint_as_float(raw[i]);
        } else if constexpr (DT == GACT_F16) {
            const float2 f = __half22float2(*(const __half2*)&raw[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        } else {
            v[2 * i] = __uint_as_float(raw[i] << 16);
            v[2 * i + 1] = __uint_as_float(raw[i] & 0xffff0000u);
        }
    }
}

// Load the 8 values of group `g` that belong to `lane`, as floats.
template <int DT>
__device__ __forceinline__ void load_group8(const void* x, int64_t n, int64_t g, int lane, float (&v)[8]) {
    uint32_t raw[RawRegs<DT>::N];
    load_raw<DT>(x, n, g, lane, 16, raw);
    raw_to_float<DT>(raw, v);
}

// warp-wide float min / max in one instruction each (sm_100a); NaN inputs are ignored, -0 orders below +0
__device__ __forceinline__ float warp_min_f32(float v) {
    float r;
    asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float warp_max_f32(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

// Warp-wide min and max of per-lane candidates.  Hardware min/max ignore NaN operands and order
// -0 below +0, so the result is the numeric extreme with a deterministic zero sign.
__device__ __forceinline__ void warp_minmax(float& mn, float& mx) {
    mn = warp_min_f32(mn);
    mx = warp_max_f32(mx);
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

// A zero extreme can be +0 or -0 depending on the reference's reduction order.  The hardware reduction
// reports -0 for the min when any -0 is present and +0 for the max when any +0 is present, so the answer is
// only open when the min is -0, or the max is +0 while the min is not +0 (an all-(+0) group has min = max = +0).
__device__ __forceinline__ bool zero_sign_ambiguous(float mn, float mx) {
    const uint32_t bmn = __float_as_uint(mn), bmx = __float_as_uint(mx);
    return bmn == 0x80000000u || (bmx == 0u && bmn != 0u);
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
    if (zero_sign_ambiguous(mn, mx)) {
        const float z = zero_sign_like_reference<DT>(v, lane);
        if (mn == 0.0f) mn = z;
        if (mx == 0.0f) mx = z;
    }
}

// Same, from the storage format.  16-bit types reduce their four packed pairs with two-wide min / max first.
template <int DT>
__device__ __forceinline__ void group_minmax_raw(const uint32_t (&raw)[RawRegs<DT>::N], int lane, float& mn, float& mx) {
    const float hi = Elem<DT>::init_hi();
    if constexpr (DT == GACT_F32) {
        mn = hi; mx = -hi;
#pragma unroll
        for (int j = 0; j < 8; j++) { mn = fminf(mn, __uint_as_float(raw[j])); mx = fmaxf(mx, __uint_as_float(raw[j])); }
    } else if constexpr (DT == GACT_F16) {
        const __half2* h = (const __half2*)raw;
        const __half2 lo = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
        const __half2 up = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
        const float2 a = __half22float2(lo), b = __half22float2(up);
        mn = fminf(hi, fminf(a.x, a.y)); mx = fmaxf(-hi, fmaxf(b.x, b.y));
    } else {
        const __nv_bfloat162* h = (const __nv_bfloat162*)raw;
        const __nv_bfloat162 lo = __hmin2(__hmin2(h[0], h[1]), __hmin2(h[2], h[3]));
        const __nv_bfloat162 up = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
        const uint32_t l = *(const uint32_t*)&lo, u = *(const uint32_t*)&up;
        mn = fminf(hi, fminf(__uint_as_float(l << 16), __uint_as_float(l & 0xffff0000u)));
        mx = fmaxf(-hi, fmaxf(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u)));
    }
    warp_minmax(mn, mx);
    if (zero_sign_ambiguous(mn, mx)) {
        float v[8];
        raw_to_float<DT>(raw, v);
        const float z = zero_sign_like_reference<DT>(v, lane);
        if (mn == 0.0f) mn = z;
        if (mx == 0.0f) mx = z;
    }
}

// scale = T( double(T(2^b - 1)) / (double(T(mx - mn)) + 2e-6) ), quantization_cuda_kernel.cu:33.
// fp16 reaches T through float, as c10::Half only constructs from float.  bf16 inputs (which the reference
// does not handle) run the fp32 pipeline on widened values: scale = fl32((2^b-1) / fl32(fl32(mx-mn) + 2e-6f)),
// kept in fp32.
template <int DT> __device__ __forceinline__ float compute_scale(float mn, float mx, int bits) {
    const float d = __fsub_rn(mx, mn);
    if (DT == GACT_BF16) return __fdiv_rn((float)((1 << bits) - 1), __fadd_rn(d, 2e-6f));
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
