// Unpack + dequantize: out = T(T(code) / scale) + min, written for the first n elements only.
//
// A warp owns a tile of 4, 8 or 16 groups (by tensor size, see launch_dequantize) = U row-blocks of the packed
// layout.  Each lane reads its 8 packed bytes per row-block with one 8-byte load - all loads of the tile
// first - and writes 8 output values per group with one streaming store (16 bytes, or 32 bytes for fp32).
//
// No per-element division.  The quotient code/scale is formed from one reciprocal per group:
//   fp16:  round_h(fl32(code * fl32(1/scale))) equals round_h(fl32(code / scale)) for every half-precision
//          scale and every code 0..255 (checked exhaustively, 65 536 x 256 cases, by the CPU test-suite);
//   fp32 / bf16 (fp32 scale):  q0 = code*r, e = fma(-q0, scale, code), q = fma(e, r, q0) with r = fl32(1/scale)
//          is the correctly rounded quotient for all 2^23 significands of scale and codes 1..255 (checked
//          exhaustively for one binade, sampled over the others); scales outside 2^-60..2^60, zero, infinite,
//          negative or NaN take the IEEE division instead (a warp-uniform branch).
// Codes become floats without a conversion instruction: a byte permute drops the code into the low mantissa
// bits of 2^23, and the 2^23 is folded into the following multiply-add.
#include "gact_common.cuh"

namespace gact {

constexpr int kDThreads = 256;
constexpr float kTwo23 = 8388608.0f;

struct DequantArgs {
    const uint8_t* packed;
    const void* qmin;
    const void* qscale;
    int64_t n, G, R;
    void* out;
    int align;               // guaranteed alignment of out in bytes: 32, 16, or 0 (element-aligned only)
};

// 2^23 + (byte `idx` of w) as a float bit pattern: bytes {w[idx], 0x00, 0x00, 0x4B}
__device__ __forceinline__ float byte_as_magic(uint32_t w, int idx) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u + (uint32_t)idx));
}

template <int DT>
__device__ __forceinline__ void store_group8_slow(void* out, int64_t n, int64_t g, int lane, const float (&o)[8]) {
    using E = Elem<DT>;
    using T = typename E::T;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int64_t i = g * kGroup + elem_pos<DT>(lane, j);
        if (i < n) ((T*)out)[i] = E::from_float(o[j]);
    }
}

// TG = groups per warp tile (a 1-bit row-block holds 8, so at least that many there)
template <int DT, int BITS, int TG>
__global__ void __launch_bounds__(kDThreads) dequantize_kernel(const DequantArgs a) {
    using E = Elem<DT>;
    using T = typename E::T;
    constexpr int WPT = 8 / BITS;
    constexpr int U = (WPT >= TG) ? 1 : TG / WPT;
    constexpr int GPW = WPT * U;
    constexpr uint32_t MASK4 = ((1u << BITS) - 1u) * 0x01010101u;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kDThreads / 32);
    const int64_t tiles = (a.R + U - 1) / U;

    for (int64_t tile = (int64_t)blockIdx.x * (kDThreads / 32) + (threadIdx.x >> 5); tile < tiles; tile += nwarps) {
        const int64_t g0 = tile * GPW;
        uint32_t lo[U], hi[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t r = tile * U + u;
            lo[u] = hi[u] = 0;
            if (r < a.R) {
                const uint2 p = ld_stream_u2(a.packed + r * kGroup + lane * 8);
                lo[u] = p.x; hi[u] = p.y;
            }
        }
        // lane k < GPW fetches scale and min of group g0+k and forms the reciprocal once
        float my_s = 1.0f, my_m = 0.0f;
        if (lane < GPW && g0 + lane < a.G) {
            my_s = load_scale<DT>(a.qscale, g0 + lane);
            my_m = E::to_float(((const T*)a.qmin)[g0 + lane]);
        }
        const float my_r = __fdiv_rn(1.0f, my_s);

#pragma unroll
        for (int k = 0; k < GPW; k++) {
            const int64_t g = g0 + k;
            if (g >= a.G) break;
            const int u = k / WPT, ni = k % WPT;
            const float s = __shfl_sync(kFull, my_s, k), m = __shfl_sync(kFull, my_m, k), r = __shfl_sync(kFull, my_r, k);
            // this group's codes as bytes: (w >> ni*BITS) & mask, four elements per word
            const uint32_t c_lo = (BITS == 8) ? lo[u] : ((lo[u] >> (ni * BITS)) & MASK4);
            const uint32_t c_hi = (BITS == 8) ? hi[u] : ((hi[u] >> (ni * BITS)) & MASK4);
            const bool full = (g + 1) * kGroup <= a.n && a.align >= 16;        // else element by element

            if (DT == GACT_F16) {
                // q = round_h(code * r), out = round_h(q + m): two elements per instruction after the multiply
                const float bias = -kTwo23 * r;                       // exact (power-of-two scaling); may be -inf/NaN with r
                const __half2 m2 = __float2half2_rn(m);
                uint32_t w[4];
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const uint32_t word = (j < 4) ? c_lo : c_hi;
                    float q0, q1;
                    if (isfinite(bias)) {
                        q0 = __fmaf_rn(byte_as_magic(word, j & 3), r, bias);          // = fl32(code * r)
                        q1 = __fmaf_rn(byte_as_magic(word, (j + 1) & 3), r, bias);
                    } else {                                                          // r is inf or NaN (scale 0 / NaN)
                        q0 = __fmul_rn(byte_as_magic(word, j & 3) - kTwo23, r);
                        q1 = __fmul_rn(byte_as_magic(word, (j + 1) & 3) - kTwo23, r);
                    }
                    const __half2 h = __hadd2(__floats2half2_rn(q0, q1), m2);
                    w[j >> 1] = *(const uint32_t*)&h;
                    if (!full) { const float2 f = __half22float2(h); o[j] = f.x; o[j + 1] = f.y; }
                }
                if (full) st_stream_u4((uint16_t*)a.out + g * kGroup + lane * 8, make_uint4(w[0], w[1], w[2], w[3]));
                else store_group8_slow<DT>(a.out, a.n, g, lane, o);
            } else {
                // fp32: correctly rounded quotient from the reciprocal (Markstein); IEEE division for unusual scales.
                // bf16 (not a reference type): fma(code, 1/scale, min) in fp32, rounded once to bf16.
                const uint32_t sb = __float_as_uint(s);
                const bool fast = (sb - 0x21800000u) < (0x5D800000u - 0x21800000u);   // 2^-60 <= s < 2^60, s > 0
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t word = (j < 4) ? c_lo : c_hi;
                    if (DT == GACT_BF16) {
                        const float c = byte_as_magic(word, j & 3) - kTwo23;
                        o[j] = __fmaf_rn(c, r, m);
                        continue;
                    }
                    const float c = byte_as_magic(word, j & 3) - kTwo23;              // exact
                    float q;
                    if (fast) {
                        const float q0 = __fmul_rn(c, r);
                        const float e = __fmaf_rn(-q0, s, c);
                        q = __fmaf_rn(e, r, q0);
                    } else {
                        q = __fdiv_rn(c, s);
                    }
                    o[j] = __fadd_rn(q, m);
                }
                if (!full) {
                    store_group8_slow<DT>(a.out, a.n, g, lane, o);
                } else if (DT == GACT_F32) {
                    float* p = (float*)a.out + g * kGroup + lane * 8;
                    if (a.align >= 32) {
                        const uint32_t w[8] = {__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3]),
                                               __float_as_uint(o[4]), __float_as_uint(o[5]), __float_as_uint(o[6]), __float_as_uint(o[7])};
                        st_stream_u8(p, w);
                    } else {
                        st_stream_u4(p, make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3])));
                        st_stream_u4(p + 4, make_uint4(__float_as_uint(o[4]), __float_as_uint(o[5]), __float_as_uint(o[6]), __float_as_uint(o[7])));
                    }
                } else {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const __nv_bfloat162 b = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
                        w[i] = *(const uint32_t*)&b;
                    }
                    st_stream_u4((uint16_t*)a.out + g * kGroup + lane * 8, make_uint4(w[0], w[1], w[2], w[3]));
                }
            }
        }
    }
}

template <int DT, int BITS, int TG> static int launch_dequantize_tile(const DequantArgs& a, cudaStream_t s) {
    constexpr int WPT = 8 / BITS;
    constexpr int U = (WPT >= TG) ? 1 : TG / WPT;
    const int64_t tiles = (a.R + U - 1) / U;
    const int64_t want = (tiles + kDThreads / 32 - 1) / (kDThreads / 32);
    const int64_t cap = (int64_t)sm_count() * 16;
    const int blocks = (int)(want < cap ? want : cap);
    dequantize_kernel<DT, BITS, TG><<<blocks, kDThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
}

// Tile size by tensor size (measured): large tiles amortise the per-tile work (scale / min fetch, reciprocal,
// broadcasts) and keep more loads in flight, but a tensor must still spread over enough warps to fill the GPU:
// 16 groups per warp (8 for fp32, whose stores are twice as wide) once that leaves half a resident wave of warps,
// else 8, else 4.
template <int DT, int BITS> static int launch_dequantize(const DequantArgs& a, cudaStream_t s) {
    const int64_t kHalfWave = (int64_t)sm_count() * 32;       // warps: half of what the SMs hold (64 resident warps each)
    constexpr int kBig = (DT == GACT_F32) ? 8 : 16;
    if (a.G >= kBig * kHalfWave) return launch_dequantize_tile<DT, BITS, kBig>(a, s);
    if (kBig > 8 && a.G >= 8 * kHalfWave) return launch_dequantize_tile<DT, BITS, 8>(a, s);
    return launch_dequantize_tile<DT, BITS, 4>(a, s);
}

template <int DT> static int dispatch_dq(const DequantArgs& a, int bits, cudaStream_t s) {
    switch (bits) {
    case 1: return launch_dequantize<DT, 1>(a, s);
    case 2: return launch_dequantize<DT, 2>(a, s);
    case 4: return launch_dequantize<DT, 4>(a, s);
    case 8: return launch_dequantize<DT, 8>(a, s);
    default: return GACT_ERR_BITS;
    }
}

}  // namespace gact

using namespace gact;

extern "C" int gact_dequantize(const void* packed, const void* qmin, const void* qscale, int dtype, int64_t n,
                               int bits, void* out, void* stream) {
    if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8)) return GACT_ERR_BITS;
    if (dtype < GACT_F32 || dtype > GACT_BF16) return GACT_ERR_DTYPE;
    if (n < 0) return GACT_ERR_SIZE;
    if (n == 0) return GACT_OK;
    if (!packed || !qmin || !qscale || !out) return GACT_ERR_NULL;
    // out only has to be aligned to its element size (e.g. a view into a larger buffer); packed keeps its vector alignment
    if (((uintptr_t)packed & 15) || ((uintptr_t)out & (dtype == GACT_F32 ? 3 : 1))) return GACT_ERR_ALIGN;
    DequantArgs a;
    a.packed = (const uint8_t*)packed; a.qmin = qmin; a.qscale = qscale; a.n = n;
    a.G = (n + kGroup - 1) / kGroup;
    a.R = (a.G + 8 / bits - 1) / (8 / bits);
    a.out = out;
    a.align = ((uintptr_t)out & 15) ? 0 : (((uintptr_t)out & 31) ? 16 : 32);
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case GACT_F32: return dispatch_dq<GACT_F32>(a, bits, s);
    case GACT_F16: return dispatch_dq<GACT_F16>(a, bits, s);
    default: return dispatch_dq<GACT_BF16>(a, bits, s);
    }
}
