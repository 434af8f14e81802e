// Unpack + dequantize: out = T(T(code) / scale) + min, written for the first n elements only.
//
// A warp owns U row-blocks of the packed layout.  Each lane reads its 8 packed bytes per row-block with
// one 8-byte (16-bit outputs) or two 4-byte (fp32) loads, and for each of the wpt groups of the row-block
// writes 8 output values with one or two 16-byte streaming stores.
#include "gact_common.cuh"

namespace gact {

constexpr int kDThreads = 256;

struct DequantArgs {
    const uint8_t* packed;
    const void* qmin;
    const void* qscale;
    int64_t n, G, R;
    void* out;
};

template <int DT>
__device__ __forceinline__ void store_group8(void* out, int64_t n, int64_t g, int lane, const float (&o)[8]) {
    using E = Elem<DT>;
    using T = typename E::T;
    const int64_t base = g * kGroup;
    if (base + kGroup <= n) {
        if (DT == GACT_F32) {
            float* p = (float*)out + base + lane * 4;
            st_stream_u4(p, make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3])));
            st_stream_u4(p + 128, make_uint4(__float_as_uint(o[4]), __float_as_uint(o[5]), __float_as_uint(o[6]), __float_as_uint(o[7])));
        } else {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const T a = E::from_float(o[2 * i]), b = E::from_float(o[2 * i + 1]);
                w[i] = (uint32_t)(*(const uint16_t*)&a) | ((uint32_t)(*(const uint16_t*)&b) << 16);
            }
            st_stream_u4((uint16_t*)out + base + lane * 8, make_uint4(w[0], w[1], w[2], w[3]));
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int64_t i = base + elem_pos<DT>(lane, j);
            if (i < n) ((T*)out)[i] = E::from_float(o[j]);
        }
    }
}

template <int DT, int BITS>
__global__ void __launch_bounds__(kDThreads) dequantize_kernel(const DequantArgs a) {
    using E = Elem<DT>;
    using T = typename E::T;
    constexpr int WPT = 8 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (kDThreads / 32);

    for (int64_t r = (int64_t)blockIdx.x * (kDThreads / 32) + (threadIdx.x >> 5); r < a.R; r += nwarps) {
        const uint8_t* row = a.packed + r * kGroup;
        uint32_t lo, hi;
        if (DT == GACT_F32) {
            lo = ld_stream_u1(row + lane * 4);
            hi = ld_stream_u1(row + 128 + lane * 4);
        } else {
            const uint2 p = ld_stream_u2(row + lane * 8);
            lo = p.x; hi = p.y;
        }
        // one (scale, min) pair per group of the row-block: lane i fetches group i's, then broadcast
        float my_s = 0.0f, my_m = 0.0f;
        const int64_t gl = r * WPT + lane;
        if (lane < WPT && gl < a.G) {
            my_s = load_scale<DT>(a.qscale, gl);
            my_m = E::to_float(((const T*)a.qmin)[gl]);
        }
#pragma unroll
        for (int ni = 0; ni < WPT; ni++) {
            const int64_t g = r * WPT + ni;
            if (g >= a.G) break;
            const float s = __shfl_sync(kFull, my_s, ni), m = __shfl_sync(kFull, my_m, ni);
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t word = (j < 4) ? lo : hi;
                const uint32_t code = (word >> ((j & 3) * 8 + ni * BITS)) & MASK;
                const float c = (float)code;                           // exact in every T (<= 255)
                o[j] = (DT != GACT_F16) ? __fadd_rn(__fdiv_rn(c, s), m)
                                        : __fadd_rn(E::round(__fdiv_rn(c, s)), m);   // final rounding on store
            }
            store_group8<DT>(a.out, a.n, g, lane, o);
        }
    }
}

template <int DT, int BITS> static int launch_dequantize(const DequantArgs& a, cudaStream_t s) {
    const int64_t want = (a.R + kDThreads / 32 - 1) / (kDThreads / 32);
    const int64_t cap = (int64_t)kSMs * 8;
    const int blocks = (int)(want < cap ? want : cap);
    dequantize_kernel<DT, BITS><<<blocks, kDThreads, 0, s>>>(a);
    return cudaGetLastError() == cudaSuccess ? GACT_OK : GACT_ERR_LAUNCH;
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
    if (((uintptr_t)packed & 15) || ((uintptr_t)out & 15)) return GACT_ERR_ALIGN;
    DequantArgs a;
    a.packed = (const uint8_t*)packed; a.qmin = qmin; a.qscale = qscale; a.n = n;
    a.G = (n + kGroup - 1) / kGroup;
    a.R = (a.G + 8 / bits - 1) / (8 / bits);
    a.out = out;
    cudaStream_t s = (cudaStream_t)stream;
    switch (dtype) {
    case GACT_F32: return dispatch_dq<GACT_F32>(a, bits, s);
    case GACT_F16: return dispatch_dq<GACT_F16>(a, bits, s);
    default: return dispatch_dq<GACT_BF16>(a, bits, s);
    }
}
