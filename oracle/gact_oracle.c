/*
 * CPU oracle for GACT's saved-tensor compression path.  TEST INFRASTRUCTURE ONLY: it is the checker
 * that the CUDA kernels are compared with (tests, the smoke check and the benchmark's CPU baseline);
 * the product never calls it and has no CPU fallback.
 *
 * It restates, in scalar C, what the reference computes on the GPU.  Each function cites the reference
 * source (paths inside the GACT repository) that it follows:
 *   gact/gact/cpp_extension/minimax_cuda_kernel.cu:23-67        per-group min / max, comparison order
 *   gact/gact/cpp_extension/quantization_cuda_kernel.cu:23-35   scale
 *   gact/gact/cpp_extension/quantization_cuda_kernel.cu:38-71   stochastic rounding + bit packing
 *   gact/gact/cpp_extension/quantization_cuda_kernel.cu:149-177 unpack + dequantize
 *   gact/gact/cpp_extension/quantization_cuda_kernel.cu:229-288 1-bit dropout-mask layout
 *   gact/gact/cpp_extension/calc_precision.cc:66-118            greedy bit allocation
 *   gact/gact/ops.py:11-69                                      zero padding to 256-element groups
 * The random stream is cuRAND's Philox4x32-10 (a published algorithm: Salmon et al., SC'11) in the
 * arrangement `curand_init(seed, subsequence, 0)` + `curand_uniform` gives.
 *
 * Parity pins: Philox + uniform against vectors produced by the CUDA toolkit's own cuRAND header
 * compiled for the host; the greedy allocator against the reference's calc_precision.cc built
 * unmodified; quantize / dequantize / mask against the reference's CUDA kernels built unmodified and
 * run on a GPU (see tests/).
 *
 * Build:  gcc -O2 -fPIC -shared -fopenmp -ffp-contract=off -o libgact_oracle.so gact_oracle.c -lm
 *         (OpenMP only spreads independent groups / row-blocks over the host cores; OMP_NUM_THREADS=1
 *         gives the scalar run.)
 *         (-ffp-contract=off matters: every rounding below is spelled out.)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GROUP 256

enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };
enum { RNG_CURAND = 0, RNG_FAST = 1, RNG_RTN = 2, RNG_EXTERNAL = 3 };
#define FAST_ROUNDS 7        /* Philox rounds of RNG_FAST */

/* ------------------------------------------------------------------------------------------------
 * 16-bit float formats, in software (round-to-nearest-even), so that no compiler/ISA feature is needed
 * ---------------------------------------------------------------------------------------------- */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return u2f(sign);
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-08f;
        return (sign ? -v : v);
    }
    if (exp == 31) return u2f(sign | 0x7f800000u | (man << 13));
    return u2f(sign | ((exp + 112) << 23) | (man << 13));
}

static uint16_t float_to_half(float f) {
    uint32_t x = f2u(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return (uint16_t)(sign | 0x7fffu);       /* NaN (canonical, as cvt.rn.f16.f32) */
    if (ax >= 0x47800000u) {                                       /* |f| >= 65536 -> inf (also inf) */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x38800000u) {                                        /* |f| < 2^-14: subnormal half or zero */
        /* round |f| / 2^-24 to an integer, ties to even */
        float a = u2f(ax);
        float scaled = a * 16777216.0f;                            /* exact: power of two */
        float r = nearbyintf(scaled);                              /* default mode = ties-to-even */
        return (uint16_t)(sign | (uint16_t)r);                     /* r <= 1024 -> carries into exponent OK */
    }
    uint32_t man = ax & 0x7fffffu, exp = (ax >> 23) - 112;
    uint32_t h = (exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;         /* may carry into exponent / to inf */
    return (uint16_t)(sign | h);
}

static float bf16_to_float(uint16_t b) { return u2f((uint32_t)b << 16); }

static uint16_t float_to_bf16(float f) {
    uint32_t x = f2u(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;           /* NaN (canonical, as cvt.rn.bf16.f32) */
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

static inline float load_elem(const void *p, int dtype, int64_t i) {
    switch (dtype) {
    case DT_F32: return ((const float *)p)[i];
    case DT_F16: return half_to_float(((const uint16_t *)p)[i]);
    default:     return bf16_to_float(((const uint16_t *)p)[i]);
    }
}

/* round a float to the storage type T and return it as float */
static inline float round_T(float v, int dtype) {
    switch (dtype) {
    case DT_F32: return v;
    case DT_F16: return half_to_float(float_to_half(v));
    default:     return bf16_to_float(float_to_bf16(v));
    }
}

static inline void store_elem(void *p, int dtype, int64_t i, float v) {
    switch (dtype) {
    case DT_F32: ((float *)p)[i] = v; break;
    case DT_F16: ((uint16_t *)p)[i] = float_to_half(v); break;
    default:     ((uint16_t *)p)[i] = float_to_bf16(v); break;
    }
}

/* exported for the tests of the conversions themselves */
uint16_t oracle_float_to_half(float f) { return float_to_half(f); }
float oracle_half_to_float(uint16_t h) { return half_to_float(h); }
uint16_t oracle_float_to_bf16(float f) { return float_to_bf16(f); }

/* ------------------------------------------------------------------------------------------------
 * Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11)
 * ---------------------------------------------------------------------------------------------- */
void oracle_philox4x32_r(const uint32_t ctr_in[4], const uint32_t key_in[2], int rounds, uint32_t out[4]) {
    uint32_t c0 = ctr_in[0], c1 = ctr_in[1], c2 = ctr_in[2], c3 = ctr_in[3];
    uint32_t k0 = key_in[0], k1 = key_in[1];
    for (int r = 0; r < rounds; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
/* the generator cuRAND uses: ten rounds */
void oracle_philox4x32_10(const uint32_t ctr_in[4], const uint32_t key_in[2], uint32_t out[4]) {
    oracle_philox4x32_r(ctr_in, key_in, 10, out);
}

/* uniform in (0, 1] from one 32-bit word, as cuRAND's curand_uniform does:
 * float(word) * 2^-32 + 2^-33, evaluated in fp32 (the product is exact, so FMA or not is the same) */
static inline float uniform_from_word(uint32_t w) {
    float f = (float)w;                       /* round-to-nearest-even */
    return f * 2.3283064365386963e-10f + 1.1641532182693481e-10f;
}

/* The `draw`-th curand_uniform() of a generator initialised with curand_init(seed, subsequence, 0):
 * word (draw mod 4) of Philox(counter = (draw div 4, 0, subseq_lo, subseq_hi), key = (seed_lo, seed_hi)).
 * Follows quantization_cuda_kernel.cu:55-56,65 where subsequence = index of the packed byte. */
float oracle_curand_uniform(uint64_t seed, uint64_t subsequence, uint32_t draw) {
    uint32_t ctr[4] = { draw >> 2, 0u, (uint32_t)subsequence, (uint32_t)(subsequence >> 32) };
    uint32_t key[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) };
    uint32_t out[4];
    oracle_philox4x32_10(ctr, key, out);
    return uniform_from_word(out[draw & 3]);
}

/* ------------------------------------------------------------------------------------------------
 * min / max of each 256-element group, in the reference's comparison order
 * (minimax_cuda_kernel.cu:29-66): lane l scans elements l, l+32, ... keeping the running value unless
 * the new one is strictly greater (smaller); then a 5-step shuffle-down tree in which the lower lane
 * keeps its own value on ties.  The order only matters for which of +0 / -0 is reported; NaN never
 * replaces a running value.  Start values are -1e30 / +1e30 converted to the storage type (so +-inf
 * for fp16, finite for fp32 and bf16).
 * ---------------------------------------------------------------------------------------------- */
static void group_minmax(const float v[GROUP], int dtype, float *mn_out, float *mx_out) {
    float mx[32], mn[32];
    float init_hi = (dtype == DT_F32) ? 1e30f : round_T(1e30f, dtype);
    for (int l = 0; l < 32; l++) {
        float a = -init_hi, b = init_hi;
        for (int k = 0; k < GROUP / 32; k++) {
            float x = v[k * 32 + l];
            a = (a < x) ? x : a;              /* std::max(a, x) */
            b = (x < b) ? x : b;              /* std::min(b, x) */
        }
        mx[l] = a; mn[l] = b;
    }
    for (int delta = 16; delta >= 1; delta >>= 1) {
        float nmx[32], nmn[32];
        for (int l = 0; l < 32; l++) {
            int src = (l + delta < 32) ? l + delta : l;   /* shfl_down past the warp returns own value */
            nmx[l] = (mx[l] < mx[src]) ? mx[src] : mx[l];
            nmn[l] = (mn[src] < mn[l]) ? mn[src] : mn[l];
        }
        memcpy(mx, nmx, sizeof mx); memcpy(mn, nmn, sizeof mn);
    }
    *mn_out = mn[0]; *mx_out = mx[0];
}

/* zero-padded group fetch (ops.py:12-19: elements past n are real zeros that take part in min/max) */
static void fetch_group(const void *x, int dtype, int64_t n, int64_t g, float v[GROUP]) {
    for (int d = 0; d < GROUP; d++) {
        int64_t i = g * GROUP + d;
        v[d] = (i < n) ? load_elem(x, dtype, i) : 0.0f;
    }
}

/* scale = T( double(T(2^b-1)) / (double(T(mx-mn)) + 2e-6) ), quantization_cuda_kernel.cu:33.
 * fp16: the double result reaches T through float (c10::Half only constructs from float).
 * bf16 (no counterpart in the reference, which skips bf16 tensors): the whole pipeline runs in fp32 on the
 * widened values: scale = fl32((2^b-1) / fl32(fl32(mx-mn) + 2e-6f)), KEPT in fp32, because a scale rounded to
 * 8 significant bits would push the largest element of a group past 2^b - 1. */
static float compute_scale(float mn, float mx, int bits, int dtype) {
    if (dtype == DT_BF16) {                       /* ours: fp32 throughout */
        float d = mx - mn;
        float den = d + 2e-6f;
        return (float)((1 << bits) - 1) / den;
    }
    float r = (dtype == DT_F16) ? round_T(mx - mn, dtype) : (mx - mn);
    double q = (double)(float)((1 << bits) - 1) / ((double)r + 2e-6);
    return (dtype == DT_F16) ? round_T((float)q, dtype) : (float)q;
}

/* storage type of the per-group scale: the input type, except fp32 for bf16 inputs */
static inline int scale_dtype(int dtype) { return dtype == DT_BF16 ? DT_F32 : dtype; }

int oracle_minimax(const void *x, int dtype, int64_t n, void *mn_out, void *mx_out) {
    int64_t G = (n + GROUP - 1) / GROUP;
    float v[GROUP];
    for (int64_t g = 0; g < G; g++) {
        float mn, mx;
        fetch_group(x, dtype, n, g, v);
        group_minmax(v, dtype, &mn, &mx);
        store_elem(mn_out, dtype, g, mn);
        store_elem(mx_out, dtype, g, mx);
    }
    return 0;
}

/* __float2int_rn: round to nearest even, saturating; NaN -> 0 */
static inline int32_t float2int_rn(float f) {
    if (f != f) return 0;
    if (f >= 2147483648.0f) return INT32_MAX;
    if (f <= -2147483648.0f) return INT32_MIN;
    return (int32_t)nearbyintf(f);
}

/* our own noise arrangement for RNG_FAST: see oracle_fast_noise below */
static float fast_noise(uint64_t seed, int64_t elem);

/* ------------------------------------------------------------------------------------------------
 * quantize: fused restatement of minimax + scale + pack.
 *   packed : R*256 bytes, R = ceil(G / (8/bits)); byte r*256+d holds element d of groups r*wpt .. r*wpt+wpt-1
 *   qmin : G values of the input dtype; qscale : G values of the input dtype (fp32 for bf16 inputs)
 *   noise (RNG_EXTERNAL): G*256 floats in [0,1], indexed like the zero-padded input
 *   fma_mode (fp32 only): 1 = (x-mn)*scale+noise evaluated as one fused multiply-add (what nvcc makes of
 *   the reference expression at its default -fmad=true), 0 = product rounded before the add.
 * ---------------------------------------------------------------------------------------------- */
int oracle_quantize(const void *x, int dtype, int64_t n, int bits, uint64_t seed, int rng_mode,
                    const float *noise, int fma_mode, uint8_t *packed, void *qmin, void *qscale) {
    if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8)) return 1;
    if (dtype < 0 || dtype > 2) return 2;
    const int wpt = 8 / bits;
    const int64_t G = (n + GROUP - 1) / GROUP;
    const int64_t R = (G + wpt - 1) / wpt;
    float *mn = (float *)malloc(sizeof(float) * (size_t)(G ? G : 1));
    float *sc = (float *)malloc(sizeof(float) * (size_t)(G ? G : 1));
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < G; g++) {
        float v[GROUP];
        float lo, hi;
        fetch_group(x, dtype, n, g, v);
        group_minmax(v, dtype, &lo, &hi);
        mn[g] = lo;
        sc[g] = compute_scale(lo, hi, bits, dtype);
        store_elem(qmin, dtype, g, mn[g]);
        store_elem(qscale, scale_dtype(dtype), g, sc[g]);
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < R; r++) {
        for (int d = 0; d < GROUP; d++) {
            const int64_t gid = r * GROUP + d;                 /* = the packed byte index = Philox subsequence */
            uint8_t byte = 0;
            for (int ni = 0; ni < wpt; ni++) {
                const int64_t g = r * wpt + ni;
                if (g >= G) break;
                const int64_t i = g * GROUP + d;
                const float xv = (i < n) ? load_elem(x, dtype, i) : 0.0f;
                float nz;
                switch (rng_mode) {
                case RNG_CURAND:   nz = oracle_curand_uniform(seed, (uint64_t)gid, (uint32_t)ni); break;
                case RNG_FAST:     nz = fast_noise(seed, i); break;
                case RNG_RTN:      nz = 0.5f; break;
                default:           nz = noise[i]; break;
                }
                const int maxc = (1 << bits) - 1;
                const int no_overflow_mode = (rng_mode == RNG_FAST || rng_mode == RNG_RTN);
                int32_t val;
                if (dtype == DT_BF16) {
                    /* ours (bf16 is not a reference type): u = fma(x - min, scale, fl32(noise - 0.5)), clamped to
                     * [0, 2^bits - 1] (NaN -> 0), then rounded to nearest even */
                    float t = xv - mn[g];
                    float nzc = nz - 0.5f;
                    float u = fmaf(t, sc[g], nzc);
                    float w = (u > 0.0f) ? u : 0.0f;
                    if (w > (float)maxc) w = (float)maxc;
                    val = float2int_rn(w);
                } else {
                    float u;
                    if (dtype == DT_F32) {
                        float t = xv - mn[g];
                        u = fma_mode ? fmaf(t, sc[g], nz) : (t * sc[g]) + nz;
                    } else {
                        float t = round_T(xv - mn[g], dtype);
                        float p = round_T(t * sc[g], dtype);
                        u = p + nz;
                    }
                    /* (double)u - 0.5, compared with 0 in double, then narrowed to float for the conversion */
                    double w = (double)u - 0.5;
                    w = (w > 0.0) ? w : 0.0;
                    val = float2int_rn((float)w);
                    /* The reference has no upper clamp (a code of 2^bits spills / wraps).  The reference stream and
                     * EXTERNAL keep that.  FAST and RTN, which are ours, cap the fp16 code at 2^bits - 1 (fp32 cannot
                     * overflow there: the noise stays below 1). */
                    if (dtype == DT_F16 && no_overflow_mode && val > maxc) val = maxc;
                }
                byte |= (uint8_t)((uint32_t)val << (ni * bits));   /* no upper clamp: overflow spills / wraps */
            }
            packed[gid] = byte;
        }
    }
    free(mn); free(sc);
    return 0;
}

/* ------------------------------------------------------------------------------------------------
 * dequantize (quantization_cuda_kernel.cu:166-175): out = T(T(code) / scale) + min, each op rounded to T
 * (fp32: IEEE divide, add; bf16, which is not a reference type: fma(code, fl32(1/scale), min) in fp32, then one
 * rounding to bf16).  Writes the first n elements.
 * ---------------------------------------------------------------------------------------------- */
int oracle_dequantize(const uint8_t *packed, const void *qmin, const void *qscale, int dtype, int64_t n,
                      int bits, void *out) {
    if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8)) return 1;
    if (dtype < 0 || dtype > 2) return 2;
    const int wpt = 8 / bits;
    const int mask = (1 << bits) - 1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        const int64_t g = i / GROUP;
        const int d = (int)(i % GROUP);
        const int64_t r = g / wpt;
        const int ni = (int)(g % wpt);
        const int code = (packed[r * GROUP + d] >> (ni * bits)) & mask;
        const float s = load_elem(qscale, scale_dtype(dtype), g), m = load_elem(qmin, dtype, g);
        if (dtype == DT_BF16) {                                  /* ours: fma(code, fl32(1/scale), min), one rounding to bf16 */
            store_elem(out, dtype, i, fmaf((float)code, 1.0f / s, m));
            continue;
        }
        const float c = round_T((float)code, dtype);             /* exact for codes <= 255 in every T */
        const float q = round_T(c / s, dtype);
        store_elem(out, dtype, i, round_T(q + m, dtype));
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------------
 * 1-bit dropout mask (quantization_cuda_kernel.cu:233-251, 280-287): element e of a 512-element block
 * blk goes to bit (t div 16) of word blk*16 + (t mod 16), t = e mod 512.  The packed mask has
 * ceil(n/512)*16 words: a partial last block still spreads its elements over all 16 of its words.  (The
 * reference allocates only ceil(n/32) words and lets the last block store and load past the allocation;
 * the two sizes agree when n is a multiple of 512.)
 * ---------------------------------------------------------------------------------------------- */
int oracle_mask_pack(const uint8_t *x, int64_t n, uint32_t *words) {
    const int64_t nwords = (n + 511) / 512 * 16;
    for (int64_t i = 0; i < nwords; i++) words[i] = 0;
    for (int64_t e = 0; e < n; e++) {
        const int64_t blk = e / 512;
        const int t = (int)(e % 512);
        const int64_t w = blk * 16 + (t % 16);
        if (w < nwords && x[e]) words[w] |= 1u << (t / 16);
    }
    return 0;
}

int oracle_mask_unpack(const uint32_t *words, int64_t n, uint8_t *out) {
    const int64_t nwords = (n + 511) / 512 * 16;
    for (int64_t e = 0; e < n; e++) {
        const int64_t blk = e / 512;
        const int t = (int)(e % 512);
        const int64_t w = blk * 16 + (t % 16);
        out[e] = (w < nwords) ? (uint8_t)((words[w] >> (t / 16)) & 1u) : 0;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------------
 * Greedy bit allocation (calc_precision.cc:66-118).  A max-heap of (float key, int64 index) ordered
 * lexicographically, exactly as std::priority_queue<std::pair<float,int64_t>> orders it: the largest key
 * pops first and equal keys pop the larger index first.
 * Returns 0, or 1 when the heap ran empty before the budget was met (the reference only asserts).
 * ---------------------------------------------------------------------------------------------- */
typedef struct { float key; int64_t idx; } heap_item;

static int item_less(heap_item a, heap_item b) {      /* std::pair operator< */
    if (a.key < b.key) return 1;
    if (b.key < a.key) return 0;
    return a.idx < b.idx;
}
static void heap_push(heap_item *h, int64_t *len, heap_item it) {
    int64_t i = (*len)++;
    h[i] = it;
    while (i > 0) {
        int64_t p = (i - 1) / 2;
        if (!item_less(h[p], h[i])) break;
        heap_item t = h[p]; h[p] = h[i]; h[i] = t; i = p;
    }
}
static heap_item heap_pop(heap_item *h, int64_t *len) {
    heap_item top = h[0];
    h[0] = h[--(*len)];
    int64_t i = 0;
    for (;;) {
        int64_t l = 2 * i + 1, r = l + 1, m = i;
        if (l < *len && item_less(h[m], h[l])) m = l;
        if (r < *len && item_less(h[m], h[r])) m = r;
        if (m == i) break;
        heap_item t = h[m]; h[m] = h[i]; h[i] = t; i = m;
    }
    return top;
}

static int next_bits(int b) { return b == 32 ? 8 : b == 8 ? 4 : b == 4 ? 2 : b == 2 ? 1 : 0; }

/* gain of stepping b -> next(b), calc_precision.cc:87-92: integer coefficients (2^b-1)^2 in int;
 * for b = 32 the reference returns -C/(2^8-1)^2 */
static double step_gain(float C, int b) {
    int nb = next_bits(b);
    int coeff_2 = ((1 << nb) - 1) * ((1 << nb) - 1);
    if (b == 32) return -(double)C / coeff_2;
    int coeff_1 = ((1 << b) - 1) * ((1 << b) - 1);
    return C * (1.0 / coeff_1 - 1.0 / coeff_2);
}

int oracle_calc_precision(int32_t *b, const float *C, const int64_t *w, int64_t L, double target) {
    heap_item *heap = (heap_item *)malloc(sizeof(heap_item) * (size_t)(L ? L : 1));
    int64_t len = 0;
    double b_sum = 0;
    int status = 0;
    for (int64_t i = 0; i < L; i++) if (b[i] > 1) {
        int delta_b = b[i] - next_bits(b[i]);
        double delta = step_gain(C[i], b[i]) / (double)(w[i] * delta_b);
        heap_item it = { (float)delta, i };
        heap_push(heap, &len, it);
        b_sum += (double)((int64_t)b[i] * w[i]);
    }
    while (b_sum > target) {
        if (len == 0) { status = 1; break; }
        heap_item top = heap_pop(heap, &len);
        int64_t i = top.idx;
        int delta_b = b[i] - next_bits(b[i]);
        b[i] = next_bits(b[i]);
        b_sum -= (double)(w[i] * delta_b);
        if (b[i] > 1) {
            int db = b[i] - next_bits(b[i]);
            double delta = step_gain(C[i], b[i]) / (double)(w[i] * db);
            heap_item it = { (float)delta, i };
            heap_push(heap, &len, it);
        }
    }
    free(heap);
    return status;
}

/* ------------------------------------------------------------------------------------------------
 * Sensitivity statistics (autoprec.py:116-119): the three squared distances between gradient vectors.
 * Accumulated in double here; the reference sums in fp32 with torch's reduction tree, so comparisons
 * against this use a relative tolerance.
 * ---------------------------------------------------------------------------------------------- */
int oracle_sq_diffs3(const float *g0, const float *g1, const float *g2, int64_t P, double out3[3]) {
    double d01 = 0, d02 = 0, d12 = 0;
    for (int64_t i = 0; i < P; i++) {
        double a = (double)(float)(g0[i] - g1[i]);
        double b = (double)(float)(g0[i] - g2[i]);
        double c = (double)(float)(g1[i] - g2[i]);
        d01 += a * a; d02 += b * b; d12 += c * c;
    }
    out3[0] = d01; out3[1] = d02; out3[2] = d12;
    return 0;
}

/* ------------------------------------------------------------------------------------------------
 * RNG_FAST (no counterpart in the reference): one Philox4x32-7 call (seven rounds: the member of the family with
 * the fewest rounds that passes BigCrush, Salmon et al., SC'11, table 2; cuRAND's ten add a safety margin that
 * rounding noise does not need) feeds 16 elements with 8 bits of noise
 * each - the 8 elements d..d+7 (d a multiple of 8) of an even group g and the same 8 positions of group g+1.
 * Block index j = (g div 2) * 32 + (d div 8), counter (j_lo, j_hi, 0, 0x46415354 "FAST"), key (seed_lo,
 * seed_hi); element (g, d) takes byte (g mod 2) * 8 + (d mod 8) of the 16 output bytes (word = byte div 4,
 * little endian); noise = (byte + 0.5) / 256, exact in fp32, in (0, 1).
 * ---------------------------------------------------------------------------------------------- */
static float fast_noise(uint64_t seed, int64_t elem) {
    const int64_t g = elem / GROUP;
    const int d = (int)(elem % GROUP);
    uint64_t j = (uint64_t)(g >> 1) * 32u + (uint64_t)(d >> 3);
    int e = (int)((g & 1) * 8 + (d & 7));
    uint32_t ctr[4] = { (uint32_t)j, (uint32_t)(j >> 32), 0u, 0x46415354u };
    uint32_t key[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) };
    uint32_t out[4];
    oracle_philox4x32_r(ctr, key, FAST_ROUNDS, out);
    uint32_t b = (out[e >> 2] >> ((e & 3) * 8)) & 0xffu;
    return ((float)b + 0.5f) * 0.00390625f;
}
float oracle_fast_noise(uint64_t seed, int64_t elem) { return fast_noise(seed, elem); }


/* ------------------------------------------------------------------------------------------------
 * Identities the division-free dequantize kernel rests on, checked by brute force (CPU tests call these).
 * (A) fp16: round_h(fl32(c * fl32(1/s))) == round_h(fl32(c / s)) for every half-precision bit pattern s and
 *     every code c in 0..255.  Returns the number of mismatches (NaN results count as equal).
 * (B) fp32: with r = fl32(1/s), q0 = fl32(c*r), e = fma(-q0, s, c), q = fma(e, r, q0) is the correctly rounded
 *     c/s.  Checked for every `stride`-th significand of s, binades 2^-60..2^59 every `bstep`-th, c in 1..255.
 * ---------------------------------------------------------------------------------------------- */
int64_t oracle_check_half_reciprocal(void) {
    int64_t bad = 0;
    for (uint32_t hs = 0; hs < 65536; hs++) {
        const float s = half_to_float((uint16_t)hs);
        const float r = 1.0f / s;
        for (int c = 0; c < 256; c++) {
            const float cf = (float)c;
            const uint16_t a = float_to_half(cf / s), b = float_to_half(cf * r);
            if ((a & 0x7fff) > 0x7c00 && (b & 0x7fff) > 0x7c00) continue;
            if (a != b) bad++;
        }
    }
    return bad;
}

int64_t oracle_check_markstein(uint32_t stride, int bstep) {
    int64_t bad = 0;
#pragma omp parallel for reduction(+:bad) schedule(static)
    for (int64_t m = 0; m < (1 << 23); m += stride) {
        for (int ex = 127 - 60; ex < 127 + 60; ex += bstep) {
            const float s = u2f(((uint32_t)ex << 23) | (uint32_t)m);
            const float r = 1.0f / s;
            for (int c = 1; c < 256; c++) {
                const float cf = (float)c;
                const float q0 = cf * r;
                const float e = fmaf(-q0, s, cf);
                const float q = fmaf(e, r, q0);
                if (f2u(q) != f2u(cf / s)) bad++;
            }
        }
    }
    return bad;
}

#ifdef _OPENMP
#include <omp.h>
int oracle_threads(void) { return omp_get_max_threads(); }
void oracle_set_threads(int t) { omp_set_num_threads(t); }
#else
int oracle_threads(void) { return 1; }
void oracle_set_threads(int t) { (void)t; }
#endif
