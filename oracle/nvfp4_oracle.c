/*
 * CPU oracle for the NVFP4 linear path: quantize_nvfp4, dequantize_nvfp4 and the
 * dequantize -> fp32 matmul restatement of scaled_mm_nvfp4.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are compared
 * against and the CPU baseline that the benchmark times; the product never calls it.
 *
 * It restates, in scalar C with IEEE-754 single precision arithmetic, the algorithm of the
 * reference's eager backend:
 *   quantize_nvfp4      comfy_kitchen/backends/eager/quantization.py:118-163
 *   fp32 -> e2m1 (RNE)  comfy_kitchen/float_utils.py:41-150  (_f32_to_floatx_unpacked, ebits=2, mbits=1)
 *   nibble packing      comfy_kitchen/float_utils.py:253-260 (pack_uint4)
 *   128x4 scale swizzle comfy_kitchen/float_utils.py:292-326 (to_blocked) / :329-352 (from_blocked)
 *   fp32 -> e4m3fn      torch's float8_e4m3fn cast used by comfy_kitchen/float_utils.py:37-38
 *   dequantize_nvfp4    comfy_kitchen/backends/eager/quantization.py:174-222
 *   scaled_mm_nvfp4     comfy_kitchen/backends/eager/quantization.py:225-249 has no CPU kernel; the
 *                       reference tests check other backends against dequantize -> F.linear
 *                       (tests/test_qdq.py:490-509), which is what nvfp4_oracle_dequant_f32 + a
 *                       fp32 matmul in oracle.py restate.
 *
 * Parity of this file is pinned by tests/test_oracle_golden.py against vectors produced by
 * running the reference eager backend (tests/golden/make_golden.py).
 *
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * No FMA contraction and no fast-math: every fp32 operation below must round exactly once.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORACLE_F32 = 0, ORACLE_F16 = 1, ORACLE_BF16 = 2 }; /* reference dtype codes, eager/quantization.py:34-42 */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ---- 16-bit float conversions ------------------------------------------------------------- */

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* fp32 -> bf16, round to nearest even (torch c10::BFloat16 round_to_nearest_even). */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0; /* NaN */
    uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)((u + bias) >> 16);
}

static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-08f;
        return bits_f32(f32_bits(v) | sign);
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* fp32 -> fp16, round to nearest even, overflow to inf. */
static inline uint16_t f32_to_f16(float f) {
    uint32_t u = f32_bits(f);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);     /* >= 65536 -> inf (65520 handled below) */
    if (a < 0x38800000u) {                                        /* < 2^-14: subnormal half */
        /* add 0.5 (exponent 126): the sum's ulp is 2^-24, so the add rounds to the fp16 subnormal grid (RNE) */
        float v = bits_f32(a) + 0.5f;
        return (uint16_t)(sign | (uint16_t)(f32_bits(v) - 0x3f000000u));
    }
    uint32_t mant_odd = (a >> 13) & 1u;
    a += ((uint32_t)(15 - 127) << 23) + 0xfffu;
    a += mant_odd;
    return (uint16_t)(sign | (uint16_t)(a >> 13));                /* may carry into inf at 65520+, as IEEE wants */
}

static inline float load_as_f32(const void* x, int dtype, int64_t i) {
    switch (dtype) {
        case ORACLE_F32: return ((const float*)x)[i];
        case ORACLE_F16: return f16_to_f32(((const uint16_t*)x)[i]);
        default: return bf16_to_f32(((const uint16_t*)x)[i]);
    }
}

/* round an fp32 value to the given dtype and return it widened back to fp32 */
static inline float round_to_dtype(float v, int dtype) {
    switch (dtype) {
        case ORACLE_F32: return v;
        case ORACLE_F16: return f16_to_f32(f32_to_f16(v));
        default: return bf16_to_f32(f32_to_bf16(v));
    }
}

static inline void store_from_f32(void* out, int dtype, int64_t i, float v) {
    switch (dtype) {
        case ORACLE_F32: ((float*)out)[i] = v; break;
        case ORACLE_F16: ((uint16_t*)out)[i] = f32_to_f16(v); break;
        default: ((uint16_t*)out)[i] = f32_to_bf16(v); break;
    }
}

/* ---- 8-bit and 4-bit float conversions ----------------------------------------------------- */

/* fp32 (>= 0 after the clamp to 448) -> float8_e4m3fn, round to nearest even; the cast torch applies
 * in _float8_round (comfy_kitchen/float_utils.py:37-38).  Values that round above 448 and NaN give 0x7f. */
static inline uint8_t f32_to_e4m3fn(float f) {
    uint32_t u = f32_bits(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7fffffffu;
    uint8_t r;
    if (a >= 0x43f00000u) {                 /* >= 480 (first value that does not round to 448), inf, NaN */
        r = 0x7f;
    } else if (a < 0x3c800000u) {           /* < 2^-6: subnormal result, grid 2^-9 */
        float v = bits_f32(a) + bits_f32(141u << 23); /* + 2^14: the sum's ulp is 2^-9 */
        r = (uint8_t)(f32_bits(v) - (141u << 23));
    } else {
        uint32_t mant_odd = (a >> 20) & 1u;
        a += ((uint32_t)(7 - 127) << 23) + 0x7ffffu;
        a += mant_odd;
        r = (uint8_t)(a >> 20);
    }
    return (uint8_t)(r | sign);
}

static inline float e4m3fn_to_f32(uint8_t b) {
    uint32_t sign = (uint32_t)(b & 0x80u) << 24;
    uint32_t exp = (b >> 3) & 0xfu;
    uint32_t man = b & 7u;
    float v;
    if (exp == 0) v = (float)man * 0.001953125f;                       /* man * 2^-9 */
    else if (exp == 15 && man == 7) v = NAN;
    else v = bits_f32(((exp + 120u) << 23) | (man << 20));
    return bits_f32(f32_bits(v) | sign);
}

/* fp32 -> e2m1 code in the low nibble (sign in bit 3), round to nearest even, saturating at 6.
 * Follows the three branches of comfy_kitchen/float_utils.py:87-150 for ebits=2, mbits=1. */
static inline uint8_t f32_to_e2m1(float f) {
    uint32_t u = f32_bits(f);
    uint8_t sign = (uint8_t)((u >> 28) & 0x8u);
    uint32_t a = u & 0x7fffffffu;
    float x = bits_f32(a);
    uint8_t r;
    if (x >= 6.0f) {
        r = 7;
    } else if (x < 1.0f) {
        float v = x + bits_f32(149u << 23);      /* + 2^22: the sum's ulp is 0.5 */
        r = (uint8_t)(f32_bits(v) - (149u << 23));
    } else {
        uint32_t mant_odd = (a >> 22) & 1u;
        a += ((uint32_t)(1 - 127) << 23) + 0x1fffffu;
        a += mant_odd;
        r = (uint8_t)(a >> 22);
    }
    return (uint8_t)(r | sign);
}

static const float E2M1_VALUES[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                      -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* ---- layout helpers ------------------------------------------------------------------------ */

static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

/* Byte offset of logical scale (r, c) in the 128x4 tiled ("swizzled") scale tensor whose padded
 * width is sf_cols; equivalent to to_blocked, comfy_kitchen/float_utils.py:292-326. */
static inline int64_t swizzled_sf_offset(int64_t r, int64_t c, int64_t sf_cols) {
    int64_t rb = r / 128, rem = r % 128, cb = c / 4;
    return ((rb * (sf_cols / 4) + cb) * 32 + rem % 32) * 16 + (rem / 32) * 4 + c % 4;
}

int64_t nvfp4_oracle_sf_offset(int64_t r, int64_t c, int64_t sf_cols) { return swizzled_sf_offset(r, c, sf_cols); }

/* ---- quantize_nvfp4 ------------------------------------------------------------------------ */

/*
 * x: [rows, cols] row-major, dtype code 0/1/2.  With pad_16x the logical input is zero-padded to
 * multiples of 16 in both dimensions (eager/quantization.py:128-136); without it rows and cols
 * must already be multiples of 16 (returns -1 otherwise).
 * q_out:  uint8 [prow, pcol/2];  sf_out: uint8 (e4m3 bits) [round_up(prow,128), round_up(pcol/16,4)], swizzled.
 */
int nvfp4_oracle_quantize(const void* x, int dtype, int64_t rows, int64_t cols, float per_tensor_scale,
                          int pad_16x, int hi_first, uint8_t* q_out, uint8_t* sf_out) {
    int64_t prow = rows, pcol = cols;
    if (pad_16x) { prow = round_up(rows, 16); pcol = round_up(cols, 16); }
    else if (rows % 16 != 0 || cols % 16 != 0) return -1;
    const int64_t nblk = pcol / 16;
    const int64_t sf_rows = round_up(prow, 128), sf_cols = round_up(nblk, 4);
    memset(sf_out, 0, (size_t)(sf_rows * sf_cols));
    const float ts = per_tensor_scale;

#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < prow; ++r) {
        for (int64_t j = 0; j < nblk; ++j) {
            float v[16];
            float amax = 0.0f;
            for (int i = 0; i < 16; ++i) {
                int64_t c = j * 16 + i;
                float e = (r < rows && c < cols) ? load_as_f32(x, dtype, r * cols + c) : 0.0f;
                v[i] = e;
                float a = fabsf(e);
                if (a > amax) amax = a;                       /* amax in the input dtype == amax of the widened values */
            }
            float bs = amax / 6.0f;                           /* :142 */
            float sbs = bs / ts;                              /* :143 */
            if (sbs > 448.0f) sbs = 448.0f;                   /* :144 clamp(max=448); NaN stays NaN */
            uint8_t s8 = f32_to_e4m3fn(sbs);                  /* :145 */
            float total = ts * e4m3fn_to_f32(s8);             /* :146 */
            sf_out[swizzled_sf_offset(r, j, sf_cols)] = s8;   /* :155,162 */
            uint8_t code[16];
            for (int i = 0; i < 16; ++i) {
                float d;
                if (total == 0.0f) d = 0.0f;                  /* :149-153 zero-scale blocks encode +0 */
                else d = v[i] / total;                        /* :152 true division */
                if (d > 6.0f) d = 6.0f;                       /* :157 */
                if (d < -6.0f) d = -6.0f;
                code[i] = f32_to_e2m1(d);                     /* :160 */
            }
            uint8_t* q = q_out + r * (pcol / 2) + j * 8;
            for (int i = 0; i < 8; ++i)                       /* float_utils.py:253-260 */
                q[i] = hi_first ? (uint8_t)((code[2 * i] << 4) | code[2 * i + 1])
                                : (uint8_t)((code[2 * i + 1] << 4) | code[2 * i]);
        }
    }
    return 0;
}

/* ---- dequantize_nvfp4 ---------------------------------------------------------------------- */

/*
 * q: uint8 [rows, pcols]; sf: swizzled e4m3 bits [round_up(rows,128), round_up(2*pcols/16,4)];
 * out: [rows, 2*pcols] in out_dtype.  Two roundings to the output dtype, as eager does:
 * total = out(out(ts) * out(bs)) (eager/quantization.py:213) then y = out(lut * total) (:216-219).
 */
int nvfp4_oracle_dequantize(const uint8_t* q, float per_tensor_scale, const uint8_t* sf, int64_t rows,
                            int64_t pcols, int out_dtype, int hi_first, void* out) {
    const int64_t cols = pcols * 2;
    if (cols % 16 != 0) return -1;
    const int64_t nblk = cols / 16;
    const int64_t sf_cols = round_up(nblk, 4);
    const float ts_o = round_to_dtype(per_tensor_scale, out_dtype);

#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t j = 0; j < nblk; ++j) {
            float bs_o = round_to_dtype(e4m3fn_to_f32(sf[swizzled_sf_offset(r, j, sf_cols)]), out_dtype);
            float total = round_to_dtype(ts_o * bs_o, out_dtype);
            for (int i = 0; i < 8; ++i) {
                uint8_t b = q[r * pcols + j * 8 + i];
                uint8_t first = hi_first ? (uint8_t)(b >> 4) : (uint8_t)(b & 0xf);
                uint8_t second = hi_first ? (uint8_t)(b & 0xf) : (uint8_t)(b >> 4);
                float l0 = round_to_dtype(E2M1_VALUES[first], out_dtype);
                float l1 = round_to_dtype(E2M1_VALUES[second], out_dtype);
                store_from_f32(out, out_dtype, r * cols + j * 16 + 2 * i, l0 * total);
                store_from_f32(out, out_dtype, r * cols + j * 16 + 2 * i + 1, l1 * total);
            }
        }
    }
    return 0;
}

/* Dequantize to fp32 for the GEMM restatement (dequantize_nvfp4(..., float32)); same as above with
 * out_dtype fp32, kept as a separate entry so the GEMM oracle reads as one call per operand. */
int nvfp4_oracle_dequant_f32(const uint8_t* q, float per_tensor_scale, const uint8_t* sf, int64_t rows,
                             int64_t pcols, int hi_first, float* out) {
    return nvfp4_oracle_dequantize(q, per_tensor_scale, sf, rows, pcols, ORACLE_F32, hi_first, out);
}

/* y[m,n] = out_dtype( sum_k a[m,k] * b[n,k] + bias[n] ), fp32 accumulation in k order, a/b already
 * dequantized to fp32.  Small-shape checker; oracle.py uses a BLAS matmul for larger shapes. */
int nvfp4_oracle_matmul_nt(const float* a, const float* b, const float* bias_or_null, int64_t M, int64_t N,
                           int64_t K, int out_dtype, void* out) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            const float* pa = a + m * K;
            const float* pb = b + n * K;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            int64_t k = 0;
            for (; k + 8 <= K; k += 8)
                for (int u = 0; u < 8; ++u) acc[u] += pa[k + u] * pb[k + u];
            float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
            for (; k < K; ++k) s += pa[k] * pb[k];
            if (bias_or_null) s += bias_or_null[n];
            store_from_f32(out, out_dtype, m * N + n, s);
        }
    }
    return 0;
}

/* fp32 array -> bf16/fp16 bits (RNE), used by oracle.py after a BLAS matmul */
void nvfp4_oracle_round_array(const float* in, int64_t n, int out_dtype, void* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) store_from_f32(out, out_dtype, i, in[i]);
}

/* widen bf16/fp16 bits to fp32 */
void nvfp4_oracle_widen_array(const void* in, int64_t n, int in_dtype, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = load_as_f32(in, in_dtype, i);
}

/* Per-tensor scale as TensorCoreNVFP4Layout.quantize computes it when none is given
 * (comfy_kitchen/tensor/nvfp4.py:66-71): amax(|x|) and the division by 448*6 are carried out in the
 * input dtype, and only the result is widened to fp32. */
float nvfp4_oracle_dynamic_scale(const void* x, int dtype, int64_t n) {
    float amax = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        float a = fabsf(load_as_f32(x, dtype, i));
        if (a > amax) amax = a;
    }
    return round_to_dtype(amax / 2688.0f, dtype);
}

/* ---- MXFP8: block 32, power-of-two (e8m0) block scales, e4m3 data ---------------------------------
 * Restates comfy_kitchen/backends/eager/quantization.py:260-364 (quantize_mxfp8, dequantize_mxfp8) and
 * e8m0_to_f32 (comfy_kitchen/float_utils.py:376-382).  One deliberate difference, stated here and checked by
 * the golden vectors: the reference takes ceil(log2(amax/448)) with a float32 log2, which rounds a quotient
 * that lies within ~2.6e-6 above a power of two down onto it (one exponent lower); this restatement takes the
 * exact ceiling, like the reference's CUDA kernel (comfy_kitchen/backends/cuda/ops/quantize_mxfp8.cu:56-64, e8m0
 * conversion rounding toward +infinity).  The reference's own tests allow +-1 on the exponent between its backends
 * (tests/test_qdq.py:431-438); on bf16 and fp16 inputs the two agree always (amax/448 cannot come that close).
 */

/* biased e8m0 exponent of a block with the given amax (> 0) */
static inline int mxfp8_biased_exponent(float amax) {
    float need = amax / 448.0f;
    const float min_scale = bits_f32(0x00400000u); /* 2^-127 */
    if (need < min_scale) need = min_scale;
    int ex;
    const float fr = frexpf(need, &ex);            /* need = fr * 2^ex, fr in [0.5, 1) */
    int ce = (fr == 0.5f) ? ex - 1 : ex;           /* exact ceil(log2(need)) */
    int biased = ce + 127;
    if (biased < 0) biased = 0;
    if (biased > 254) biased = 254;
    return biased;
}

int mxfp8_oracle_quantize(const void* x, int dtype, int64_t rows, int64_t cols, int pad_32x, uint8_t* q_out,
                          uint8_t* sf_out) {
    const int64_t prow = pad_32x ? round_up(rows, 32) : rows;
    const int64_t pcol = pad_32x ? round_up(cols, 32) : cols;
    if (pcol % 32 != 0) return 1;
    const int64_t nblk = pcol / 32;
    const int64_t sf_rows = round_up(prow, 128), sf_cols = round_up(nblk, 4);
    memset(sf_out, 0, (size_t)(sf_rows * sf_cols));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < prow; ++r) {
        for (int64_t b = 0; b < nblk; ++b) {
            float v[32];
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) {
                const int64_t c = b * 32 + i;
                v[i] = (r < rows && c < cols) ? load_as_f32(x, dtype, r * cols + c) : 0.0f;
                const float a = fabsf(v[i]);
                if (a > amax) amax = a;
            }
            uint8_t* q = q_out + r * pcol + b * 32;
            if (amax == 0.0f) {                       /* zero block: scale byte 0, data +0 */
                memset(q, 0, 32);
                continue;
            }
            const int biased = mxfp8_biased_exponent(amax);
            sf_out[swizzled_sf_offset(r, b, sf_cols)] = (uint8_t)biased;
            /* e8m0_to_f32 maps a biased exponent of 0 to 0.0, not 2^-127: the division below then yields
             * +-inf (clamped to +-448) and, for zero elements, the default NaN (sign set on the CPU) */
            const float scale = biased == 0 ? 0.0f : bits_f32((uint32_t)biased << 23);
            for (int i = 0; i < 32; ++i) {
                float d = v[i] / scale;
                if (d != d) { q[i] = 0xff; continue; }
                if (d > 448.0f) d = 448.0f;
                if (d < -448.0f) d = -448.0f;
                q[i] = f32_to_e4m3fn(d);
            }
        }
    }
    return 0;
}

int mxfp8_oracle_dequantize(const uint8_t* q, const uint8_t* sf, int64_t rows, int64_t cols, int out_dtype, void* out) {
    if (cols % 32 != 0) return 1;
    const int64_t nblk = cols / 32;
    const int64_t sf_cols = round_up(nblk, 4);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) {
            const uint8_t e = sf[swizzled_sf_offset(r, c / 32, sf_cols)];
            const float scale = e == 0 ? 0.0f : bits_f32((uint32_t)e << 23);
            store_from_f32(out, out_dtype, r * cols + c, e4m3fn_to_f32(q[r * cols + c]) * scale);
        }
    return 0;
}

/* Number of OpenMP threads the loops above use from now on (a launcher may have exported OMP_NUM_THREADS=1). */
void nvfp4_oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int nvfp4_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
