// quantize_nvfp4 / dequantize_nvfp4 / dynamic per-tensor scale for sm_100a.
//
// Bandwidth-bound kernels.  Arithmetic reproduces the reference eager backend bit for bit
// (comfy_kitchen/backends/eager/quantization.py:118-222): amax in the input dtype, three IEEE fp32
// divisions (amax/6, /per_tensor_scale, x/(per_tensor_scale*block_scale)), RNE to e4m3 and e2m1.
// Compiled without fast-math; every rounding below is explicit (__fdiv_rn, __fmul_rn, fmaf).
//
// Work decomposition of the quantizer: one warp handles a "unit" of 4 rows x 64 columns.  The 4 rows
// are r0 + {0,32,64,96} inside one 128-row band and the 64 columns are one group of 4 scale blocks, so
// the 16 block scales of a unit are exactly one 16-byte element of the 128x4 tiled scale tensor
// (comfy_kitchen/float_utils.py:292-326) and the kernel writes that tensor, zero padding included,
// with 16-byte aligned groups of four 4-byte stores and no separate layout pass or memset.
// Lane l owns row r0 + 32*(l/8) and the 8 elements at column 64*cbg + 8*(l%8): a warp load covers
// four fully used 128-byte lines (16-bit inputs), a warp store four full 32-byte sectors of packed output.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace ckb {
namespace {

constexpr int kUnitsPerWarp = 4;   // consecutive 64-column groups a warp has in flight
constexpr int kWarpsPerBlock = 8;

// ---- conversions ------------------------------------------------------------------------------

__device__ __forceinline__ uint8_t f32_to_e4m3_rne(float v) {
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(__half(h));
}

// Eight fp32 values -> eight e2m1 codes, element 2i in the high nibble of byte i (RNE, saturating at 6).
__device__ __forceinline__ uint32_t pack8_e2m1_hi_first(const float (&d)[8]) {
    uint32_t w;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %1, %2;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %3, %4;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %5, %6;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %7, %8;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}"
        : "=r"(w)
        : "f"(d[0]), "f"(d[1]), "f"(d[2]), "f"(d[3]), "f"(d[4]), "f"(d[5]), "f"(d[6]), "f"(d[7]));
    return w;
}

__device__ __forceinline__ uint32_t swap_nibbles32(uint32_t w) {
    return ((w & 0x0f0f0f0fu) << 4) | ((w >> 4) & 0x0f0f0f0fu);
}

// ---- input traits: 8 consecutive elements of one row ---------------------------------------------

template <int DT>
struct Input;

template <>
struct Input<CK_B200_DTYPE_BF16> {
    static constexpr int kBytes = 2;
    struct Raw { uint4 v; };
    static __device__ __forceinline__ Raw zero() { return Raw{make_uint4(0, 0, 0, 0)}; }
    static __device__ __forceinline__ Raw load_vec(const void* p) { return Raw{ldg_stream16(p)}; }
    static __device__ __forceinline__ void set(Raw& r, int i, const void* base, int64_t idx) {
        uint32_t h = ((const unsigned short*)base)[idx];
        uint32_t* w = &r.v.x + (i >> 1);
        *w |= h << ((i & 1) * 16);
    }
    // widened values and the block-local amax, which is taken in bf16 and is exact in fp32
    static __device__ __forceinline__ float unpack(const Raw& r, float (&f)[8]) {
        const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
        uint32_t m = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            __nv_bfloat162 cur = *reinterpret_cast<__nv_bfloat162*>(&m);
            cur = __hmax2(cur, a);
            m = *reinterpret_cast<uint32_t*>(&cur);
        }
        float lo = __uint_as_float(m << 16), hi = __uint_as_float(m & 0xffff0000u);
        return fmaxf(lo, hi);
    }
};

template <>
struct Input<CK_B200_DTYPE_F16> {
    static constexpr int kBytes = 2;
    struct Raw { uint4 v; };
    static __device__ __forceinline__ Raw zero() { return Raw{make_uint4(0, 0, 0, 0)}; }
    static __device__ __forceinline__ Raw load_vec(const void* p) { return Raw{ldg_stream16(p)}; }
    static __device__ __forceinline__ void set(Raw& r, int i, const void* base, int64_t idx) {
        uint32_t h = ((const unsigned short*)base)[idx];
        uint32_t* w = &r.v.x + (i >> 1);
        *w |= h << ((i & 1) * 16);
    }
    static __device__ __forceinline__ float unpack(const Raw& r, float (&f)[8]) {
        const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
            m = fmaxf(m, fmaxf(fabsf(p.x), fabsf(p.y)));   // widening is exact and monotone: same amax as in fp16
        }
        return m;
    }
};

template <>
struct Input<CK_B200_DTYPE_F32> {
    static constexpr int kBytes = 4;
    struct Raw { uint4 v[2]; };
    static __device__ __forceinline__ Raw zero() { return Raw{{make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}}; }
    static __device__ __forceinline__ Raw load_vec(const void* p) {
        return Raw{{ldg_stream16(p), ldg_stream16((const char*)p + 16)}};
    }
    static __device__ __forceinline__ void set(Raw& r, int i, const void* base, int64_t idx) {
        (&r.v[0].x)[i] = ((const uint32_t*)base)[idx];
    }
    static __device__ __forceinline__ float unpack(const Raw& r, float (&f)[8]) {
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            f[i] = __uint_as_float((&r.v[0].x)[i]);
            m = fmaxf(m, fabsf(f[i]));
        }
        return m;
    }
};

// ---- exact division by a shared divisor ----------------------------------------------------------

// Correctly rounded x / t from r = RN(1/t): two rounds of residual correction (Markstein).  The first
// round turns the two-ulp estimate x*r into a faithful quotient, the second makes it the correctly
// rounded one.  Valid while no intermediate leaves the normal range: the caller checks
// 2^-64 <= t <= 2^64 and |x| <= 2^20 * t and otherwise takes the IEEE division.  The sign of the
// result is forced to the sign of x so that -0 (and negative values that round to zero) stay negative.
__device__ __forceinline__ float div_shared(float x, float t, float r) {
    float q = __fmul_rn(x, r);
    q = fmaf(fmaf(-t, q, x), r, q);
    q = fmaf(fmaf(-t, q, x), r, q);
    return __uint_as_float((__float_as_uint(q) & 0x7fffffffu) | (__float_as_uint(x) & 0x80000000u));
}

// ---- quantize -------------------------------------------------------------------------------------

struct QuantArgs {
    const void* x;
    const float* pts;
    uint8_t* q;
    uint8_t* sf;
    int64_t rows, cols;      // logical input
    int64_t prow, pcol;      // padded (output) shape
    int64_t row_groups;      // roundup(prow,128)/4 : number of (band, d3) groups
    int sf_cbg;              // scale tensor width / 4
    int tasks_per_group;     // ceil(sf_cbg / kUnitsPerWarp)
    int hi_first;
};

template <int DT, bool VEC, int VARIANT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) quantize_nvfp4_kernel(const QuantArgs a) {
    using In = Input<DT>;
    const int lane = threadIdx.x & 31;
    const int64_t task = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (task >= a.row_groups * a.tasks_per_group) return;
    const int64_t group = task / a.tasks_per_group;
    const int cbg0 = (int)(task % a.tasks_per_group) * kUnitsPerWarp;
    const int d4 = lane >> 3, sub = lane & 7;
    const int64_t band = group >> 5;
    const int d3 = (int)(group & 31);
    const int64_t r = band * 128 + d3 + 32 * d4;
    const float ts = __ldg(a.pts);
    const bool row_in = r < a.rows;

    typename In::Raw raw[kUnitsPerWarp];
#pragma unroll
    for (int u = 0; u < kUnitsPerWarp; ++u) {
        const int64_t c0 = (int64_t)(cbg0 + u) * 64 + sub * 8;
        raw[u] = In::zero();
        if (row_in && c0 < a.cols) {
            if (VEC) {   // cols % 8 == 0 and 16-byte aligned base: the whole vector is inside the row
                raw[u] = In::load_vec((const char*)a.x + (r * a.cols + c0) * In::kBytes);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (c0 + i < a.cols) In::set(raw[u], i, a.x, r * a.cols + c0 + i);
            }
        }
    }

#pragma unroll
    for (int u = 0; u < kUnitsPerWarp; ++u) {
        const int cbg = cbg0 + u;
        if (cbg >= a.sf_cbg) break;   // uniform across the warp
        const int64_t c0 = (int64_t)cbg * 64 + sub * 8;
        float f[8];
        float amax = In::unpack(raw[u], f);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));   // the two halves of a 16-element block

        // block scale: e4m3( min(amax / 6 / ts, 448) ), and the decode scale t = ts * float(e4m3)
        const bool inside = (r < a.prow) && (c0 < a.pcol);
        uint32_t s8 = 0;
        float t = 0.0f;
        if (inside) {
            float sbs = __fdiv_rn(__fdiv_rn(amax, 6.0f), ts);
            sbs = fminf(sbs, 448.0f);
            s8 = f32_to_e4m3_rne(sbs);
            t = __fmul_rn(ts, e4m3_to_f32((uint8_t)s8));
        }

        uint32_t word = 0;
        if (t != 0.0f) {   // zero decode scale: every element encodes +0 (eager/quantization.py:149-153)
            float d[8];
            bool fast = false;
            if (VARIANT == 1) fast = (t >= 0x1p-64f) && (t <= 0x1p64f) && (amax <= t * 1048576.0f);
            if (fast) {
                const float rcp = __frcp_rn(t);
#pragma unroll
                for (int i = 0; i < 8; ++i) d[i] = div_shared(f[i], t, rcp);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) d[i] = __fdiv_rn(f[i], t);
            }
            word = pack8_e2m1_hi_first(d);   // satfinite clamps to +-6 like the reference's clamp before rounding
            if (!a.hi_first) word = swap_nibbles32(word);
        }
        if (inside) *reinterpret_cast<uint32_t*>(a.q + r * (a.pcol >> 1) + (c0 >> 1)) = word;

        // gather the four block scales of this row (lanes sub = 0,2,4,6) into one 32-bit word on lane sub = 0
        uint32_t sfw = (sub & 1) ? 0u : (s8 << (8 * (sub >> 1)));
        sfw |= __shfl_xor_sync(0xffffffffu, sfw, 2);
        sfw |= __shfl_xor_sync(0xffffffffu, sfw, 4);
        if (sub == 0)
            *reinterpret_cast<uint32_t*>(a.sf + ((band * a.sf_cbg + cbg) * 32 + d3) * 16 + d4 * 4) = sfw;
    }
}

template <int DT>
int launch_quantize(const QuantArgs& a, bool vec, int variant, cudaStream_t stream) {
    const int64_t tasks = a.row_groups * a.tasks_per_group;
    const int64_t blocks = ceil_div64(tasks, kWarpsPerBlock);
    if (blocks <= 0) return CK_B200_OK;
    if (blocks > 0x7fffffffll) return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: tensor too large");
    dim3 grid((unsigned)blocks), block(kWarpsPerBlock * 32);
    if (vec) {
        if (variant == 0) quantize_nvfp4_kernel<DT, true, 0><<<grid, block, 0, stream>>>(a);
        else quantize_nvfp4_kernel<DT, true, 1><<<grid, block, 0, stream>>>(a);
    } else {
        if (variant == 0) quantize_nvfp4_kernel<DT, false, 0><<<grid, block, 0, stream>>>(a);
        else quantize_nvfp4_kernel<DT, false, 1><<<grid, block, 0, stream>>>(a);
    }
    g_launches.fetch_add(1);
    CKB_CUDA_OK(cudaGetLastError());
    return CK_B200_OK;
}

// ---- dequantize -----------------------------------------------------------------------------------

template <int DT>
struct Output;
template <>
struct Output<CK_B200_DTYPE_BF16> {
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ void store8(void* out, int64_t idx, const float (&y)[8]) {
        uint4 o;
        uint32_t* w = &o.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 p = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>((char*)out + idx * 2) = o;
    }
};
template <>
struct Output<CK_B200_DTYPE_F16> {
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ void store8(void* out, int64_t idx, const float (&y)[8]) {
        uint4 o;
        uint32_t* w = &o.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 p = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>((char*)out + idx * 2) = o;
    }
};
template <>
struct Output<CK_B200_DTYPE_F32> {
    static __device__ __forceinline__ float round(float v) { return v; }
    static __device__ __forceinline__ void store8(void* out, int64_t idx, const float (&y)[8]) {
        float4* p = reinterpret_cast<float4*>((char*)out + idx * 4);
        p[0] = make_float4(y[0], y[1], y[2], y[3]);
        p[1] = make_float4(y[4], y[5], y[6], y[7]);
    }
};

// One thread decodes 4 packed bytes (half of a 16-element block).  Rounding follows the eager backend:
// total = out(out(ts) * out(block_scale)), y = out(lut * total)  (eager/quantization.py:213-219).
template <int DT>
__global__ void __launch_bounds__(256) dequantize_nvfp4_kernel(const uint8_t* __restrict__ q,
                                                               const float* __restrict__ pts,
                                                               const uint8_t* __restrict__ sf, void* __restrict__ out,
                                                               int64_t rows, int64_t words_per_row, int sf_cbg,
                                                               int hi_first) {
    using Out = Output<DT>;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * words_per_row) return;
    const int64_t r = gid / words_per_row;
    const int64_t h = gid % words_per_row;
    uint32_t w = ldg_stream4(q + gid * 4);
    if (!hi_first) w = swap_nibbles32(w);
    const float ts_o = Out::round(__ldg(pts));
    const float bs_o = Out::round(e4m3_to_f32(__ldg(sf + sf_offset(r, (int)(h >> 1), sf_cbg))));
    const float total = Out::round(__fmul_rn(ts_o, bs_o));
    float y[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t h2;
        uint16_t byte = (uint16_t)((w >> (8 * i)) & 0xffu);
        // low nibble -> low half, high nibble -> high half
        asm("{\n.reg .b8 b, z;\nmov.b16 {b, z}, %1;\ncvt.rn.f16x2.e2m1x2 %0, b;\n}" : "=r"(h2) : "h"(byte));
        float2 p = __half22float2(*reinterpret_cast<__half2*>(&h2));
        y[2 * i] = Out::round(__fmul_rn(p.y, total));       // element 2i sits in the high nibble
        y[2 * i + 1] = Out::round(__fmul_rn(p.x, total));
    }
    Out::store8(out, r * (words_per_row * 8) + h * 8, y);
}

// ---- dynamic per-tensor scale ---------------------------------------------------------------------

template <int DT>
__global__ void __launch_bounds__(256) amax_kernel(const void* __restrict__ x, int64_t n, uint32_t* __restrict__ acc) {
    float m = 0.0f;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v;
        if (DT == CK_B200_DTYPE_F32) v = ((const float*)x)[i];
        else if (DT == CK_B200_DTYPE_F16) v = __half2float(((const __half*)x)[i]);
        else v = __bfloat162float(((const __nv_bfloat16*)x)[i]);
        m = fmaxf(m, fabsf(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(acc, __float_as_uint(m));   // non-negative floats order like their bits
}

template <int DT>
__global__ void finalize_scale_kernel(float* scale) {
    // amax / (448 * 6) evaluated in the input dtype (comfy_kitchen/tensor/nvfp4.py:66-71)
    *scale = Output<DT>::round(__fdiv_rn(*scale, 2688.0f));
}

}  // namespace
}  // namespace ckb

using namespace ckb;

extern "C" int ck_b200_quantize_nvfp4(const void* x_dev, int x_dtype, const float* per_tensor_scale_dev,
                                      void* q_out_dev, void* sf_out_dev, int64_t rows, int64_t cols, int pad_16x,
                                      int hi_first, void* stream) {
    if (int rc = check_device(nullptr)) return rc;
    if (!x_dev || !per_tensor_scale_dev || !q_out_dev || !sf_out_dev)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: null pointer");
    if (rows < 0 || cols < 0) return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: negative shape");
    if (!pad_16x && (rows % 16 != 0 || cols % 16 != 0))
        return fail(CK_B200_ERR_INVALID_ARGUMENT,
                    "quantize_nvfp4: rows and cols must be divisible by 16 without pad_16x, got %lld x %lld",
                    (long long)rows, (long long)cols);
    if (x_dtype < 0 || x_dtype > 2) return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: dtype code %d", x_dtype);
    QuantArgs a;
    a.x = x_dev;
    a.pts = per_tensor_scale_dev;
    a.q = (uint8_t*)q_out_dev;
    a.sf = (uint8_t*)sf_out_dev;
    a.rows = rows;
    a.cols = cols;
    a.prow = pad_16x ? round_up64(rows, 16) : rows;
    a.pcol = pad_16x ? round_up64(cols, 16) : cols;
    a.row_groups = round_up64(a.prow, 128) / 4;
    const int64_t sf_cols = round_up64(a.pcol / 16, 4);
    if (sf_cols / 4 > 0x3fffffff) return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: too many columns");
    a.sf_cbg = (int)(sf_cols / 4);
    a.tasks_per_group = (int)ceil_div64(a.sf_cbg, kUnitsPerWarp);
    a.hi_first = hi_first ? 1 : 0;
    if (a.prow == 0 || a.pcol == 0) return CK_B200_OK;
    if (((uintptr_t)q_out_dev & 3) || ((uintptr_t)sf_out_dev & 3))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: outputs must be 4-byte aligned");
    const bool vec = (cols % 8 == 0) && (((uintptr_t)x_dev & 15) == 0);
    const int variant = g_quant_variant.load() ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    switch (x_dtype) {
        case CK_B200_DTYPE_F32: return launch_quantize<CK_B200_DTYPE_F32>(a, vec, variant, s);
        case CK_B200_DTYPE_F16: return launch_quantize<CK_B200_DTYPE_F16>(a, vec, variant, s);
        default: return launch_quantize<CK_B200_DTYPE_BF16>(a, vec, variant, s);
    }
}

extern "C" int ck_b200_dequantize_nvfp4(const void* q_dev, const float* per_tensor_scale_dev, const void* sf_dev,
                                        void* out_dev, int out_dtype, int64_t rows, int64_t packed_cols, int hi_first,
                                        void* stream) {
    if (int rc = check_device(nullptr)) return rc;
    if (!q_dev || !per_tensor_scale_dev || !sf_dev || !out_dev)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_nvfp4: null pointer");
    if (rows < 0 || packed_cols < 0 || packed_cols % 8 != 0)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_nvfp4: packed column count %lld must be a multiple of 8",
                    (long long)packed_cols);
    if (out_dtype < 0 || out_dtype > 2)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_nvfp4: dtype code %d", out_dtype);
    if (((uintptr_t)q_dev & 3) || ((uintptr_t)out_dev & 15))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_nvfp4: q must be 4-byte and out 16-byte aligned");
    if (rows == 0 || packed_cols == 0) return CK_B200_OK;
    const int64_t words_per_row = packed_cols / 4;
    const int64_t total = rows * words_per_row;
    const int64_t blocks = ceil_div64(total, 256);
    if (blocks > 0x7fffffffll) return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_nvfp4: tensor too large");
    const int sf_cbg = (int)(round_up64(packed_cols / 8, 4) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    const uint8_t* q = (const uint8_t*)q_dev;
    const uint8_t* sf = (const uint8_t*)sf_dev;
    const int hf = hi_first ? 1 : 0;
    switch (out_dtype) {
        case CK_B200_DTYPE_F32:
            dequantize_nvfp4_kernel<CK_B200_DTYPE_F32><<<(unsigned)blocks, 256, 0, s>>>(q, per_tensor_scale_dev, sf, out_dev, rows, words_per_row, sf_cbg, hf);
            break;
        case CK_B200_DTYPE_F16:
            dequantize_nvfp4_kernel<CK_B200_DTYPE_F16><<<(unsigned)blocks, 256, 0, s>>>(q, per_tensor_scale_dev, sf, out_dev, rows, words_per_row, sf_cbg, hf);
            break;
        default:
            dequantize_nvfp4_kernel<CK_B200_DTYPE_BF16><<<(unsigned)blocks, 256, 0, s>>>(q, per_tensor_scale_dev, sf, out_dev, rows, words_per_row, sf_cbg, hf);
            break;
    }
    g_launches.fetch_add(1);
    CKB_CUDA_OK(cudaGetLastError());
    return CK_B200_OK;
}

extern "C" int ck_b200_dynamic_scale_nvfp4(const void* x_dev, int x_dtype, int64_t numel, float* scale_out_dev,
                                           void* stream) {
    int sms = 0;
    if (int rc = check_device(&sms)) return rc;
    if (!x_dev || !scale_out_dev) return fail(CK_B200_ERR_INVALID_ARGUMENT, "dynamic_scale_nvfp4: null pointer");
    if (numel < 0 || x_dtype < 0 || x_dtype > 2)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dynamic_scale_nvfp4: bad numel or dtype code");
    cudaStream_t s = (cudaStream_t)stream;
    CKB_CUDA_OK(cudaMemsetAsync(scale_out_dev, 0, sizeof(float), s));
    if (numel > 0) {
        int64_t want = ceil_div64(numel, 256 * 8);
        unsigned blocks = (unsigned)(want < (int64_t)sms * 8 ? (want < 1 ? 1 : want) : (int64_t)sms * 8);
        uint32_t* acc = reinterpret_cast<uint32_t*>(scale_out_dev);
        switch (x_dtype) {
            case CK_B200_DTYPE_F32: amax_kernel<CK_B200_DTYPE_F32><<<blocks, 256, 0, s>>>(x_dev, numel, acc); break;
            case CK_B200_DTYPE_F16: amax_kernel<CK_B200_DTYPE_F16><<<blocks, 256, 0, s>>>(x_dev, numel, acc); break;
            default: amax_kernel<CK_B200_DTYPE_BF16><<<blocks, 256, 0, s>>>(x_dev, numel, acc); break;
        }
        g_launches.fetch_add(1);
    }
    switch (x_dtype) {
        case CK_B200_DTYPE_F32: finalize_scale_kernel<CK_B200_DTYPE_F32><<<1, 1, 0, s>>>(scale_out_dev); break;
        case CK_B200_DTYPE_F16: finalize_scale_kernel<CK_B200_DTYPE_F16><<<1, 1, 0, s>>>(scale_out_dev); break;
        default: finalize_scale_kernel<CK_B200_DTYPE_BF16><<<1, 1, 0, s>>>(scale_out_dev); break;
    }
    g_launches.fetch_add(1);
    CKB_CUDA_OK(cudaGetLastError());
    return CK_B200_OK;
}
