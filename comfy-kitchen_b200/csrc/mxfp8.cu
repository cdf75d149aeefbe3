// MXFP8 quantizer and dequantizer for sm_100a: e4m3 data, one power-of-two (e8m0) scale per 32 elements, scales in
// the same 128x4 tiled layout as the NVFP4 path.
//
// Semantics follow the reference eager backend (comfy_kitchen/backends/eager/quantization.py:260-364):
//   amax per block in the input dtype -> need = max(fp32(amax) / 448, 2^-127) -> biased exponent
//   clamp(ceil(log2(need)) + 127, 0, 254) -> data = e4m3_rne(clamp(x / 2^(e-127), +-448)); all-zero blocks store
//   scale byte 0 and +0 data.  The ceiling is taken exactly (the reference evaluates log2 in float32, which can land
//   one exponent lower for quotients within ~2.6e-6 above a power of two; impossible for 16-bit inputs).  A biased
//   exponent of 0 decodes to 0.0 in the reference (float_utils.py:376-382), so such blocks divide by zero there:
//   +-448 for non-zero elements and NaN (0xff) for zeros; reproduced here.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace ckb {
namespace {

struct MxQuantArgs {
    const void* x;
    uint8_t* q;
    uint8_t* sf;
    int rows, cols;      // logical input
    int prow, pcol;      // padded output shape (multiples of 32 when padding was asked for)
    int row_groups;      // roundup(prow, 128) / 4
    int sf_cbg;          // 512-byte scale chunks per 128-row band = ceil(pcol / 128)
    int units_per_warp;  // 128-column units a warp walks
    int vec_ok;          // rows start 16-byte aligned and cols % 8 == 0
};

template <int DT>
__device__ __forceinline__ float widen_at(const void* x, int64_t i) {
    if (DT == CK_B200_DTYPE_F32) return ((const float*)x)[i];
    if (DT == CK_B200_DTYPE_F16) return __half2float(((const __half*)x)[i]);
    return __bfloat162float(((const __nv_bfloat16*)x)[i]);
}

// 16 consecutive elements of one row, widened; zero outside the input
template <int DT>
__device__ __forceinline__ void load16(const MxQuantArgs& a, bool row_in, int64_t row_off, int c0, float (&f)[16]) {
    if (row_in && a.vec_ok && c0 + 16 <= a.cols) {
        if (DT == CK_B200_DTYPE_F32) {
            const uint4* p = reinterpret_cast<const uint4*>((const float*)a.x + row_off + c0);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 w = ldg_stream16(p + v);
                f[4 * v] = __uint_as_float(w.x);
                f[4 * v + 1] = __uint_as_float(w.y);
                f[4 * v + 2] = __uint_as_float(w.z);
                f[4 * v + 3] = __uint_as_float(w.w);
            }
        } else {
            const uint4* p = reinterpret_cast<const uint4*>((const unsigned short*)a.x + row_off + c0);
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const uint4 w = ldg_stream16(p + v);
                const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (DT == CK_B200_DTYPE_BF16) {
                        f[8 * v + 2 * i] = __uint_as_float(ws[i] << 16);
                        f[8 * v + 2 * i + 1] = __uint_as_float(ws[i] & 0xffff0000u);
                    } else {
                        const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&ws[i]));
                        f[8 * v + 2 * i] = h.x;
                        f[8 * v + 2 * i + 1] = h.y;
                    }
                }
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = (row_in && c0 + i < a.cols) ? widen_at<DT>(a.x, row_off + c0 + i) : 0.0f;
    }
}

// Biased e8m0 exponent for a block amax > 0: clamp(ceil(log2(max(amax / 448, 2^-127))) + 127, 0, 254), exact.
__device__ __forceinline__ int biased_exponent(float amax) {
    float need = __fdiv_rn(amax, 448.0f);
    need = fmaxf(need, __uint_as_float(0x00400000u));   // 2^-127
    const uint32_t b = __float_as_uint(need);
    const int e = (int)(b >> 23), mant = (int)(b & 0x7fffffu);
    // normal: 2^(e-127) * (1 + mant/2^23); subnormal (e == 0): only [2^-127, 2^-126) can occur here
    int biased = (e == 0) ? ((mant == 0x400000) ? 0 : 1) : e + (mant != 0 ? 1 : 0);
    return min(biased, 254);
}

// Four rows (r0 + 32*d4) x 128 columns per warp step; a lane owns 16 consecutive elements, two lanes a block.
template <int DT>
__global__ void __launch_bounds__(256) quantize_mxfp8_kernel(const MxQuantArgs a) {
    allow_dependent_launch();
    const int lane = threadIdx.x;
    const int group = blockIdx.x * blockDim.z + threadIdx.z;
    const int seg = blockIdx.y * blockDim.y + threadIdx.y;
    if (group >= a.row_groups) return;
    const int u_begin = seg * a.units_per_warp;
    const int u_end = min(a.sf_cbg, u_begin + a.units_per_warp);
    if (u_begin >= u_end) return;
    grid_dependency_wait();
    const int d4 = lane >> 3, sub = lane & 7;
    const int band = group >> 5, d3 = group & 31;
    const int r = band * 128 + d3 + 32 * d4;
    const bool row_in = r < a.rows, row_out = r < a.prow;
    const int64_t row_off = (int64_t)r * a.cols;
    uint8_t* q_row = a.q + (int64_t)r * a.pcol;
    uint8_t* sf_row = a.sf + (((int64_t)band * a.sf_cbg) * 32 + d3) * 16 + d4 * 4;
    for (int u = u_begin; u < u_end; ++u) {
        const int c0 = u * 128 + sub * 16;
        float f[16];
        load16<DT>(a, row_in, row_off, c0, f);
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(f[i]));
        const float amax = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        uint32_t words[4] = {0u, 0u, 0u, 0u};
        uint32_t s8 = 0;
        if (amax != 0.0f) {
            const int biased = biased_exponent(amax);
            s8 = (uint32_t)biased;
            if (biased != 0) {
                // x / 2^(biased-127) as a product with the exact reciprocal power of two
                const float inv = (biased == 254) ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(254 - biased) << 23);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint16_t lo, hi;
                    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(__fmul_rn(f[4 * i + 1], inv)), "f"(__fmul_rn(f[4 * i], inv)));
                    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(__fmul_rn(f[4 * i + 3], inv)), "f"(__fmul_rn(f[4 * i + 2], inv)));
                    words[i] = (uint32_t)lo | ((uint32_t)hi << 16);
                }
            } else {
                // decode scale 0.0 in the reference: x / 0 = +-inf -> +-448, 0 / 0 = NaN with the sign bit set
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t code = f[i] > 0.0f ? 0x7eu : f[i] < 0.0f ? 0xfeu : 0xffu;
                    words[i >> 2] |= code << (8 * (i & 3));
                }
            }
        }
        if (row_out && c0 < a.pcol) *reinterpret_cast<uint4*>(q_row + c0) = make_uint4(words[0], words[1], words[2], words[3]);
        // scale byte of block b = sub / 2 of this unit sits on the even lanes: gather the row's four into one word
        uint32_t sfw = (sub & 1) ? 0u : (((row_out && c0 < a.pcol) ? s8 : 0u) << (8 * (sub >> 1)));
        sfw |= __shfl_xor_sync(0xffffffffu, sfw, 2);
        sfw |= __shfl_xor_sync(0xffffffffu, sfw, 4);
        if (sub == 0) *reinterpret_cast<uint32_t*>(sf_row + (int64_t)u * 512) = sfw;   // rows >= prow: zero padding
    }
}

// One warp per row, a lane decodes 16 bytes (16 elements, half a block) per step.
template <int DT>
__global__ void __launch_bounds__(256) dequantize_mxfp8_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf,
                                                               void* __restrict__ out, int rows, int cols, int sf_cbg) {
    allow_dependent_launch();
    const int lane = threadIdx.x;
    const int r = blockIdx.x * 8 + threadIdx.y;
    if (r >= rows) return;
    grid_dependency_wait();
    const uint8_t* sf_row = sf + ((int64_t)(r >> 7) * sf_cbg * 32 + (r & 31)) * 16 + ((r & 127) >> 5) * 4;
    const uint8_t* q_row = q + (int64_t)r * cols;
    for (int c0 = (blockIdx.y * 32 + lane) * 16; c0 < cols; c0 += gridDim.y * 32 * 16) {
        const uint4 w = ldg_stream16(q_row + c0);
        const int blk = c0 >> 5;
        const uint32_t e = __ldg(sf_row + (blk >> 2) * 512 + (blk & 3));
        const float scale = e == 0 ? 0.0f : __uint_as_float(e << 23);   // e8m0_to_f32: exponent 0 decodes to 0.0
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        float y[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t h_lo, h_hi;
            asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h_lo) : "h"((uint16_t)(ws[i] & 0xffffu)));
            asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h_hi) : "h"((uint16_t)(ws[i] >> 16)));
            const float2 a = __half22float2(*reinterpret_cast<__half2*>(&h_lo));
            const float2 b = __half22float2(*reinterpret_cast<__half2*>(&h_hi));
            y[4 * i] = __fmul_rn(a.x, scale);
            y[4 * i + 1] = __fmul_rn(a.y, scale);
            y[4 * i + 2] = __fmul_rn(b.x, scale);
            y[4 * i + 3] = __fmul_rn(b.y, scale);
        }
        const int64_t o = (int64_t)r * cols + c0;
        if (DT == CK_B200_DTYPE_F32) {
            float4* p = reinterpret_cast<float4*>((float*)out + o);
#pragma unroll
            for (int i = 0; i < 4; ++i) p[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
        } else {
            uint32_t pk[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (DT == CK_B200_DTYPE_BF16) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
                    pk[i] = *reinterpret_cast<uint32_t*>(&v);
                } else {
                    __half2 v = __floats2half2_rn(y[2 * i], y[2 * i + 1]);
                    pk[i] = *reinterpret_cast<uint32_t*>(&v);
                }
            }
            uint4* p = reinterpret_cast<uint4*>((unsigned short*)out + o);
            p[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            p[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
    }
}

template <int DT>
int launch_quantize_mxfp8(const MxQuantArgs& a0, int sms, cudaStream_t stream) {
    MxQuantArgs a = a0;
    // enough warps for ~4 waves of 8-warp blocks, at least two units per warp when the row is long enough
    const int64_t want_warps = (int64_t)sms * 4 * 8 * 4;
    int segs = (int)ceil_div64(want_warps, a.row_groups);
    if (segs < 1) segs = 1;
    if (segs > a.sf_cbg) segs = a.sf_cbg;
    a.units_per_warp = (int)ceil_div64(a.sf_cbg, segs);
    segs = (int)ceil_div64(a.sf_cbg, a.units_per_warp);
    const int wy = segs >= 4 ? 4 : segs >= 2 ? 2 : 1;
    const int wz = 8 / wy;
    dim3 block(32, wy, wz);
    dim3 grid((unsigned)ceil_div64(a.row_groups, wz), (unsigned)ceil_div64(segs, wy));
    const cudaError_t err = launch_dependent(kLaunchFamilyQuantize, quantize_mxfp8_kernel<DT>, grid, block, 0, stream, a);
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
    return CK_B200_OK;
}

}  // namespace
}  // namespace ckb

using namespace ckb;

extern "C" int ck_b200_quantize_mxfp8(const void* x_dev, int x_dtype, void* q_out_dev, void* sf_out_dev, int64_t rows,
                                      int64_t cols, int pad_32x, void* stream) {
    int sms = 0;
    if (int rc = check_device(&sms)) return rc;
    if (!x_dev || !q_out_dev || !sf_out_dev) return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_mxfp8: null pointer");
    if (rows < 0 || cols < 0 || rows > 0x3fffff00ll || cols > 0x3fffff00ll)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_mxfp8: rows and cols must be in [0, 2^30)");
    if (!pad_32x && (rows % 32 != 0 || cols % 32 != 0))
        return fail(CK_B200_ERR_INVALID_ARGUMENT,
                    "quantize_mxfp8: rows and cols must be divisible by 32 without pad_32x, got %lld x %lld",
                    (long long)rows, (long long)cols);
    if (x_dtype < 0 || x_dtype > 2) return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_mxfp8: dtype code %d", x_dtype);
    if (((uintptr_t)q_out_dev & 15) || ((uintptr_t)sf_out_dev & 3))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_mxfp8: q must be 16-byte and scales 4-byte aligned");
    MxQuantArgs a;
    a.x = x_dev;
    a.q = (uint8_t*)q_out_dev;
    a.sf = (uint8_t*)sf_out_dev;
    a.rows = (int)rows;
    a.cols = (int)cols;
    a.prow = (int)(pad_32x ? round_up64(rows, 32) : rows);
    a.pcol = (int)(pad_32x ? round_up64(cols, 32) : cols);
    if (a.prow == 0 || a.pcol == 0) return CK_B200_OK;
    a.row_groups = (int)(round_up64(a.prow, 128) / 4);
    a.sf_cbg = (int)ceil_div64(a.pcol, 128);
    a.units_per_warp = 1;
    const int elt = x_dtype == CK_B200_DTYPE_F32 ? 4 : 2;
    a.vec_ok = ((((uintptr_t)x_dev) & 15) == 0 && (cols * elt) % 16 == 0) ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    switch (x_dtype) {
        case CK_B200_DTYPE_F32: return launch_quantize_mxfp8<CK_B200_DTYPE_F32>(a, sms, s);
        case CK_B200_DTYPE_F16: return launch_quantize_mxfp8<CK_B200_DTYPE_F16>(a, sms, s);
        default: return launch_quantize_mxfp8<CK_B200_DTYPE_BF16>(a, sms, s);
    }
}

extern "C" int ck_b200_dequantize_mxfp8(const void* q_dev, const void* sf_dev, void* out_dev, int out_dtype, int64_t rows,
                                        int64_t cols, void* stream) {
    if (int rc = check_device(nullptr)) return rc;
    if (!q_dev || !sf_dev || !out_dev) return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_mxfp8: null pointer");
    if (rows < 0 || cols < 0 || cols % 32 != 0 || rows > 0x3fffff00ll || cols > 0x3fffff00ll)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_mxfp8: cols = %lld must be a multiple of 32", (long long)cols);
    if (out_dtype < 0 || out_dtype > 2) return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_mxfp8: dtype code %d", out_dtype);
    if (((uintptr_t)q_dev & 15) || ((uintptr_t)out_dev & 15))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_mxfp8: q and out must be 16-byte aligned");
    if (rows == 0 || cols == 0) return CK_B200_OK;
    const int sf_cbg = (int)ceil_div64(cols, 128);
    const int64_t col_chunks = ceil_div64(cols, 32 * 16);
    const dim3 grid((unsigned)ceil_div64(rows, 8), (unsigned)(col_chunks < 65535 ? col_chunks : 65535));
    const dim3 block(32, 8);
    cudaStream_t s = (cudaStream_t)stream;
    const uint8_t* q = (const uint8_t*)q_dev;
    const uint8_t* sf = (const uint8_t*)sf_dev;
    cudaError_t err;
    switch (out_dtype) {
        case CK_B200_DTYPE_F32:
            err = launch_dependent(kLaunchFamilyQuantize, dequantize_mxfp8_kernel<CK_B200_DTYPE_F32>, grid, block, 0, s, q, sf, out_dev, (int)rows, (int)cols, sf_cbg);
            break;
        case CK_B200_DTYPE_F16:
            err = launch_dependent(kLaunchFamilyQuantize, dequantize_mxfp8_kernel<CK_B200_DTYPE_F16>, grid, block, 0, s, q, sf, out_dev, (int)rows, (int)cols, sf_cbg);
            break;
        default:
            err = launch_dependent(kLaunchFamilyQuantize, dequantize_mxfp8_kernel<CK_B200_DTYPE_BF16>, grid, block, 0, s, q, sf, out_dev, (int)rows, (int)cols, sf_cbg);
            break;
    }
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
    return CK_B200_OK;
}
