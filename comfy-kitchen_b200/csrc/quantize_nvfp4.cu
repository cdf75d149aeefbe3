// quantize_nvfp4 / dequantize_nvfp4 / dynamic per-tensor scale for sm_100a.
//
// Bandwidth-bound kernels.  Arithmetic reproduces the reference eager backend bit for bit
// (comfy_kitchen/backends/eager/quantization.py:118-222): amax in the input dtype, three IEEE fp32
// divisions (amax/6, /per_tensor_scale, x/(per_tensor_scale*block_scale)), RNE to e4m3 and e2m1.
// Compiled without fast-math; every rounding below is explicit (__fdiv_rn, __fmul_rn, fmaf).  The common path
// obtains the three correctly rounded quotients without a division instruction (a correctly rounded reciprocal
// and residual corrections in fused arithmetic); anything unusual (infinities, operands outside the range where
// that is exact, zero scales) takes IEEE divisions, chosen by warp votes.
//
// Work decomposition of the quantizer: one warp handles a "unit" of 4 rows x 64 columns.  The 4 rows
// are r0 + {0,32,64,96} inside one 128-row band and the 64 columns are one group of 4 scale blocks, so
// the 16 block scales of a unit are exactly one 16-byte element of the 128x4 tiled scale tensor
// (comfy_kitchen/float_utils.py:292-326) and the kernel writes that tensor, zero padding included,
// with 16-byte aligned groups of four 4-byte stores and no separate layout pass or memset.
// Lane l owns row r0 + 32*(l/8) and the 8 elements at column 64*cbg + 8*(l%8): a warp load covers
// four fully used 128-byte lines (16-bit inputs), a warp store four full 32-byte sectors of packed output.
#include <mutex>

#include "quantize_nvfp4_device.cuh"

namespace ckb {
namespace {

// Launch geometry: block (32, WX, WY) with WX * WY = kWarpsPerBlock; warp (wx, wy) of block (bx, by, bz) handles
// segment bx*WX + wx of row group (bz*65535 + by)*WY + wy, so no thread divides anything.
template <int DT, bool VEC, int VARIANT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, kBlocksPerSM) quantize_nvfp4_kernel(const QuantArgs a) {
    allow_dependent_launch();
    const int lane = threadIdx.x;
    const int seg = blockIdx.x * blockDim.y + threadIdx.y;
    // row groups are handed out last band first: the bottom band is the one that may hold padding rows, whose
    // warps take the slower edge walk and should not be the ones the kernel ends on
    const int group = a.row_groups - 1 - (int)((blockIdx.z * 65535 + blockIdx.y) * blockDim.z + threadIdx.z);
    if (seg >= a.segments || group < 0) return;   // whole warps
    grid_dependency_wait();
    quantize_segment<DT, VEC, VARIANT>(a, seg, group, lane, __ldg(a.pts));
}

// Mid-sized inputs (20 MB to 0.25 GB of bf16): the units of all row groups, taken as one sequence (group after group, bottom band first), are cut
// into one equal, even-sized range per resident warp.  Every warp then walks a long stretch (a range crosses at most
// a few row-group boundaries, where the walk starts afresh) and the grid is exactly one full wave, instead of several
// waves of short segments, each paying the load latency with a part-filled ring.
template <int DT, bool VEC, int VARIANT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, kBlocksPerSM)
quantize_nvfp4_flat_kernel(const QuantArgs a, int per_warp, long long total_units) {
    allow_dependent_launch();
    const int lane = threadIdx.x;
    long long pos = ((long long)blockIdx.x * kWarpsPerBlock + threadIdx.y) * per_warp;
    const long long end = min(total_units, pos + per_warp);
    if (pos >= end) return;   // whole warps
    grid_dependency_wait();
    const float ts = __ldg(a.pts);
    while (pos < end) {
        const int gi = (int)(pos / a.sf_cbg);
        const int u0 = (int)(pos - (long long)gi * a.sf_cbg);
        const int u1 = (int)min((long long)a.sf_cbg, (long long)u0 + (end - pos));
        quantize_units<DT, VEC, VARIANT>(a, u0, u1, a.row_groups - 1 - gi, lane, ts);
        pos += u1 - u0;
    }
}

template <int DT, bool VEC, int VARIANT>
cudaError_t launch_quantize_flat(const QuantArgs& a, int resident_warps, cudaStream_t stream) {
    const long long total = (long long)a.row_groups * a.sf_cbg;
    const int per_warp = (int)round_up64(ceil_div64(total, resident_warps), 2);
    const unsigned blocks = (unsigned)ceil_div64(ceil_div64(total, per_warp), kWarpsPerBlock);
    return launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_flat_kernel<DT, VEC, VARIANT>, dim3(blocks),
                            dim3(32, kWarpsPerBlock), 0, stream, a, per_warp, total);
}

// Inputs of up to about 32 MB with rows and columns multiples of 128: the whole input in flight at once, parked in
// shared memory (quantize_nvfp4_onchip_kernel, defined with the dynamic quantizer below).  Sets *launched.
template <int DT>
int launch_quantize_onchip(const QuantArgs& a, int sms, cudaStream_t stream, bool* launched);

template <int DT>
int launch_quantize(QuantArgs a, bool vec, int variant, int sms, cudaStream_t stream) {
    if (a.row_groups <= 0 || a.sf_cbg <= 0) return CK_B200_OK;
    if (vec && variant == 2 && g_quant_onchip.load()) {
        bool launched = false;
        if (int rc = launch_quantize_onchip<DT>(a, sms, stream, &launched)) return rc;
        if (launched) return CK_B200_OK;
    }
    {
        // one wave of long walks once every resident warp gets at least `kFlatMinUnits` units; rows with an odd
        // number of units stay on the segment geometry (ranges would start on odd units)
        const long long total = (long long)a.row_groups * a.sf_cbg;
        const int resident_warps = kBlocksPerSM * sms * kWarpsPerBlock;
        // and only up to kFlatMaxUnits per warp: beyond that the segment geometry, whose resident blocks work on one
        // compact region of the input at a time, measured faster (65536 x 12288: 5.7 TB/s against 4.1 with one wave
        // of 886-unit ranges and 5.5 with seven waves of 128-unit ranges)
        constexpr int kFlatMaxUnits = 128;
        if (g_quant_flat.load() && vec && a.sf_cbg % 2 == 0 && total >= (long long)resident_warps * g_quant_flat.load() &&
            total <= (long long)resident_warps * kFlatMaxUnits) {
            a.seg_units = a.sf_cbg;
            a.segments = 1;
            cudaError_t err;
            if (variant == 0) err = launch_quantize_flat<DT, true, 0>(a, resident_warps, stream);
            else if (variant == 2) err = launch_quantize_flat<DT, true, 2>(a, resident_warps, stream);
            else err = launch_quantize_flat<DT, true, 1>(a, resident_warps, stream);
            g_launches.fetch_add(1);
            CKB_CUDA_OK(err);
            return CK_B200_OK;
        }
    }
    // Cut rows into segments of `su` units (even, at least the prefetch ring) so that the blocks fill whole waves
    // of the kBlocksPerSM blocks an SM holds: among the candidates within 4 % of the best balance take the longest segment
    // (longer walks amortise the per-warp set-up).
    const int resident = kBlocksPerSM * sms;
    int best_su = kRing, best_wx = 1;
    double best_eff = -1.0;
    for (int pass = 0; pass < 2; ++pass)
    for (int su = kRing; ; su += 2) {
        if (su > a.sf_cbg) su = (int)round_up64(a.sf_cbg, 2) < kRing ? kRing : (int)round_up64(a.sf_cbg, 2);
        const int segs = (int)ceil_div64(a.sf_cbg, su);
        // warps of a block side by side along the row while that idles no more than an eighth of them
        int wx = kWarpsPerBlock;
        while (wx > 1 && (int)round_up64(segs, wx) * 7 > segs * 8) wx >>= 1;
        const int64_t ctas = ceil_div64(segs, wx) * ceil_div64(a.row_groups, kWarpsPerBlock / wx);
        const double waves = (double)ctas / resident;
        const double eff = waves / (double)ceil_div64(ctas, resident) * ((double)a.sf_cbg / ((double)segs * su)) *
                           ((double)segs / (double)round_up64(segs, wx));
        if (pass == 0) {
            if (eff > best_eff) best_eff = eff;
        } else if (eff >= 0.96 * best_eff) {
            best_su = su;
            best_wx = wx;
        }
        if (su >= a.sf_cbg || su >= 256) break;
    }
    a.seg_units = best_su;
    a.segments = (int)ceil_div64(a.sf_cbg, best_su);
    const int wx = best_wx;
    const int wy = kWarpsPerBlock / wx;
    const int64_t gy_total = ceil_div64(a.row_groups, wy);
    dim3 block(32, wx, wy);
    dim3 grid((unsigned)ceil_div64(a.segments, wx), (unsigned)(gy_total < 65535 ? gy_total : 65535),
              (unsigned)ceil_div64(gy_total, 65535));
    cudaError_t err;
    if (vec) {
        if (variant == 0) err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_kernel<DT, true, 0>, grid, block, 0, stream, a);
        else if (variant == 2) err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_kernel<DT, true, 2>, grid, block, 0, stream, a);
        else err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_kernel<DT, true, 1>, grid, block, 0, stream, a);
    } else {
        if (variant == 0) err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_kernel<DT, false, 0>, grid, block, 0, stream, a);
        else if (variant == 2) err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_kernel<DT, false, 2>, grid, block, 0, stream, a);
        else err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_kernel<DT, false, 1>, grid, block, 0, stream, a);
    }
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
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

// One thread decodes 4 packed bytes (half of a 16-element block) at a time, kDequantIter of them per pass so that their
// loads are in flight together.  Block (32, 8): a warp owns one row, its lanes consecutive 4-byte words (16-byte
// outputs), so loads and stores are fully coalesced and nothing is divided.  Rounding follows the eager backend:
// total = out(out(ts) * out(block_scale)), y = out(lut * total)  (eager/quantization.py:213-219).
constexpr int kDequantIter = 4;
template <int DT>
__global__ void __launch_bounds__(256) dequantize_nvfp4_kernel(const uint8_t* __restrict__ q,
                                                               const float* __restrict__ pts,
                                                               const uint8_t* __restrict__ sf, void* __restrict__ out,
                                                               int rows, int words_per_row, int sf_cbg, int hi_first) {
    using Out = Output<DT>;
    const int lane = threadIdx.x;
    const int r = blockIdx.x * 8 + threadIdx.y;
    if (r >= rows) return;   // whole warps
    grid_dependency_wait();
    const float ts_o = Out::round(__ldg(pts));
    // scale (r, c) lives at sf_row + (c / 4) * 512 + c % 4 in the 128x4 tiled layout
    const uint8_t* sf_row = sf + ((int64_t)(r >> 7) * sf_cbg * 32 + (r & 31)) * 16 + ((r & 127) >> 5) * 4;
    const uint8_t* q_row = q + (int64_t)r * words_per_row * 4;
    const int64_t out_row = (int64_t)r * words_per_row * 8;
    for (int base = blockIdx.y * (32 * kDequantIter); base < words_per_row; base += gridDim.y * (32 * kDequantIter)) {
        uint32_t w[kDequantIter];
        uint32_t sb[kDequantIter];
#pragma unroll
        for (int i = 0; i < kDequantIter; ++i) {
            const int wi = base + lane + 32 * i;
            w[i] = 0;
            sb[i] = 0;
            if (wi < words_per_row) {
                w[i] = ldg_stream4(q_row + wi * 4);
                const int c = wi >> 1;
                sb[i] = __ldg(sf_row + (c >> 2) * 512 + (c & 3));
            }
        }
#pragma unroll
        for (int i = 0; i < kDequantIter; ++i) {
            const int wi = base + lane + 32 * i;
            if (wi >= words_per_row) break;
            uint32_t word = w[i];
            if (!hi_first) word = swap_nibbles32(word);
            const float bs_o = Out::round(e4m3_to_f32((uint8_t)sb[i]));
            const float total = Out::round(__fmul_rn(ts_o, bs_o));
            float y[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t h2;
                uint16_t byte = (uint16_t)((word >> (8 * k)) & 0xffu);
                // low nibble -> low half, high nibble -> high half
                asm("{\n.reg .b8 b, z;\nmov.b16 {b, z}, %1;\ncvt.rn.f16x2.e2m1x2 %0, b;\n}" : "=r"(h2) : "h"(byte));
                float2 p = __half22float2(*reinterpret_cast<__half2*>(&h2));
                y[2 * k] = Out::round(__fmul_rn(p.y, total));       // element 2k sits in the high nibble
                y[2 * k + 1] = Out::round(__fmul_rn(p.x, total));
            }
            Out::store8(out, out_row + (int64_t)wi * 8, y);
        }
    }
}

// ---- dynamic per-tensor scale ---------------------------------------------------------------------

// amax(|x|) over the whole tensor into *acc (bits of a non-negative float, combined with atomicMax).  16-byte loads,
// four in flight per thread; the maximum is taken in the input dtype, which widening to fp32 preserves exactly.
template <int DT>
__global__ void __launch_bounds__(256) amax_kernel(const void* __restrict__ x, int64_t n, uint32_t* __restrict__ acc) {
    constexpr int kPerVec = (DT == CK_B200_DTYPE_F32) ? 4 : 8;
    float m = 0.0f;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const int64_t vecs = aligned ? n / kPerVec : 0;
    auto fold = [&](const uint4& v) {
        if (DT == CK_B200_DTYPE_BF16) {
            const uint32_t p = maxabs_bf16x2(maxabs_bf16x2(v.x, v.y), maxabs_bf16x2(v.z, v.w));
            m = fmaxf(m, fmaxf(__uint_as_float((p << 16) & 0x7fff0000u), __uint_as_float(p & 0x7fff0000u)));
        } else if (DT == CK_B200_DTYPE_F16) {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            __half2 h = __habs2(*reinterpret_cast<const __half2*>(&w[0]));
#pragma unroll
            for (int i = 1; i < 4; ++i) h = __hmax2(h, __habs2(*reinterpret_cast<const __half2*>(&w[i])));
            const float2 p = __half22float2(h);
            m = fmaxf(m, fmaxf(p.x, p.y));
        } else {
            m = fmaxf(fmaxf(m, fabsf(__uint_as_float(v.x))), fabsf(__uint_as_float(v.y)));
            m = fmaxf(fmaxf(m, fabsf(__uint_as_float(v.z))), fabsf(__uint_as_float(v.w)));
        }
    };
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    int64_t i = tid;
    for (; i + 3 * stride < vecs; i += 4 * stride) {
        const uint4 a = ldg_stream16(xv + i), b = ldg_stream16(xv + i + stride), c = ldg_stream16(xv + i + 2 * stride),
                    d = ldg_stream16(xv + i + 3 * stride);
        fold(a);
        fold(b);
        fold(c);
        fold(d);
    }
    for (; i < vecs; i += stride) fold(ldg_stream16(xv + i));
    for (int64_t j = vecs * kPerVec + tid; j < n; j += stride) {   // tail, or everything when the base is unaligned
        float v;
        if (DT == CK_B200_DTYPE_F32) v = ((const float*)x)[j];
        else if (DT == CK_B200_DTYPE_F16) v = __half2float(((const __half*)x)[j]);
        else v = __bfloat162float(((const __nv_bfloat16*)x)[j]);
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

// ---- per-tensor scale and quantization in one launch --------------------------------------------------------
//
// TensorCoreNVFP4Layout.quantize derives the per-tensor scale from the tensor itself when the caller gives none
// (comfy_kitchen/tensor/nvfp4.py:66-71): amax(|x|) / (448 * 6) in x's dtype.  As separate kernels that is a full read
// of x from HBM for the maximum and a second one for the quantizer.  quantize_nvfp4_dynamic_kernel does both in one
// launch of the one-wave geometry above: every warp first takes the maximum over the range of units it will
// quantize (which leaves x in the 126 MB L2), the blocks meet at a grid-wide counter, and every warp then
// quantizes its range from L2 with the scale all blocks now agree on.  The grid never exceeds the blocks that are
// resident at once, so the blocks can wait for one another; the wait is bounded all the same (about a second),
// after which the block records WAIT_QUANT_GRID in the status word and returns without quantizing.
//
// DynamicSync lives in 16 bytes of caller memory that are zero before the first launch; the last block past the
// meeting point leaves them zero again, so any sequence of launches and graph replays on one stream works.
struct DynamicSync {
    uint32_t amax_bits;   // bits of the running maximum (non-negative floats order like their bits)
    uint32_t arrived;     // blocks that have contributed their maximum
    uint32_t departed;    // blocks that have read the final maximum
    uint32_t pad;
};
constexpr int WAIT_QUANT_GRID = 8;
__device__ int g_quant_status = 0;

// The grid-wide meeting point of the dynamic quantizer, run by one thread per block: contributes the block's maximum,
// waits (bounded) until every block has, and returns the per-tensor scale amax / (448 * 6) evaluated in the input
// dtype (comfy_kitchen/tensor/nvfp4.py:66-71), or a negative value when the wait ran out (WAIT_QUANT_GRID is then in
// the status word).  Block 0 publishes the scale; the last block past the point leaves the counters zero.
template <int DT>
__device__ __forceinline__ float grid_meet(DynamicSync* sync, float block_max, unsigned expected_blocks, long long wait_cycles,
                                           float* scale_out) {
    atomicMax(&sync->amax_bits, __float_as_uint(block_max));
    __threadfence();
    atomicAdd(&sync->arrived, 1u);
    float ts = -1.0f;
    const long long start = clock64();
    for (;;) {
        uint32_t n;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(n) : "l"(&sync->arrived) : "memory");
        if (n >= expected_blocks) {
            uint32_t bits;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(bits) : "l"(&sync->amax_bits) : "memory");
            ts = Output<DT>::round(__fdiv_rn(__uint_as_float(bits), 2688.0f));
            break;
        }
        if (clock64() - start > wait_cycles) {
            atomicCAS(&g_quant_status, 0, WAIT_QUANT_GRID);
            break;
        }
        __nanosleep(64);
    }
    if (ts >= 0.0f) {
        if (blockIdx.x == 0) *scale_out = ts;
        if (atomicAdd(&sync->departed, 1u) + 1u == expected_blocks) {
            sync->amax_bits = 0u;
            sync->departed = 0u;
            __threadfence();
            sync->arrived = 0u;
        }
    }
    return ts;
}

template <int DT>
__device__ __forceinline__ float raw_amax(const typename Input<DT>::Raw& r) {
    if constexpr (DT == CK_B200_DTYPE_BF16) {
        const uint32_t p = maxabs_bf16x2(maxabs_bf16x2(r.v.x, r.v.y), maxabs_bf16x2(r.v.z, r.v.w));
        return fmaxf(__uint_as_float((p << 16) & 0x7fff0000u), __uint_as_float(p & 0x7fff0000u));
    } else {
        return Pairs<DT>::half_amax(r);
    }
}

// Maximum of |x| over the part of units [pos, end) of the flat unit sequence that this lane owns.  The range is
// walked from its end to its start: the quantizing pass that follows walks it from the start, so what this pass
// read last - the part of the range most likely to be still in L2 - is what that pass reads first.
template <int DT>
__device__ __forceinline__ float range_amax(const QuantArgs& a, long long pos, long long end, int lane) {
    using In = Input<DT>;
    constexpr int kUnitBytes = 64 * In::kBytes;
    float m = 0.0f;
    const int sub = lane & 7;
    while (end > pos) {
        const int gi = (int)((end - 1) / a.sf_cbg);
        const long long base = (long long)gi * a.sf_cbg;
        const int u1 = (int)(end - base);
        const int u0 = (int)(max(pos, base) - base);
        const int group = a.row_groups - 1 - gi;
        const int r = (group >> 5) * 128 + (group & 31) + 32 * (lane >> 3);
        if (r < a.rows) {
            const char* p = (const char*)a.x + ((int64_t)r * a.cols + sub * 8) * In::kBytes;
            // units whose eight columns of this lane lie inside the row (cols is a multiple of 8 on this path)
            const int u_in = min(u1, (a.cols - sub * 8 + 63) / 64);
            int u = u_in;
            for (; u - 4 >= u0; u -= 4) {
                const typename In::Raw r0 = In::load_vec(p + (int64_t)(u - 1) * kUnitBytes),
                                       r1 = In::load_vec(p + (int64_t)(u - 2) * kUnitBytes),
                                       r2 = In::load_vec(p + (int64_t)(u - 3) * kUnitBytes),
                                       r3 = In::load_vec(p + (int64_t)(u - 4) * kUnitBytes);
                m = fmaxf(fmaxf(m, fmaxf(raw_amax<DT>(r0), raw_amax<DT>(r1))), fmaxf(raw_amax<DT>(r2), raw_amax<DT>(r3)));
            }
            for (; u > u0; --u) m = fmaxf(m, raw_amax<DT>(In::load_vec(p + (int64_t)(u - 1) * kUnitBytes)));
        }
        end = base + u0;
    }
    return m;
}

template <int DT, int VARIANT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, kBlocksPerSM)
quantize_nvfp4_dynamic_kernel(const QuantArgs a, float* __restrict__ scale_out, DynamicSync* __restrict__ sync, int per_warp,
                              long long total_units, unsigned expected_blocks, long long wait_cycles) {
    allow_dependent_launch();
    __shared__ float s_max[kWarpsPerBlock];
    __shared__ float s_ts;
    const int lane = threadIdx.x, warp = threadIdx.y;
    const long long pos = ((long long)blockIdx.x * kWarpsPerBlock + warp) * per_warp;
    const long long end = min(total_units, pos + per_warp);
    grid_dependency_wait();
    // phase 1: this warp's share of the maximum
    float m = pos < end ? range_amax<DT>(a, pos, end, lane) : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_max[warp] = m;
    __syncthreads();
    if (warp == 0 && lane == 0) {
        float bm = s_max[0];
#pragma unroll
        for (int w = 1; w < kWarpsPerBlock; ++w) bm = fmaxf(bm, s_max[w]);
        s_ts = grid_meet<DT>(sync, bm, expected_blocks, wait_cycles, scale_out);
    }
    __syncthreads();
    const float ts = s_ts;
    if (ts < 0.0f || pos >= end) return;
    // phase 2: the quantizer's walk over the same range, now served by L2
    long long p = pos;
    while (p < end) {
        const int gi = (int)(p / a.sf_cbg);
        const int u0 = (int)(p - (long long)gi * a.sf_cbg);
        const int u1 = (int)min((long long)a.sf_cbg, (long long)u0 + (end - p));
        quantize_units<DT, true, VARIANT>(a, u0, u1, a.row_groups - 1 - gi, lane, ts);
        p += u1 - u0;
    }
}


// ---- inputs that fit the SMs' shared memory: the whole input in flight at once ------------------------------------
//
// Up to about 32 MB of 16-bit input (18 units per warp, 72 KB of shared memory per block, three blocks per SM - the
// 28 MB activation of a Flux-class block is exactly this size) every warp asks for its whole range at once with
// 16-byte asynchronous copies into shared memory (no registers held, so nothing limits how much is in flight), one
// copy group per pair of units, and quantizes pair after pair as the groups land.  A register ring over the same range
// needs three rounds of HBM latency (6 + 6 + 4 units); this needs one, which is what a 9 us kernel is made of.
// Interior shapes only (rows and columns multiples of 128: no padding rows, whole pairs of units).
// DYNAMIC: the per-tensor scale is derived from the input itself (the layout's amax / (448 * 6)): the maximum is
// taken over the parked range, the blocks meet at the grid-wide counter, and the parked range is quantized with the
// scale all blocks agree on - x is read from HBM once and from nowhere else.
constexpr int kOnchipMaxUnits = 18;   // units per warp that can be parked (72 KB per block)
constexpr int kOnchipMaxPairs = kOnchipMaxUnits / 2;

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Every warp commits kOnchipMaxPairs groups (empty ones at the end): group `pair` has landed once at most
// kOnchipMaxPairs - 1 - pair younger groups are pending.
__device__ __forceinline__ void cp_async_wait_pair(int pair) {
    switch (pair) {
        case 0: cp_async_wait<8>(); break;
        case 1: cp_async_wait<7>(); break;
        case 2: cp_async_wait<6>(); break;
        case 3: cp_async_wait<5>(); break;
        case 4: cp_async_wait<4>(); break;
        case 5: cp_async_wait<3>(); break;
        case 6: cp_async_wait<2>(); break;
        case 7: cp_async_wait<1>(); break;
        default: cp_async_wait<0>(); break;
    }
}
static_assert(kOnchipMaxPairs == 9, "cp_async_wait_pair covers nine groups");

template <int DT, bool DYNAMIC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, kBlocksPerSM)
quantize_nvfp4_onchip_kernel(const QuantArgs a, float* __restrict__ scale_out, DynamicSync* __restrict__ sync, int per_warp,
                             long long total_units, unsigned expected_blocks, long long wait_cycles) {
    using In = Input<DT>;
    using Raw = typename In::Raw;
    static_assert(In::kBytes == 2, "16-bit inputs");
    constexpr int kUnitBytes = 64 * In::kBytes;
    extern __shared__ uint4 stash_all[];
    allow_dependent_launch();
    __shared__ float s_max[kWarpsPerBlock];
    __shared__ float s_ts;
    const int lane = threadIdx.x, warp = threadIdx.y;
    uint4* stash = stash_all + (size_t)warp * per_warp * 32 + lane;   // [unit of the range][lane]
    const uint32_t stash_u32 = smem_u32(stash);
    const long long pos = ((long long)blockIdx.x * kWarpsPerBlock + warp) * per_warp;
    const long long end = min(total_units, pos + per_warp);
    const int sub = lane & 7;
    grid_dependency_wait();
    // phase 1: ask for the whole range
    int npairs = 0;
    {
        long long p = pos;
        while (p < end) {
            const int gi = (int)(p / a.sf_cbg);
            const int u0 = (int)(p - (long long)gi * a.sf_cbg);
            const int u1 = (int)min((long long)a.sf_cbg, (long long)u0 + (end - p));
            const int group = a.row_groups - 1 - gi;
            const int r = (group >> 5) * 128 + (group & 31) + 32 * (lane >> 3);
            const char* src = (const char*)a.x + ((int64_t)r * a.cols + u0 * 64 + sub * 8) * In::kBytes;
            for (int u = u0; u < u1; u += 2, ++npairs, src += 2 * kUnitBytes) {
                cp_async_16(stash_u32 + (uint32_t)(2 * npairs) * 512u, src);
                cp_async_16(stash_u32 + (uint32_t)(2 * npairs + 1) * 512u, src + kUnitBytes);
                cp_async_commit();
            }
            p += u1 - u0;
        }
        for (int k = npairs; k < kOnchipMaxPairs; ++k) cp_async_commit();
    }
    float ts;
    if constexpr (DYNAMIC) {
        cp_async_wait<0>();
        float m = 0.0f;
        for (int j = 0; j < 2 * npairs; ++j) {
            Raw v;
            v.v = stash[j * 32];
            m = fmaxf(m, raw_amax<DT>(v));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) s_max[warp] = m;
        __syncthreads();
        if (warp == 0 && lane == 0) {
            float bm = s_max[0];
#pragma unroll
            for (int w = 1; w < kWarpsPerBlock; ++w) bm = fmaxf(bm, s_max[w]);
            s_ts = grid_meet<DT>(sync, bm, expected_blocks, wait_cycles, scale_out);
        }
        __syncthreads();
        ts = s_ts;
        if (ts < 0.0f) return;
    } else {
        ts = __ldg(a.pts);
    }
    if (pos >= end) return;
    // phase 2: quantize the parked range pair by pair (each lane reads back only what it asked for itself)
    LaneCtx c;
    c.sub = sub;
    c.odd = sub & 1;
    c.ts = ts;
    c.ts_in_range = ts >= 0x1p-60f && ts <= 0x1p60f;
    c.rcp_ts = c.ts_in_range ? __frcp_rn(ts) : 0.0f;
    c.row_in = c.row_out = true;
    c.hi_first = a.hi_first != 0;
    c.cols = a.cols;
    c.pcol = a.pcol;
    const int x_unit = c.odd ? 1 : 0, y_unit = 1 - x_unit;
    long long p = pos;
    int pair = 0;
    while (p < end) {
        const int gi = (int)(p / a.sf_cbg);
        const int u0 = (int)(p - (long long)gi * a.sf_cbg);
        const int u1 = (int)min((long long)a.sf_cbg, (long long)u0 + (end - p));
        const int group = a.row_groups - 1 - gi;
        const int band = group >> 5, d3 = group & 31, d4 = lane >> 3;
        const int r = band * 128 + d3 + 32 * d4;
        uint8_t* q_row = a.q + (int64_t)r * (a.pcol >> 1) + sub * 4;
        uint8_t* sf_row = a.sf + (((int64_t)band * a.sf_cbg) * 32 + d3) * 16 + d4 * 4 + (int64_t)(sub & 1) * 512;
        for (int u = u0; u < u1; u += 2, ++pair) {
            if constexpr (!DYNAMIC) cp_async_wait_pair(pair);
            Raw raw_x, raw_y;
            raw_x.v = stash[(2 * pair + x_unit) * 32];
            raw_y.v = stash[(2 * pair + y_unit) * 32];
            uint32_t wx, wy, s8;
            if (c.hi_first) quantize_pair_xy<DT, true>(c, raw_x, raw_y, wx, wy, s8);
            else quantize_pair_xy<DT, false>(c, raw_x, raw_y, wx, wy, s8);
            *reinterpret_cast<uint32_t*>(q_row + (u + x_unit) * 32) = wx;
            *reinterpret_cast<uint32_t*>(q_row + (u + y_unit) * 32) = wy;
            const uint32_t sfw = gather_scale_word(s8, sub);
            if (sub < 2) *reinterpret_cast<uint32_t*>(sf_row + (int64_t)u * 512) = sfw;
        }
        p += u1 - u0;
    }
}


// Resident blocks of the dynamic kernel per SM (cached per device and dtype); never more than kBlocksPerSM.
template <int DT>
int dynamic_blocks_per_sm(int* out) {
    static std::mutex mu;
    static int cache[64] = {0};
    int dev = 0;
    CKB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(CK_B200_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == 0) {
        int n = 0;
        CKB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quantize_nvfp4_dynamic_kernel<DT, 2>,
                                                                  kWarpsPerBlock * 32, 0));
        cache[dev] = n < 1 ? -1 : (n > kBlocksPerSM ? kBlocksPerSM : n);
    }
    if (cache[dev] < 0) return fail(CK_B200_ERR_CUDA, "the dynamic quantizer kernel does not fit on this device");
    *out = cache[dev];
    return CK_B200_OK;
}

// Opt the on-chip kernels in to 72 KB per block, once per device, dtype and form.
template <int DT, bool DYNAMIC>
int onchip_ready() {
    static std::mutex mu;
    static int cache[64] = {0};
    int dev = 0;
    CKB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(CK_B200_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == 0) {
        constexpr int kBytes = kWarpsPerBlock * kOnchipMaxUnits * 512;
        CKB_CUDA_OK(cudaFuncSetAttribute(quantize_nvfp4_onchip_kernel<DT, DYNAMIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
        int n = 0;
        CKB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quantize_nvfp4_onchip_kernel<DT, DYNAMIC>,
                                                                  kWarpsPerBlock * 32, kBytes));
        cache[dev] = n >= kBlocksPerSM ? 1 : -1;
    }
    return cache[dev] > 0 ? CK_B200_OK : -1;   // -1: not an error, the caller takes the other variant
}

template <int DT>
int launch_quantize_onchip(const QuantArgs& a_in, int sms, cudaStream_t stream, bool* launched) {
    *launched = false;
    if constexpr (DT != CK_B200_DTYPE_F32) {
        QuantArgs a = a_in;
        const long long total = (long long)a.row_groups * a.sf_cbg;
        const long long resident_warps = (long long)kBlocksPerSM * sms * kWarpsPerBlock;
        int per_warp = (int)round_up64(ceil_div64(total, resident_warps), 2);
        if (per_warp < 2) per_warp = 2;
        if (per_warp > kOnchipMaxUnits || a.sf_cbg % 2 != 0 || a.rows % 128 != 0 || a.cols % 128 != 0 || a.rows != a.prow ||
            a.cols != a.pcol)
            return CK_B200_OK;
        const int ready = onchip_ready<DT, false>();
        if (ready > 0) return ready;
        if (ready != CK_B200_OK) return CK_B200_OK;   // does not fit three to an SM on this device: the other kernels
        const unsigned blocks = (unsigned)ceil_div64(ceil_div64(total, per_warp), kWarpsPerBlock);
        a.seg_units = a.sf_cbg;
        a.segments = 1;
        const cudaError_t err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_onchip_kernel<DT, false>, dim3(blocks),
                                                 dim3(32, kWarpsPerBlock), (size_t)kWarpsPerBlock * per_warp * 512, stream, a,
                                                 (float*)nullptr, (DynamicSync*)nullptr, per_warp, total, 0u, 0ll);
        g_launches.fetch_add(1);
        CKB_CUDA_OK(err);
        *launched = true;
    }
    return CK_B200_OK;
}

template <int DT>
int launch_quantize_dynamic(QuantArgs a, float* scale_out, void* sync, int sms, cudaStream_t stream) {
    int per_sm = 0;
    if (int rc = dynamic_blocks_per_sm<DT>(&per_sm)) return rc;
    const long long total = (long long)a.row_groups * a.sf_cbg;
    const long long resident_warps = (long long)per_sm * sms * kWarpsPerBlock;
    int per_warp = (int)round_up64(ceil_div64(total, resident_warps), 2);
    if (per_warp < 2) per_warp = 2;
    const unsigned blocks = (unsigned)ceil_div64(ceil_div64(total, per_warp), kWarpsPerBlock);
    a.seg_units = a.sf_cbg;
    a.segments = 1;
    // test hook: expect arrivals that never come and give up after about 0.1 s instead of 1 s
    const int extra = g_quant_sync_test.load();
    const long long wait_cycles = extra > 0 ? 200000000ll : 2000000000ll;
    const unsigned expected = blocks + (unsigned)(extra > 0 ? extra : 0);
    cudaError_t err = cudaSuccess;
    bool launched = false;
    if constexpr (DT != CK_B200_DTYPE_F32) {
        // small enough to stay on chip between the phases, and no padding anywhere
        if (g_dynamic_smem.load() && per_sm == kBlocksPerSM && per_warp <= kOnchipMaxUnits && a.rows % 128 == 0 &&
            a.cols % 128 == 0 && a.rows == a.prow && a.cols == a.pcol) {
            const int ready = onchip_ready<DT, true>();
            if (ready > 0) return ready;
            if (ready == CK_B200_OK) {
                err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_onchip_kernel<DT, true>, dim3(blocks),
                                       dim3(32, kWarpsPerBlock), (size_t)kWarpsPerBlock * per_warp * 512, stream, a, scale_out,
                                       (DynamicSync*)sync, per_warp, total, expected, wait_cycles);
                launched = true;
            }
        }
    }
    if (!launched)
        err = launch_dependent(kLaunchFamilyQuantize, quantize_nvfp4_dynamic_kernel<DT, 2>, dim3(blocks),
                               dim3(32, kWarpsPerBlock), 0, stream, a, scale_out, (DynamicSync*)sync, per_warp, total,
                               expected, wait_cycles);
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
    return CK_B200_OK;
}

}  // namespace
}  // namespace ckb

using namespace ckb;

extern "C" int ck_b200_quantize_nvfp4(const void* x_dev, int x_dtype, const float* per_tensor_scale_dev,
                                      void* q_out_dev, void* sf_out_dev, int64_t rows, int64_t cols, int pad_16x,
                                      int hi_first, void* stream) {
    int sms = 0;
    if (int rc = check_device(&sms)) return rc;
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
    if (rows > 0x3fffff00ll || cols > 0x3fffff00ll)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: rows and cols must be below 2^30");
    a.rows = (int)rows;
    a.cols = (int)cols;
    a.prow = (int)(pad_16x ? round_up64(rows, 16) : rows);
    a.pcol = (int)(pad_16x ? round_up64(cols, 16) : cols);
    a.row_groups = (int)(round_up64(a.prow, 128) / 4);
    const int64_t sf_cols = round_up64(a.pcol / 16, 4);
    a.sf_cbg = (int)(sf_cols / 4);
    a.seg_units = a.segments = 0;
    a.hi_first = hi_first ? 1 : 0;
    if (a.prow == 0 || a.pcol == 0) return CK_B200_OK;
    if (((uintptr_t)q_out_dev & 3) || ((uintptr_t)sf_out_dev & 3))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4: outputs must be 4-byte aligned");
    const bool vec = (cols % 8 == 0) && (((uintptr_t)x_dev & 15) == 0);
    const int variant = g_quant_variant.load();
    cudaStream_t s = (cudaStream_t)stream;
    switch (x_dtype) {
        case CK_B200_DTYPE_F32: return launch_quantize<CK_B200_DTYPE_F32>(a, vec, variant, sms, s);
        case CK_B200_DTYPE_F16: return launch_quantize<CK_B200_DTYPE_F16>(a, vec, variant, sms, s);
        default: return launch_quantize<CK_B200_DTYPE_BF16>(a, vec, variant, sms, s);
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
    if (rows > 0x3fffff00ll || words_per_row > 0x3fffff00ll)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "dequantize_nvfp4: rows and packed columns must be below 2^30");
    const int64_t col_chunks = ceil_div64(words_per_row, 32 * kDequantIter);
    const dim3 grid((unsigned)ceil_div64(rows, 8), (unsigned)(col_chunks < 65535 ? col_chunks : 65535));
    const dim3 block(32, 8);
    const int sf_cbg = (int)(round_up64(packed_cols / 8, 4) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    const uint8_t* q = (const uint8_t*)q_dev;
    const uint8_t* sf = (const uint8_t*)sf_dev;
    const int hf = hi_first ? 1 : 0;
    cudaError_t err;
    switch (out_dtype) {
        case CK_B200_DTYPE_F32:
            err = launch_dependent(kLaunchFamilyQuantize, dequantize_nvfp4_kernel<CK_B200_DTYPE_F32>, grid, block, 0, s, q, per_tensor_scale_dev, sf, out_dev, (int)rows, (int)words_per_row, sf_cbg, hf);
            break;
        case CK_B200_DTYPE_F16:
            err = launch_dependent(kLaunchFamilyQuantize, dequantize_nvfp4_kernel<CK_B200_DTYPE_F16>, grid, block, 0, s, q, per_tensor_scale_dev, sf, out_dev, (int)rows, (int)words_per_row, sf_cbg, hf);
            break;
        default:
            err = launch_dependent(kLaunchFamilyQuantize, dequantize_nvfp4_kernel<CK_B200_DTYPE_BF16>, grid, block, 0, s, q, per_tensor_scale_dev, sf, out_dev, (int)rows, (int)words_per_row, sf_cbg, hf);
            break;
    }
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
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

namespace ckb {
int read_quant_status(int* out) {
    int v = 0;
    CKB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_quant_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        CKB_CUDA_OK(cudaMemcpyToSymbol(g_quant_status, &zero, sizeof(int)));
    }
    *out = v;
    return CK_B200_OK;
}
}  // namespace ckb

extern "C" int ck_b200_quantize_nvfp4_dynamic(const void* x_dev, int x_dtype, float* scale_out_dev, void* q_out_dev,
                                              void* sf_out_dev, int64_t rows, int64_t cols, int pad_16x, int hi_first,
                                              void* sync_dev, void* stream) {
    int sms = 0;
    if (int rc = check_device(&sms)) return rc;
    if (!x_dev || !scale_out_dev || !q_out_dev || !sf_out_dev)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4_dynamic: null pointer");
    if (rows < 0 || cols < 0 || rows > 0x3fffff00ll || cols > 0x3fffff00ll)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4_dynamic: rows and cols must be in [0, 2^30)");
    if (!pad_16x && (rows % 16 != 0 || cols % 16 != 0))
        return fail(CK_B200_ERR_INVALID_ARGUMENT,
                    "quantize_nvfp4_dynamic: rows and cols must be divisible by 16 without pad_16x, got %lld x %lld",
                    (long long)rows, (long long)cols);
    if (x_dtype < 0 || x_dtype > 2)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4_dynamic: dtype code %d", x_dtype);
    if (sync_dev && ((uintptr_t)sync_dev & 15))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "quantize_nvfp4_dynamic: the sync words must be 16-byte aligned");
    const int64_t prow = pad_16x ? round_up64(rows, 16) : rows, pcol = pad_16x ? round_up64(cols, 16) : cols;
    const int64_t sf_cbg = round_up64(pcol / 16, 4) / 4;
    const int64_t in_bytes = rows * cols * (x_dtype == CK_B200_DTYPE_F32 ? 4 : 2);
    const bool vec = (cols % 8 == 0) && (((uintptr_t)x_dev & 15) == 0);
    // one launch while x is about the size of the L2 or smaller (the first pass walks each warp's range backwards, so
    // the second pass starts on what L2 still holds) and the one-wave geometry applies;
    // otherwise the reduction kernel, the scale and the quantizer as separate launches: same bits either way
    const bool one_launch = sync_dev && vec && sf_cbg % 2 == 0 && prow > 0 && pcol > 0 && g_quant_variant.load() == 2 &&
                            in_bytes <= (int64_t)g_dynamic_fused_max_mb.load() * 1000000ll &&
                            !(((uintptr_t)q_out_dev & 3) || ((uintptr_t)sf_out_dev & 3));
    if (!one_launch) {
        if (int rc = ck_b200_dynamic_scale_nvfp4(x_dev, x_dtype, rows * cols, scale_out_dev, stream)) return rc;
        return ck_b200_quantize_nvfp4(x_dev, x_dtype, scale_out_dev, q_out_dev, sf_out_dev, rows, cols, pad_16x, hi_first,
                                      stream);
    }
    QuantArgs a;
    a.x = x_dev;
    a.pts = scale_out_dev;   // not read by the kernel: the scale is handed over inside it
    a.q = (uint8_t*)q_out_dev;
    a.sf = (uint8_t*)sf_out_dev;
    a.rows = (int)rows;
    a.cols = (int)cols;
    a.prow = (int)prow;
    a.pcol = (int)pcol;
    a.row_groups = (int)(round_up64(prow, 128) / 4);
    a.sf_cbg = (int)sf_cbg;
    a.seg_units = a.segments = 0;
    a.hi_first = hi_first ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    switch (x_dtype) {
        case CK_B200_DTYPE_F32: return launch_quantize_dynamic<CK_B200_DTYPE_F32>(a, scale_out_dev, sync_dev, sms, s);
        case CK_B200_DTYPE_F16: return launch_quantize_dynamic<CK_B200_DTYPE_F16>(a, scale_out_dev, sync_dev, sms, s);
        default: return launch_quantize_dynamic<CK_B200_DTYPE_BF16>(a, scale_out_dev, sync_dev, sms, s);
    }
}
