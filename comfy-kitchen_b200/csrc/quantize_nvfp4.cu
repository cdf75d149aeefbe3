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
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace ckb {
namespace {

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

// ---- packed pairs of fp32 (sm_100 f32x2 arithmetic: one instruction, two results) ---------------------------

typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pack2(float lo, float hi) {
    f32x2_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2_t pack2_bits(uint32_t lo, uint32_t hi) {
    f32x2_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2_t mul2_rn(f32x2_t a, f32x2_t b) {
    f32x2_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2_t fma2_rn(f32x2_t a, f32x2_t b, f32x2_t c) {
    f32x2_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2_t fma2_rm(f32x2_t a, f32x2_t b, f32x2_t c) {   // rounds toward minus infinity
    f32x2_t r;
    asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// max(|a|, |b|) per 16-bit half; the sign bits of the result are meaningless (xor of the inputs' signs)
__device__ __forceinline__ uint32_t maxabs_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Widened pairs of the eight elements of a unit, and the amax of the block that this lane derives.  The two lanes
// of a pair each hold eight elements of two units; lane "X" data is the unit whose block the lane derives, lane "Y"
// data the other unit, whose block the partner lane derives.  block_amax returns max(own X half, partner's Y half).
template <int DT>
struct Pairs;

template <>
struct Pairs<CK_B200_DTYPE_BF16> {
    using Raw = Input<CK_B200_DTYPE_BF16>::Raw;
    static __device__ __forceinline__ void widen(const Raw& r, f32x2_t (&f)[4]) {
        const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = pack2_bits(w[i] << 16, w[i] & 0xffff0000u);
    }
    static __device__ __forceinline__ float block_amax(const Raw& x, const Raw& y) {
        const uint32_t mx = maxabs_bf16x2(maxabs_bf16x2(x.v.x, x.v.y), maxabs_bf16x2(x.v.z, x.v.w));
        const uint32_t my = maxabs_bf16x2(maxabs_bf16x2(y.v.x, y.v.y), maxabs_bf16x2(y.v.z, y.v.w));
        // low half: this lane's X elements, high half: its Y elements
        const uint32_t mine = maxabs_bf16x2(__byte_perm(mx, my, 0x5410), __byte_perm(mx, my, 0x7632));
        const uint32_t theirs = __shfl_xor_sync(0xffffffffu, mine, 1);
        const uint32_t both = maxabs_bf16x2(mine, __byte_perm(theirs, theirs, 0x1032));   // low: X half, partner's Y half
        return __uint_as_float((both << 16) & 0x7fff0000u);
    }
};

template <>
struct Pairs<CK_B200_DTYPE_F16> {
    using Raw = Input<CK_B200_DTYPE_F16>::Raw;
    static __device__ __forceinline__ void widen(const Raw& r, f32x2_t (&f)[4]) {
        const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[i] = pack2(p.x, p.y);
        }
    }
    static __device__ __forceinline__ float half_amax(const Raw& r) {
        const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
        __half2 m = __habs2(*reinterpret_cast<const __half2*>(&w[0]));
#pragma unroll
        for (int i = 1; i < 4; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __half2*>(&w[i])));
        const float2 p = __half22float2(m);
        return fmaxf(p.x, p.y);
    }
    static __device__ __forceinline__ float block_amax(const Raw& x, const Raw& y) {
        return fmaxf(half_amax(x), __shfl_xor_sync(0xffffffffu, half_amax(y), 1));
    }
};

template <>
struct Pairs<CK_B200_DTYPE_F32> {
    using Raw = Input<CK_B200_DTYPE_F32>::Raw;
    static __device__ __forceinline__ void widen(const Raw& r, f32x2_t (&f)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = pack2_bits((&r.v[0].x)[2 * i], (&r.v[0].x)[2 * i + 1]);
    }
    static __device__ __forceinline__ float half_amax(const Raw& r) {
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(__uint_as_float((&r.v[0].x)[i])));
        return m;
    }
    static __device__ __forceinline__ float block_amax(const Raw& x, const Raw& y) {
        return fmaxf(half_amax(x), __shfl_xor_sync(0xffffffffu, half_amax(y), 1));
    }
};

// ---- exact arithmetic helpers ---------------------------------------------------------------------

// Correctly rounded a / b from rb = RN(1/b): two rounds of residual correction (Markstein).  The first round
// turns the two-ulp estimate a*rb into a faithful quotient, the second makes it the correctly rounded one.
// Valid while no intermediate leaves the normal range (the callers check the operand ranges).
__device__ __forceinline__ float div_by_reciprocal(float a, float b, float rb) {
    float q = __fmul_rn(a, rb);
    q = fmaf(fmaf(-b, q, a), rb, q);
    q = fmaf(fmaf(-b, q, a), rb, q);
    return q;
}

__device__ __forceinline__ float rcp_approx(float v) {   // one MUFU instruction, at most 1 ulp off for normal v
    float r;
    asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

// Block scale byte and decode scale t = ts * float(byte) for a block whose amax is given
// (eager/quantization.py:142-146): e4m3( min(amax / 6 / ts, 448) ).  `fast`: amax and ts are inside
// [2^-60, 2^60], where the reciprocal-based divisions below are exact; otherwise IEEE divisions.
__device__ __forceinline__ void block_scale(float amax, float ts, float rcp_ts, bool fast, uint32_t& s8, float& t) {
    float sbs;
    if (fast) {
        const float bs = div_by_reciprocal(amax, 6.0f, 0x1.555556p-3f);   // RN(1/6)
        sbs = div_by_reciprocal(bs, ts, rcp_ts);
    } else {
        sbs = __fdiv_rn(__fdiv_rn(amax, 6.0f), ts);
    }
    sbs = fminf(sbs, 448.0f);
    s8 = f32_to_e4m3_rne(sbs);
    t = __fmul_rn(ts, e4m3_to_f32((uint8_t)s8));
}

// block_scale for an ordinary block (finite, non-negative quotient) with the conversions written as the two
// instructions they are: no NaN handling, no branches.  Same results as block_scale(..., fast = true, ...) there.
__device__ __forceinline__ void block_scale_ordinary(float amax, float ts, float rcp_ts, uint32_t& s8, float& t) {
    const float bs = div_by_reciprocal(amax, 6.0f, 0x1.555556p-3f);   // RN(1/6)
    const float sbs = fminf(div_by_reciprocal(bs, ts, rcp_ts), 448.0f);
    uint16_t pk;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pk) : "f"(0.0f), "f"(sbs));   // second operand -> low byte
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(pk));
    s8 = pk & 0xffu;
    t = __fmul_rn(ts, __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu))));
}

// Eight elements -> packed e2m1 word (element 2i in the high nibble), exactly as RNE(e2m1)(RN(x / t)), by IEEE
// division.  Zero decode scale: every element encodes +0 (eager/quantization.py:149-153).
__device__ __forceinline__ uint32_t quantize8_exact(const float (&f)[8], float t) {
    if (t == 0.0f) return 0u;
    float d[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) d[i] = __fdiv_rn(f[i], t);
    return pack8_e2m1_hi_first(d);   // satfinite clamps to +-6 like the reference's clamp before rounding
}

// The same word for a decode scale in [2^-100, 2^100] without the IEEE division routine: r = RN(1/t), then each
// quotient by two rounds of residual correction.  The sign of x is forced onto the result so that -0 and negative
// values that round to zero keep their sign bit.
__device__ __forceinline__ uint32_t quantize8_reciprocal(const float (&f)[8], float t) {
    const float r = __frcp_rn(t);
    float d[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float q = div_by_reciprocal(f[i], t, r);
        d[i] = __uint_as_float((__float_as_uint(q) & 0x7fffffffu) | (__float_as_uint(f[i]) & 0x80000000u));
    }
    return pack8_e2m1_hi_first(d);
}

// The same word from a bracket instead of a division.  With r within 1 ulp of 1/t, x*(r - 8ulp) and x*(r + 8ulp)
// (round-to-nearest products) lie below and above x/t in magnitude with the sign of x, so RN(x/t) lies between
// them; conversion to e2m1 is monotone, hence equal codes for the two bounds are the code of RN(x/t).  The
// bounds are 17 ulp apart, so they disagree only for quotients within 2^-19 of a rounding boundary; the caller
// then falls back to quantize8_exact.  Needs t and r in the normal range: the caller passes r = 0 (which makes
// the two words differ or the flag below fire) unless t is in [2^-100, 2^100].
__device__ __forceinline__ bool quantize8_bracket(const float (&f)[8], float r, uint32_t& word) {
    const float r_lo = __uint_as_float(__float_as_uint(r) - 8u);
    const float r_hi = __uint_as_float(__float_as_uint(r) + 8u);
    float d[8], e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        d[i] = __fmul_rn(f[i], r_lo);
        e[i] = __fmul_rn(f[i], r_hi);
    }
    word = pack8_e2m1_hi_first(d);
    return (word == pack8_e2m1_hi_first(e)) && (r != 0.0f);
}

// The same word with one division-free correctly rounded quotient per element: r = RN(1/t), q0 = x*r (within two
// ulp), residual x - t*q0 by a fused multiply-add, q = q0 + residual*r (one round of Markstein's correction, which
// yields RN(x/t) from a correctly rounded reciprocal).  The residual is rounded toward minus infinity: where it is
// exact that changes nothing except that an exact zero comes out as -0, which lets the last step keep the sign of
// a -0 input (-0 + -0 = -0, -0 + +0 = +0) without a separate sign fix-up.  Needs t in [2^-100, 2^100].
__device__ __forceinline__ uint32_t quantize8_markstein(const float (&f)[8], float t, float r) {
    float d[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float q0 = __fmul_rn(f[i], r);
        d[i] = __fmaf_rn(__fmaf_rd(-t, q0, f[i]), r, q0);
    }
    return pack8_e2m1_hi_first(d);
}

// RN(1/t) for normal t without the range checks of the library routine: one MUFU reciprocal (within 1 ulp) and one
// Newton step in fused arithmetic.  Equal to __frcp_rn for every fp32 in [2^-69, 2^69] (checked exhaustively on a B200).
__device__ __forceinline__ float rcp_rn_normal(float t) {
    float r0;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(t));
    return fmaf(r0, fmaf(-t, r0, 1.0f), r0);
}

// quantize8_markstein on four packed pairs: three packed instructions per two elements.
__device__ __forceinline__ uint32_t quantize8_markstein_packed(const f32x2_t (&f)[4], float t, float r) {
    const f32x2_t tt = pack2(-t, -t), rr = pack2(r, r);
    float d[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const f32x2_t q0 = mul2_rn(f[i], rr);
        unpack2(fma2_rn(fma2_rm(tt, q0, f[i]), rr, q0), d[2 * i], d[2 * i + 1]);
    }
    return pack8_e2m1_hi_first(d);
}

// ---- quantize -------------------------------------------------------------------------------------

struct QuantArgs {
    const void* x;
    const float* pts;
    uint8_t* q;
    uint8_t* sf;
    int rows, cols;          // logical input
    int prow, pcol;          // padded (output) shape
    int row_groups;          // roundup(prow,128)/4 : number of (band, d3) groups
    int sf_cbg;              // scale tensor width / 4 = units per row
    int seg_units;           // units per warp (even); a row is cut into `segments` such pieces
    int segments;
    int hi_first;
};

// Ring depth and resident blocks per SM (which sets the register budget).  Measured on a B200: 6 units x 3 blocks
// (78 registers, no spills) is as fast as or faster than 6 x 4 (64 registers with spills in the loop), 4 x 4, 8 x 3 and
// 10 x 2 at every size from 28 MB to 1.6 GB; all of them end at 5.6-5.75 TB/s on the largest inputs.
#ifndef CKB_QUANT_RING
#define CKB_QUANT_RING 6
#endif
#ifndef CKB_QUANT_BLOCKS_PER_SM
#define CKB_QUANT_BLOCKS_PER_SM 3
#endif
constexpr int kBlocksPerSM = CKB_QUANT_BLOCKS_PER_SM;   // resident blocks the register budget is set for
constexpr int kRing = CKB_QUANT_RING;   // units a thread keeps in flight (16-byte loads), processed two at a time

// State of one lane for one segment walk.
struct LaneCtx {
    const char* x_row;   // first element of this lane's row
    uint8_t* q_row;      // first packed byte of this lane's output row
    uint8_t* sf_row;     // this lane's row inside scale chunk 0 of the band (chunks are 512 bytes apart)
    float ts, rcp_ts;
    bool ts_in_range, row_in, row_out, odd, hi_first;
    int sub, cols, pcol;
};

// One pair of units (A, B) held by a warp: the two lanes that share a 16-element block split the per-block work.
// The even lane derives scale byte, decode scale and reciprocal for the block of unit A, the odd lane for the
// block of unit B, and they swap the results with shuffles.  `mine_in`: the block this lane derives lies inside
// the padded output.  Returns the two packed words and leaves this lane's scale byte in s8.
// Rare cases (operands outside the exact-reciprocal range, quotients next to a rounding boundary) are found with a
// warp vote, so the common path has no divergent branch.
template <int DT, int VARIANT>
__device__ __forceinline__ void quantize_pair(const LaneCtx& c, const typename Input<DT>::Raw& raw_a,
                                              const typename Input<DT>::Raw& raw_b, bool mine_in, uint32_t& word_a,
                                              uint32_t& word_b, uint32_t& s8) {
    using In = Input<DT>;
    const bool odd = c.odd;
    float fa[8], fb[8];
    const float half_a = In::unpack(raw_a, fa);
    const float half_b = In::unpack(raw_b, fb);
    // amax of the block this lane is responsible for: its own half and the partner's half
    const float other_half = __shfl_xor_sync(0xffffffffu, odd ? half_a : half_b, 1);
    const float amax = fmaxf(odd ? half_b : half_a, other_half);
    s8 = 0;
    float t = 0.0f, rcp = 0.0f;
    if (VARIANT != 0) {
        const bool fast = c.ts_in_range && amax >= 0x1p-60f && amax <= 0x1p60f;
        if (__all_sync(0xffffffffu, fast && mine_in)) {
            block_scale(amax, c.ts, c.rcp_ts, true, s8, t);
            rcp = VARIANT == 2 ? __frcp_rn(t) : rcp_approx(t);
            // t is zero (block scale rounded to zero) or, never with these ranges, outside [2^-100, 2^100]: flag it
            if (!(t >= 0x1p-100f && t <= 0x1p100f)) rcp = 0.0f;
        } else if (mine_in) {
            block_scale(amax, c.ts, c.rcp_ts, fast, s8, t);
            // the residual form also needs finite elements (inf - inf otherwise): only blocks with amax in range
            if (VARIANT == 2) { if (fast && t >= 0x1p-100f && t <= 0x1p100f) rcp = __frcp_rn(t); }
            else if (t >= 0x1p-100f && t <= 0x1p100f) rcp = rcp_approx(t);
        }
    } else if (mine_in) {
        block_scale(amax, c.ts, 0.0f, false, s8, t);
    }
    const float t_other = __shfl_xor_sync(0xffffffffu, t, 1);
    const float t_a = odd ? t_other : t, t_b = odd ? t : t_other;
    if (VARIANT == 2) {
        const float rcp_other = __shfl_xor_sync(0xffffffffu, rcp, 1);
        const float rcp_a = odd ? rcp_other : rcp, rcp_b = odd ? rcp : rcp_other;
        if (__all_sync(0xffffffffu, rcp_a != 0.0f && rcp_b != 0.0f)) {
            word_a = quantize8_markstein(fa, t_a, rcp_a);
            word_b = quantize8_markstein(fb, t_b, rcp_b);
        } else {   // a decode scale that is zero or out of range
            word_a = (rcp_a != 0.0f) ? quantize8_markstein(fa, t_a, rcp_a) : quantize8_exact(fa, t_a);
            word_b = (rcp_b != 0.0f) ? quantize8_markstein(fb, t_b, rcp_b) : quantize8_exact(fb, t_b);
        }
    } else if (VARIANT == 1) {
        const float rcp_other = __shfl_xor_sync(0xffffffffu, rcp, 1);
        const float rcp_a = odd ? rcp_other : rcp, rcp_b = odd ? rcp : rcp_other;
        const bool ok_a = quantize8_bracket(fa, rcp_a, word_a);
        const bool ok_b = quantize8_bracket(fb, rcp_b, word_b);
        if (__any_sync(0xffffffffu, !(ok_a && ok_b))) {
            // next to a rounding boundary (exact ties are common when the per-tensor scale is amax/2688), or a
            // decode scale that is zero or out of range (flagged by a zero reciprocal)
            if (!ok_a) word_a = (rcp_a != 0.0f) ? quantize8_reciprocal(fa, t_a) : quantize8_exact(fa, t_a);
            if (!ok_b) word_b = (rcp_b != 0.0f) ? quantize8_reciprocal(fb, t_b) : quantize8_exact(fb, t_b);
        }
    } else {
        word_a = quantize8_exact(fa, t_a);
        word_b = quantize8_exact(fb, t_b);
    }
    if (!c.hi_first) {
        word_a = swap_nibbles32(word_a);
        word_b = swap_nibbles32(word_b);
    }
}

// The four block scales of a row and unit sit on lanes of equal parity (even: unit A, odd: unit B): gather them
// into one 32-bit word on lane sub = 0 (A) and sub = 1 (B).
__device__ __forceinline__ uint32_t gather_scale_word(uint32_t s8, int sub) {
    uint32_t sfw = s8 << (8 * (sub >> 1));
    sfw |= __shfl_xor_sync(0xffffffffu, sfw, 2);
    sfw |= __shfl_xor_sync(0xffffffffu, sfw, 4);
    return sfw;
}

// Interior segment: every row of the warp and every column of units [u_begin, u_end) is inside the input and the
// output and the segment holds whole pairs.  The main loop has no bounds checks: all addresses are the three
// running pointers plus immediates, and each consumed pair of registers is refilled with the units kRing ahead.
template <int DT, int VARIANT>
__device__ __forceinline__ void walk_interior(const LaneCtx& c, int u_begin, int u_end) {
    using In = Input<DT>;
    using Raw = typename In::Raw;
    constexpr int kUnitBytes = 64 * In::kBytes;   // input bytes of one unit in one row
    const int sub = c.sub;
    const char* xp = c.x_row + (u_begin * 64 + sub * 8) * In::kBytes;
    uint8_t* qp = c.q_row + u_begin * 32 + sub * 4;
    uint8_t* sp = c.sf_row + (u_begin + (sub & 1)) * 512;   // lane sub = 1 stores unit B's scales
    const bool sf_lane = sub < 2;
    int remaining = u_end - u_begin;

    Raw raw[kRing];
#pragma unroll
    for (int k = 0; k < kRing; ++k)
        if (k < remaining) raw[k] = In::load_vec(xp + k * kUnitBytes);
        else raw[k] = In::zero();

    auto consume = [&](int k) {
        uint32_t wa, wb, s8;
        quantize_pair<DT, VARIANT>(c, raw[k], raw[k + 1], true, wa, wb, s8);
        *reinterpret_cast<uint32_t*>(qp + k * 32) = wa;
        *reinterpret_cast<uint32_t*>(qp + k * 32 + 32) = wb;
        const uint32_t sfw = gather_scale_word(s8, sub);
        if (sf_lane) *reinterpret_cast<uint32_t*>(sp + k * 512) = sfw;
    };

    for (; remaining >= 2 * kRing; remaining -= kRing) {
#pragma unroll
        for (int k = 0; k < kRing; k += 2) {
            consume(k);
            raw[k] = In::load_vec(xp + (kRing + k) * kUnitBytes);
            raw[k + 1] = In::load_vec(xp + (kRing + k + 1) * kUnitBytes);
        }
        xp += kRing * kUnitBytes;
        qp += kRing * 32;
        sp += kRing * 512;
    }
    // at most two more rounds: the first may still refill part of the ring
#pragma unroll 1
    for (; remaining > 0; remaining -= kRing) {
#pragma unroll
        for (int k = 0; k < kRing; k += 2) {
            if (k < remaining) consume(k);                    // uniform
            if (kRing + k < remaining) {                      // uniform; pairs are whole
                raw[k] = In::load_vec(xp + (kRing + k) * kUnitBytes);
                raw[k + 1] = In::load_vec(xp + (kRing + k + 1) * kUnitBytes);
            }
        }
        xp += kRing * kUnitBytes;
        qp += kRing * 32;
        sp += kRing * 512;
    }
}

// The pair of units of quantize_pair with lane-relative roles and no rare-path work in the common case: `raw_x` is the
// unit whose block this lane derives (unit A on even lanes, unit B on odd lanes), `raw_y` the other one, so nothing
// is selected by lane parity - the caller's addresses differ instead.  Everything is computed as if the block were
// ordinary (finite, per-tensor scale and amax inside the exact-reciprocal range, or an all-zero block); one vote
// at the end sends the whole warp to IEEE arithmetic otherwise.  Returns this lane's scale byte in s8.
template <int DT, bool HI_FIRST>
__device__ __forceinline__ void quantize_pair_xy(const LaneCtx& c, const typename Input<DT>::Raw& raw_x,
                                                 const typename Input<DT>::Raw& raw_y, uint32_t& word_x,
                                                 uint32_t& word_y, uint32_t& s8) {
    using In = Input<DT>;
    const float amax = Pairs<DT>::block_amax(raw_x, raw_y);
    const bool ordinary = c.ts_in_range && (amax == 0.0f || (amax >= 0x1p-60f && amax <= 0x1p60f));
    float t;
    block_scale_ordinary(amax, c.ts, c.rcp_ts, s8, t);   // t is 0 or inside [2^-69, 2^69] for an ordinary block
    const float r = rcp_rn_normal(t);
    const float t_y = __shfl_xor_sync(0xffffffffu, t, 1);
    const float r_y = __shfl_xor_sync(0xffffffffu, r, 1);
    f32x2_t fx[4], fy[4];
    Pairs<DT>::widen(raw_x, fx);
    Pairs<DT>::widen(raw_y, fy);
    word_x = quantize8_markstein_packed(fx, t, r);
    word_y = quantize8_markstein_packed(fy, t_y, r_y);
    // zero decode scale: every element encodes +0 (the arithmetic above produced infinities or NaNs there)
    word_x = (t == 0.0f) ? 0u : word_x;
    word_y = (t_y == 0.0f) ? 0u : word_y;
    if (!__all_sync(0xffffffffu, ordinary)) {
        float gx[8], gy[8], t2;
        In::unpack(raw_x, gx);
        In::unpack(raw_y, gy);
        block_scale(amax, c.ts, 0.0f, false, s8, t2);
        const float t2_y = __shfl_xor_sync(0xffffffffu, t2, 1);
        word_x = quantize8_exact(gx, t2);
        word_y = quantize8_exact(gy, t2_y);
    }
    if (!HI_FIRST) {
        word_x = swap_nibbles32(word_x);
        word_y = swap_nibbles32(word_y);
    }
}

// walk_interior for quantize_pair_xy: even lanes keep unit A of a pair in raw[k] and unit B in raw[k + 1], odd lanes
// the other way round, by a per-lane offset on the load and store addresses.
// ROWS_IN = false: some of the warp's rows lie in the zero padding below the input (they are still rows of the
// output); their lanes skip the loads and quantize zeros.
template <int DT, bool ROWS_IN, bool HI_FIRST>
__device__ __forceinline__ void walk_interior_xy(const LaneCtx& c, int u_begin, int u_end) {
    using In = Input<DT>;
    using Raw = typename In::Raw;
    constexpr int kUnitBytes = 64 * In::kBytes;
    const int sub = c.sub;
    const int x_unit = c.odd ? 1 : 0, y_unit = 1 - x_unit;
    const char* xp = c.x_row + (u_begin * 64 + sub * 8) * In::kBytes;
    const char* xp_x = xp + x_unit * kUnitBytes;
    const char* xp_y = xp + y_unit * kUnitBytes;
    uint8_t* qp_x = c.q_row + (u_begin + x_unit) * 32 + sub * 4;
    uint8_t* qp_y = c.q_row + (u_begin + y_unit) * 32 + sub * 4;
    uint8_t* sp = c.sf_row + (u_begin + (sub & 1)) * 512;   // lane sub = 1 stores unit B's scales
    const bool sf_lane = sub < 2;
    int remaining = u_end - u_begin;   // even
    auto load = [&](const char* p) -> Raw { return (ROWS_IN || c.row_in) ? In::load_vec(p) : In::zero(); };

    Raw raw[kRing];
#pragma unroll
    for (int k = 0; k < kRing; k += 2) {
        if (k < remaining) {
            raw[k] = load(xp_x + k * kUnitBytes);
            raw[k + 1] = load(xp_y + k * kUnitBytes);
        } else {
            raw[k] = In::zero();
            raw[k + 1] = In::zero();
        }
    }

    auto consume = [&](int k) {
        uint32_t wx, wy, s8;
        quantize_pair_xy<DT, HI_FIRST>(c, raw[k], raw[k + 1], wx, wy, s8);
        *reinterpret_cast<uint32_t*>(qp_x + k * 32) = wx;
        *reinterpret_cast<uint32_t*>(qp_y + k * 32) = wy;
        const uint32_t sfw = gather_scale_word(s8, sub);
        if (sf_lane) *reinterpret_cast<uint32_t*>(sp + k * 512) = sfw;
    };
    auto advance = [&] {
        xp_x += kRing * kUnitBytes;
        xp_y += kRing * kUnitBytes;
        qp_x += kRing * 32;
        qp_y += kRing * 32;
        sp += kRing * 512;
    };

    for (; remaining >= 2 * kRing; remaining -= kRing) {
#pragma unroll
        for (int k = 0; k < kRing; k += 2) {
            consume(k);
            raw[k] = load(xp_x + (kRing + k) * kUnitBytes);
            raw[k + 1] = load(xp_y + (kRing + k) * kUnitBytes);
        }
        advance();
    }
#pragma unroll 1
    for (; remaining > 0; remaining -= kRing) {
#pragma unroll
        for (int k = 0; k < kRing; k += 2) {
            if (k < remaining) consume(k);                    // uniform
            if (kRing + k < remaining) {                      // uniform; pairs are whole
                raw[k] = load(xp_x + (kRing + k) * kUnitBytes);
                raw[k + 1] = load(xp_y + (kRing + k) * kUnitBytes);
            }
        }
        advance();
    }
}

// Edge segment: rows past the input, ragged columns, padding to 16x16 and to whole scale chunks.
template <int DT, bool VEC, int VARIANT>
__device__ __forceinline__ void walk_edge(const LaneCtx& c, int u_begin, int u_end) {
    using In = Input<DT>;
    using Raw = typename In::Raw;
    const int sub = c.sub;
    const bool odd = c.odd;

    auto load_unit = [&](int cbg) -> Raw {
        Raw v = In::zero();
        const int c0 = cbg * 64 + sub * 8;
        if (c.row_in && cbg < u_end && c0 < c.cols) {
            if (VEC) {   // cols % 8 == 0 and 16-byte aligned base: the whole vector is inside the row
                v = In::load_vec(c.x_row + c0 * In::kBytes);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (c0 + i < c.cols) In::set(v, i, c.x_row, c0 + i);
            }
        }
        return v;
    };

    Raw raw[kRing];
#pragma unroll
    for (int k = 0; k < kRing; ++k) raw[k] = load_unit(u_begin + k);

#pragma unroll 1
    for (int base = u_begin; base < u_end; base += kRing) {
#pragma unroll
        for (int k = 0; k < kRing; k += 2) {
            const int cbg_a = base + k;
            const int cbg_b = cbg_a + 1;   // may be the segment's end: then unit B belongs to no one here
            if (cbg_a < u_end) {           // uniform across the warp
                const bool b_valid = cbg_b < u_end;
                const int cbg_mine = odd ? cbg_b : cbg_a;
                const bool mine_in = c.row_out && cbg_mine < u_end && cbg_mine * 64 + sub * 8 < c.pcol;
                uint32_t word_a, word_b, s8;
                quantize_pair<DT, VARIANT>(c, raw[k], raw[k + 1], mine_in, word_a, word_b, s8);
                const int byte_col = cbg_a * 32 + sub * 4;
                if (c.row_out && byte_col * 2 < c.pcol) *reinterpret_cast<uint32_t*>(c.q_row + byte_col) = word_a;
                if (c.row_out && b_valid && (byte_col + 32) * 2 < c.pcol)
                    *reinterpret_cast<uint32_t*>(c.q_row + byte_col + 32) = word_b;
                const uint32_t sfw = gather_scale_word(s8, sub);
                // lanes 0 and 1 of each group of eight store: lane 1 adds 512 bytes (unit B's chunk)
                if (sub < 2 && (sub == 0 || b_valid))
                    *reinterpret_cast<uint32_t*>(c.sf_row + (cbg_a + sub) * 512) = sfw;
            }
            raw[k] = load_unit(base + kRing + k);
            raw[k + 1] = load_unit(base + kRing + k + 1);
        }
    }
}

// One warp walks a segment of one row group: it keeps kRing units in flight in registers and, each time it has
// consumed a pair of units, issues the loads that refill those registers, so loads and arithmetic overlap inside
// the warp and the bytes in flight per SM stay high for the whole life of the block.
// Launch geometry: block (32, WX, WY) with WX * WY = kWarpsPerBlock; warp (wx, wy) of block (bx, by, bz) handles
// segment bx*WX + wx of row group (bz*65535 + by)*WY + wy, so no thread divides anything.
template <int DT, bool VEC, int VARIANT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, kBlocksPerSM) quantize_nvfp4_kernel(const QuantArgs a) {
    using In = Input<DT>;
    allow_dependent_launch();
    const int lane = threadIdx.x;
    const int seg = blockIdx.x * blockDim.y + threadIdx.y;
    // row groups are handed out last band first: the bottom band is the one that may hold padding rows, whose
    // warps take the slower edge walk and should not be the ones the kernel ends on
    const int group = a.row_groups - 1 - (int)((blockIdx.z * 65535 + blockIdx.y) * blockDim.z + threadIdx.z);
    if (seg >= a.segments || group < 0) return;   // whole warps
    const int u_begin = seg * a.seg_units;
    const int u_end = min(a.sf_cbg, u_begin + a.seg_units);
    const int d4 = lane >> 3;
    const int band = group >> 5;
    const int d3 = group & 31;
    const int r = band * 128 + d3 + 32 * d4;
    LaneCtx c;
    c.sub = lane & 7;
    c.odd = c.sub & 1;
    grid_dependency_wait();
    c.ts = __ldg(a.pts);
    c.ts_in_range = c.ts >= 0x1p-60f && c.ts <= 0x1p60f;
    c.rcp_ts = (VARIANT != 0 && c.ts_in_range) ? __frcp_rn(c.ts) : 0.0f;
    c.row_in = r < a.rows;
    c.row_out = r < a.prow;
    c.hi_first = a.hi_first != 0;
    c.cols = a.cols;
    c.pcol = a.pcol;
    c.x_row = (const char*)a.x + (int64_t)r * a.cols * In::kBytes;
    c.q_row = a.q + (int64_t)r * (a.pcol >> 1);
    c.sf_row = a.sf + (((int64_t)band * a.sf_cbg) * 32 + d3) * 16 + d4 * 4;
    // rows of the warp are r0 + {0,32,64,96}: all inside the input iff the last one is; segments hold whole pairs
    const bool whole_pairs = VEC && (u_end * 64 <= a.cols) && ((u_end - u_begin) % 2 == 0);
    const bool interior = whole_pairs && (band * 128 + d3 + 96 < a.rows);
    if (interior && VARIANT == 2) {
        if (c.hi_first) walk_interior_xy<DT, true, true>(c, u_begin, u_end);
        else walk_interior_xy<DT, true, false>(c, u_begin, u_end);
    } else if (VARIANT == 2 && whole_pairs && (band * 128 + d3 + 96 < a.prow)) {
        if (c.hi_first) walk_interior_xy<DT, false, true>(c, u_begin, u_end);
        else walk_interior_xy<DT, false, false>(c, u_begin, u_end);
    }
    else if (interior) walk_interior<DT, VARIANT>(c, u_begin, u_end);
    else walk_edge<DT, VEC, VARIANT>(c, u_begin, u_end);
}

template <int DT>
int launch_quantize(QuantArgs a, bool vec, int variant, int sms, cudaStream_t stream) {
    if (a.row_groups <= 0 || a.sf_cbg <= 0) return CK_B200_OK;
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
