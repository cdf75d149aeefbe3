// scaled_mm_nvfp4 for sm_100a: block-scaled FP4 GEMM on the 5th-generation tensor cores.
//
//   out[M,N] = out_dtype( alpha * sum_k e2m1(a[m,k]) e4m3(sfa[m,k/16]) e2m1(b[n,k]) e4m3(sfb[n,k/16]) + bias[n] )
//
// Two kernels share this structure.  gemm_nvfp4_pair_kernel (default for M, N > 128): clusters of two CTAs compute
// 256 x 256 tiles with cta_group::2 instructions, each CTA loading its 128 rows of A and its half of B.
// gemm_nvfp4_kernel<BN> (everything else, and split-K for M <= 128): one CTA per 128 x BN tile.  Both take a format
// parameter: NVFP4 (above) or MXFP8 (e4m3 bytes, e8m0 scale per 32 elements, kind::mxf8f6f4).  No TMA multicast anywhere.
//
// Structure of gemm_nvfp4_kernel (one persistent CTA per SM, 6 warps):
//   warp 0   producer: TMA tile loads of packed A/B (128-byte swizzle) and plain bulk copies of the
//            scale-factor chunks into a ring of shared-memory stages (mbarrier complete_tx).
//   warp 1   MMA issuer: copies the stage's scale factors shared -> tensor memory (tcgen05.cp), issues
//            tcgen05.mma.kind::mxf4nvf4.block_scale (128 x BN x 64 per instruction, fp32 accumulators in
//            tensor memory) and commits stage-release / accumulator-ready barriers.
//   warps 2-5 epilogue: tcgen05.ld of the accumulator quadrant the warp may access, alpha and bias,
//            conversion, then either a swizzled shared-memory staging tile written out with a TMA store
//            (16-bit outputs: full 64-byte row segments) or direct 16-byte stores (fp32 output).
// Warps 0 and 1 run their loops with all lanes (uniform control flow keeps descriptor and address arithmetic
// on the uniform datapath) and predicate only the issuing instructions on one elected lane.
//
// Tensor memory (512 columns) holds two accumulators so the epilogue of tile i overlaps the main loop of
// tile i+1.  With BN = 128 they are disjoint.  With BN = 256 two full accumulators plus the scale factors
// do not fit, so the accumulators overlap in 64 columns ([0,256) and [192,448)): the epilogue drains the
// shared columns first and releases them through their own barrier, after which the next tile's MMAs may start.
//
// The scale tensors are in the 128x4 tiled layout of cuBLAS (comfy_kitchen/float_utils.py:292-326): the
// scales of 128 rows x 64 K-elements are one contiguous 512-byte chunk shaped 32 x 16 bytes, which is
// exactly the source shape of tcgen05.cp.32x128b.warpx4, so no repacking happens anywhere.
//
// Every wait on an mbarrier is bounded: when it runs out the kernel records a code in a device status
// word, all roles leave their loops, tensor memory is released and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "common.cuh"
#include "quantize_nvfp4_device.cuh"

namespace ckb {
namespace {

__device__ int g_device_status = 0;
// What the counting build of the CTA-pair kernel last measured: {cycles, nanoseconds} of CTA 0's epilogue role (its
// ratio is the SM clock inside the kernel), cycles the MMA role waited for loaded stages and for an accumulator, and
// the MMA role's total.
__device__ long long g_gemm_counters[5] = {0, 0, 0, 0, 0};

constexpr int BM = 128;             // rows of A per tile = tensor-memory lanes
constexpr int BK_BYTES = 128;       // packed bytes of K per stage = 256 elements = one swizzle row
constexpr int CHUNKS = 4;           // 64-element MMA steps per stage
constexpr int SF_CHUNK_BYTES = 512; // scales of 128 rows x 64 elements
constexpr int NUM_THREADS = 192;
constexpr int EPI_COLS = 32;        // accumulator columns per epilogue step
constexpr int STAGING_BYTES_PER_WARP = 32 * EPI_COLS * 2;   // 32 rows x 32 sixteen-bit outputs
constexpr long long WAIT_LIMIT_CYCLES = 3000000000ll;   // about 1.5 s

enum WaitCode { WAIT_STAGE_EMPTY = 1, WAIT_STAGE_FULL = 2, WAIT_ACC_EMPTY = 3, WAIT_ACC_FULL = 4, WAIT_OVERLAP = 5,
                WAIT_PEER_BARRIER = 6, WAIT_QUANT_BAND = 7 /* 8: the dynamic quantizer's meeting point */ };

struct GemmArgs {
    const uint8_t* sfa;
    const uint8_t* sfb;
    const float* tsa;
    const float* tsb;
    const float* alpha;   // may be null
    const void* bias;     // may be null
    void* out;
    int bias_dtype, out_dtype;
    int M, N;
    int sf_cbg;           // 512-byte chunks per 128-row band = ceil(K / 64)
    int sfb_bands;        // 128-row bands in the B scale tensor
    int k_iters;          // ceil(K / 256)
    int m_tiles, n_tiles;
    int raster_group;     // tiles are walked in groups of this many tile rows (all N tiles of a group before the next)
    int splits;           // split-K: every tile is computed by `splits` work items over k_per_split stages each,
    int k_per_split;      //          which leave fp32 partial sums in `partial` for splitk_reduce_kernel
    float* partial;       // [splits, M, N] fp32 scratch (split-K only)
    int a_box_bytes;      // bytes one TMA load of A delivers per stage in the 1-CTA kernel: the box covers only
                          // 32 or 64 rows when M is that small (the rows above stay unwritten and feed accumulator
                          // rows that are never stored)
    int tma_store;        // non-zero: 16-bit output written through shared memory and TMA stores
    int debug;            // non-zero: CTA 0 prints the cycles its roles spent waiting
    int early_weights;    // one-CTA kernel: non-zero = B and its scales of the first ring of stages are requested before
                          // the wait for the preceding kernel of the stream (the caller's promise: nothing in flight
                          // writes them)
    // fused all-gather (CTA-pair kernel, 16-bit output): `out` is this rank's column block inside its own
    // [M, ld_out] matrix and every staged tile is also stored to the same block of the other ranks' matrices
    int64_t ld_out;       // row stride of the output matrix in elements (N for a plain GEMM)
    int n_peers;
    uint8_t* peer_out[7]; // origin of the column block in each peer's matrix, as mapped into this process
};

// AROWS < 128 (with BN = 64: the configuration for one short tile row, M <= 64): A's share of a stage shrinks to the rows
// that exist, tiles are 64 columns wide and two CTAs fit on an SM, so that N / 64 (times the K splits) CTAs of short
// rings have the weight's bytes in flight on every SM at once.  The MMA still reads 128 rows of A; the rows past AROWS
// are whatever follows in shared memory and feed accumulator rows that are never stored.
template <int BN, int AROWS = BM>
struct Cfg {
    static constexpr bool kSkinny = BN < 128;
    static constexpr int kCtasPerSm = kSkinny ? 2 : 1;
    static constexpr int kBands = kSkinny ? 1 : BN / 128;         // 128-row bands of B scales per tile
    static constexpr int kABytes = AROWS * BK_BYTES;              // 16 KiB for full tiles
    static constexpr int kBBytes = BN * BK_BYTES;
    static constexpr int kSfaBytes = CHUNKS * SF_CHUNK_BYTES;     // 2 KiB
    static constexpr int kSfbBytes = kBands * CHUNKS * SF_CHUNK_BYTES;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kStagingBytes = 4 * STAGING_BYTES_PER_WARP;   // 8 KiB, one tile per epilogue warp
    static constexpr int kBarrierBytes = 256;
    // two CTAs per SM: (228 KiB - 1 KiB reserved per CTA) / 2
    static constexpr int kSmemBudget = kSkinny ? 115712 : 232448;
    // as many stages as fit: 6 (128 x 128) or 4 (128 x 256) with full A tiles; 6 / 5 for 64-column tiles with 32 / 64 A rows
    static constexpr int kStages = (kSmemBudget - kStagingBytes - 1024 - kBarrierBytes) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*alignment slack*/ + kBarrierBytes;
    static_assert(!kSkinny || (kStageBytes >= BM * BK_BYTES && kABytes % 1024 == 0),
                  "the MMA's 128 A rows stay inside the stage; B stays 1024-byte aligned");
    static_assert(kStages >= 3 && 2 * kStages + 5 <= 30, "ring depth and barrier room");
    // tensor-memory columns: two accumulators (overlapping by kOverlapCols when BN = 256), then two alternating
    // scale-factor regions, each holding the scales of two 64-element steps
    static constexpr int kOverlapCols = (BN == 256) ? 64 : 0;
    static constexpr int kAcc1Col = BN - kOverlapCols;
    static constexpr int kSfCol0 = kAcc1Col + BN;
    static constexpr int kSfaColsHalf = 2 * 4;
    static constexpr int kSfbColsHalf = 2 * 4 * kBands;
    static constexpr int kSfRegionCols = kSfaColsHalf + kSfbColsHalf;
    static constexpr int kTmemCols = kSkinny ? 256 : 512;         // per CTA; kCtasPerSm of them share the SM's 512
    static_assert(kSfCol0 + 2 * kSfRegionCols <= kTmemCols, "tensor memory budget");
    static_assert(kSmemBytes <= kSmemBudget, "shared memory budget");
    // instruction descriptor of tcgen05.mma.kind::mxf4nvf4.block_scale: A,B = packed e2m1 (format 1), K-major,
    // UE4M3 scales, N >> 3 at bit 17, M >> 4 at bit 24
    static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (0u << 23) |
                                       ((uint32_t)(BM >> 4) << 24);
    // kind::mxf8f6f4.block_scale: A,B = e4m3 (format 0), UE8M0 scales (bit 23); the byte of the four-byte scale cell
    // that an instruction uses is chosen per instruction: b_sf_id at bit 4, a_sf_id at bit 29
    static constexpr uint32_t kIdescMx = ((uint32_t)(BN >> 3) << 17) | (1u << 23) | ((uint32_t)(BM >> 4) << 24);
};

// ---- PTX wrappers -----------------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the wait was given up (here or, as seen through *abort_flag, elsewhere).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(&g_device_status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// Brings a tensor map (a kernel parameter) into the cache the TMA unit reads it from, ahead of its first use.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x),
                 "r"(y), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest N store groups have finished reading their shared-memory source
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Untiled bulk copy shared memory -> global memory (own or peer-mapped): 16-byte aligned addresses, size a multiple of 16.
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make generic-proxy shared-memory writes visible to the async proxy (TMA store reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_tmem,
                                       uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_mma_mx(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// One lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
    return pred != 0;
}

// Shared-memory matrix descriptor (sm_100 version 1), split in two 32-bit halves so that the issuing warp only
// adds to the low half.  Addresses and offsets are in 16-byte units.
//   low  = (address >> 4) | (leading byte offset >> 4) << 16
//   high = (stride byte offset >> 4) | version 1 << 14 | layout << 29
//   operands: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
//   scale chunks: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
constexpr uint32_t LAYOUT_SWIZZLE_NONE = 0, LAYOUT_SWIZZLE_128B = 2, LAYOUT_SWIZZLE_64B = 4;
constexpr uint32_t desc_hi(uint32_t sbo_bytes, uint32_t layout) { return (sbo_bytes >> 4) | (1u << 14) | (layout << 29); }
constexpr uint32_t kOperandDescHi = desc_hi(1024, LAYOUT_SWIZZLE_128B);
constexpr uint32_t kOperandDescLoFlags = (16u >> 4) << 16;
constexpr uint32_t kSfDescHi = desc_hi(128, LAYOUT_SWIZZLE_NONE);
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// ---- epilogue helpers -----------------------------------------------------------------------------

__device__ __forceinline__ float bias_at(const void* bias, int dtype, int n) {
    if (dtype == CK_B200_DTYPE_BF16) return __bfloat162float(((const __nv_bfloat16*)bias)[n]);
    if (dtype == CK_B200_DTYPE_F16) return __half2float(((const __half*)bias)[n]);
    return ((const float*)bias)[n];
}

// alpha * acc (+ bias) for 32 consecutive columns starting at n0
__device__ __forceinline__ void scale_row32(const GemmArgs& g, int n0, const uint32_t (&acc)[32], float alpha,
                                            float (&y)[32]) {
#pragma unroll
    for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(acc[i]) * alpha;
    if (g.bias) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (n0 + i < g.N) y[i] += bias_at(g.bias, g.bias_dtype, n0 + i);
    }
}

__device__ __forceinline__ uint32_t pack16(float a, float b, int out_dtype) {
    if (out_dtype == CK_B200_DTYPE_BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Direct global stores of 32 consecutive outputs of one row (n0 % 32 == 0; N % 8 == 0 so groups of 8 columns are
// either fully inside or fully outside).
__device__ __forceinline__ void st_global_v4(void* p, const uint4& v) {
    asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void store_row32(const GemmArgs& g, int64_t row, int n0, const float (&y)[32]) {
    if (g.out_dtype == CK_B200_DTYPE_F32) {
        float* p = (float*)g.out + row * g.N + n0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (n0 + 4 * j < g.N)
                *reinterpret_cast<float4*>(p + 4 * j) = make_float4(y[4 * j], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]);
    } else {
        uint16_t* p = (uint16_t*)g.out + row * g.N + n0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (n0 + 8 * j >= g.N) break;
            uint4 o;
            uint32_t* w = &o.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = pack16(y[8 * j + 2 * i], y[8 * j + 2 * i + 1], g.out_dtype);
            *reinterpret_cast<uint4*>(p + 8 * j) = o;
        }
    }
}

// Tile order: groups of `raster_group` tile rows; inside a group the tile row index runs fastest, then N.  The CTAs
// that run concurrently then share a few A row blocks and a few B column blocks, so a group's A rows stay in L2
// while B streams past them, instead of all of A cycling through L2 once per tile column.
__device__ __forceinline__ void tile_coords(const GemmArgs& g, int tile, int& tm, int& tn) {
    const int per_group = g.raster_group * g.n_tiles;
    const int grp = tile / per_group;
    const int within = tile - grp * per_group;
    const int m0 = grp * g.raster_group;
    const int rows = min(g.raster_group, g.m_tiles - m0);
    tn = within / rows;
    tm = m0 + (within - tn * rows);
}

// ---- kernel -----------------------------------------------------------------------------------------

// FMT 0: NVFP4 (packed e2m1, e4m3 scales per 16 elements, 256 elements of K per stage).
// FMT 1: MXFP8 (e4m3 bytes, e8m0 scales per 32 elements, 128 elements of K per stage): the same 128-byte operand rows
// and 32-byte steps per instruction, but one scale chunk per stage, whose four bytes per row serve the four instructions.
template <int BN, bool DBG, int FMT = 0, int AROWS = BM>
__global__ void __launch_bounds__(NUM_THREADS, (Cfg<BN, AROWS>::kCtasPerSm))
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_out, const GemmArgs g) {
    using C = Cfg<BN, AROWS>;
    static_assert(!C::kSkinny || FMT == 0, "64-column tiles: NVFP4 only");
    constexpr bool MX = (FMT == 1);
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = smem + C::kStages * C::kStageBytes;      // 4 x 2 KiB, 64-byte swizzled rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::kStagingBytes);
    uint64_t* full_bar = bars;                                  // [kStages]  producer -> MMA
    uint64_t* empty_bar = bars + C::kStages;                    // [kStages]  MMA -> producer
    uint64_t* acc_full_bar = bars + 2 * C::kStages;             // [2] MMA -> epilogue
    uint64_t* acc_empty_bar = acc_full_bar + 2;                 // [2] epilogue -> MMA: accumulator drained
    uint64_t* overlap_bar = acc_empty_bar + 2;                  // [1] epilogue -> MMA: shared columns drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(overlap_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    allow_dependent_launch();
    if (threadIdx.x == 32) {   // the maps are parameters: nothing a preceding kernel writes
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        if (g.tma_store) prefetch_tensormap(&tmap_out);
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&acc_full_bar[s]), 1);
            mbar_init(smem_u32(&acc_empty_bar[s]), 128);
        }
        mbar_init(smem_u32(overlap_bar), 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // tensor-memory allocation is a warp-wide operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)C::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_items = g.m_tiles * g.n_tiles * g.splits;
    // Barriers and tensor memory are set up while the previous kernel drains.  With early_weights the roles that
    // read or write what a preceding kernel may touch (activations, their scales, the tensor scales, bias, output,
    // partial sums) wait by themselves, and the producer asks for the weight's first stages before it does.
    const bool early = g.early_weights != 0;
    if (!early) grid_dependency_wait();

    // cycle counters of the debug build (DBG): compiled out otherwise
    auto now = [] { return DBG ? clock64() : 0ll; };

    if (warp == 0) {
        // ---------------- producer ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        bool waited_for_grid = !early;
        long long waited = 0;
        const long long t_begin = now();
        if (early && (int)blockIdx.x >= total_items) grid_dependency_wait();
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            const int tile = item / g.splits;
            const int kb0 = (item - tile * g.splits) * g.k_per_split, kb1 = min(g.k_iters, kb0 + g.k_per_split);
            int tm, tn;
            tile_coords(g, tile, tm, tn);
            // first 128-row band of B scales of this tile (a 64-column tile uses half of one band's chunks)
            const int band0 = C::kSkinny ? (tn * BN) / 128 : tn * C::kBands;
            int sfb_present = 0;
#pragma unroll
            for (int b = 0; b < C::kBands; ++b)
                if (band0 + b < g.sfb_bands) ++sfb_present;
            const uint8_t* sfa_src = g.sfa + (int64_t)tm * g.sf_cbg * SF_CHUNK_BYTES;
            const uint8_t* sfb_src = g.sfb + (int64_t)band0 * g.sf_cbg * SF_CHUNK_BYTES;
            __syncwarp();
            // one stage's loads in two parts: what belongs to the weight, and what a preceding kernel may have written
            auto load_weight_part = [&](int kb, int stg) {
                const uint32_t st = smem_u32(smem) + stg * C::kStageBytes;
                const uint32_t bar = smem_u32(&full_bar[0]) + stg * 8;
                const int chunk0 = MX ? kb : kb * CHUNKS;   // first scale chunk of this stage
                const int nchunk = MX ? 1 : min(CHUNKS, g.sf_cbg - kb * CHUNKS);
                const uint32_t sf_bytes = nchunk * SF_CHUNK_BYTES;
                mbar_expect_tx(bar, g.a_box_bytes + C::kBBytes + (1 + sfb_present) * sf_bytes);
                tma_load_2d(st + C::kABytes, &tmap_b, kb * BK_BYTES, tn * BN, bar);
#pragma unroll
                for (int b = 0; b < C::kBands; ++b)
                    if (b < sfb_present)
                        bulk_load(st + C::kABytes + C::kBBytes + C::kSfaBytes + b * C::kSfaBytes,
                                  sfb_src + ((int64_t)b * g.sf_cbg + chunk0) * SF_CHUNK_BYTES, sf_bytes, bar);
            };
            auto load_activation_part = [&](int kb, int stg) {
                const uint32_t st = smem_u32(smem) + stg * C::kStageBytes;
                const uint32_t bar = smem_u32(&full_bar[0]) + stg * 8;
                const int chunk0 = MX ? kb : kb * CHUNKS;
                const int nchunk = MX ? 1 : min(CHUNKS, g.sf_cbg - kb * CHUNKS);
                tma_load_2d(st, &tmap_a, kb * BK_BYTES, tm * BM, bar);
                bulk_load(st + C::kABytes + C::kBBytes, sfa_src + (int64_t)chunk0 * SF_CHUNK_BYTES, nchunk * SF_CHUNK_BYTES, bar);
            };
            int kb = kb0;
            if (!waited_for_grid) {
                // the CTA's first work item: every stage of the ring is free.  Weight parts of as many stages as the
                // ring holds, then the wait for the preceding kernel, then the activation parts.
                const int n_pre = min(C::kStages, kb1 - kb0);
                if (elect_one())
                    for (int i = 0; i < n_pre; ++i) load_weight_part(kb0 + i, i);
                __syncwarp();
                grid_dependency_wait();
                waited_for_grid = true;
                if (elect_one())
                    for (int i = 0; i < n_pre; ++i) load_activation_part(kb0 + i, i);
                __syncwarp();
                kb = kb0 + n_pre;
                stage = n_pre;
                if (stage == C::kStages) { stage = 0; phase ^= 1; }
            }
            for (; kb < kb1; ++kb) {
                const long long t0 = now();
                ok = mbar_wait(smem_u32(&empty_bar[0]) + stage * 8, phase ^ 1, abort_flag, WAIT_STAGE_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                waited += now() - t0;
                if (!ok) break;
                if (elect_one()) {
                    load_weight_part(kb, stage);
                    load_activation_part(kb, stage);
                }
                __syncwarp();
                if (++stage == C::kStages) { stage = 0; phase ^= 1; }
            }
        }
        if (DBG && (g.debug & 1) && blockIdx.x == 0 && lane == 0)
            printf("[gemm bn%d cta0] producer: total %lld cycles, waiting for free stages %lld\n", BN, now() - t_begin,
                   waited);
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int stage = 0, acc = 0, local_tile = 0;
        uint32_t phase = 0, acc_phase = 0;
        bool ok = true;
        long long wait_acc = 0, wait_full = 0;
        const long long t_begin = now();
        const uint32_t smem_enc = smem_u32(smem) >> 4;   // descriptor addresses are in 16-byte units
        const uint32_t sf_t0 = tmem_base + C::kSfCol0;
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++local_tile) {
            const int kb0 = (item % g.splits) * g.k_per_split, kb1 = min(g.k_iters, kb0 + g.k_per_split);
            // a 64-column tile's scales are two of the four tensor-memory columns its band's chunk fills (32 rows of the
            // band per column): the instruction reads from the column its first row sits in
            uint32_t sfb_col = 0;
            if (C::kSkinny) {
                int tm, tn;
                tile_coords(g, item / g.splits, tm, tn);
                sfb_col = (uint32_t)(((tn * BN) % 128) / 32);
            }
            long long t0 = now();
            // the accumulator's own columns: drained by the epilogue two tiles ago
            ok = mbar_wait(smem_u32(&acc_empty_bar[acc]), acc_phase ^ 1, abort_flag, WAIT_ACC_EMPTY);
            // the columns shared with the other accumulator: drained first by the previous tile's epilogue
            if (C::kOverlapCols > 0 && local_tile > 0 && ok)
                ok = mbar_wait(smem_u32(overlap_bar), (uint32_t)(local_tile - 1) & 1u, abort_flag, WAIT_OVERLAP);
            ok = __all_sync(0xffffffffu, ok);
            wait_acc += now() - t0;
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * C::kAcc1Col;
            for (int kb = kb0; kb < kb1; ++kb) {
                t0 = now();
                ok = mbar_wait(smem_u32(&full_bar[0]) + stage * 8, phase, abort_flag, WAIT_STAGE_FULL);
                ok = __all_sync(0xffffffffu, ok);
                wait_full += now() - t0;
                if (!ok) break;
                tc_fence_after();
                const uint32_t st_enc = smem_enc + stage * (C::kStageBytes >> 4);
                const uint32_t a_lo = st_enc | kOperandDescLoFlags;
                const uint32_t b_lo = a_lo + (C::kABytes >> 4);
                const uint32_t sfa_lo = st_enc + ((C::kABytes + C::kBBytes) >> 4);
                const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
                const int nchunk = min(CHUNKS, g.sf_cbg - kb * CHUNKS);
                if (MX) {
                    if (elect_one()) {
                        // one chunk per 128-row band per stage: cell (row, column) holds the scales of the stage's four
                        // 32-element blocks, one byte per instruction; the two regions alternate between stages
                        const uint32_t region = sf_t0 + (uint32_t)(kb & 1) * C::kSfRegionCols;
                        const uint32_t sfa_t = region, sfb_t = region + C::kSfaColsHalf;
                        tc_cp_sf(sfa_t, desc64(sfa_lo, kSfDescHi));
#pragma unroll
                        for (int b = 0; b < C::kBands; ++b)
                            tc_cp_sf(sfb_t + 4 * b, desc64(sfb_lo + (b * C::kSfaBytes) / 16, kSfDescHi));
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            tc_mma_mx(d_tmem, desc64(a_lo + 2 * j, kOperandDescHi), desc64(b_lo + 2 * j, kOperandDescHi),
                                      C::kIdescMx | ((uint32_t)j << 29) | ((uint32_t)j << 4), sfa_t, sfb_t,
                                      (j != 0 || kb != kb0) ? 1u : 0u);
                        tc_commit(smem_u32(&empty_bar[0]) + stage * 8);
                    }
                } else if (elect_one()) {
                    // scale factors of step j go to region j/2 (the two regions alternate, so a copy never
                    // overwrites scales that the MMAs issued just before it still read)
#pragma unroll
                    for (int j = 0; j < CHUNKS; ++j) {
                        if (j < nchunk) {
                            const uint32_t sfa_t = sf_t0 + (j >> 1) * C::kSfRegionCols + (j & 1) * 4;
                            const uint32_t sfb_t =
                                sf_t0 + (j >> 1) * C::kSfRegionCols + C::kSfaColsHalf + (j & 1) * 4 * C::kBands;
                            tc_cp_sf(sfa_t, desc64(sfa_lo + j * (SF_CHUNK_BYTES >> 4), kSfDescHi));
#pragma unroll
                            for (int b = 0; b < C::kBands; ++b)
                                tc_cp_sf(sfb_t + 4 * b,
                                         desc64(sfb_lo + (b * C::kSfaBytes + j * SF_CHUNK_BYTES) / 16, kSfDescHi));
                        }
                    }
#pragma unroll
                    for (int j = 0; j < CHUNKS; ++j) {
                        if (j < nchunk) {
                            const uint32_t sfa_t = sf_t0 + (j >> 1) * C::kSfRegionCols + (j & 1) * 4;
                            const uint32_t sfb_t =
                                sf_t0 + (j >> 1) * C::kSfRegionCols + C::kSfaColsHalf + (j & 1) * 4 * C::kBands;
                            // 64 elements of K = 32 bytes = 2 descriptor address units inside the swizzle row
                            tc_mma(d_tmem, desc64(a_lo + 2 * j, kOperandDescHi), desc64(b_lo + 2 * j, kOperandDescHi),
                                   C::kIdesc, sfa_t, sfb_t + sfb_col, (j != 0 || kb != kb0) ? 1u : 0u);
                        }
                    }
                    tc_commit(smem_u32(&empty_bar[0]) + stage * 8);   // stage reusable once these MMAs have read it
                }
                __syncwarp();
                if (++stage == C::kStages) { stage = 0; phase ^= 1; }
            }
            if (!ok) break;
            if (elect_one()) tc_commit(smem_u32(&acc_full_bar[acc]));   // accumulator complete
            __syncwarp();
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if (DBG && (g.debug & 1) && blockIdx.x == 0 && lane == 0)
            printf("[gemm bn%d cta0] mma: total %lld cycles, waiting for accumulator %lld, for loaded stages %lld\n", BN,
                   now() - t_begin, wait_acc, wait_full);
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quad = warp & 3;   // tensor-memory lanes [32*quad, 32*quad+32) are the ones this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        long long wait_acc = 0;
        const long long t_begin = now();
        if (early) grid_dependency_wait();   // before the tensor scales are read and anything is stored
        const float alpha = g.alpha ? __ldg(g.alpha) : __fmul_rn(__ldg(g.tsa), __ldg(g.tsb));
        uint8_t* my_staging = staging + quad * STAGING_BYTES_PER_WARP;
        const uint32_t my_staging_u32 = smem_u32(my_staging);
        constexpr int kSteps = BN / EPI_COLS;
        constexpr int kOverlapSteps = C::kOverlapCols / EPI_COLS;
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            const int tile = item / g.splits;
            const int split = item - tile * g.splits;
            int tm, tn;
            tile_coords(g, tile, tm, tn);
            const long long tw = now();
            ok = mbar_wait(smem_u32(&acc_full_bar[acc]), acc_phase, abort_flag, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            wait_acc += now() - tw;
            if (!ok) break;
            tc_fence_after();
            const int row0 = tm * BM + quad * 32;
            const int64_t row = (int64_t)row0 + lane;
            const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * C::kAcc1Col;
            // accumulator 0 shares its last columns with accumulator 1's first ones: drain those first
            const int first_step = (C::kOverlapCols > 0 && acc == 0) ? kSteps - kOverlapSteps : 0;
            auto emit = [&](int s, const uint32_t (&v)[32]) {
                const int n0 = tn * BN + s * EPI_COLS;
                if (g.splits > 1) {   // split-K: raw fp32 partial sums; alpha, bias and rounding happen in the reduction
                    if (row < g.M && n0 < g.N) {
                        float* p = g.partial + ((int64_t)split * g.M + row) * g.N + n0;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (n0 + 4 * j < g.N)
                                *reinterpret_cast<uint4*>(p + 4 * j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                    return;
                }
                float y[32];
                scale_row32(g, n0, v, alpha, y);
                if (g.tma_store) {
                    // 32 rows x 64 bytes, 16-byte pieces XOR-swizzled with (row/2)%4: the 64-byte swizzle of the
                    // output tensor map, and conflict-free for these stores
                    if (lane == 0) tma_store_wait_read<0>();   // the previous store has read the staging tile
                    __syncwarp();
                    uint8_t* rowp = my_staging + lane * 64;
                    const int sw = (lane >> 1) & 3;
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        uint4 o;
                        o.x = pack16(y[8 * p + 0], y[8 * p + 1], g.out_dtype);
                        o.y = pack16(y[8 * p + 2], y[8 * p + 3], g.out_dtype);
                        o.z = pack16(y[8 * p + 4], y[8 * p + 5], g.out_dtype);
                        o.w = pack16(y[8 * p + 6], y[8 * p + 7], g.out_dtype);
                        *reinterpret_cast<uint4*>(rowp + ((p ^ sw) << 4)) = o;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && n0 < g.N && row0 < g.M) {   // the store clips rows >= M and columns >= N itself
                        tma_store_2d(&tmap_out, n0, row0, my_staging_u32);
                        tma_store_commit();
                    }
                } else if (row < g.M && n0 < g.N) {
                    store_row32(g, row, n0, y);
                }
            };
            int i = 0;
            if (C::kOverlapCols > 0) {
                // both steps of the shared columns are fetched before anything else so that they can be handed to
                // the next tile's MMAs as early as possible
                static_assert(C::kOverlapCols == 0 || kOverlapSteps == 2, "two epilogue steps cover the shared columns");
                uint32_t v0[32], v1[32];
                const int s0 = first_step % kSteps, s1 = (first_step + 1) % kSteps;
                tc_ld32(t_acc + s0 * EPI_COLS, v0);
                tc_ld32(t_acc + s1 * EPI_COLS, v1);
                tc_wait_ld();
                tc_fence_before();
                mbar_arrive(smem_u32(overlap_bar));
                emit(s0, v0);
                emit(s1, v1);
                i = 2;
            }
#pragma unroll 1
            for (; i < kSteps; ++i) {
                const int s = (first_step + i) % kSteps;
                uint32_t v[32];
                tc_ld32(t_acc + s * EPI_COLS, v);
                tc_wait_ld();
                emit(s, v);
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&acc_empty_bar[acc]));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if (g.tma_store && lane == 0) tma_store_wait_all();   // global writes complete before the CTA exits
        if (DBG && (g.debug & 1) && blockIdx.x == 0 && threadIdx.x == 64)
            printf("[gemm bn%d cta0] epilogue: total %lld cycles, waiting for accumulators %lld\n", BN, now() - t_begin,
                   wait_acc);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
                     : "memory");
    }
}

// ---- 2-CTA kernel ---------------------------------------------------------------------------------
//
// The same pipeline on pairs of CTAs (thread-block clusters of 2, tcgen05 cta_group::2): a pair computes a
// 256 x 256 tile.  CTA r of the pair loads A rows [128 r, 128 r + 128) of the tile, HALF of the B tile (its rows
// [128 r, 128 r + 128) of N), its own 128 rows of A scales and all 256 rows of B scales; one MMA instruction issued
// by CTA 0 runs on both SMs (each reads the other half of B from its peer's shared memory) and each CTA keeps the
// fp32 accumulators of its 128 rows x 256 columns in its own tensor memory.  Per SM and 256 K-elements that is
// 38 KB of loads instead of 54 KB, which is what the 1-CTA kernel's main loop waits for.
//   * Loads of both CTAs signal CTA 0's "full" barrier (TMA .cta_group::2 lets the mbarrier live in the peer CTA);
//     none of them is a multicast load.
//   * CTA 0's MMA warp frees a stage, and publishes an accumulator, in both CTAs with one tcgen05.commit per CTA.
//   * Epilogue warps of both CTAs report drained accumulators to CTA 0 with remote mbarrier arrives.
// Scale chunks are fetched as 2-D tiles (a [chunks, 128 x u32] view of the tiled scale tensor, box of 4 chunks).

// KB = packed bytes of K per stage and row: 128 (256 elements, 128-byte swizzle, 5 stages of 38 KiB) or 64
// (128 elements, 64-byte swizzle, 11 stages of 19 KiB).  The finer stages keep more bytes in flight for the same
// shared memory (10 of 11 stages instead of 4 of 5 while one is being consumed), which hides more load latency.
// GATHER (the kernel that also delivers its tiles to the other ranks): the epilogue assembles whole 512-byte tile rows
// in shared memory, 32 rows per warp with a 16-byte pad per row (conflict-free 16-byte stores by 32 lanes), and one
// stage of the ring pays for that.
constexpr int kGatherRowPitch = 512 + 16;
template <int KB, bool GATHER = false>
struct PairCfg {
    static_assert(KB == 128 || KB == 64, "stage width");
    static constexpr int kChunks = KB / 32;                         // 64-element MMA steps per stage
    static constexpr int kA = BM * KB;                              // this CTA's 128 rows of A
    static constexpr int kB = 128 * KB;                             // this CTA's half of the 256 B rows
    static constexpr int kSfa = kChunks * SF_CHUNK_BYTES;
    static constexpr int kSfb = 2 * kChunks * SF_CHUNK_BYTES;       // both 128-row bands of the B tile
    static constexpr int kStageBytes = kA + kB + kSfa + kSfb;       // 38 KiB or 19 KiB
    static constexpr int kStagingBytes = GATHER ? 4 * 32 * kGatherRowPitch     // 32 full tile rows per epilogue warp
                                                : 4 * 4 * STAGING_BYTES_PER_WARP;   // four staging tiles per epilogue warp
    static constexpr int kStages = (232448 - 1024 - 256 - kStagingBytes) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
    static constexpr uint32_t kLayout = (KB == 128) ? LAYOUT_SWIZZLE_128B : LAYOUT_SWIZZLE_64B;
    static constexpr uint32_t kDescHi = desc_hi(8 * KB, kLayout);   // 8-row groups are 8 * KB bytes apart
    static_assert(kStageBytes % 1024 == 0, "stages stay 1024-byte aligned");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
    static_assert(2 * kStages + 5 <= 32, "barriers fit their 256 bytes");
};
constexpr int kAccCol1_2 = 192, kSfCol0_2 = 448, kSfRegion2 = 24;   // tensor-memory plan of the BN = 256 kernel
constexpr uint32_t kIdesc2 = (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_tmem,
                                            uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_mma_pair_mx(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
constexpr uint32_t kIdesc2Mx = ((uint32_t)(256 >> 3) << 17) | (1u << 23) | ((uint32_t)(256 >> 4) << 24);

// ---- activation quantizer inside the pair kernel --------------------------------------------------------
//
// gemm_nvfp4_pair_kernel<.., QDT >= 0> carries eight more warps per CTA that quantize the activation matrix (dtype
// code QDT) into the packed operand and scale tensor the kernel's own TMA loads read: the quantizer, which is bound
// by HBM, then runs beside the tensor-core main loop instead of in front of it.  Tiles are walked one row block
// after the other, so the first wave of tiles needs only the first few 128-row bands and the quantizer warps (which
// take the bands in the same order and never wait for anything) stay ahead of the loads from then on.
// Measured on a B200 (M = 4608, eager launches): 3072 -> 9216 takes 66-68 us against 64-66 us for the quantizer kernel
// followed by the GEMM kernel, 12288 -> 3072 takes 96-97 us against 87-89 us.  Eight warps per SM walk a segment at a
// time (loads, arithmetic, stores, release, in sequence) and move about 1 TB/s where the stand-alone quantizer, with
// 24 resident warps per SM, moves 4-5 TB/s; the producers then wait for bands (a quarter of their time) and the main
// loop starves.  The path is therefore off by default (CK_B200_TUNE_LINEAR_FUSED) and kept for shapes and parts
// where the balance differs; its results are bit-identical to the separate kernels.
//
// Progress is published per band as a counter in a small sync area of the caller's workspace, bumped with one
// atomic add per finished segment.  The counters are zero when a kernel starts: the caller zeroes the area once, and
// the last CTA to leave a kernel zeroes what the kernel used, so replays of a captured launch work like fresh ones.
// A producer warp polls its band's counter (bounded, like every wait here) before the first load of a tile, then
// orders its TMA loads after what it has seen with a proxy fence.  Calls that share a workspace must not overlap
// on the GPU (they would also share the quantized operand).
constexpr int kQuantWarps = 8;
struct FusedQuantSync {
    uint32_t exits;        // CTAs that have left the kernel
    uint32_t bands_done;   // bands completely quantized
    uint32_t band[2];      // [bands] warps done with their segment of the band
};
struct FusedQuant {
    QuantArgs q;
    FusedQuantSync* sync;
    int bands;
};

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// FMT as in gemm_nvfp4_kernel: 0 = NVFP4, 1 = MXFP8 (one scale chunk per stage and band instead of KB / 32).
// QDT: -1 = operands come quantized; otherwise the dtype code of the activations that eight extra warps quantize.
// GATHER: every finished tile also goes to the same place of the other ranks' output matrices (g.peer_out), as
// 512-byte row segments copied out of shared memory by bulk async copies (no load of any kind from peer memory).
template <int KB, bool DBG, int FMT = 0, int QDT = -1, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(QDT >= 0 ? NUM_THREADS + kQuantWarps * 32 : NUM_THREADS, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                       const __grid_constant__ CUtensorMap tmap_out, const GemmArgs g, const FusedQuant fq) {
    constexpr bool QF = QDT >= 0;
    using P = PairCfg<KB, GATHER>;
    constexpr int kStages2 = P::kStages, kStageBytes2 = P::kStageBytes, kA2 = P::kA, kB2 = P::kB, kSfa2 = P::kSfa;
    constexpr int kChunks = P::kChunks;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = smem + kStages2 * kStageBytes2;
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + P::kStagingBytes);
    uint64_t* full_bar = bars;                       // [kStages2] used in CTA 0: loads of both CTAs -> MMA
    uint64_t* empty_bar = bars + kStages2;           // [kStages2] in each CTA: MMA -> this CTA's producer
    uint64_t* acc_full_bar = bars + 2 * kStages2;    // [2] in each CTA: MMA -> this CTA's epilogue
    uint64_t* acc_empty_bar = acc_full_bar + 2;      // [2] used in CTA 0: epilogues of both CTAs -> MMA
    uint64_t* overlap_bar = acc_empty_bar + 2;       // [1] used in CTA 0
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(overlap_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    allow_dependent_launch();
    if (threadIdx.x == 32) {   // the maps are parameters: nothing a preceding kernel writes
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        prefetch_tensormap(&tmap_sfa);
        prefetch_tensormap(&tmap_sfb);
        if (g.tma_store) prefetch_tensormap(&tmap_out);
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 2);     // one expect_tx arrive from each CTA's producer
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&acc_full_bar[s]), 1);
            mbar_init(smem_u32(&acc_empty_bar[s]), 8);   // one arrive per epilogue warp of both CTAs
        }
        mbar_init(smem_u32(overlap_bar), 8);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // the same warp of both CTAs allocates the pair's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();   // barriers of both CTAs are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_wait();   // barriers and tensor memory are set up while the previous kernel drains

    const int total_tiles = g.m_tiles * g.n_tiles;   // 256 x 256 tiles
    constexpr bool MX = (FMT == 1);
    constexpr int kSfChunks = MX ? 1 : kChunks;                       // scale chunks per stage and 128-row band
    constexpr uint32_t kTxBytes = kA2 + kB2 + 3 * kSfChunks * SF_CHUNK_BYTES;   // per CTA and stage
    const int k_stages = (g.sf_cbg + kSfChunks - 1) / kSfChunks;   // stages per tile
    auto now = [] { return DBG ? clock64() : 0ll; };

    if (warp == 0) {
        // ---------------- producer (both CTAs) ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        long long waited = 0;
        const long long t_begin = now();
        const uint32_t full0 = map_to_cta(smem_u32(&full_bar[0]), 0);   // CTA 0's barriers
        bool q_all_ready = false;
        long long q_waited = 0;
        const uint32_t q_band_target = QF ? (uint32_t)(32 * fq.q.segments) : 0u;
        const uint32_t q_all_target = QF ? (uint32_t)fq.bands : 0u;
        uint32_t q_pre_all = 0, q_pre_band = 0;
        bool q_have_pre = false;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
            int tm, tn;
            tile_coords(g, tile, tm, tn);
            const int a_row = (tm * 2 + (int)rank) * BM;                 // this CTA's A rows; also its scale band
            const int b_row = tn * 256 + (int)rank * 128;                // this CTA's half of the B tile
            const int sfa_chunk0 = (tm * 2 + (int)rank) * g.sf_cbg;
            const int sfb_chunk0 = tn * 2 * g.sf_cbg;
            if (QF && !q_all_ready) {
                // this CTA's A rows and their scales are one band of the activation matrix: wait until the
                // quantizer warps (of any CTA) have finished it.  The counters were read ahead while the previous
                // tile's loads were in flight, so the common case costs no round trip to L2 here.
                const int band = tm * 2 + (int)rank;
                const long long t0 = now();
                const uint32_t all_v = q_have_pre ? q_pre_all : ld_relaxed_u32(&fq.sync->bands_done);
                uint32_t band_v = q_band_target;
                if (band < fq.bands) band_v = q_have_pre ? q_pre_band : ld_relaxed_u32(&fq.sync->band[band]);
                if (all_v == q_all_target) {
                    q_all_ready = true;
                } else if (band_v != q_band_target) {
                    const long long start = clock64();
                    while (ld_relaxed_u32(&fq.sync->band[band]) != q_band_target) {
                        if (*abort_flag) { ok = false; break; }
                        if (clock64() - start > WAIT_LIMIT_CYCLES) {
                            *abort_flag = 1;
                            atomicCAS(&g_device_status, 0, (int)WAIT_QUANT_BAND);
                            ok = false;
                            break;
                        }
                        __nanosleep(64);
                    }
                }
                ok = __all_sync(0xffffffffu, ok);
                __threadfence();           // acquire: pairs with the quantizer warps' release of the band
                fence_proxy_async_all();   // the TMA loads below read what those warps wrote with plain stores
                q_waited += now() - t0;
                if (!ok) break;
            }
            for (int kb = 0; kb < k_stages; ++kb) {
                const long long t0 = now();
                ok = mbar_wait(smem_u32(&empty_bar[0]) + stage * 8, phase ^ 1, abort_flag, WAIT_STAGE_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
                waited += now() - t0;
                if (!ok) break;
                const uint32_t st = smem_u32(smem) + stage * kStageBytes2;
                const uint32_t bar = full0 + stage * 8;
                if (elect_one()) {
                    mbar_expect_tx_cluster(bar, kTxBytes);   // every box is transferred in full (zero fill past the ends)
                    tma_load_2d_pair(st, &tmap_a, kb * KB, a_row, bar);
                    tma_load_2d_pair(st + kA2, &tmap_b, kb * KB, b_row, bar);
                    tma_load_2d_pair(st + kA2 + kB2, &tmap_sfa, 0, sfa_chunk0 + kb * kSfChunks, bar);
                    tma_load_2d_pair(st + kA2 + kB2 + kSfa2, &tmap_sfb, 0, sfb_chunk0 + kb * kSfChunks, bar);
                    tma_load_2d_pair(st + kA2 + kB2 + kSfa2 + kSfa2, &tmap_sfb, 0, sfb_chunk0 + g.sf_cbg + kb * kSfChunks, bar);
                }
                if (QF && kb == 0 && !q_all_ready) {
                    // read ahead the counters the next tile will ask for
                    const int next = tile + num_pairs;
                    q_have_pre = false;
                    if (next < total_tiles) {
                        int nm, nn;
                        tile_coords(g, next, nm, nn);
                        const int nb = nm * 2 + (int)rank;
                        q_pre_all = ld_relaxed_u32(&fq.sync->bands_done);
                        q_pre_band = nb < fq.bands ? ld_relaxed_u32(&fq.sync->band[nb]) : q_band_target;
                        q_have_pre = true;
                    }
                }
                __syncwarp();
                if (++stage == kStages2) { stage = 0; phase ^= 1; }
            }
        }
        if (DBG && (g.debug & 1) && pair == 0 && lane == 0)
            printf("[gemm pair cta%u] producer: total %lld cycles, waiting for free stages %lld, for quantized bands %lld\n",
                   rank, now() - t_begin, waited, q_waited);
    } else if (warp == 1 && rank == 0) {
        // ---------------- MMA issuer (CTA 0 of the pair) ----------------
        int stage = 0, acc = 0, local_tile = 0;
        uint32_t phase = 0, acc_phase = 0;
        bool ok = true;
        long long wait_acc = 0, wait_full = 0;
        const long long t_begin = now();
        const uint32_t smem_enc = (smem_u32(smem) >> 4) & 0x3fffu;
        const uint32_t sf_t0 = tmem_base + kSfCol0_2;
        const uint32_t empty_peer = map_to_cta(smem_u32(&empty_bar[0]), 1);
        const uint32_t acc_full_peer = map_to_cta(smem_u32(&acc_full_bar[0]), 1);
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++local_tile) {
            long long t0 = now();
            ok = mbar_wait(smem_u32(&acc_empty_bar[acc]), acc_phase ^ 1, abort_flag, WAIT_ACC_EMPTY);
            if (local_tile > 0 && ok)
                ok = mbar_wait(smem_u32(overlap_bar), (uint32_t)(local_tile - 1) & 1u, abort_flag, WAIT_OVERLAP);
            ok = __all_sync(0xffffffffu, ok);
            wait_acc += now() - t0;
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * kAccCol1_2;
            for (int kb = 0; kb < k_stages; ++kb) {
                t0 = now();
                ok = mbar_wait(smem_u32(&full_bar[0]) + stage * 8, phase, abort_flag, WAIT_STAGE_FULL);
                ok = __all_sync(0xffffffffu, ok);
                wait_full += now() - t0;
                if (!ok) break;
                tc_fence_after();
                const uint32_t st_enc = smem_enc + stage * (kStageBytes2 >> 4);
                const uint32_t a_lo = st_enc | kOperandDescLoFlags;
                const uint32_t b_lo = a_lo + (kA2 >> 4);
                const uint32_t sfa_lo = st_enc + ((kA2 + kB2) >> 4);
                const uint32_t sfb_lo = sfa_lo + (kSfa2 >> 4);
                const int nchunk = min(kChunks, g.sf_cbg - kb * kChunks);
                // scale factors of 64-element step j of the tile go to region (j/2) % 2: two alternating regions,
                // each holding two steps
                const int region0 = (kChunks == 2) ? (kb & 1) : 0;
                if (MX) {
                    if (elect_one()) {
                        // one chunk per band and stage; its four bytes per row serve the stage's four instructions
                        const uint32_t sfa_t = sf_t0 + (uint32_t)(kb & 1) * kSfRegion2, sfb_t = sfa_t + 8;
                        tc_cp_sf_pair(sfa_t, desc64(sfa_lo, kSfDescHi));
                        tc_cp_sf_pair(sfb_t, desc64(sfb_lo, kSfDescHi));
                        tc_cp_sf_pair(sfb_t + 4, desc64(sfb_lo + kSfa2 / 16, kSfDescHi));
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            tc_mma_pair_mx(d_tmem, desc64(a_lo + 2 * j, P::kDescHi), desc64(b_lo + 2 * j, P::kDescHi),
                                           kIdesc2Mx | ((uint32_t)j << 29) | ((uint32_t)j << 4), sfa_t, sfb_t,
                                           (j != 0 || kb != 0) ? 1u : 0u);
                        tc_commit_pair(smem_u32(&empty_bar[0]) + stage * 8);
                        tc_commit_pair(empty_peer + stage * 8);
                    }
                } else if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < kChunks; ++j) {
                        if (j < nchunk) {
                            const uint32_t sf_r = sf_t0 + (region0 + (j >> 1)) * kSfRegion2;
                            const uint32_t sfa_t = sf_r + (j & 1) * 4;
                            const uint32_t sfb_t = sf_r + 8 + (j & 1) * 8;
                            tc_cp_sf_pair(sfa_t, desc64(sfa_lo + j * (SF_CHUNK_BYTES >> 4), kSfDescHi));
                            tc_cp_sf_pair(sfb_t, desc64(sfb_lo + j * (SF_CHUNK_BYTES >> 4), kSfDescHi));
                            tc_cp_sf_pair(sfb_t + 4, desc64(sfb_lo + (kSfa2 + j * SF_CHUNK_BYTES) / 16, kSfDescHi));
                        }
                    }
#pragma unroll
                    for (int j = 0; j < kChunks; ++j) {
                        if (j < nchunk) {
                            const uint32_t sf_r = sf_t0 + (region0 + (j >> 1)) * kSfRegion2;
                            const uint32_t sfa_t = sf_r + (j & 1) * 4;
                            const uint32_t sfb_t = sf_r + 8 + (j & 1) * 8;
                            tc_mma_pair(d_tmem, desc64(a_lo + 2 * j, P::kDescHi), desc64(b_lo + 2 * j, P::kDescHi), kIdesc2,
                                        sfa_t, sfb_t, (j != 0 || kb != 0) ? 1u : 0u);
                        }
                    }
                    tc_commit_pair(smem_u32(&empty_bar[0]) + stage * 8);   // this CTA's producer
                    tc_commit_pair(empty_peer + stage * 8);                // the peer's producer
                }
                __syncwarp();
                if (++stage == kStages2) { stage = 0; phase ^= 1; }
            }
            if (!ok) break;
            if (elect_one()) {
                tc_commit_pair(smem_u32(&acc_full_bar[acc]));
                tc_commit_pair(acc_full_peer + acc * 8);
            }
            __syncwarp();
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if (DBG && pair == 0 && lane == 0) {
            const long long cyc = now() - t_begin;
            if ((g.debug & 1)) printf("[gemm pair cta0] mma: total %lld cycles, waiting for accumulator %lld, for loaded stages %lld\n", cyc,
                   wait_acc, wait_full);
            g_gemm_counters[2] = wait_full;
            g_gemm_counters[3] = wait_acc;
            g_gemm_counters[4] = cyc;
        }
    } else if (QF && warp >= NUM_THREADS / 32) {
        // ---------------- activation quantizer (eight warps of both CTAs) ----------------
        if constexpr (QF) {
            const long long t_begin = now();
            const float ts = __ldg(fq.q.pts);
            const int per_band = 32 * fq.q.segments;
            const int items = fq.bands * per_band;
            const int stride = (int)gridDim.x * kQuantWarps;
            for (int item = (int)blockIdx.x * kQuantWarps + (warp - NUM_THREADS / 32); item < items; item += stride) {
                const int band = item / per_band;
                const int rem = item - band * per_band;
                quantize_segment<QDT, true, 2>(fq.q, rem >> 5, band * 32 + (rem & 31), lane, ts);
                // release by one lane: the warp barrier orders the other lanes' stores before lane 0's fence, which
                // is cumulative; the other lanes go on to the next segment's loads meanwhile
                __syncwarp();
                if (lane == 0) {
                    __threadfence();
                    if (atomicAdd(&fq.sync->band[band], 1u) + 1u == (uint32_t)per_band) atomicAdd(&fq.sync->bands_done, 1u);
                }
            }
            if (DBG && (g.debug & 1) && pair == 0 && threadIdx.x == NUM_THREADS)
                printf("[gemm pair cta%u] quantizer: total %lld cycles\n", rank, now() - t_begin);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        const int quad = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        long long wait_acc = 0;
        auto now_ns = [] {
            long long t = 0;
            if (DBG) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            return t;
        };
        const long long t_begin = now();
        const long long t_begin_ns = now_ns();
        const float alpha = g.alpha ? __ldg(g.alpha) : __fmul_rn(__ldg(g.tsa), __ldg(g.tsb));
        uint8_t* my_staging = staging + quad * 4 * STAGING_BYTES_PER_WARP;   // four tiles per warp: the i-th emitted step uses tile i % 4
        uint8_t* gather_rows = staging + quad * 32 * kGatherRowPitch;        // GATHER: this warp's 32 tile rows
        const uint32_t acc_empty0 = map_to_cta(smem_u32(&acc_empty_bar[0]), 0);
        const uint32_t overlap0 = map_to_cta(smem_u32(overlap_bar), 0);
        constexpr int kSteps = 256 / EPI_COLS;
        constexpr int kOverlapSteps = 64 / EPI_COLS;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
            int tm, tn;
            tile_coords(g, tile, tm, tn);
            const long long tw = now();
            ok = mbar_wait(smem_u32(&acc_full_bar[acc]), acc_phase, abort_flag, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            wait_acc += now() - tw;
            if (!ok) break;
            tc_fence_after();
            const int row0 = (tm * 2 + (int)rank) * BM + quad * 32;
            const int64_t row = (int64_t)row0 + lane;
            const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * kAccCol1_2;
            // order of the eight 32-column steps: accumulator 0 starts with the two steps whose columns it shares
            // with accumulator 1 (6, 7), then finishes that group of four (4, 5) before 0..3, so that every four
            // consecutive steps cover 128 adjacent columns
            auto step_at = [&](int i) { return (acc == 0) ? ((i < 4) ? 4 + (i ^ 2) : i - 4) : i; };
            auto emit = [&](int i, int s, const uint32_t (&v)[32]) {
                const int n0 = tn * 256 + s * EPI_COLS;
                float y[32];
                scale_row32(g, n0, v, alpha, y);
                if constexpr (GATHER) {
                    // this lane's row of the tile: 64 bytes at column offset 32 s of its 512-byte row
                    uint8_t* rowp = gather_rows + lane * kGatherRowPitch + s * (EPI_COLS * 2);
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        uint4 o;
                        o.x = pack16(y[8 * p + 0], y[8 * p + 1], g.out_dtype);
                        o.y = pack16(y[8 * p + 2], y[8 * p + 3], g.out_dtype);
                        o.z = pack16(y[8 * p + 4], y[8 * p + 5], g.out_dtype);
                        o.w = pack16(y[8 * p + 6], y[8 * p + 7], g.out_dtype);
                        *reinterpret_cast<uint4*>(rowp + (p << 4)) = o;
                    }
                } else if (g.tma_store) {
                    // Four staging tiles per warp, taken in the order in which the steps are emitted (i, not the column
                    // step s: accumulator 0 walks the steps as 6,7,4,5,0,1,2,3, and indexing by s would hand a tile out
                    // again two steps later, while the TMA store that reads it may still be in flight - its last rows
                    // then carry the later step's values).  With i the store that last used the tile is always the one
                    // issued four steps ago, which wait_group.read 3 has retired.
                    if (lane == 0) tma_store_wait_read<3>();
                    __syncwarp();
                    uint8_t* tile_smem = my_staging + (i & 3) * STAGING_BYTES_PER_WARP;
                    uint8_t* rowp = tile_smem + lane * 64;
                    const int sw = (lane >> 1) & 3;
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        uint4 o;
                        o.x = pack16(y[8 * p + 0], y[8 * p + 1], g.out_dtype);
                        o.y = pack16(y[8 * p + 2], y[8 * p + 3], g.out_dtype);
                        o.z = pack16(y[8 * p + 4], y[8 * p + 5], g.out_dtype);
                        o.w = pack16(y[8 * p + 6], y[8 * p + 7], g.out_dtype);
                        *reinterpret_cast<uint4*>(rowp + ((p ^ sw) << 4)) = o;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && n0 < g.N && row0 < g.M) {
                        tma_store_2d(&tmap_out, n0, row0, smem_u32(tile_smem));
                        tma_store_commit();
                    }
                } else if (row < g.M && n0 < g.N) {
                    store_row32(g, row, n0, y);
                }
            };
            if constexpr (GATHER) bulk_wait_read_all();   // the previous tile's copies have read this lane's row
            {
                // both steps of the columns shared by the two accumulators are fetched first and handed to the
                // next tile's MMAs before any output work
                static_assert(kOverlapSteps == 2 && kSteps == 8, "two of eight epilogue steps cover the shared columns");
                uint32_t v0[32], v1[32];
                const int s0 = step_at(0), s1 = step_at(1);
                tc_ld32(t_acc + s0 * EPI_COLS, v0);
                tc_ld32(t_acc + s1 * EPI_COLS, v1);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(overlap0);
                emit(0, s0, v0);
                emit(1, s1, v1);
            }
            {
                // the other six steps, two register sets deep: the fetch of step i + 1 is in flight while step i is
                // converted and stored, and the accumulator goes back to the MMA warp as soon as the last fetch
                // has landed in registers, before the last step's output work
                uint32_t va[32], vb[32];
                tc_ld32(t_acc + step_at(2) * EPI_COLS, va);
#pragma unroll 1
                for (int i = 2; i < kSteps; i += 2) {
                    tc_wait_ld();
                    tc_ld32(t_acc + step_at(i + 1) * EPI_COLS, vb);
                    emit(i, step_at(i), va);
                    tc_wait_ld();
                    if (i + 2 < kSteps) {
                        tc_ld32(t_acc + step_at(i + 2) * EPI_COLS, va);
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(acc_empty0 + acc * 8);
                    }
                    emit(i + 1, step_at(i + 1), vb);
                }
            }
            if constexpr (GATHER) {
                // The lane's 512-byte row of the tile is complete in shared memory (written by this lane alone): one bulk
                // copy takes it to this rank's matrix and one to the same place in every other rank's.  The copies run
                // on the async proxy while the warp goes on to the next tile.
                fence_proxy_async_smem();
                const int col0 = tn * 256;
                const int bytes = min(256, g.N - col0) * 2;
                if (row < g.M && bytes > 0) {
                    const uint32_t src = smem_u32(gather_rows + lane * kGatherRowPitch);
                    const int64_t off = (row * g.ld_out + col0) * 2;
                    bulk_store(reinterpret_cast<uint8_t*>(g.out) + off, src, (uint32_t)bytes);
#pragma unroll 1
                    for (int p = 0; p < g.n_peers; ++p) bulk_store(g.peer_out[p] + off, src, (uint32_t)bytes);
                }
                bulk_commit();
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if constexpr (GATHER) bulk_wait_all();   // every copy has been performed before the CTA exits
        else if (g.tma_store && lane == 0) tma_store_wait_all();
        if (DBG && pair == 0 && threadIdx.x == 64) {
            const long long cyc = now() - t_begin, ns = now_ns() - t_begin_ns;
            if ((g.debug & 1)) printf("[gemm pair cta%u] epilogue: total %lld cycles in %lld ns, waiting for accumulators %lld\n", rank, cyc,
                   ns, wait_acc);
            if (rank == 0) {
                g_gemm_counters[0] = cyc;
                g_gemm_counters[1] = ns;
            }
        }
    }

    tc_fence_before();
    cluster_sync_all();   // no CTA of the pair leaves while the other may still read its shared memory or signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    if (QF) {
        // every warp of this CTA is past its last use of the counters; the last CTA out leaves them zero for the
        // next kernel
        __shared__ uint32_t s_last;
        if (threadIdx.x == 0) {
            __threadfence();
            s_last = (atomicAdd(&fq.sync->exits, 1u) + 1u == gridDim.x) ? 1u : 0u;
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int i = threadIdx.x; i < fq.bands; i += blockDim.x) fq.sync->band[i] = 0u;
            if (threadIdx.x == 0) {
                fq.sync->bands_done = 0u;
                fq.sync->exits = 0u;
            }
        }
    }
}

// ---- barrier between the ranks of one node (kernel) ---------------------------------------------------

struct BarrierArgs {
    uint32_t* flags[8];   // flags[r]: rank r's array of `world` counters (flags[rank] is local memory)
    uint32_t* epoch;      // local: barriers completed so far
    int world, rank;
};

// One block.  Thread t signals rank t (writes the new epoch into slot `rank` of its array) and waits until rank t
// has signalled this rank.  The wait is bounded (two seconds): on expiry the kernel records WAIT_PEER_BARRIER in
// the status word and returns, so a missing peer leaves the context usable.
__global__ void peer_barrier_kernel(const BarrierArgs b) {
    const int t = threadIdx.x;
    const uint32_t target = *b.epoch + 1;
    if (t < b.world && t != b.rank) {
        __threadfence_system();   // this GPU's earlier stores to the peers are ordered before the signal
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(b.flags[t] + b.rank), "r"(target) : "memory");
        const uint32_t* mine = b.flags[b.rank] + t;
        unsigned long long t0, now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - target) >= 0) break;
            __nanosleep(200);
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - t0 > 2000000000ull) {
                atomicCAS(&g_device_status, 0, (int)WAIT_PEER_BARRIER);
                break;
            }
        }
    }
    __syncthreads();
    if (t == 0) *b.epoch = target;
}

// ---- split-K reduction ----------------------------------------------------------------------------

// out[m,n] = out_dtype( alpha * sum_s partial[s,m,n] + bias[n] ), four columns per thread (N % 8 == 0).
// ---- one short tile row, K split over a thread-block cluster ------------------------------------------
//
// M <= 64: a 128-column tile of the output is computed by a cluster of CS CTAs, each over 1/CS of K (two CTAs per SM,
// short rings), so the serial chain of stages per CTA - which is what a small-M GEMM spends its time in once the
// weight streams at the HBM rate - is CS times shorter.  The partial sums never leave the SMs: every CTA writes the
// 32-column steps it does not own into the owner's shared memory (distributed shared memory), one cluster barrier,
// and every CTA adds up the steps it owns in rank order (the order of splitk_reduce_kernel, so the bits equal the
// two-kernel split-K with the same number of splits), applies alpha and bias and stores.  One launch, no scratch.
template <int AROWS, int CS>
struct ClusterCfg {
    static_assert(CS == 2 || CS == 4, "cluster size");
    static_assert(AROWS == 32 || AROWS == 64, "A rows per stage");
    static constexpr int kABytes = AROWS * BK_BYTES;
    static constexpr int kBBytes = 128 * BK_BYTES;
    static constexpr int kSfBytes = CHUNKS * SF_CHUNK_BYTES;
    static constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;
    static constexpr int kStepsOwned = 4 / CS;                            // 32-column steps a rank adds up
    static constexpr int kSlotBytes = AROWS * kStepsOwned * EPI_COLS * 4; // what one sender leaves with an owner
    static constexpr int kExchangeBytes = (CS - 1) * kSlotBytes;
    static constexpr int kSmemBudget = 115712;                            // two CTAs per SM
    static constexpr int kStages = (kSmemBudget - kExchangeBytes - 1024 - 256) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kExchangeBytes + 1024 + 256;
    static constexpr int kSfCol0 = 128, kSfRegionCols = 16, kTmemCols = 256;
    static_assert(kStages >= 3 && 2 * kStages + 1 <= 28, "ring depth and barrier room");
    static_assert(kStageBytes >= BM * BK_BYTES && kStageBytes % 1024 == 0 && kABytes % 1024 == 0, "stage layout");
};

__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <int AROWS, int CS>
__global__ void __cluster_dims__(CS, 1, 1) __launch_bounds__(NUM_THREADS, 2)
gemm_nvfp4_cluster_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const GemmArgs g) {
    using C = ClusterCfg<AROWS, CS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* exchange = smem + C::kStages * C::kStageBytes;     // [CS - 1 senders][AROWS][kStepsOwned * 32] fp32
    uint64_t* bars = reinterpret_cast<uint64_t*>(exchange + C::kExchangeBytes);
    uint64_t* full_bar = bars;                                  // [kStages] producer -> MMA
    uint64_t* empty_bar = bars + C::kStages;                    // [kStages] MMA -> producer
    uint64_t* acc_full_bar = bars + 2 * C::kStages;             // [1] MMA -> epilogue
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int tn = blockIdx.x / CS;                             // one tile row: the tile index is the column block
    allow_dependent_launch();
    if (threadIdx.x == 32) {
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(acc_full_bar), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)C::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    cluster_sync_all();   // every CTA of the cluster has started before any of them writes into another's shared memory
    const bool early = g.early_weights != 0;
    if (!early) grid_dependency_wait();

    const int kb0 = (int)rank * g.k_per_split, kb1 = min(g.k_iters, kb0 + g.k_per_split);   // never empty (host)
    bool ok = true;

    if (warp == 0) {
        // ---------------- producer ----------------
        const int band0 = tn;                                   // 128-column tiles: one band of B scales each
        const bool sfb_present = band0 < g.sfb_bands;
        const uint8_t* sfb_src = g.sfb + (int64_t)band0 * g.sf_cbg * SF_CHUNK_BYTES;
        auto load_weight_part = [&](int kb, int stg) {
            const uint32_t st = smem_u32(smem) + stg * C::kStageBytes;
            const uint32_t bar = smem_u32(&full_bar[0]) + stg * 8;
            const uint32_t sf_bytes = (uint32_t)min(CHUNKS, g.sf_cbg - kb * CHUNKS) * SF_CHUNK_BYTES;
            mbar_expect_tx(bar, g.a_box_bytes + C::kBBytes + (sfb_present ? 2u : 1u) * sf_bytes);
            tma_load_2d(st + C::kABytes, &tmap_b, kb * BK_BYTES, tn * 128, bar);
            if (sfb_present)
                bulk_load(st + C::kABytes + C::kBBytes + C::kSfBytes, sfb_src + (int64_t)kb * CHUNKS * SF_CHUNK_BYTES, sf_bytes, bar);
        };
        auto load_activation_part = [&](int kb, int stg) {
            const uint32_t st = smem_u32(smem) + stg * C::kStageBytes;
            const uint32_t bar = smem_u32(&full_bar[0]) + stg * 8;
            const uint32_t sf_bytes = (uint32_t)min(CHUNKS, g.sf_cbg - kb * CHUNKS) * SF_CHUNK_BYTES;
            tma_load_2d(st, &tmap_a, kb * BK_BYTES, 0, bar);
            bulk_load(st + C::kABytes + C::kBBytes, g.sfa + (int64_t)kb * CHUNKS * SF_CHUNK_BYTES, sf_bytes, bar);
        };
        int stage = 0, kb = kb0;
        uint32_t phase = 0;
        if (early) {
            // the weight's first stages before the wait for the preceding kernel, the activations after it
            const int n_pre = min(C::kStages, kb1 - kb0);
            if (elect_one())
                for (int i = 0; i < n_pre; ++i) load_weight_part(kb0 + i, i);
            __syncwarp();
            grid_dependency_wait();
            if (elect_one())
                for (int i = 0; i < n_pre; ++i) load_activation_part(kb0 + i, i);
            __syncwarp();
            kb = kb0 + n_pre;
            stage = n_pre;
            if (stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        for (; kb < kb1; ++kb) {
            ok = mbar_wait(smem_u32(&empty_bar[0]) + stage * 8, phase ^ 1, abort_flag, WAIT_STAGE_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (elect_one()) {
                load_weight_part(kb, stage);
                load_activation_part(kb, stage);
            }
            __syncwarp();
            if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int stage = 0;
        uint32_t phase = 0;
        const uint32_t smem_enc = smem_u32(smem) >> 4;
        const uint32_t sf_t0 = tmem_base + C::kSfCol0;
        for (int kb = kb0; kb < kb1; ++kb) {
            ok = mbar_wait(smem_u32(&full_bar[0]) + stage * 8, phase, abort_flag, WAIT_STAGE_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st_enc = smem_enc + stage * (C::kStageBytes >> 4);
            const uint32_t a_lo = st_enc | kOperandDescLoFlags;
            const uint32_t b_lo = a_lo + (C::kABytes >> 4);
            const uint32_t sfa_lo = st_enc + ((C::kABytes + C::kBBytes) >> 4);
            const uint32_t sfb_lo = sfa_lo + (C::kSfBytes >> 4);
            const int nchunk = min(CHUNKS, g.sf_cbg - kb * CHUNKS);
            if (elect_one()) {
#pragma unroll
                for (int j = 0; j < CHUNKS; ++j) {
                    if (j < nchunk) {
                        const uint32_t sfa_t = sf_t0 + (j >> 1) * C::kSfRegionCols + (j & 1) * 4;
                        tc_cp_sf(sfa_t, desc64(sfa_lo + j * (SF_CHUNK_BYTES >> 4), kSfDescHi));
                        tc_cp_sf(sfa_t + 8, desc64(sfb_lo + j * (SF_CHUNK_BYTES >> 4), kSfDescHi));
                    }
                }
#pragma unroll
                for (int j = 0; j < CHUNKS; ++j) {
                    if (j < nchunk) {
                        const uint32_t sfa_t = sf_t0 + (j >> 1) * C::kSfRegionCols + (j & 1) * 4;
                        tc_mma(tmem_base, desc64(a_lo + 2 * j, kOperandDescHi), desc64(b_lo + 2 * j, kOperandDescHi),
                               Cfg<128>::kIdesc, sfa_t, sfa_t + 8, (j != 0 || kb != kb0) ? 1u : 0u);
                    }
                }
                tc_commit(smem_u32(&empty_bar[0]) + stage * 8);
            }
            __syncwarp();
            if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok && elect_one()) tc_commit(smem_u32(acc_full_bar));
        __syncwarp();
    }

    // ---------------- epilogue, part 1 (warps whose tensor-memory lanes hold existing rows) ----------------
    const int quad = warp & 3;
    const bool epi = warp >= 2 && quad * 32 < AROWS;
    const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16);
    const int row = quad * 32 + lane;
    if (epi) {
        if (early) grid_dependency_wait();   // before tensor scales and bias are read and anything is stored
        ok = mbar_wait(smem_u32(acc_full_bar), 0, abort_flag, WAIT_ACC_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
#pragma unroll 1
            for (int s = 0; s < 4; ++s) {
                const uint32_t owner = (uint32_t)(s / C::kStepsOwned);
                if (owner == rank) continue;
                uint32_t v[32];
                tc_ld32(t_acc + s * EPI_COLS, v);
                tc_wait_ld();
                // slot of this sender in the owner's exchange area: senders in rank order, the owner left out
                const uint32_t slot = rank < owner ? rank : rank - 1;
                const uint32_t local = smem_u32(exchange) + slot * C::kSlotBytes +
                                       (uint32_t)row * (C::kStepsOwned * EPI_COLS * 4) + (uint32_t)(s % C::kStepsOwned) * (EPI_COLS * 4);
                const uint32_t remote = map_to_cta(local, owner);
#pragma unroll
                for (int j = 0; j < 8; ++j) st_cluster_v4(remote + 16 * j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
        }
    }
    // Every thread of every CTA of the cluster, whatever happened above: partial sums delivered and visible.
    cluster_sync_all();
    // ---------------- epilogue, part 2: add up the owned steps in rank order, scale, store ----------------
    if (epi && ok && !*abort_flag) {
        const float alpha = g.alpha ? __ldg(g.alpha) : __fmul_rn(__ldg(g.tsa), __ldg(g.tsb));
#pragma unroll 1
        for (int so = 0; so < C::kStepsOwned; ++so) {
            const int s = (int)rank * C::kStepsOwned + so;
            uint32_t own[32];
            tc_ld32(t_acc + s * EPI_COLS, own);
            tc_wait_ld();
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.f;
#pragma unroll
            for (int src = 0; src < CS; ++src) {
                if ((uint32_t)src == rank) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] += __uint_as_float(own[i]);
                } else {
                    const uint32_t slot = (uint32_t)src < rank ? (uint32_t)src : (uint32_t)src - 1;
                    const float4* p = reinterpret_cast<const float4*>(exchange + slot * C::kSlotBytes +
                                                                      row * (C::kStepsOwned * EPI_COLS * 4) + so * (EPI_COLS * 4));
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 t = p[j];
                        acc[4 * j] += t.x; acc[4 * j + 1] += t.y; acc[4 * j + 2] += t.z; acc[4 * j + 3] += t.w;
                    }
                }
            }
            const int n0 = tn * 128 + s * EPI_COLS;
            if (row < g.M && n0 < g.N) {
                uint32_t bits[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) bits[i] = __float_as_uint(acc[i]);
                float y[32];
                scale_row32(g, n0, bits, alpha, y);
                store_row32(g, row, n0, y);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
                     : "memory");
    }
}

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, int splits, int M, int N,
                                                            const float* tsa, const float* tsb, const float* alpha_ptr,
                                                            const void* bias, int bias_dtype, void* out, int out_dtype) {
    allow_dependent_launch();
    const int64_t quads = (int64_t)M * N / 4;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= quads) return;
    grid_dependency_wait();
    const float alpha = alpha_ptr ? __ldg(alpha_ptr) : __fmul_rn(__ldg(tsa), __ldg(tsb));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(partial) + (int64_t)s * quads + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float y[4] = {acc.x * alpha, acc.y * alpha, acc.z * alpha, acc.w * alpha};
    const int n = (int)((i * 4) % N);
    if (bias) {
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] += bias_at(bias, bias_dtype, n + j);
    }
    if (out_dtype == CK_B200_DTYPE_F32) {
        reinterpret_cast<float4*>(out)[i] = make_float4(y[0], y[1], y[2], y[3]);
    } else {
        uint2 o;
        o.x = pack16(y[0], y[1], out_dtype);
        o.y = pack16(y[2], y[3], out_dtype);
        reinterpret_cast<uint2*>(out)[i] = o;
    }
}

// ---- host side --------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// Packed operand [rows, k_bytes] row-major, boxes of 128 bytes x box_rows rows, 128-byte swizzle, zero fill.
int make_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t k_bytes, int box_rows,
                     int box_bytes = BK_BYTES) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)k_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled (operand) failed with CUresult %d", (int)r);
    return CK_B200_OK;
}

// Tensor maps of operands that stay where they are over many calls (a resident weight and its scales) are kept in a
// small per-process table keyed by kind, address, shape and box, so the driver call happens once per weight.  A map
// only describes memory (base, extents, strides), so a stale entry for a freed and reused address is still a valid
// description of whatever matrix of that shape now lives there.
template <typename Build>
int cached_map(CUtensorMap* map, int kind, const void* ptr, int64_t d0, int64_t d1, int b0, int b1, Build build) {
    struct Entry {
        const void* ptr;
        int64_t d0, d1;
        int b0, b1, dev, kind;
        CUtensorMap map;
    };
    constexpr int kEntries = 512;
    static std::mutex mu;
    static Entry table[kEntries] = {};
    int dev = 0;
    CKB_CUDA_OK(cudaGetDevice(&dev));
    const size_t h = ((((uint64_t)reinterpret_cast<uintptr_t>(ptr) >> 8) + (uint64_t)kind) * 0x9E3779B97F4A7C15ull >> 40) % kEntries;
    {
        std::lock_guard<std::mutex> lock(mu);
        const Entry& e = table[h];
        if (e.ptr == ptr && e.d0 == d0 && e.d1 == d1 && e.b0 == b0 && e.b1 == b1 && e.dev == dev && e.kind == kind) {
            *map = e.map;
            return CK_B200_OK;
        }
    }
    if (int rc = build()) return rc;
    std::lock_guard<std::mutex> lock(mu);
    table[h] = Entry{ptr, d0, d1, b0, b1, dev, kind, *map};
    return CK_B200_OK;
}
int cached_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t k_bytes, int box_rows, int box_bytes = BK_BYTES) {
    return cached_map(map, 1, ptr, rows, k_bytes, box_rows, box_bytes,
                      [&] { return make_operand_map(map, ptr, rows, k_bytes, box_rows, box_bytes); });
}

// 16-bit output [M, N] row-major, boxes of 32 columns (64 bytes) x 32 rows, 64-byte swizzle.
int make_output_map(CUtensorMap* map, void* ptr, int64_t M, int64_t N, int64_t ld) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)EPI_COLS, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
    return CK_B200_OK;
}

// Tiled scale tensor seen as [chunks, 128 x u32] (one 512-byte chunk per row), boxes of box_chunks chunks, no swizzle.
int make_scale_map(CUtensorMap* map, const void* ptr, int64_t chunks, int box_chunks) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {128, (cuuint64_t)chunks};
    cuuint64_t strides[1] = {(cuuint64_t)SF_CHUNK_BYTES};
    cuuint32_t box[2] = {128, (cuuint32_t)box_chunks};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with CUresult %d", (int)r);
    return CK_B200_OK;
}

int cached_scale_map(CUtensorMap* map, const void* ptr, int64_t chunks, int box_chunks) {
    return cached_map(map, 2, ptr, chunks, 0, box_chunks, 0, [&] { return make_scale_map(map, ptr, chunks, box_chunks); });
}

// Pairs of CTAs that can be resident at once (clusters of 2 need two free SMs of one GPC), cached per device.
template <int KB, int QDT = -1, bool GATHER = false>
int max_active_pairs(int* out) {
    constexpr int kSmemBytes2 = PairCfg<KB, GATHER>::kSmemBytes;
    constexpr int kThreads = QDT >= 0 ? NUM_THREADS + kQuantWarps * 32 : NUM_THREADS;
    static std::mutex mu;
    static int cache[64] = {0};
    int dev = 0, sms = 0;
    CKB_CUDA_OK(cudaGetDevice(&dev));
    if (int rc = check_device(&sms)) return rc;   // also bounds the device ordinal
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == 0) {
        auto kernel = gemm_nvfp4_pair_kernel<KB, false, 0, QDT, GATHER>;
        CKB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes2));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)sms);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kSmemBytes2;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        CKB_CUDA_OK(cudaOccupancyMaxActiveClusters(&n, (const void*)kernel, &cfg));
        cache[dev] = n > 0 ? n : -1;
    }
    if (cache[dev] < 0) return fail(CK_B200_ERR_CUDA, "no CTA pair of the GEMM kernel fits on this device");
    *out = cache[dev];
    return CK_B200_OK;
}

// QDT >= 0: the kernel also quantizes the activations described by *fused (dtype code QDT) into `a` and g.sfa.
template <int KB, int FMT = 0, int QDT = -1, bool GATHER = false>
int launch_gemm_pair(const void* a, const void* b, GemmArgs g, int64_t K, cudaStream_t stream,
                     const FusedQuant* fused = nullptr) {
    using P = PairCfg<KB, GATHER>;
    constexpr int kSmemBytes2 = P::kSmemBytes;
    constexpr int kSfChunks = FMT == 1 ? 1 : P::kChunks;
    constexpr int kThreads = QDT >= 0 ? NUM_THREADS + kQuantWarps * 32 : NUM_THREADS;
    const int64_t row_bytes = FMT == 1 ? K : K / 2;
    auto kernel = g.debug ? gemm_nvfp4_pair_kernel<KB, true, FMT, QDT, GATHER> : gemm_nvfp4_pair_kernel<KB, false, FMT, QDT, GATHER>;
    int pairs = 0;
    if (int rc = max_active_pairs<KB, QDT, GATHER>(&pairs)) return rc;
    FusedQuant fq{};
    if (QDT >= 0) {
        if (!fused) return fail(CK_B200_ERR_INVALID_ARGUMENT, "fused quantizer: missing description");
        fq = *fused;
    }
    {
        // opting in to large dynamic shared memory is per function (this template instance, with or without counters)
        // and per device: once
        static std::mutex mu;
        static bool done[2][64] = {};
        int dev = 0;
        CKB_CUDA_OK(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !done[g.debug ? 1 : 0][dev]) {
            cudaError_t attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes2);
            if (attr_err != cudaSuccess)
                return fail(CK_B200_ERR_CUDA, "cudaFuncSetAttribute(shared memory %d) failed: %s", kSmemBytes2,
                            cudaGetErrorString(attr_err));
            if (dev >= 0 && dev < 64) done[g.debug ? 1 : 0][dev] = true;
        }
    }
    CUtensorMap ma, mb, msa, msb, mo;
    if (int rc = make_operand_map(&ma, a, g.M, row_bytes, BM, KB)) return rc;
    if (int rc = cached_operand_map(&mb, b, g.N, row_bytes, 128, KB)) return rc;   // the resident weight and its scales
    if (int rc = make_scale_map(&msa, g.sfa, ceil_div64(g.M, 128) * g.sf_cbg, kSfChunks)) return rc;
    if (int rc = cached_scale_map(&msb, g.sfb, ceil_div64(g.N, 128) * g.sf_cbg, kSfChunks)) return rc;
    g.tma_store = (g.out_dtype != CK_B200_DTYPE_F32 && !GATHER) ? 1 : 0;   // GATHER copies rows out itself
    if (g.tma_store) {
        if (int rc = make_output_map(&mo, g.out, g.M, g.N, g.ld_out)) return rc;
    } else {
        mo = ma;   // not used by the kernel
    }
    g.m_tiles = (int)ceil_div64(g.M, 256);
    g.n_tiles = (int)ceil_div64(g.N, 256);
    const int64_t row_block_bytes = 256ll * row_bytes;
    int64_t group = (8ll << 20) / (row_block_bytes > 0 ? row_block_bytes : 1);
    if (group < 4) group = 4;
    g.raster_group = (int)(group < g.m_tiles ? group : g.m_tiles);
    // with the quantizer inside, tiles go row block by row block: the first wave then waits for a few bands only.
    // Delivering tiles to the other ranks: row block by row block too, so that at any time the stores of all CTAs fall
    // into a few megabytes of each peer's matrix.  Peer-mapped memory is translated in 2 MiB pages and the translation
    // cache covers a few GiB: walking all rows once per tile column touched every page again and again, and once the
    // matrices mapped from the peers exceeded that reach the stores fell from ~500 to below 100 GB/s.
    if (QDT >= 0 || GATHER) g.raster_group = 1;
    g.splits = 1;
    g.k_per_split = g.k_iters;
    g.partial = nullptr;
    g_last_splits.store(1);
    const int64_t tiles = (int64_t)g.m_tiles * g.n_tiles;
    // a caller that runs two of these kernels side by side (two streams) gives each a share of the CTA pairs
    const int cap = g_gemm_max_pairs.load();
    if (cap > 0 && cap < pairs) pairs = cap;
    const unsigned grid = 2u * (unsigned)(tiles < pairs ? tiles : pairs);
    const cudaError_t err = launch_dependent(kLaunchFamilyGemm, kernel, dim3(grid), dim3(kThreads), kSmemBytes2, stream, ma, mb, msa, msb, mo, g, fq);
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
    return CK_B200_OK;
}

// Split-K factor for a problem with one tile row (M <= 128): as many work items as SMs, at least two stages per
// item, and partial sums that fit the scratch buffer.
int choose_splits(int n_tiles, int k_iters, int sms, int64_t M, int64_t N, size_t scratch_bytes) {
    int s = sms / (n_tiles > 0 ? n_tiles : 1);
    if (s > k_iters / 2) s = k_iters / 2;
    if (s > 16) s = 16;
    while (s > 1 && (size_t)s * (size_t)M * (size_t)N * 4 > scratch_bytes) --s;
    return s < 1 ? 1 : s;
}

// Scratch of a split-K launch: room for the fp32 partial sums.
struct SplitScratch {
    float* partial = nullptr;
    size_t partial_bytes = 0;
};

template <int BN, int FMT = 0, int AROWS = BM>
int launch_gemm(const void* a, const void* b, GemmArgs g, int64_t K, int sms, cudaStream_t stream, SplitScratch scratch) {
    using C = Cfg<BN, AROWS>;
    auto kernel = g.debug ? gemm_nvfp4_kernel<BN, true, FMT, AROWS> : gemm_nvfp4_kernel<BN, false, FMT, AROWS>;
    if (AROWS < BM && g.M > AROWS) return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm: %d rows do not fit this tile configuration", g.M);
    const int capacity = sms * C::kCtasPerSm;   // CTAs resident at once
    const int64_t row_bytes = FMT == 1 ? K : K / 2;   // e4m3 bytes or packed e2m1 nibbles
    // opting in to large dynamic shared memory is per function and per device: once
    {
        static std::mutex mu;
        static bool done[2][64] = {};
        int dev = 0;
        CKB_CUDA_OK(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !done[g.debug ? 1 : 0][dev]) {
            cudaError_t attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
            if (attr_err != cudaSuccess)
                return fail(CK_B200_ERR_CUDA, "cudaFuncSetAttribute(shared memory %d) failed: %s", C::kSmemBytes,
                            cudaGetErrorString(attr_err));
            // all of the SM's configurable memory as shared memory, so that kCtasPerSm CTAs fit
            if (C::kCtasPerSm > 1)
                CKB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            if (dev >= 0 && dev < 64) done[g.debug ? 1 : 0][dev] = true;
        }
    }
    CUtensorMap ma, mb, mo;
    const int a_box_rows = g.M <= 32 ? 32 : g.M <= 64 ? 64 : BM;   // never more than AROWS (checked above)
    g.a_box_bytes = a_box_rows * BK_BYTES;
    if (int rc = make_operand_map(&ma, a, g.M, row_bytes, a_box_rows)) return rc;
    if (int rc = cached_operand_map(&mb, b, g.N, row_bytes, BN)) return rc;   // the weight: the same matrix call after call
    g.m_tiles = (int)ceil_div64(g.M, BM);
    g.n_tiles = (int)ceil_div64(g.N, BN);
    // as many tile rows per group as keep the group's A rows (with room for B and the output) inside the 126 MB L2
    const int64_t row_block_bytes = (int64_t)BM * row_bytes;
    int64_t group = (8ll << 20) / (row_block_bytes > 0 ? row_block_bytes : 1);
    if (group < 8) group = 8;
    g.raster_group = (int)(group < g.m_tiles ? group : g.m_tiles);
    g.splits = 1;
    g.k_per_split = g.k_iters;
    g.partial = nullptr;
    g.early_weights = (g.m_tiles == 1 && g_weights_resident.load() != 0) ? 1 : 0;
    if (g.m_tiles == 1 && scratch.partial != nullptr) {
        g.splits = choose_splits(g.n_tiles, g.k_iters, capacity, g.M, g.N, scratch.partial_bytes);
        if (g.splits > 1) {
            g.k_per_split = (int)ceil_div64(g.k_iters, g.splits);
            g.splits = (int)ceil_div64(g.k_iters, g.k_per_split);   // no empty work items
        }
        if (g.splits > 1) g.partial = scratch.partial;
    }
    // split-K items write fp32 partial sums and the reduction kernel stores the output: no output map
    g.tma_store = (g.out_dtype != CK_B200_DTYPE_F32 && g.splits == 1) ? 1 : 0;
    if (g.tma_store) {
        if (int rc = make_output_map(&mo, g.out, g.M, g.N, g.ld_out)) return rc;
    } else {
        mo = ma;   // not used by the kernel
    }
    g_last_splits.store(g.splits);
    const int64_t items = (int64_t)g.m_tiles * g.n_tiles * g.splits;
    const unsigned grid = (unsigned)(items < capacity ? items : capacity);
    const cudaError_t err = launch_dependent(kLaunchFamilyGemm, kernel, dim3(grid), dim3(NUM_THREADS), C::kSmemBytes, stream, ma, mb, mo, g);
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
    if (g.splits > 1) {
        const int64_t quads = (int64_t)g.M * g.N / 4;
        const cudaError_t err2 = launch_dependent(kLaunchFamilyGemm, splitk_reduce_kernel, dim3((unsigned)ceil_div64(quads, 256)), dim3(256), 0,
                                                  stream, g.partial, g.splits, g.M, g.N, g.tsa, g.tsb, g.alpha, g.bias,
                                                  g.bias_dtype, g.out, g.out_dtype);
        g_launches.fetch_add(1);
        CKB_CUDA_OK(err2);
    }
    return CK_B200_OK;
}


// M <= 64 on clusters that split K (gemm_nvfp4_cluster_kernel).  Returns CK_B200_OK with *taken = false when the
// shape does not suit it (the caller then takes the other small-M paths).
template <int AROWS, int CS>
int launch_gemm_cluster(const void* a, const void* b, GemmArgs g, int64_t K, cudaStream_t stream) {
    using C = ClusterCfg<AROWS, CS>;
    auto kernel = gemm_nvfp4_cluster_kernel<AROWS, CS>;
    {
        static std::mutex mu;
        static bool done[64] = {};
        int dev = 0;
        CKB_CUDA_OK(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !done[dev]) {
            CKB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
            CKB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            if (dev >= 0 && dev < 64) done[dev] = true;
        }
    }
    const int64_t row_bytes = K / 2;
    CUtensorMap ma, mb;
    g.a_box_bytes = AROWS * BK_BYTES;
    if (int rc = make_operand_map(&ma, a, g.M, row_bytes, AROWS)) return rc;
    if (int rc = cached_operand_map(&mb, b, g.N, row_bytes, 128)) return rc;
    g.m_tiles = 1;
    g.n_tiles = (int)ceil_div64(g.N, 128);
    g.raster_group = 1;
    g.splits = CS;
    g.k_per_split = (int)ceil_div64(g.k_iters, CS);
    g.partial = nullptr;
    g.tma_store = 0;
    g.early_weights = g_weights_resident.load() != 0 ? 1 : 0;
    g_last_splits.store(CS);
    const cudaError_t err = launch_dependent(kLaunchFamilyGemm, kernel, dim3((unsigned)(g.n_tiles * CS)), dim3(NUM_THREADS),
                                             C::kSmemBytes, stream, ma, mb, g);
    g_launches.fetch_add(1);
    CKB_CUDA_OK(err);
    return CK_B200_OK;
}

// Cluster size for a one-tile-row problem: the largest of 4 and 2 whose CTAs are all resident at once (two per SM)
// and get at least two stages each with no empty rank; 0 = none.
int choose_cluster_split(int64_t N, int k_iters, int sms) {
    const int64_t tiles = ceil_div64(N, 128);
    for (int cs = 4; cs >= 2; cs /= 2) {
        const int per = (int)ceil_div64(k_iters, cs);
        if (tiles * cs <= 2ll * sms && per >= 2 && (int64_t)(cs - 1) * per < k_iters) return cs;
    }
    return 0;
}

}  // namespace
}  // namespace ckb

using namespace ckb;

namespace {
// Where a fused all-gather sends the output besides `out_dev`: the column block's origin in every other rank's matrix.
struct GatherSpec {
    int64_t ld;
    int n_peers;
    uint8_t* peers[7];
};

int scaled_mm_impl(const void* a_dev, const void* sfa_dev, const void* b_dev, const void* sfb_dev,
                   const float* tensor_scale_a_dev, const float* tensor_scale_b_dev, const float* alpha_dev_or_null,
                   const void* bias_dev_or_null, int bias_dtype, void* out_dev, int out_dtype, int64_t M, int64_t N,
                   int64_t K, SplitScratch scratch, void* stream,
                   const GatherSpec* gather = nullptr, const FusedQuant* fused = nullptr, int fused_dtype = -1,
                   bool force_scratch = false) {
    int sms = 0;
    if (int rc = check_device(&sms)) return rc;
    if (!a_dev || !sfa_dev || !b_dev || !sfb_dev || !out_dev)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: null pointer");
    if (!alpha_dev_or_null && (!tensor_scale_a_dev || !tensor_scale_b_dev))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: need both tensor scales or alpha");
    if (M < 0 || N < 0 || K < 0) return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: negative shape");
    if (K % 32 != 0)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: K = %lld must be a multiple of 32", (long long)K);
    if (N % 8 != 0)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: N = %lld must be a multiple of 8", (long long)N);
    if (out_dtype < 0 || out_dtype > 2 || (bias_dev_or_null && (bias_dtype < 0 || bias_dtype > 2)))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: bad dtype code");
    if (M > 0x7fffff00ll || N > 0x7fffff00ll || K > 0x7fffff00ll)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: dimension too large");
    if (((uintptr_t)a_dev & 15) || ((uintptr_t)b_dev & 15) || ((uintptr_t)sfa_dev & 15) || ((uintptr_t)sfb_dev & 15) ||
        ((uintptr_t)out_dev & 15))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: operands, scales and output must be 16-byte aligned");
    if (M == 0 || N == 0) return CK_B200_OK;
    if (K == 0) return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: K must be positive");

    GemmArgs g;
    g.sfa = (const uint8_t*)sfa_dev;
    g.sfb = (const uint8_t*)sfb_dev;
    g.tsa = tensor_scale_a_dev;
    g.tsb = tensor_scale_b_dev;
    g.alpha = alpha_dev_or_null;
    g.bias = bias_dev_or_null;
    g.out = out_dev;
    g.bias_dtype = bias_dtype;
    g.out_dtype = out_dtype;
    g.M = (int)M;
    g.N = (int)N;
    g.sf_cbg = (int)ceil_div64(K, 64);
    g.sfb_bands = (int)ceil_div64(N, 128);
    g.k_iters = (int)ceil_div64(K, 256);
    g.m_tiles = g.n_tiles = 0;
    g.splits = 1;
    g.k_per_split = g.k_iters;
    g.partial = nullptr;
    g.a_box_bytes = BM * BK_BYTES;
    g.raster_group = 1;
    g.tma_store = 0;
    g.ld_out = N;
    g.n_peers = 0;
    for (int p = 0; p < 7; ++p) g.peer_out[p] = nullptr;
    g.debug = g_gemm_debug.load();
    g.early_weights = 0;
    int variant = g_gemm_variant.load();
    // CTA pairs with 256x256 tiles when the problem has more than one tile row and column; otherwise one CTA per
    // tile, 128x256 (half the operand traffic per flop of 128x128) unless N is a single 128-column tile
    // variant 5 = the short-row configuration where it applies (M <= 64), the automatic choice elsewhere
    // (automatic: when the 64-column tiles alone fill the SMs, so that K is not split - measured on M = 16: with fewer
    // tiles the 128-column configuration and its smaller number of K splits is equal or 3-4 % faster)
    const bool skinny = M <= 64 && (variant == 5 || (variant == 0 && g_gemm_skinny.load() != 0 && N >= 64ll * sms));
    // variant 6 = K split over a thread-block cluster, partial sums exchanged through shared memory (M <= 64, 16-byte
    // aligned rows of packed K)
    int cluster_split = 0;
    if (M <= 64 && K % 32 == 0 && (variant == 6 || (variant == 0 && g_gemm_cluster_split.load() != 0)) && !force_scratch)
        cluster_split = choose_cluster_split(N, g.k_iters, sms);
    if (variant == 0 || variant == 5 || variant == 6) variant = (M > 128 && N > 128) ? 3 : (N > 128) ? 2 : 1;
    cudaStream_t s = (cudaStream_t)stream;
    if ((uintptr_t)scratch.partial & 15)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4: workspace must be 16-byte aligned");
    if (gather) {
        if (out_dtype == CK_B200_DTYPE_F32 || M <= 128 || N <= 128)
            return fail(CK_B200_ERR_INVALID_ARGUMENT,
                        "scaled_mm_nvfp4_all_gather: needs a 16-bit output, M > 128 and more than 128 local columns");
        g.ld_out = gather->ld;
        g.n_peers = gather->n_peers;
        for (int p = 0; p < gather->n_peers; ++p) g.peer_out[p] = gather->peers[p];
        return launch_gemm_pair<128, 0, -1, true>(a_dev, b_dev, g, K, s);
    }
    if (fused) {
        if (M <= 128 || N <= 128)
            return fail(CK_B200_ERR_INVALID_ARGUMENT, "fused quantizer: needs M > 128 and N > 128");
        if (fused_dtype == CK_B200_DTYPE_BF16)
            return launch_gemm_pair<128, 0, CK_B200_DTYPE_BF16>(a_dev, b_dev, g, K, s, fused);
        if (fused_dtype == CK_B200_DTYPE_F16)
            return launch_gemm_pair<128, 0, CK_B200_DTYPE_F16>(a_dev, b_dev, g, K, s, fused);
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "fused quantizer: activations must be bf16 or fp16");
    }
    if (variant == 4 && M > 128) return launch_gemm_pair<64>(a_dev, b_dev, g, K, s);
    if (variant == 3 && M > 128) return launch_gemm_pair<128>(a_dev, b_dev, g, K, s);
    if (variant == 2 && M > 128) return launch_gemm<256>(a_dev, b_dev, g, K, sms, s, scratch);
    // one short tile row: 64-column tiles, two CTAs per SM (every SM streams its share of the weight from the start)
    if (cluster_split == 2 && M <= 32) return launch_gemm_cluster<32, 2>(a_dev, b_dev, g, K, s);
    if (cluster_split == 2 && M <= 64) return launch_gemm_cluster<64, 2>(a_dev, b_dev, g, K, s);
    if (cluster_split == 4 && M <= 32) return launch_gemm_cluster<32, 4>(a_dev, b_dev, g, K, s);
    if (cluster_split == 4 && M <= 64) return launch_gemm_cluster<64, 4>(a_dev, b_dev, g, K, s);
    if (skinny && M <= 32) return launch_gemm<64, 0, 32>(a_dev, b_dev, g, K, sms, s, scratch);
    if (skinny && M <= 64) return launch_gemm<64, 0, 64>(a_dev, b_dev, g, K, sms, s, scratch);
    // one tile row: 128-column tiles give the most work items, and split-K (with scratch) fills the remaining SMs
    return launch_gemm<128>(a_dev, b_dev, g, K, sms, s, scratch);
}

SplitScratch scratch_from_workspace(void* workspace_dev, size_t workspace_bytes) {
    SplitScratch sc;
    if (workspace_dev && workspace_bytes > 0) {
        sc.partial = (float*)workspace_dev;
        sc.partial_bytes = workspace_bytes;
    }
    return sc;
}
}  // namespace

extern "C" int ck_b200_scaled_mm_nvfp4(const void* a_dev, const void* sfa_dev, const void* b_dev, const void* sfb_dev,
                                       const float* tensor_scale_a_dev, const float* tensor_scale_b_dev,
                                       const float* alpha_dev_or_null, const void* bias_dev_or_null, int bias_dtype,
                                       void* out_dev, int out_dtype, int64_t M, int64_t N, int64_t K, void* workspace_dev,
                                       size_t workspace_bytes, void* stream) {
    return scaled_mm_impl(a_dev, sfa_dev, b_dev, sfb_dev, tensor_scale_a_dev, tensor_scale_b_dev, alpha_dev_or_null,
                          bias_dev_or_null, bias_dtype, out_dev, out_dtype, M, N, K,
                          scratch_from_workspace(workspace_dev, workspace_bytes), stream);
}



// ---- GEMM that quantizes its own activations -------------------------------------------------------------

namespace ckb {
constexpr size_t kFusedSyncBytes = 32768;
constexpr int64_t kFusedMaxBands = (int64_t)(kFusedSyncBytes - sizeof(FusedQuantSync)) / 4;
size_t fused_sync_bytes() { return kFusedSyncBytes; }

bool fused_linear_supported(int x_dtype, const void* x_dev, int64_t M, int64_t N, int64_t K, int out_dtype) {
    return (x_dtype == CK_B200_DTYPE_BF16 || x_dtype == CK_B200_DTYPE_F16) && M > 128 && N > 128 && K % 32 == 0 &&
           K >= 384 && (((uintptr_t)x_dev & 15) == 0) && ceil_div64(M, 128) <= kFusedMaxBands && K < 0x3fffff00ll &&
           out_dtype >= 0;
}

int fused_linear_launch(const void* x_dev, int x_dtype, int64_t M, int64_t K, const float* ts_x_dev, void* qx_dev,
                        void* sfx_dev, void* sync_dev, const void* w_q_dev, const void* w_sf_dev,
                        const float* w_scale_dev, int64_t N, const void* bias_dev_or_null, int bias_dtype, void* out_dev,
                        int out_dtype, void* stream) {
    if (!x_dev || !ts_x_dev || !qx_dev || !sfx_dev || !sync_dev || ((uintptr_t)sync_dev & 3))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "fused linear: null or misaligned pointer");
    FusedQuant fq;
    QuantArgs& a = fq.q;
    a.x = x_dev;
    a.pts = ts_x_dev;
    a.q = (uint8_t*)qx_dev;
    a.sf = (uint8_t*)sfx_dev;
    a.rows = (int)M;
    a.cols = (int)K;
    a.prow = (int)round_up64(M, 16);
    a.pcol = (int)K;   // K % 32 == 0
    a.row_groups = (int)(round_up64(a.prow, 128) / 4);
    a.sf_cbg = (int)(round_up64(K / 16, 4) / 4);
    // about eight segments per row, each an even number of units and at least one prefetch ring long: short
    // enough that the bands finish one after the other, in the order in which the tiles need them
    int su = (int)round_up64(ceil_div64(a.sf_cbg, 8), 2);
    if (su < kRing) su = kRing;
    a.seg_units = su;
    a.segments = (int)ceil_div64(a.sf_cbg, su);
    a.hi_first = 1;
    fq.sync = (FusedQuantSync*)sync_dev;
    fq.bands = a.row_groups / 32;
    return scaled_mm_impl(qx_dev, sfx_dev, w_q_dev, w_sf_dev, ts_x_dev, w_scale_dev, nullptr, bias_dev_or_null,
                          bias_dtype, out_dev, out_dtype, M, N, K, SplitScratch{}, stream, nullptr, &fq, x_dtype);
}
}  // namespace ckb

// ---- GEMM fused with the all-gather of its column blocks ----------------------------------------------

extern "C" int ck_b200_scaled_mm_nvfp4_all_gather(const void* a_dev, const void* sfa_dev, const void* b_dev,
                                                  const void* sfb_dev, const float* tensor_scale_a_dev,
                                                  const float* tensor_scale_b_dev, const float* alpha_dev_or_null,
                                                  const void* bias_dev_or_null, int bias_dtype, void* const* out_ptrs,
                                                  int world, int rank, int out_dtype, int64_t M, int64_t N_local,
                                                  int64_t K, void* stream) {
    if (!out_ptrs || world < 1 || world > 8 || rank < 0 || rank >= world)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4_all_gather: need 1..8 ranks and 0 <= rank < world");
    if (N_local < 0 || N_local % 8 != 0)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4_all_gather: N_local must be a multiple of 8");
    GatherSpec spec;
    spec.ld = (int64_t)world * N_local;
    spec.n_peers = 0;
    const int64_t block_bytes = (int64_t)rank * N_local * 2;   // 16-bit outputs only
    for (int r = 0; r < world; ++r) {
        if (!out_ptrs[r] || ((uintptr_t)out_ptrs[r] & 15))
            return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_nvfp4_all_gather: output %d is null or not 16-byte aligned", r);
        // start with the rank after this one so that the ranks do not all write to the same peer at once
        const int peer = (rank + 1 + r) % world;
        if (peer != rank) spec.peers[spec.n_peers++] = (uint8_t*)out_ptrs[peer] + block_bytes;
    }
    void* own = (uint8_t*)out_ptrs[rank] + block_bytes;
    return scaled_mm_impl(a_dev, sfa_dev, b_dev, sfb_dev, tensor_scale_a_dev, tensor_scale_b_dev, alpha_dev_or_null,
                          bias_dev_or_null, bias_dtype, own, out_dtype, M, N_local, K, SplitScratch{}, stream, &spec);
}

// ---- barrier between the ranks of one node ------------------------------------------------------------

extern "C" int ck_b200_peer_barrier(void* const* flag_ptrs, int world, int rank, void* epoch_dev, void* stream) {
    if (int rc = check_device(nullptr)) return rc;
    if (!flag_ptrs || !epoch_dev || world < 1 || world > 8 || rank < 0 || rank >= world)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "peer_barrier: need 1..8 ranks, 0 <= rank < world and non-null pointers");
    BarrierArgs b;
    for (int r = 0; r < 8; ++r) b.flags[r] = r < world ? (uint32_t*)flag_ptrs[r] : nullptr;
    for (int r = 0; r < world; ++r)
        if (!b.flags[r] || ((uintptr_t)b.flags[r] & 3))
            return fail(CK_B200_ERR_INVALID_ARGUMENT, "peer_barrier: flag array %d is null or misaligned", r);
    b.epoch = (uint32_t*)epoch_dev;
    b.world = world;
    b.rank = rank;
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(b);
    g_launches.fetch_add(1);
    CKB_CUDA_OK(cudaGetLastError());
    return CK_B200_OK;
}

// ---- MXFP8 GEMM ----------------------------------------------------------------------------------------

namespace {
static __device__ float g_unit_alpha = 1.0f;   // MXFP8 has no per-tensor scales: the epilogue multiplies by this

int unit_alpha_address(const float** out) {
    static std::mutex mu;
    static void* cache[64] = {nullptr};
    int dev = 0;
    CKB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(CK_B200_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_unit_alpha);
        if (e != cudaSuccess || p == nullptr)
            return fail(CK_B200_ERR_CUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        cache[dev] = p;
    }
    *out = reinterpret_cast<const float*>(cache[dev]);
    return CK_B200_OK;
}
}  // namespace

extern "C" int ck_b200_scaled_mm_mxfp8(const void* a_dev, const void* sfa_dev, const void* b_dev, const void* sfb_dev,
                                       const void* bias_dev_or_null, int bias_dtype, void* out_dev, int out_dtype,
                                       int64_t M, int64_t N, int64_t K, void* workspace_dev, size_t workspace_bytes,
                                       void* stream) {
    int sms = 0;
    if (int rc = check_device(&sms)) return rc;
    if (!a_dev || !sfa_dev || !b_dev || !sfb_dev || !out_dev)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_mxfp8: null pointer");
    if (M < 0 || N < 0 || K < 0 || M > 0x7fffff00ll || N > 0x7fffff00ll || K > 0x7fffff00ll)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_mxfp8: bad shape");
    if (K % 32 != 0 || N % 8 != 0)
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_mxfp8: K = %lld must be a multiple of 32 and N = %lld of 8",
                    (long long)K, (long long)N);
    if (out_dtype < 0 || out_dtype > 2 || (bias_dev_or_null && (bias_dtype < 0 || bias_dtype > 2)))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_mxfp8: bad dtype code");
    if (((uintptr_t)a_dev & 15) || ((uintptr_t)b_dev & 15) || ((uintptr_t)sfa_dev & 15) || ((uintptr_t)sfb_dev & 15) ||
        ((uintptr_t)out_dev & 15) || ((uintptr_t)workspace_dev & 15))
        return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_mxfp8: operands, scales, output and workspace must be 16-byte aligned");
    if (M == 0 || N == 0) return CK_B200_OK;
    if (K == 0) return fail(CK_B200_ERR_INVALID_ARGUMENT, "scaled_mm_mxfp8: K must be positive");
    const float* one = nullptr;
    if (int rc = unit_alpha_address(&one)) return rc;
    GemmArgs g;
    g.sfa = (const uint8_t*)sfa_dev;
    g.sfb = (const uint8_t*)sfb_dev;
    g.tsa = g.tsb = nullptr;
    g.alpha = one;
    g.bias = bias_dev_or_null;
    g.out = out_dev;
    g.bias_dtype = bias_dtype;
    g.out_dtype = out_dtype;
    g.M = (int)M;
    g.N = (int)N;
    g.sf_cbg = (int)ceil_div64(K, 128);    // one 512-byte chunk = 128 rows x 4 blocks of 32 elements
    g.sfb_bands = (int)ceil_div64(N, 128);
    g.k_iters = (int)ceil_div64(K, 128);   // 128 elements = 128 bytes of K per stage
    g.m_tiles = g.n_tiles = 0;
    g.splits = 1;
    g.k_per_split = g.k_iters;
    g.partial = nullptr;
    g.a_box_bytes = BM * BK_BYTES;
    g.raster_group = 1;
    g.tma_store = 0;
    g.ld_out = N;
    g.n_peers = 0;
    for (int p = 0; p < 7; ++p) g.peer_out[p] = nullptr;
    g.debug = g_gemm_debug.load();
    cudaStream_t s = (cudaStream_t)stream;
    const SplitScratch scratch = scratch_from_workspace(workspace_dev, workspace_bytes);
    // the same choice of tiles as the NVFP4 entry point; variants 1 and 2 force the 1-CTA kernels
    int variant = g_gemm_variant.load();
    if (variant == 0 || variant > 3) variant = (M > 128 && N > 128) ? 3 : (N > 128) ? 2 : 1;
    if (variant == 3 && M > 128) return launch_gemm_pair<128, 1>(a_dev, b_dev, g, K, s);
    if (variant == 2 && M > 128) return launch_gemm<256, 1>(a_dev, b_dev, g, K, sms, s, scratch);
    return launch_gemm<128, 1>(a_dev, b_dev, g, K, sms, s, scratch);
}

// ---- entry point with built-in scratch --------------------------------------------------------------

namespace {
constexpr size_t kStaticScratchBytes = 8u << 20;
// Split-K partial sums for callers that cannot hand over device memory of their own.  Lives in the library image:
// every device that loads the library holds these 8 MiB until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device, looked up once per device.  In host code the array's
// name is only a handle for the runtime, not a device pointer, so it is never passed to a kernel directly.
int static_scratch_address(unsigned char** out) {
    static std::mutex mu;
    static void* cache[64] = {nullptr};
    int dev = 0;
    CKB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(CK_B200_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(CK_B200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        cache[dev] = p;
    }
    *out = reinterpret_cast<unsigned char*>(cache[dev]);
    return CK_B200_OK;
}
}  // namespace

extern "C" int ck_b200_scaled_mm_nvfp4_static_scratch(const void* a_dev, const void* sfa_dev, const void* b_dev,
                                                      const void* sfb_dev, const float* tensor_scale_a_dev,
                                                      const float* tensor_scale_b_dev, const float* alpha_dev_or_null,
                                                      const void* bias_dev_or_null, int bias_dtype, void* out_dev,
                                                      int out_dtype, int64_t M, int64_t N, int64_t K, void* stream) {
    if (M > 128)
        return fail(CK_B200_ERR_INVALID_ARGUMENT,
                    "scaled_mm_nvfp4_static_scratch: M = %lld is beyond the limit of 128 rows (larger problems need no "
                    "scratch: use ck_b200_scaled_mm_nvfp4)", (long long)M);
    if (M > 0 && N > 0 && (size_t)M * (size_t)N * 4 * 2 > kStaticScratchBytes)
        return fail(CK_B200_ERR_INVALID_ARGUMENT,
                    "scaled_mm_nvfp4_static_scratch: M * N = %lld is beyond the limit of %lld outputs (two fp32 partial "
                    "sums per output must fit the %lld-byte built-in scratch)",
                    (long long)(M * N), (long long)(kStaticScratchBytes / 8), (long long)kStaticScratchBytes);
    unsigned char* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    return scaled_mm_impl(a_dev, sfa_dev, b_dev, sfb_dev, tensor_scale_a_dev, tensor_scale_b_dev, alpha_dev_or_null,
                          bias_dev_or_null, bias_dtype, out_dev, out_dtype, M, N, K,
                          scratch_from_workspace(scratch, kStaticScratchBytes), stream, nullptr, nullptr, -1,
                          /*force_scratch=*/true);   // this entry point's path is the one through its scratch array
}

extern "C" int ck_b200_read_gemm_counters(long long* out5) {
    if (int rc = check_device(nullptr)) return rc;
    if (!out5) return fail(CK_B200_ERR_INVALID_ARGUMENT, "read_gemm_counters: null pointer");
    CKB_CUDA_OK(cudaDeviceSynchronize());
    CKB_CUDA_OK(cudaMemcpyFromSymbol(out5, g_gemm_counters, 5 * sizeof(long long)));
    return CK_B200_OK;
}

extern "C" int ck_b200_read_device_status(int* status_out) {
    if (int rc = check_device(nullptr)) return rc;
    if (!status_out) return fail(CK_B200_ERR_INVALID_ARGUMENT, "read_device_status: null pointer");
    CKB_CUDA_OK(cudaDeviceSynchronize());
    int v = 0;
    CKB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    const int zero = 0;
    CKB_CUDA_OK(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    int vq = 0;   // the quantizer kernels keep their own word (another translation unit)
    if (int rc = read_quant_status(&vq)) return rc;
    if (v == 0) v = vq;
    *status_out = v;
    return v == 0 ? CK_B200_OK : fail(CK_B200_ERR_DEVICE_STATUS, "a kernel gave up on bounded wait %d", v);
}
