// scaled_mm_nvfp4 for sm_100a: block-scaled FP4 GEMM on the 5th-generation tensor cores.
//
//   out[M,N] = out_dtype( alpha * sum_k e2m1(a[m,k]) e4m3(sfa[m,k/16]) e2m1(b[n,k]) e4m3(sfb[n,k/16]) + bias[n] )
//
// Structure (one persistent CTA per SM, 6 warps, no cluster, no multicast):
//   warp 0   producer: one lane issues TMA tile loads of packed A/B (128-byte swizzle) and plain bulk
//            copies of the scale-factor chunks into a ring of shared-memory stages (mbarrier complete_tx).
//   warp 1   MMA issuer: one lane copies the stage's scale factors shared -> tensor memory (tcgen05.cp),
//            issues tcgen05.mma.kind::mxf4nvf4.block_scale (128 x BN x 64 per instruction, fp32
//            accumulators in tensor memory) and commits stage release / accumulator-ready barriers.
//   warps 2-5 epilogue: tcgen05.ld of the accumulator quadrant that the warp may access, alpha and bias,
//            conversion to the output dtype, 16-byte global stores.  With BN = 128 two accumulator
//            buffers let the epilogue of tile i overlap the main loop of tile i+1.
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

namespace ckb {
namespace {

__device__ int g_device_status = 0;

constexpr int BM = 128;             // rows of A per tile = tensor-memory lanes
constexpr int BK_BYTES = 128;       // packed bytes of K per stage = 256 elements = one swizzle row
constexpr int CHUNKS = 4;           // 64-element MMA steps per stage
constexpr int SF_CHUNK_BYTES = 512; // scales of 128 rows x 64 elements
constexpr int NUM_THREADS = 192;
constexpr long long WAIT_LIMIT_CYCLES = 3000000000ll;   // about 1.5 s

enum WaitCode { WAIT_STAGE_EMPTY = 1, WAIT_STAGE_FULL = 2, WAIT_ACC_EMPTY = 3, WAIT_ACC_FULL = 4 };

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
};

template <int BN>
struct Cfg {
    static constexpr int kStages = (BN == 128) ? 6 : 4;
    static constexpr int kAccStages = (BN == 128) ? 2 : 1;
    static constexpr int kBands = BN / 128;                       // 128-row bands of B per tile
    static constexpr int kABytes = BM * BK_BYTES;                 // 16 KiB
    static constexpr int kBBytes = BN * BK_BYTES;
    static constexpr int kSfaBytes = CHUNKS * SF_CHUNK_BYTES;     // 2 KiB
    static constexpr int kSfbBytes = kBands * CHUNKS * SF_CHUNK_BYTES;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    // tensor-memory columns: accumulators, then two alternating scale-factor regions
    static constexpr int kSfaCols = CHUNKS * 4;
    static constexpr int kSfbCols = CHUNKS * 4 * kBands;
    static constexpr int kSfCol0 = kAccStages * BN;
    static constexpr int kTmemCols = 512;
    static_assert(kSfCol0 + 2 * (kSfaCols + kSfbCols) <= kTmemCols, "tensor memory budget");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
    // instruction descriptor of tcgen05.mma.kind::mxf4nvf4.block_scale: A,B = packed e2m1 (format 1), K-major,
    // UE4M3 scales, N >> 3 at bit 17, M >> 4 at bit 24
    static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (0u << 23) |
                                       ((uint32_t)(BM >> 4) << 24);
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

// Shared-memory matrix descriptor (sm_100 version 1).  Addresses and offsets are in 16-byte units.
//   operands: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
//   scale chunks: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
           (1ull << 46) | ((uint64_t)layout << 61);
}
constexpr uint32_t LAYOUT_SWIZZLE_NONE = 0, LAYOUT_SWIZZLE_128B = 2;

// ---- epilogue helpers -----------------------------------------------------------------------------

__device__ __forceinline__ float bias_at(const void* bias, int dtype, int n) {
    if (dtype == CK_B200_DTYPE_BF16) return __bfloat162float(((const __nv_bfloat16*)bias)[n]);
    if (dtype == CK_B200_DTYPE_F16) return __half2float(((const __half*)bias)[n]);
    return ((const float*)bias)[n];
}

// Store 32 consecutive outputs of one row starting at column n0 (n0 % 32 == 0); N % 8 == 0 so groups of
// 8 columns are either fully inside or fully outside.
__device__ __forceinline__ void store_row32(const GemmArgs& g, int64_t row, int n0, const uint32_t (&acc)[32],
                                            float alpha) {
    float y[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(acc[i]) * alpha;
    if (g.bias) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (n0 + i < g.N) y[i] += bias_at(g.bias, g.bias_dtype, n0 + i);
    }
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
            for (int i = 0; i < 4; ++i) {
                if (g.out_dtype == CK_B200_DTYPE_BF16) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(y[8 * j + 2 * i], y[8 * j + 2 * i + 1]);
                    w[i] = *reinterpret_cast<uint32_t*>(&v);
                } else {
                    __half2 v = __floats2half2_rn(y[8 * j + 2 * i], y[8 * j + 2 * i + 1]);
                    w[i] = *reinterpret_cast<uint32_t*>(&v);
                }
            }
            *reinterpret_cast<uint4*>(p + 8 * j) = o;
        }
    }
}

// ---- kernel -----------------------------------------------------------------------------------------

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const GemmArgs g) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
    uint64_t* full_bar = bars;                                  // [kStages]  producer -> MMA
    uint64_t* empty_bar = bars + C::kStages;                    // [kStages]  MMA -> producer
    uint64_t* acc_full_bar = bars + 2 * C::kStages;             // [kAccStages] MMA -> epilogue
    uint64_t* acc_empty_bar = acc_full_bar + C::kAccStages;     // [kAccStages] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + C::kAccStages);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < C::kAccStages; ++s) {
            mbar_init(smem_u32(&acc_full_bar[s]), 1);
            mbar_init(smem_u32(&acc_empty_bar[s]), 128);
        }
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

    const int total_tiles = g.m_tiles * g.n_tiles;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int tm = tile % g.m_tiles, tn = tile / g.m_tiles;
                for (int kb = 0; kb < g.k_iters; ++kb) {
                    ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, WAIT_STAGE_EMPTY);
                    if (!ok) break;
                    uint8_t* st = smem + stage * C::kStageBytes;
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    const int nchunk = min(CHUNKS, g.sf_cbg - kb * CHUNKS);
                    int sfb_present = 0;
#pragma unroll
                    for (int b = 0; b < C::kBands; ++b)
                        if (tn * C::kBands + b < g.sfb_bands) ++sfb_present;
                    mbar_expect_tx(bar, C::kABytes + C::kBBytes + (1 + sfb_present) * nchunk * SF_CHUNK_BYTES);
                    tma_load_2d(smem_u32(st), &tmap_a, kb * BK_BYTES, tm * BM, bar);
                    tma_load_2d(smem_u32(st + C::kABytes), &tmap_b, kb * BK_BYTES, tn * BN, bar);
                    bulk_load(smem_u32(st + C::kABytes + C::kBBytes),
                              g.sfa + ((int64_t)tm * g.sf_cbg + kb * CHUNKS) * SF_CHUNK_BYTES, nchunk * SF_CHUNK_BYTES, bar);
#pragma unroll
                    for (int b = 0; b < C::kBands; ++b) {
                        const int band = tn * C::kBands + b;
                        if (band < g.sfb_bands)
                            bulk_load(smem_u32(st + C::kABytes + C::kBBytes + C::kSfaBytes + b * C::kSfaBytes),
                                      g.sfb + ((int64_t)band * g.sf_cbg + kb * CHUNKS) * SF_CHUNK_BYTES,
                                      nchunk * SF_CHUNK_BYTES, bar);
                    }
                    if (++stage == C::kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0, acc = 0, sfbuf = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                ok = mbar_wait(smem_u32(&acc_empty_bar[acc]), acc_phase ^ 1, abort_flag, WAIT_ACC_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < g.k_iters; ++kb) {
                    ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, WAIT_STAGE_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + stage * C::kStageBytes);
                    const int nchunk = min(CHUNKS, g.sf_cbg - kb * CHUNKS);
                    const uint32_t sfa_t = tmem_base + C::kSfCol0 + sfbuf * (C::kSfaCols + C::kSfbCols);
                    const uint32_t sfb_t = sfa_t + C::kSfaCols;
                    for (int j = 0; j < nchunk; ++j) {
                        tc_cp_sf(sfa_t + 4 * j,
                                 smem_desc(st + C::kABytes + C::kBBytes + j * SF_CHUNK_BYTES, 0, 128, LAYOUT_SWIZZLE_NONE));
#pragma unroll
                        for (int b = 0; b < C::kBands; ++b)
                            tc_cp_sf(sfb_t + 4 * C::kBands * j + 4 * b,
                                     smem_desc(st + C::kABytes + C::kBBytes + C::kSfaBytes + b * C::kSfaBytes +
                                                   j * SF_CHUNK_BYTES,
                                               0, 128, LAYOUT_SWIZZLE_NONE));
                    }
                    const uint64_t adesc = smem_desc(st, 16, 1024, LAYOUT_SWIZZLE_128B);
                    const uint64_t bdesc = smem_desc(st + C::kABytes, 16, 1024, LAYOUT_SWIZZLE_128B);
                    for (int j = 0; j < nchunk; ++j) {
                        // 64 elements of K = 32 bytes = 2 descriptor address units inside the swizzle row
                        tc_mma(d_tmem, adesc + 2 * j, bdesc + 2 * j, C::kIdesc, sfa_t + 4 * j,
                               sfb_t + 4 * C::kBands * j, (kb | j) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&empty_bar[stage]));   // stage reusable once these MMAs have read it
                    sfbuf ^= 1;
                    if (++stage == C::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(smem_u32(&acc_full_bar[acc]));      // accumulator complete
                if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quad = warp & 3;   // tensor-memory lanes [32*quad, 32*quad+32) are the ones this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        float alpha = 0.0f;
        bool alpha_loaded = false;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int tm = tile % g.m_tiles, tn = tile / g.m_tiles;
            if (!alpha_loaded) {
                alpha = g.alpha ? __ldg(g.alpha) : __fmul_rn(__ldg(g.tsa), __ldg(g.tsb));
                alpha_loaded = true;
            }
            ok = mbar_wait(smem_u32(&acc_full_bar[acc]), acc_phase, abort_flag, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int64_t row = (int64_t)tm * BM + quad * 32 + lane;
            const uint32_t t0 = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                tc_ld32(t0 + c, v);
                tc_wait_ld();
                const int n0 = tn * BN + c;
                if (row < g.M && n0 < g.N) store_row32(g, row, n0, v, alpha);
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&acc_empty_bar[acc]));
            if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
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
int make_operand_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t k_bytes, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)k_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k_bytes};
    cuuint32_t box[2] = {(cuuint32_t)BK_BYTES, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CK_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return CK_B200_OK;
}

template <int BN>
int launch_gemm(const void* a, const void* b, GemmArgs g, int64_t K, int sms, cudaStream_t stream) {
    using C = Cfg<BN>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    // opting in to large dynamic shared memory is per function and per device; doing it on every call is cheap
    attr_err = cudaFuncSetAttribute(gemm_nvfp4_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    (void)once;
    if (attr_err != cudaSuccess)
        return fail(CK_B200_ERR_CUDA, "cudaFuncSetAttribute(shared memory %d) failed: %s", C::kSmemBytes,
                    cudaGetErrorString(attr_err));
    CUtensorMap ma, mb;
    if (int rc = make_operand_map(&ma, a, g.M, K / 2, BM)) return rc;
    if (int rc = make_operand_map(&mb, b, g.N, K / 2, BN)) return rc;
    g.m_tiles = (int)ceil_div64(g.M, BM);
    g.n_tiles = (int)ceil_div64(g.N, BN);
    const int64_t tiles = (int64_t)g.m_tiles * g.n_tiles;
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    gemm_nvfp4_kernel<BN><<<grid, NUM_THREADS, C::kSmemBytes, stream>>>(ma, mb, g);
    g_launches.fetch_add(1);
    CKB_CUDA_OK(cudaGetLastError());
    return CK_B200_OK;
}

}  // namespace
}  // namespace ckb

using namespace ckb;

extern "C" int ck_b200_scaled_mm_nvfp4(const void* a_dev, const void* sfa_dev, const void* b_dev, const void* sfb_dev,
                                       const float* tensor_scale_a_dev, const float* tensor_scale_b_dev,
                                       const float* alpha_dev_or_null, const void* bias_dev_or_null, int bias_dtype,
                                       void* out_dev, int out_dtype, int64_t M, int64_t N, int64_t K, void* workspace_dev,
                                       size_t workspace_bytes, void* stream) {
    (void)workspace_dev;
    (void)workspace_bytes;
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
    int variant = g_gemm_variant.load();
    if (variant == 0) variant = (N > 128) ? 2 : 1;   // 128x256 tiles halve the operand traffic per flop
    cudaStream_t s = (cudaStream_t)stream;
    if (variant == 2) return launch_gemm<256>(a_dev, b_dev, g, K, sms, s);
    return launch_gemm<128>(a_dev, b_dev, g, K, sms, s);
}

extern "C" int ck_b200_read_device_status(int* status_out) {
    if (int rc = check_device(nullptr)) return rc;
    if (!status_out) return fail(CK_B200_ERR_INVALID_ARGUMENT, "read_device_status: null pointer");
    CKB_CUDA_OK(cudaDeviceSynchronize());
    int v = 0;
    CKB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    const int zero = 0;
    CKB_CUDA_OK(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    *status_out = v;
    return v == 0 ? CK_B200_OK : fail(CK_B200_ERR_DEVICE_STATUS, "a kernel gave up on bounded wait %d", v);
}
