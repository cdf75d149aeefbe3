// Shared host/device helpers of libck_b200: error reporting, launch accounting, PTX wrappers (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/ck_b200.h"

namespace ckb {

// ---- host side --------------------------------------------------------------------------------

// Per-thread message of the last failure, returned by ck_b200_last_error().
char* last_error_buffer();
int fail(int code, const char* fmt, ...);
// Number of kernels this library has launched in this process.
extern std::atomic<long long> g_launches;
// Tuning switches (ck_b200_set_tuning).
extern std::atomic<int> g_quant_variant;
extern std::atomic<int> g_gemm_variant;
extern std::atomic<int> g_gemm_debug;
extern std::atomic<int> g_dependent_launch;
extern std::atomic<int> g_gemm_max_pairs;   // > 0: the CTA-pair GEMM launches at most this many pairs (CK_B200_TUNE_GEMM_MAX_PAIRS)
extern std::atomic<int> g_gemm_skinny;      // non-zero: M <= 64 takes the 64-column, two-CTAs-per-SM configuration (CK_B200_TUNE_GEMM_SKINNY)
extern std::atomic<int> g_gemm_cluster_split;   // non-zero: M <= 64 splits K over a thread-block cluster (CK_B200_TUNE_GEMM_CLUSTER_SPLITK)
extern std::atomic<int> g_weights_resident;   // the caller's promise behind GemmArgs::early_weights (CK_B200_TUNE_WEIGHTS_RESIDENT)
extern std::atomic<int> g_last_splits;   // K-splits of the most recent GEMM launch (CK_B200_QUERY_LAST_GEMM_SPLITS)

// Checks that the current device is compute capability 10.x (cached per device ordinal).
int check_device(int* sm_count_out);

// The CTA-pair GEMM with the activation quantizer inside (gemm_nvfp4_sm100.cu): whether a linear can take that
// path, the bytes of its sync area, and the launch.  qx / sfx receive the quantized activations (rows padded to 16).
extern std::atomic<int> g_linear_fused;
extern std::atomic<int> g_quant_flat;   // 0 = off, else the least units per warp for the one-wave quantizer geometry
extern std::atomic<int> g_quant_sync_test;       // > 0: the dynamic quantizer expects that many arrivals too many (tests)
extern std::atomic<int> g_quant_onchip;           // non-zero: inputs that fit the SMs' shared memory are quantized from there
extern std::atomic<int> g_dynamic_smem;           // non-zero: small inputs are parked in shared memory between the two phases
extern std::atomic<int> g_dynamic_fused_max_mb;  // largest input (10^6 bytes) the dynamic quantizer handles in one launch
// Status word of the quantizer kernels (its own translation unit): reads and clears it.
int read_quant_status(int* out);
bool fused_linear_supported(int x_dtype, const void* x_dev, int64_t M, int64_t N, int64_t K, int out_dtype);
size_t fused_sync_bytes();
int fused_linear_launch(const void* x_dev, int x_dtype, int64_t M, int64_t K, const float* ts_x_dev, void* qx_dev,
                        void* sfx_dev, void* sync_dev, const void* w_q_dev, const void* w_sf_dev,
                        const float* w_scale_dev, int64_t N, const void* bias_dev_or_null, int bias_dtype, void* out_dev,
                        int out_dtype, void* stream);

#define CKB_CUDA_OK(expr)                                                                              \
    do {                                                                                               \
        cudaError_t e__ = (expr);                                                                      \
        if (e__ != cudaSuccess)                                                                        \
            return ::ckb::fail(CK_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));     \
    } while (0)

static inline int64_t round_up64(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
static inline int64_t ceil_div64(int64_t x, int64_t m) { return (x + m - 1) / m; }

// ---- device side ------------------------------------------------------------------------------

#ifdef __CUDACC__

// Launch with programmatic stream serialisation: the grid may be scheduled while the previous kernel on the
// stream is still draining, and runs its prologue up to grid_dependency_wait() before that kernel has finished.
// Every kernel launched through here calls allow_dependent_launch() first thing and grid_dependency_wait() before
// its first access to global memory, so ordering and visibility are those of a plain in-stream launch.
// `family` selects the bit of the CK_B200_TUNE_DEPENDENT_LAUNCH mask that enables the attribute for this kernel.
constexpr int kLaunchFamilyGemm = 1, kLaunchFamilyQuantize = 2;
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(int family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (g_dependent_launch.load() & family) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The next kernel on the stream may start being scheduled (it still waits for this grid to finish and flush
// before it touches memory).
__device__ __forceinline__ void allow_dependent_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Returns once every kernel this grid depends on has completed and its writes are visible.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Byte offset of logical scale (r, c) in the 128x4 tiled scale tensor with cbg_count groups of 4 columns.
__device__ __forceinline__ int64_t sf_offset(int64_t r, int c, int cbg_count) {
    int64_t rb = r >> 7;
    int rem = (int)(r & 127);
    return ((rb * cbg_count + (c >> 2)) * 32 + (rem & 31)) * 16 + (rem >> 5) * 4 + (c & 3);
}

// 16-byte streaming load through the read-only path, not allocating in L1.
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

#endif  // __CUDACC__

}  // namespace ckb
