// Library-wide entry points of libck_b200: error text, queries, tuning switches.
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace ckb {

std::atomic<long long> g_launches{0};
std::atomic<int> g_quant_variant{2};
std::atomic<int> g_dependent_launch{1};
std::atomic<int> g_gemm_variant{0};
std::atomic<int> g_gemm_debug{0};
std::atomic<int> g_last_splits{1};
std::atomic<int> g_gemm_max_pairs{0};
std::atomic<int> g_gemm_skinny{1};
std::atomic<int> g_weights_resident{0};
std::atomic<int> g_gemm_cluster_split{0};
std::atomic<int> g_linear_fused{0};
std::atomic<int> g_quant_flat{12};
std::atomic<int> g_quant_sync_test{0};
std::atomic<int> g_dynamic_fused_max_mb{128};
std::atomic<int> g_dynamic_smem{1};
std::atomic<int> g_quant_onchip{0};

char* last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

namespace {
struct DeviceInfo {
    bool known = false;
    int major = 0, minor = 0, sms = 0;
};
std::mutex g_dev_mutex;
DeviceInfo g_dev[64];
}  // namespace

int check_device(int* sm_count_out) {
    int dev = 0;
    CKB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(CK_B200_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", dev);
    DeviceInfo info;
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!g_dev[dev].known) {
            CKB_CUDA_OK(cudaDeviceGetAttribute(&g_dev[dev].major, cudaDevAttrComputeCapabilityMajor, dev));
            CKB_CUDA_OK(cudaDeviceGetAttribute(&g_dev[dev].minor, cudaDevAttrComputeCapabilityMinor, dev));
            CKB_CUDA_OK(cudaDeviceGetAttribute(&g_dev[dev].sms, cudaDevAttrMultiProcessorCount, dev));
            g_dev[dev].known = true;
        }
        info = g_dev[dev];
    }
    if (info.major != 10)
        return fail(CK_B200_ERR_UNSUPPORTED_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev,
                    info.major, info.minor);
    if (sm_count_out) *sm_count_out = info.sms;
    return CK_B200_OK;
}

}  // namespace ckb

extern "C" {

const char* ck_b200_last_error(void) { return ckb::last_error_buffer(); }

int64_t ck_b200_query(int what) {
    switch (what) {
        case CK_B200_QUERY_ABI_VERSION: return 2;
        case CK_B200_QUERY_SM_COUNT: {
            int sms = 0;
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess) return -1;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
            return sms;
        }
        case CK_B200_QUERY_WORKSPACE_BYTES: return 64ll << 20;
        case CK_B200_QUERY_COMPUTE_CAPABILITY: {
            int dev = 0, major = 0, minor = 0;
            if (cudaGetDevice(&dev) != cudaSuccess) return -1;
            if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
            if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -1;
            return major * 10 + minor;
        }
        case CK_B200_QUERY_GEMM_LAUNCHES: return ckb::g_launches.load();
        case CK_B200_QUERY_LAST_GEMM_SPLITS: return ckb::g_last_splits.load();
        default: return -1;
    }
}

int ck_b200_set_tuning(int key, int value) {
    switch (key) {
        case CK_B200_TUNE_QUANT_VARIANT: return ckb::g_quant_variant.exchange(value);
        case CK_B200_TUNE_DEPENDENT_LAUNCH: return ckb::g_dependent_launch.exchange(value);
        case CK_B200_TUNE_GEMM_VARIANT: return ckb::g_gemm_variant.exchange(value);
        case CK_B200_TUNE_GEMM_DEBUG: return ckb::g_gemm_debug.exchange(value);
        case CK_B200_TUNE_LINEAR_FUSED: return ckb::g_linear_fused.exchange(value);
        case CK_B200_TUNE_QUANT_FLAT: return ckb::g_quant_flat.exchange(value);
        case CK_B200_TUNE_QUANT_SYNC_TEST: return ckb::g_quant_sync_test.exchange(value);
        case CK_B200_TUNE_DYNAMIC_FUSED_MAX_MB: return ckb::g_dynamic_fused_max_mb.exchange(value);
        case CK_B200_TUNE_DYNAMIC_SMEM: return ckb::g_dynamic_smem.exchange(value);
        case CK_B200_TUNE_GEMM_MAX_PAIRS: return ckb::g_gemm_max_pairs.exchange(value);
        case CK_B200_TUNE_QUANT_ONCHIP: return ckb::g_quant_onchip.exchange(value);
        case CK_B200_TUNE_GEMM_CLUSTER_SPLITK: return ckb::g_gemm_cluster_split.exchange(value);
        case CK_B200_TUNE_WEIGHTS_RESIDENT: return ckb::g_weights_resident.exchange(value);
        case CK_B200_TUNE_GEMM_SKINNY: return ckb::g_gemm_skinny.exchange(value);
        default: return -1;
    }
}

// ---- memory that the other ranks of a node can address (CUDA IPC) --------------------------------------------

int ck_b200_peer_alloc(size_t bytes, void** ptr_out, void* handle_out) {
    if (int rc = ckb::check_device(nullptr)) return rc;
    if (!ptr_out || !handle_out || bytes == 0)
        return ckb::fail(CK_B200_ERR_INVALID_ARGUMENT, "peer_alloc: null pointer or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == CK_B200_PEER_HANDLE_BYTES, "handle size");
    void* p = nullptr;
    CKB_CUDA_OK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        return ckb::fail(CK_B200_ERR_CUDA, "peer_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return CK_B200_OK;
}

int ck_b200_peer_open(const void* handle, void** ptr_out) {
    if (int rc = ckb::check_device(nullptr)) return rc;
    if (!handle || !ptr_out) return ckb::fail(CK_B200_ERR_INVALID_ARGUMENT, "peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    CKB_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return CK_B200_OK;
}

int ck_b200_peer_close(void* ptr) {
    if (!ptr) return CK_B200_OK;
    CKB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return CK_B200_OK;
}

int ck_b200_peer_free(void* ptr) {
    if (!ptr) return CK_B200_OK;
    CKB_CUDA_OK(cudaFree(ptr));
    return CK_B200_OK;
}

// ---- the whole linear in one call -------------------------------------------------------------------------------

namespace {
struct LinearPlan {
    int64_t prow;          // activation rows after padding to 16
    size_t scale_off, dyn_sync_off, q_off, sf_off, sync_off, end;   // byte offsets inside the workspace
};
LinearPlan plan_linear(int64_t M, int64_t K) {
    LinearPlan p;
    p.prow = ckb::round_up64(M, 16);
    p.scale_off = 0;
    p.dyn_sync_off = 64;   // 16 bytes of counters of the dynamic quantizer: zero once, like the area at sync_off
    // the sync area of the fused kernel sits at the same place for every shape, so that nothing but that kernel
    // ever writes there when linears of different shapes share one workspace
    p.sync_off = 256;
    p.q_off = p.sync_off + ckb::fused_sync_bytes();
    p.sf_off = p.q_off + (size_t)ckb::round_up64(p.prow * (K / 2), 256);
    p.end = p.sf_off + (size_t)ckb::round_up64(ckb::round_up64(p.prow, 128) * ckb::round_up64(K / 16, 4), 256);
    return p;
}
}  // namespace

int64_t ck_b200_linear_nvfp4_workspace_bytes(int64_t M, int64_t K) {
    if (M < 0 || K < 0 || K % 32 != 0) return -1;
    return (int64_t)plan_linear(M, K).end;
}

int ck_b200_linear_nvfp4(const void* x_dev, int x_dtype, int64_t M, int64_t K, const float* input_scale_dev_or_null,
                         const void* w_q_dev, const void* w_sf_dev, const float* w_scale_dev, int64_t N,
                         const void* bias_dev_or_null, int bias_dtype, void* out_dev, int out_dtype,
                         void* workspace_dev, size_t workspace_bytes, void* stream) {
    if (M < 0 || N < 0 || K < 0 || K % 32 != 0)
        return ckb::fail(CK_B200_ERR_INVALID_ARGUMENT, "linear_nvfp4: K = %lld must be a non-negative multiple of 32",
                         (long long)K);
    if (M == 0 || N == 0) return CK_B200_OK;
    const LinearPlan p = plan_linear(M, K);
    if (!workspace_dev || ((uintptr_t)workspace_dev & 255) || workspace_bytes < p.end)
        return ckb::fail(CK_B200_ERR_INVALID_ARGUMENT,
                         "linear_nvfp4: workspace must be 256-byte aligned and hold %lld bytes "
                         "(ck_b200_linear_nvfp4_workspace_bytes)", (long long)p.end);
    char* ws = (char*)workspace_dev;
    const float* ts_x = input_scale_dev_or_null;
    float* dyn = (float*)(ws + p.scale_off);
    void* qx = ws + p.q_off;
    void* sfx = ws + p.sf_off;
    // on request, for more than one tile row and column: the GEMM kernel quantizes the activations itself
    const bool in_gemm = ckb::g_linear_fused.load() && ckb::g_gemm_variant.load() == 0 &&
                         ckb::fused_linear_supported(x_dtype, x_dev, M, N, K, out_dtype);
    if (in_gemm) {
        if (!ts_x) {
            if (int rc = ck_b200_dynamic_scale_nvfp4(x_dev, x_dtype, M * K, dyn, stream)) return rc;
            ts_x = dyn;
        }
        return ckb::fused_linear_launch(x_dev, x_dtype, M, K, ts_x, qx, sfx, ws + p.sync_off, w_q_dev, w_sf_dev,
                                        w_scale_dev, N, bias_dev_or_null, bias_dtype, out_dev, out_dtype, stream);
    }
    if (!ts_x) {
        // no scale given: derived from x like the layout does, in the same launch as the quantizer where x fits the L2
        if (int rc = ck_b200_quantize_nvfp4_dynamic(x_dev, x_dtype, dyn, qx, sfx, M, K, /*pad_16x=*/1, /*hi_first=*/1,
                                                    ws + p.dyn_sync_off, stream))
            return rc;
        ts_x = dyn;
    } else if (int rc = ck_b200_quantize_nvfp4(x_dev, x_dtype, ts_x, qx, sfx, M, K, /*pad_16x=*/1, /*hi_first=*/1, stream)) {
        return rc;
    }
    // what is left of the workspace serves the split-K reduction of small-M problems
    const size_t rest = workspace_bytes - p.end;
    return ck_b200_scaled_mm_nvfp4(qx, sfx, w_q_dev, w_sf_dev, ts_x, w_scale_dev, nullptr, bias_dev_or_null, bias_dtype,
                                   out_dev, out_dtype, M, N, K, rest >= (1u << 20) ? ws + p.end : nullptr,
                                   rest >= (1u << 20) ? rest : 0, stream);
}

}  // extern "C"
