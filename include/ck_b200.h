/*
 * C ABI of libck_b200.so: the NVFP4 linear path (quantize_nvfp4, dequantize_nvfp4, scaled_mm_nvfp4)
 * for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a native binding of comfy-kitchen would call in place of the reference's
 * extern "C" launchers.  Every pointer named *_dev is device memory on the current CUDA device;
 * `stream` is a cudaStream_t passed as void*.  Calls only enqueue work: they never synchronise,
 * never allocate device memory and may be captured in a CUDA graph (the ck_b200_peer_* set-up calls excepted).  Every function returns 0 on
 * success and a non-zero CK_B200_ERR_* code otherwise; nothing throws across this boundary and the
 * message for the calling thread's last failure is available from ck_b200_last_error().
 *
 * Dtype codes follow the reference table (comfy_kitchen/backends/eager/quantization.py:34-42,
 * comfy_kitchen/backends/cuda/dtype_dispatch.cuh:36-42): 0 = float32, 1 = float16, 2 = bfloat16.
 */
#ifndef CK_B200_H_
#define CK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CK_B200_DTYPE_F32 0
#define CK_B200_DTYPE_F16 1
#define CK_B200_DTYPE_BF16 2

#define CK_B200_OK 0
#define CK_B200_ERR_INVALID_ARGUMENT 1 /* shape / alignment / dtype rejected before any launch */
#define CK_B200_ERR_CUDA 2             /* a CUDA runtime or driver call failed */
#define CK_B200_ERR_UNSUPPORTED_DEVICE 3 /* the current device is not compute capability 10.x */
#define CK_B200_ERR_DEVICE_STATUS 4    /* a kernel reported a bounded wait that ran out */

/*
 * Block-quantize a row-major [rows, cols] matrix to NVFP4.
 * Replaces launch_quantize_nvfp4_kernel (comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu:323-384);
 * arithmetic follows the eager backend bit for bit (comfy_kitchen/backends/eager/quantization.py:118-163).
 *
 *   x_dev                 [rows, cols] contiguous, dtype code x_dtype (0/1/2)
 *   per_tensor_scale_dev  one float32
 *   pad_16x               non-zero: rows and cols are zero-padded up to multiples of 16 (prow, pcol);
 *                         zero: rows and cols must already be multiples of 16
 *   q_out_dev             uint8 [prow, pcol/2]; element 2i in the high nibble when hi_first != 0
 *   sf_out_dev            e4m3 bytes [roundup(prow,128), roundup(pcol/16,4)] in the 128x4 tiled layout
 *                         (comfy_kitchen/float_utils.py:292-326); the kernel writes the zero padding itself
 */
int ck_b200_quantize_nvfp4(const void* x_dev, int x_dtype, const float* per_tensor_scale_dev, void* q_out_dev,
                           void* sf_out_dev, int64_t rows, int64_t cols, int pad_16x, int hi_first, void* stream);

/*
 * Inverse of the above.  Replaces launch_dequantize_nvfp4_kernel
 * (comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu:386-435); rounding follows the eager backend
 * (two roundings to the output dtype, comfy_kitchen/backends/eager/quantization.py:174-222).
 *
 *   q_dev    uint8 [rows, packed_cols];  sf_dev  e4m3 bytes [roundup(rows,128), roundup(packed_cols/8,4)] tiled
 *   out_dev  [rows, 2*packed_cols] of dtype code out_dtype (0/1/2).  packed_cols must be a multiple of 8.
 */
int ck_b200_dequantize_nvfp4(const void* q_dev, const float* per_tensor_scale_dev, const void* sf_dev,
                             void* out_dev, int out_dtype, int64_t rows, int64_t packed_cols, int hi_first,
                             void* stream);

/*
 * out[M,N] = out_dtype( alpha * (A . B^T with per-16 e4m3 block scales) + bias ), fp32 accumulation,
 * alpha = *tensor_scale_a_dev * *tensor_scale_b_dev unless alpha_dev_or_null is given.
 * Replaces launch_cublas_gemm_blockwise_fp4_kernel (comfy_kitchen/backends/cuda/ops/cublas_gemm_nvfp4.cu:295-340),
 * i.e. the cuBLASLt call behind scaled_mm_nvfp4 (comfy_kitchen/backends/eager/quantization.py:225-249).
 *
 *   a_dev [M, K/2], b_dev [N, K/2] packed e2m1 (both with the same nibble order), 16-byte aligned
 *   sfa_dev [roundup(M,128), roundup(K/16,4)], sfb_dev [roundup(N,128), roundup(K/16,4)] tiled e4m3 bytes
 *   bias_dev_or_null [N] of dtype code bias_dtype (1 or 2; 0 also accepted)
 *   out_dev [M, N] row-major of dtype code out_dtype (1 or 2; 0 also accepted)
 *   K % 32 == 0 and N % 8 == 0 (the reference's constraints, comfy_kitchen/backends/cuda/__init__.py:1779,3621-3625)
 *   workspace_dev / workspace_bytes: scratch for split-K reductions; may be NULL / 0, in which case
 *   shapes that would use split-K run unsplit.  ck_b200_query(CK_B200_QUERY_WORKSPACE_BYTES) gives a
 *   size that is always enough.  Calls that share a workspace must not overlap on the GPU.
 */
int ck_b200_scaled_mm_nvfp4(const void* a_dev, const void* sfa_dev, const void* b_dev, const void* sfb_dev,
                            const float* tensor_scale_a_dev, const float* tensor_scale_b_dev,
                            const float* alpha_dev_or_null, const void* bias_dev_or_null, int bias_dtype,
                            void* out_dev, int out_dtype, int64_t M, int64_t N, int64_t K, void* workspace_dev,
                            size_t workspace_bytes, void* stream);

/*
 * scaled_mm_nvfp4 for small M with the split-K scratch built into the library.  No counterpart in the reference.
 *
 * Who needs it: code that may launch kernels but may not obtain device memory at the point of the call - a plugin
 * running inside another framework's captured or pre-planned execution, a real-time loop with a frozen memory plan,
 * a host that keeps the CUDA allocator to itself.  Such callers have no workspace to pass to
 * ck_b200_scaled_mm_nvfp4, and without one a problem with M <= 128 runs unsplit on a fraction of the SMs.
 * Here the fp32 partial sums go to an 8 MiB array that is part of the library image (every GPU that loads the
 * library holds it until the process exits); the call itself performs no allocation of any kind.
 *
 * Same arguments and result as ck_b200_scaled_mm_nvfp4 minus the workspace.  Limits, rejected with
 * CK_B200_ERR_INVALID_ARGUMENT and a message: M <= 128, and M * N <= 1 048 576 outputs (two partial sums each).
 * The first call on each device looks the array's device address up (with that device current): make that call
 * before starting a stream capture.  All calls share the one array and it is not cleared between calls (every word
 * that is read has been written by the same call first): two such calls that overlap on the GPU - different streams,
 * or graph branches - race on it; calls on one stream are ordered and safe.
 */
int ck_b200_scaled_mm_nvfp4_static_scratch(const void* a_dev, const void* sfa_dev, const void* b_dev,
                                           const void* sfb_dev, const float* tensor_scale_a_dev,
                                           const float* tensor_scale_b_dev, const float* alpha_dev_or_null,
                                           const void* bias_dev_or_null, int bias_dtype, void* out_dev, int out_dtype,
                                           int64_t M, int64_t N, int64_t K, void* stream);

/*
 * scaled_mm_nvfp4 of a column-parallel (N-sharded) linear fused with the all-gather of its output: the calling rank
 * computes columns [rank*N_local, (rank+1)*N_local) of the [M, world*N_local] result and the kernel's epilogue
 * stores every finished tile into that column block of EVERY rank's matrix (bulk copies of 512-byte tile rows out of
 * shared memory, to its own memory and to peer memory over NVLink), so no separate collective runs afterwards.  No
 * counterpart in the reference, which is single-GPU (the multi-GPU form of comfy_kitchen/tensor/nvfp4.py:212-260).
 * Keep the peers' memory mapped into one process within about 12 GiB: peer memory is translated in 2 MiB pages through
 * a cache of limited reach; measured on B200s, 7.7 GiB mapped per rank takes these stores at 584 GB/s per rank, 16.8 GiB
 * at 202 GB/s (five times slower than an NCCL all-gather of the same blocks).  The Python layer enforces that bound
 * (PeerGroup.map_limit_bytes); a native caller has to.
 *
 *   out_ptrs   host array of `world` pointers: out_ptrs[r] is rank r's [M, world*N_local] 16-bit matrix as
 *              addressable from this device (own memory for r == rank; ck_b200_peer_open mappings otherwise)
 *   b_dev, sfb_dev, bias_dev_or_null   this rank's shard: [N_local, K/2], its tiled scales, [N_local]
 *   out_dtype  1 or 2;  M > 128 and N_local > 128 (the CTA-pair kernel), N_local % 8 == 0;  1 <= world <= 8
 * The stores to the peers are complete when the kernel has finished; a rank may read its matrix after a
 * ck_b200_peer_barrier that follows the call on every rank (and must not overwrite a peer's matrix before that
 * peer is done with it: a barrier before the call).
 */
int ck_b200_scaled_mm_nvfp4_all_gather(const void* a_dev, const void* sfa_dev, const void* b_dev, const void* sfb_dev,
                                       const float* tensor_scale_a_dev, const float* tensor_scale_b_dev,
                                       const float* alpha_dev_or_null, const void* bias_dev_or_null, int bias_dtype,
                                       void* const* out_ptrs, int world, int rank, int out_dtype, int64_t M,
                                       int64_t N_local, int64_t K, void* stream);

/*
 * Barrier between the ranks of one node, enqueued on `stream` (one small kernel per rank; no host involvement, so it
 * can be captured in a CUDA graph).  flag_ptrs[r] is rank r's array of `world` zero-initialised uint32 counters in
 * peer-addressable memory, epoch_dev one zero-initialised uint32 in this rank's memory; every rank must enqueue the
 * same sequence of barriers.  One rank per GPU: the kernels of different ranks wait for one another.  The wait is
 * bounded (2 s): on expiry the kernel records code 6 in the status word (ck_b200_read_device_status) and returns.
 * No counterpart in the reference.
 */
int ck_b200_peer_barrier(void* const* flag_ptrs, int world, int rank, void* epoch_dev, void* stream);

/*
 * Device memory the other ranks of the node can map (CUDA IPC), for the two calls above.  Set-up calls: they
 * allocate, synchronise and are not for the hot path.  peer_alloc returns zeroed memory on the current device and
 * writes its CK_B200_PEER_HANDLE_BYTES-byte handle, which the caller ships to the other processes (any transport);
 * peer_open maps such a handle from another process; peer_close / peer_free undo them.  No counterpart in the reference.
 */
#define CK_B200_PEER_HANDLE_BYTES 64
int ck_b200_peer_alloc(size_t bytes, void** ptr_out, void* handle_out);
int ck_b200_peer_open(const void* handle, void** ptr_out);
int ck_b200_peer_close(void* ptr);
int ck_b200_peer_free(void* ptr);

/*
 * The whole NVFP4 linear of the reference layer (samples/nvfp4_linear.py:77-80 through
 * comfy_kitchen/tensor/nvfp4.py:53-84,212-260) in one call: per-tensor activation scale (given, or derived from x like
 * the layout does), quantize_nvfp4 of x with rows padded to 16, scaled_mm_nvfp4 with the resident quantized weight,
 * bias and output rounding.  Enqueues three to five kernels; the quantized activation lives in the caller's workspace.
 *
 *   x_dev [M, K] of dtype code x_dtype, K % 32 == 0;  input_scale_dev_or_null: one float32, or NULL for the dynamic scale
 *   w_q_dev [N, K/2], w_sf_dev tiled e4m3 [roundup(N,128), roundup(K/16,4)], w_scale_dev one float32, N % 8 == 0
 *   out_dev [M, N] of dtype code out_dtype;  bias_dev_or_null [N]
 *   workspace_dev: 256-byte aligned, at least ck_b200_linear_nvfp4_workspace_bytes(M, K) bytes; anything beyond that
 *   (1 MiB or more) is used for the split-K reduction when M <= 128
 *
 * Optional (CK_B200_TUNE_LINEAR_FUSED = 1; off by default because it measured slower on B200): with M > 128, N > 128
 * and bf16 / fp16 activations the call is ONE kernel: the CTA-pair GEMM carries eight extra warps per CTA that
 * quantize x into the workspace while the tensor-core main loop runs, and each tile's loads wait (bounded) for the
 * 128-row band of x they read.  Results are bit-identical to the separate operators.  The progress
 * words live in bytes [256, 256 + 32 KiB) of the workspace, which only that kernel writes, and the counters of the
 * dynamic quantizer (input_scale_dev_or_null == NULL) in bytes [64, 80): zero the first 33 KiB once when the
 * workspace is allocated (they then stay consistent over any sequence of calls, shapes and graph replays).  Calls
 * that share a workspace must not overlap on the GPU.
 */
int64_t ck_b200_linear_nvfp4_workspace_bytes(int64_t M, int64_t K);
int ck_b200_linear_nvfp4(const void* x_dev, int x_dtype, int64_t M, int64_t K, const float* input_scale_dev_or_null,
                         const void* w_q_dev, const void* w_sf_dev, const float* w_scale_dev, int64_t N,
                         const void* bias_dev_or_null, int bias_dtype, void* out_dev, int out_dtype,
                         void* workspace_dev, size_t workspace_bytes, void* stream);

/*
 * MXFP8, the sibling format of the same path: e4m3 data with one power-of-two (e8m0) scale per 32 elements, scales in
 * the same 128x4 tiled layout.  Replace launch_quantize_mxfp8_kernel (comfy_kitchen/backends/cuda/ops/quantize_mxfp8.cu:40-139)
 * and the eager dequantize_mxfp8 / scaled_mm_mxfp8 (comfy_kitchen/backends/eager/quantization.py:260-405; the
 * reference has no CUDA GEMM for this format, its eager path calls cuBLASLt through torch).
 *
 *   quantize:   x_dev [rows, cols] (dtype code 0/1/2) -> q_out_dev e4m3 bytes [prow, pcol] and sf_out_dev e8m0 bytes
 *               [roundup(prow,128), roundup(pcol/32,4)] tiled, prow/pcol = rows/cols rounded up to 32 when pad_32x,
 *               otherwise rows and cols must be multiples of 32; the kernel writes all padding itself
 *   dequantize: out_dev [rows, cols] of dtype code out_dtype = out(e4m3 * 2^(e-127)), cols % 32 == 0
 *   scaled_mm:  out[M,N] = out_dtype(A . B^T + bias), A [M,K] and B [N,K] e4m3 bytes, fp32 accumulation;
 *               K % 32 == 0, N % 8 == 0; workspace as for ck_b200_scaled_mm_nvfp4 (split-K for M <= 128)
 */
int ck_b200_quantize_mxfp8(const void* x_dev, int x_dtype, void* q_out_dev, void* sf_out_dev, int64_t rows, int64_t cols,
                           int pad_32x, void* stream);
int ck_b200_dequantize_mxfp8(const void* q_dev, const void* sf_dev, void* out_dev, int out_dtype, int64_t rows,
                             int64_t cols, void* stream);
int ck_b200_scaled_mm_mxfp8(const void* a_dev, const void* sfa_dev, const void* b_dev, const void* sfb_dev,
                            const void* bias_dev_or_null, int bias_dtype, void* out_dev, int out_dtype, int64_t M,
                            int64_t N, int64_t K, void* workspace_dev, size_t workspace_bytes, void* stream);

/*
 * amax(|x|) / (448*6) computed in the input dtype and widened to float32, the per-tensor scale
 * TensorCoreNVFP4Layout.quantize derives when the caller gives none (comfy_kitchen/tensor/nvfp4.py:66-71).
 * scale_out_dev receives one float32.  Two launches on `stream` (reduce, finalise); no host sync.
 */
int ck_b200_dynamic_scale_nvfp4(const void* x_dev, int x_dtype, int64_t numel, float* scale_out_dev, void* stream);

/*
 * quantize_nvfp4 with the per-tensor scale derived from x itself, as TensorCoreNVFP4Layout.quantize does when the
 * caller gives none (comfy_kitchen/tensor/nvfp4.py:53-84: scale = amax(|x|) / (448*6) in x's dtype, then
 * ck.quantize_nvfp4(x, scale)).  Same outputs, bit for bit, as ck_b200_dynamic_scale_nvfp4 followed by
 * ck_b200_quantize_nvfp4; scale_out_dev receives the float32 scale (the GEMM's tensor_scale_a).
 * While x is about the size of the L2 or smaller (CK_B200_TUNE_DYNAMIC_FUSED_MAX_MB, default 128) this is ONE kernel launch:
 * every warp takes the maximum over the part of x it will quantize, walking it backwards, the blocks meet at a grid-wide
 * counter, then every warp quantizes its part forwards - from what L2 still holds of it, or, up to about 32 MB of 16-bit
 * input, from shared memory, where the first pass parked it: the second read of x from HBM is gone or shortened.
 * Larger or oddly shaped inputs (an odd number of 64-column units, unaligned base) take the separate kernels inside
 * the same call.
 *   sync_dev   16 bytes, 16-byte aligned, zero before the first call; the kernel leaves them zero.  Calls that share
 *              them must be ordered on one stream.  NULL selects the separate kernels.
 * The meeting point is a bounded wait (about a second): if it runs out, the blocks record code 8 in the status word
 * (ck_b200_read_device_status) and return without writing the outputs.
 */
int ck_b200_quantize_nvfp4_dynamic(const void* x_dev, int x_dtype, float* scale_out_dev, void* q_out_dev,
                                   void* sf_out_dev, int64_t rows, int64_t cols, int pad_16x, int hi_first,
                                   void* sync_dev, void* stream);

/* Message describing the calling thread's last failure ("" if none).  Counterpart of the
 * std::runtime_error text of the reference launchers (comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu:380-383). */
const char* ck_b200_last_error(void);

#define CK_B200_QUERY_ABI_VERSION 0
#define CK_B200_QUERY_SM_COUNT 1          /* of the current device */
#define CK_B200_QUERY_WORKSPACE_BYTES 2   /* split-K workspace that is always enough */
#define CK_B200_QUERY_COMPUTE_CAPABILITY 3 /* major*10 + minor of the current device */
#define CK_B200_QUERY_GEMM_LAUNCHES 4     /* kernels launched by this library in this process (all entry points) */
#define CK_B200_QUERY_LAST_GEMM_SPLITS 5  /* pieces along K the most recent GEMM launch of this process was cut into
                                             (1 = no split-K); for tests and tuning */
/* Small integer facts about the library / current device; -1 for an unknown key.  Counterpart of the
 * module attributes of the reference extension (comfy_kitchen/backends/cuda/dlpack_bindings.cpp:3738). */
int64_t ck_b200_query(int what);

/*
 * Device-side status word of the current device: 0 when no kernel of this library gave up on a bounded
 * wait since the last call, otherwise a code naming the wait.  Synchronises the device; meant for tests
 * and debugging (the reference has no counterpart: its GEMM is a library call).
 */
int ck_b200_read_device_status(int* status_out);

/*
 * What the counting build of the CTA-pair GEMM (CK_B200_TUNE_GEMM_DEBUG = 1) measured in its most recent launch on the
 * current device, for CTA pair 0: out5[0] cycles and out5[1] nanoseconds of the epilogue role (their ratio is the SM
 * clock inside the kernel, which NVML's samples do not resolve), out5[2] cycles the MMA role waited for loaded stages,
 * out5[3] cycles it waited for an accumulator, out5[4] the MMA role's total cycles.  Synchronises the device; for
 * benchmarks.  No counterpart in the reference (its GEMM is a library call).
 */
int ck_b200_read_gemm_counters(long long* out5);

/* Tuning switches used by tests and benchmarks to select kernel variants: key/value integers,
 * returns the previous value or -1 for an unknown key.  No counterpart in the reference (its
 * environment switches, comfy_kitchen/backends/cuda/__init__.py:212-215, do not touch this path). */
#define CK_B200_TUNE_QUANT_VARIANT 0 /* 0 = IEEE divisions, 1 = reciprocal bracket + exact fallback, 2 = one-round residual correction (default) */
#define CK_B200_TUNE_GEMM_VARIANT 1  /* GEMM tile configuration; 0 = automatic, 1 = 128x128 one CTA, 2 = 128x256 one CTA, 3 = 256x256 CTA
                                        pair, 4 = the same with half-width stages, 5 = 128x64 with two CTAs per SM where M <= 64,
                                        6 = K split over a cluster where M <= 64 */
#define CK_B200_TUNE_GEMM_DEBUG 2    /* non-zero: the counting build of the GEMM kernels runs; 1 = its first CTA also prints the
                                        cycles its roles spent waiting, 2 = counters only (ck_b200_read_gemm_counters) */
#define CK_B200_TUNE_DEPENDENT_LAUNCH 3 /* non-zero (default): kernels are launched with programmatic stream
                                          serialisation, so a kernel's set-up overlaps the previous kernel's tail */
#define CK_B200_TUNE_LINEAR_FUSED 4  /* non-zero: ck_b200_linear_nvfp4 quantizes the activations inside the GEMM kernel
                                        when the shape allows it (default 0: separate kernels, which measured faster) */
#define CK_B200_TUNE_QUANT_FLAT 5     /* quantize_nvfp4 launch geometry: 0 = segments of rows in several waves; n > 0
                                        (default 12) = one wave of equal ranges when every resident warp gets n to 128 units */
#define CK_B200_TUNE_QUANT_SYNC_TEST 6 /* tests only: n > 0 makes the dynamic quantizer wait for n blocks that do not
                                        exist and give up after about 0.1 s (the wait then runs out by design) */
#define CK_B200_TUNE_DYNAMIC_FUSED_MAX_MB 7 /* largest input, in 10^6 bytes, that ck_b200_quantize_nvfp4_dynamic handles
                                             in one launch (default 128; measured with the backward / forward walk: 57 MB
                                             26 us against 33 with separate kernels, 113 MB 51 against 57, 336 MB 148
                                             against 136) */
#define CK_B200_TUNE_DYNAMIC_SMEM 8 /* non-zero (default): inputs of up to about 32 MB with rows and columns multiples of
                                     128 stay in shared memory between the two phases of ck_b200_quantize_nvfp4_dynamic */
#define CK_B200_TUNE_GEMM_MAX_PAIRS 9 /* n > 0: the CTA-pair GEMM (and its all-gather form) launches at most n pairs of CTAs
                                       instead of one per pair of SMs, so that two such kernels on two streams run side by
                                       side; 0 (default) = all */
#define CK_B200_TUNE_QUANT_ONCHIP 10 /* non-zero: quantize_nvfp4 of a 16-bit input of up to about 32 MB with rows and columns
                                       multiples of 128 asks for the whole input at once (asynchronous copies into shared
                                       memory) instead of walking it with a register ring.  Off by default: alone it takes
                                       the same time, and its 72 KB of shared memory per block keep it from running beside
                                       a GEMM's CTAs (a step whose quantizers overlap its GEMMs is 3.7 % slower with it) */
#define CK_B200_TUNE_GEMM_SKINNY 11 /* non-zero (default): a GEMM with M <= 64 and at least one 64-column tile per SM (N >= 64 x SMs) runs
                                      on 64-column tiles with two CTAs per SM (twice the CTAs of the 128-column configuration,
                                      each with a short ring); GEMM variant 5 forces that configuration for every M <= 64 */
#define CK_B200_TUNE_WEIGHTS_RESIDENT 12 /* A promise by the caller, off by default: when a GEMM with M <= 128 is enqueued, nothing that is
                                           still in flight on the GPU writes its B operand or B scales (weights quantized when the
                                           model was loaded, and synchronised since).  The kernel then requests the first stages of the
                                           weight BEFORE it waits for the preceding kernel of the stream, so a stack of small-M layers
                                           streams layer i+1's weight under layer i's tail.  Activations, their scales, tensor scales,
                                           bias and every store still wait. */
#define CK_B200_TUNE_GEMM_CLUSTER_SPLITK 13 /* non-zero: a GEMM with M <= 64 splits K over a thread-block cluster of 2 or 4 CTAs that exchange
                                              their partial sums through shared memory (one launch, no scratch); also GEMM variant 6 */
int ck_b200_set_tuning(int key, int value);

#ifdef __cplusplus
}
#endif
#endif /* CK_B200_H_ */
