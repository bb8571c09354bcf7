/*
 * quest_b200 - C ABI of the B200 (sm_100a) implementation of QuEST's W4A4 inference linear layer.
 *
 * Every entry point below replaces one launcher that the reference's torch C++ bindings call
 * (gemm-quest/quest/{quantize,matmul,fused_matmul_dequantize}.cpp).  Names, argument order and
 * argument meaning are the reference's; the differences are:
 *   - C linkage (the reference declares them with C++ linkage inside its extension),
 *   - every function returns an int status (QB200_OK == 0) instead of void / an ignored int,
 *   - `do_dequantize` is an int (0/1) instead of a C++ bool.
 *
 * Conventions shared by all entry points
 *   - All pointers are DEVICE pointers owned by the caller.  Nothing is allocated or freed here.
 *   - Work is only enqueued on `stream`; no call synchronises the device.  The current device
 *     must be the one that owns the buffers (the Python wrapper sets it).
 *   - Matrices are dense row-major.  "packed int4" means one byte holds two two's-complement
 *     4-bit codes: column 2j in the low nibble, column 2j+1 in the high nibble.
 *   - bf16 means __nv_bfloat16, int32 means int32_t.
 *   - All calls may be captured in a CUDA graph (no allocation, no synchronisation; tensor maps
 *     are passed by value as kernel parameters).
 */
#ifndef QUEST_B200_H_
#define QUEST_B200_H_

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    QB200_OK = 0,
    QB200_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive size, misaligned buffer */
    QB200_ERR_UNSUPPORTED = 2,      /* shape outside what the kernels cover (see each function) */
    QB200_ERR_CUDA = 3,             /* a CUDA runtime call or kernel launch failed */
    QB200_ERR_DRIVER = 4,           /* cuTensorMapEncodeTiled unavailable or failed */
    QB200_ERR_DEVICE_TIMEOUT = 5,   /* a bounded in-kernel wait gave up (reported by quest_b200_device_status) */
    QB200_ERR_SCRATCH_LIMIT = 6     /* the no-allocation entry point was asked for more scratch than its static buffer */
};

/* Human-readable text for a status code. */
const char* quest_b200_error_string(int status);

/* Library version (major * 100 + minor). */
int quest_b200_version(void);

/*
 * Reads and clears the device-side status word of the current device.  The GEMM kernel's waits on
 * mbarriers are bounded; if one gives up, the kernel records QB200_ERR_DEVICE_TIMEOUT here, drains
 * and returns instead of hanging.  Synchronises the device.  *status receives the recorded code.
 */
int quest_b200_device_status(int* status);

/*
 * Test support: launches the fused GEMM with its TMA producer switched off and the limit of every bounded in-kernel
 * wait shortened to wait_limit_cycles (SM clock cycles, at least one million; a few million = a few milliseconds), so that the waits of the
 * consumer warps run out by construction - no trap, no fault, no unbounded spin.  The kernel records
 * QB200_ERR_DEVICE_TIMEOUT, releases what it holds and returns; mat_d is not written.  Synchronises the stream and
 * restores the normal limit before returning.  The caller then reads quest_b200_device_status(), which reports
 * (site << 8) | QB200_ERR_DEVICE_TIMEOUT once and clears it.  No counterpart in the reference (its kernels have no
 * waits of this kind).
 */
int quest_b200_test_bounded_wait_cuda(void* mat_d, const void* mat_a, const void* mat_b, const void* vec_a_add,
                                      const void* vec_b_add, const void* vec_a_mul, const void* vec_b_mul, int M, int K,
                                      int N, long long wait_limit_cycles, cudaStream_t stream);

/*
 * scale[m] = bf16( sqrt(mean_k x[m,k]^2) * (2.513930578568423 * 2 / 15) + 1e-8 )
 * Replaces find_scale_int4_cuda_bf16, gemm-quest/quest/quantize.cpp:5-11
 * (kernel gemm-quest/quest/quantize_kernel.cu:38-117).
 *   scale_ptr : bf16 [batch_size]          x_ptr : bf16 [batch_size, group_size]
 */
int find_scale_int4_cuda_bf16(void* scale_ptr, const void* x_ptr, int group_size, int batch_size,
                              cudaStream_t stream);

/*
 * q = clamp(floor(x / scale), -8, 7) per row, with optional outputs (pass NULL to skip):
 *   x_int_ptr          int8  [batch_size, group_size]      dense codes
 *   x_int_packed_ptr   uint8 [batch_size, group_size / 2]  packed codes (group_size must be even)
 *   x_int_row_sum_ptr  int32 [batch_size]                  sum of the codes of each row
 * If do_dequantize != 0, x is overwritten in place by bf16((q + 0.5) * scale).
 * Replaces quantize_int4_cuda_bf16, gemm-quest/quest/quantize.cpp:28-38
 * (kernel gemm-quest/quest/quantize_kernel.cu:120-261).
 */
int quantize_int4_cuda_bf16(void* x_ptr, const void* scale_ptr, void* x_int_ptr, void* x_int_packed_ptr,
                            void* x_int_row_sum_ptr, int group_size, int batch_size, int do_dequantize,
                            cudaStream_t stream);

/*
 * D[m,n] = bf16( float(2*C[m,n] + a_add[m] + b_add[n]) * (0.5f * a_mul[m] * b_mul[n]) )
 * Replaces add_mul_vv_cuda_bf16, gemm-quest/quest/quantize.cpp:73-83
 * (kernel gemm-quest/quest/quantize_kernel.cu:264-341).
 *   mat_d bf16 [size_a,size_b]; vec_a_add int32 [size_a]; vec_a_mul bf16 [size_a];
 *   vec_b_add int32 [size_b]; vec_b_mul bf16 [size_b]; mat_c int32 [size_a,size_b]
 */
int add_mul_vv_cuda_bf16(void* mat_d, const void* vec_a_add, const void* vec_a_mul, const void* vec_b_add,
                         const void* vec_b_mul, const void* mat_c, int size_a, int size_b, cudaStream_t stream);

/*
 * C[M,N] (int32) = A[M,K] . B[N,K]^T, both operands packed int4 (A: [M,K/2] bytes, B: [N,K/2] bytes).
 * The accumulators are exact.  Requires K % 32 == 0 (16-byte row pitch, as the reference's CUTLASS
 * kernel does), K < 131072, and 16-byte aligned A and B.
 * Replaces matmul_int4_int4t_int32_cuda, gemm-quest/quest/matmul.cpp:5-13
 * (kernel gemm-quest/quest/matmul_kernel.cu:8-63).
 */
int matmul_int4_int4t_int32_cuda(void* mat_c, const void* mat_a, const void* mat_b, int M, int K, int N,
                                 cudaStream_t stream);

/*
 * D[M,N] (bf16) = add_mul_vv(vec_a_add, vec_a_mul, vec_b_add, vec_b_mul, A . B^T) in one kernel:
 *   D[m,n] = bf16( float(2*acc + vec_a_add[m] + vec_b_add[n]) * (0.5f * vec_a_mul[m] * vec_b_mul[n]) )
 * with exact int32 accumulators (the reference's fused epilogue rounds the accumulator to fp16
 * first, gemm-quest/include/symmetric/epilogue/thread/linear_combination_dequant.h:133-144; this
 * library evaluates the exact expression of add_mul_vv instead).  Same shape rules as the int32 GEMM.
 * Replaces fused_matmul_dequantize_int4_int4t_bf16_cuda,
 * gemm-quest/quest/fused_matmul_dequantize.cpp:5-17 (kernel .../fused_matmul_dequantize_kernel.cu:4-57).
 *   vec_a_add int32 [M], vec_b_add int32 [N], vec_a_mul bf16 [M], vec_b_mul bf16 [N]
 */
int fused_matmul_dequantize_int4_int4t_bf16_cuda(void* mat_d, const void* mat_a, const void* mat_b,
                                                 const void* vec_a_add, const void* vec_b_add,
                                                 const void* vec_a_mul, const void* vec_b_mul, int M, int K,
                                                 int N, cudaStream_t stream);

/*
 * As above, but the output tile columns are written into a wider row-major matrix: element (m,n)
 * goes to mat_d[m * ld_d + n].  Used by the column-sharded multi-GPU layer, where each rank
 * computes N_local output columns of a [M, N_total] result (ld_d = N_total, mat_d already offset
 * to the rank's first column).  ld_d and the offset must keep 16-byte alignment of each row segment
 * for the vector store path; otherwise a scalar store path is used.
 * No counterpart in the reference (its inference path is single-GPU).
 */
int fused_matmul_dequantize_int4_int4t_bf16_strided_cuda(void* mat_d, long long ld_d, const void* mat_a,
                                                         const void* mat_b, const void* vec_a_add,
                                                         const void* vec_b_add, const void* vec_a_mul,
                                                         const void* vec_b_mul, int M, int K, int N,
                                                         cudaStream_t stream);

/*
 * The fused GEMM + epilogue for callers that cannot allocate device memory at the time of the call: code that runs
 * while a stream is being captured, a process whose memory is handed out in full to a framework allocator at start-up,
 * a real-time loop that may not block in the driver.  The ordinary entry points obtain their split-K scratch with
 * cudaMalloc on first use; this one keeps it in a fixed 8 MiB array in device memory (static storage of the library,
 * held by every GPU that loads it until the process exits) and calls no allocating routine on any path.
 *   splits = 0   the library chooses the number of K ranges and never asks for more than the array holds: where its
 *                usual choice would not fit it takes fewer ranges, down to 1 (the kernels that need no scratch).
 *   splits >= 2  that many ranges; QB200_ERR_SCRATCH_LIMIT, and nothing is launched, if
 *                tiles x splits x rows-per-tile > 8192  (tiles = ceil(M/128) * ceil(N/256),
 *                rows-per-tile = min(128, M rounded up to 8)), or if there are more than 1024 tiles.
 *   splits = 1   never split.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that call before any
 * stream capture.  All calls on a device share the one array and its tile counters: two split-K launches of this entry
 * point that overlap on the GPU (different streams) race and corrupt each other's sums - keep them on one stream or
 * order them with events.  The array is separate from the ordinary entry points' buffer, so a launch of this entry
 * point may overlap one of theirs.  No counterpart in the reference.
 */
int fused_matmul_dequantize_int4_int4t_bf16_noalloc_cuda(void* mat_d, const void* mat_a, const void* mat_b,
                                                         const void* vec_a_add, const void* vec_b_add,
                                                         const void* vec_a_mul, const void* vec_b_mul, int M, int K,
                                                         int N, int splits, cudaStream_t stream);

/*
 * Same GEMM + epilogue, with every output tile stored into n_dst (1..8) matrices of identical shape and row
 * stride: mat_d_list[0] is normally the caller's own buffer and mat_d_list[1..] are the buffers of the other GPUs
 * of the node, mapped into this process (peer or symmetric memory), each already offset to the caller's first
 * output column.  The stores are ordinary (peer) stores issued from the epilogue while later tiles are still
 * being computed; the caller synchronises the GPUs afterwards (the kernel itself does not wait for anyone).
 * mat_d_list is a HOST array; it is copied into the kernel parameters.
 * No counterpart in the reference.
 */
int fused_matmul_dequantize_int4_int4t_bf16_push_cuda(void* const* mat_d_list, int n_dst, long long ld_d,
                                                      const void* mat_a, const void* mat_b, const void* vec_a_add,
                                                      const void* vec_b_add, const void* vec_a_mul,
                                                      const void* vec_b_mul, int M, int K, int N,
                                                      cudaStream_t stream);

/*
 * The int8-operand route of the layer (no counterpart in the reference; an internal format between this library's
 * two kernels).  hadamard_quantize_a8_cuda_bf16 is hadamard_quantize_int4_cuda_bf16 with another output: instead of
 * packed int4 it writes the operand the GEMM's tensor cores consume - int8 = 16 x code, [batch_size, group_size]
 * row-major, and inside every group of 32 consecutive K positions the 16 even positions first, then the 16 odd
 * ones - so that the GEMM need not unpack A.  Only shapes the tcgen05 quantiser can tile (group_size a multiple of
 * 128, see quest_b200_prefers_a8); QB200_ERR_UNSUPPORTED otherwise.  fused_matmul_dequantize_a8_int4t_bf16_cuda is the
 * fused GEMM + epilogue taking that operand (mat_b stays packed int4; K a multiple of 128; always the 256 x 256 tile
 * kernel).  quest_b200_prefers_a8 returns 1 where this route is the faster one for an [M, K] x [N, K]^T layer (what
 * quest_b200.layer.linear_forward asks before choosing), else 0; QB200_A8=0|1 in the environment overrides it.
 */
int hadamard_quantize_a8_cuda_bf16(void* a8_ptr, void* scale_ptr, void* x_int_row_sum_ptr, const void* x_ptr,
                                   int group_size, int batch_size, int block, cudaStream_t stream);
int fused_matmul_dequantize_a8_int4t_bf16_cuda(void* mat_d, const void* mat_a8, const void* mat_b,
                                               const void* vec_a_add, const void* vec_b_add, const void* vec_a_mul,
                                               const void* vec_b_mul, int M, int K, int N, cudaStream_t stream);
int quest_b200_prefers_a8(int M, int K, int N);

/*
 * Fused block-Hadamard + scale + int4 quantise + pack + row-sum of bf16 activations, one pass over
 * x.  Per row: xh = bf16(H_block . x) blockwise along K (Sylvester order, entries +-bf16(block^-0.5)),
 * scale = find_scale(xh), codes = quantize(xh, scale).  Replaces the three launches of the reference's
 * layer code, gemm-quest/benchmarks/utils.py:89-100 (cuBLAS Hadamard GEMM, find_scale_int4,
 * quantize_int4).  block in {64, 128, 256}; group_size % block == 0; group_size <= 65536.
 *   x_int_packed_ptr uint8 [batch_size, group_size/2]; scale_ptr bf16 [batch_size];
 *   x_int_row_sum_ptr int32 [batch_size] (may be NULL); x_ptr bf16 [batch_size, group_size] (read only)
 */
int hadamard_quantize_int4_cuda_bf16(void* x_int_packed_ptr, void* scale_ptr, void* x_int_row_sum_ptr,
                                     const void* x_ptr, int group_size, int batch_size, int block,
                                     cudaStream_t stream);

/*
 * hadamard_quantize_int4_cuda_bf16 with the producer of its input fused in: the rows that are transformed and quantised
 * are computed on the fly, so the producer's own kernels and one write + one read of [batch_size, group_size] bf16
 * disappear.  Outputs and their meaning are those of hadamard_quantize_int4_cuda_bf16 applied to y.
 *   rmsnorm_...   y = bf16( bf16(x * rsqrt(mean_k(x^2) + eps)) * norm_weight )    norm_weight bf16 [group_size]
 *                 (the model's RMSNorm, src/models/llama.py:64-76, feeding c_attn / w1 / w2)
 *   silu_mul_...  y = bf16( bf16(silu(gate)) * up ),  silu(v) = v / (1 + exp(-v)) in fp32    gate, up bf16 [batch, group]
 *                 (the SwiGLU product feeding c_proj, src/models/llama.py:118)
 * group_size a multiple of block and at most 32768; 16-byte aligned pointers; QB200_ERR_UNSUPPORTED otherwise.
 * No counterpart in the reference's op package (its layer code quantises a materialised activation tensor).
 */
int rmsnorm_hadamard_quantize_int4_cuda_bf16(void* x_int_packed_ptr, void* scale_ptr, void* x_int_row_sum_ptr,
                                             const void* x_ptr, const void* norm_weight_ptr, float eps, int group_size,
                                             int batch_size, int block, cudaStream_t stream);
int silu_mul_hadamard_quantize_int4_cuda_bf16(void* x_int_packed_ptr, void* scale_ptr, void* x_int_row_sum_ptr,
                                              const void* gate_ptr, const void* up_ptr, int group_size, int batch_size,
                                              int block, cudaStream_t stream);

/*
 * The whole layer in one call: hadamard_quantize_int4_cuda_bf16 into the caller's workspaces (a_int_packed uint8
 * [M, K/2], a_scale bf16 [M], a_int_row_sum int32 [M]; all required), then the fused GEMM + epilogue into mat_d
 * bf16 [M, N] - what gemm-quest/benchmarks/utils.py:89-100 does with four launches.  The GEMM kernel is launched with a
 * programmatic dependency on the quantiser: its blocks are scheduled while the quantiser's last blocks still run, set up
 * their barriers and tensor memory, request their first weights (which do not depend on the activations) and wait on the
 * device for the quantiser's end before they touch its outputs, so the gap between the two kernels disappears (at up to
 * 16 rows the layer costs little more than one launch).  Results are those of the two calls made one after the other.
 * w4a4_linear_hadamard_a8_bf16_cuda is the same for the int8-operand route (hadamard_quantize_a8_cuda_bf16 into a_int8
 * uint8 [M, K], then fused_matmul_dequantize_a8_int4t_bf16_cuda).  No counterpart in the reference.
 */
int w4a4_linear_hadamard_bf16_cuda(void* mat_d, const void* x, const void* w_int_packed, const void* w_add,
                                   const void* w_scale, void* a_int_packed, void* a_scale, void* a_int_row_sum, int M,
                                   int K, int N, int block, cudaStream_t stream);
int w4a4_linear_hadamard_a8_bf16_cuda(void* mat_d, const void* x, const void* w_int_packed, const void* w_add,
                                      const void* w_scale, void* a_int8, void* a_scale, void* a_int_row_sum, int M,
                                      int K, int N, int block, cudaStream_t stream);

/*
 * Layer mode, a state of the calling host thread.  Between quest_b200_begin_layer and quest_b200_end_layer the calls
 * hadamard_quantize_int4_cuda_bf16 / hadamard_quantize_a8_cuda_bf16 followed by a fused GEMM entry point
 * (fused_matmul_dequantize_*) launch their kernels as the one-call layer entry points above do - those are exactly
 * begin, the two calls, end: with programmatic dependencies where that was measured faster (the tcgen05 quantiser behind
 * the kernel before it and the GEMM behind that quantiser; behind the small CUDA-core quantiser only the GEMM, and only
 * below 3 M activation elements).  The GEMM then reads its weights (mat_b) before it waits on the device for the kernel
 * before it: the caller promises that between begin and end nothing else is launched into the stream between the
 * quantiser and the GEMM.  The package's column-sharded layer uses the pair around its quantiser and its push GEMM.
 * QB200_DEPENDENT_LAUNCH=0..3 in the environment forces the launches (bit 0 GEMM, bit 1 quantiser dependent).  No
 * counterpart in the reference.
 */
int quest_b200_begin_layer(void);
int quest_b200_end_layer(void);

/*
 * Copies one block of bf16 [rows, cols] (row stride ld elements in the source and in every destination) from src to
 * n_dst <= 7 destinations with one launch.  The column-sharded layer uses it for its few-row exchange: the block a rank
 * has computed goes into every peer's output buffer (peer memory mapped into this address space; plain 16-byte stores).
 * cols and ld must be multiples of 8 and every pointer 16-byte aligned (QB200_ERR_UNSUPPORTED otherwise).  No counterpart
 * in the reference.
 */
int quest_b200_copy_block_to_peers_cuda(const void* src, void* const* dsts, int n_dst, int rows, int cols, long long ld,
                                        cudaStream_t stream);

/*
 * out = bf16(H_block . x) blockwise along the last dimension (out may alias x).
 * weight_side == 0: entries +-bf16(block^-0.5), the activation-side matrix of
 * gemm-quest/benchmarks/utils.py:17,89-90.  weight_side != 0: entries +-fp32(block^-0.5), the
 * weight-side call hadamard_transform(..., scale=2**-3.5) of gemm-quest/benchmarks/utils.py:38-39.
 */
int hadamard_transform_cuda_bf16(void* out_ptr, const void* x_ptr, int group_size, int batch_size, int block,
                                 int weight_side, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* QUEST_B200_H_ */
