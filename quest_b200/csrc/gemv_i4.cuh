// int4 x int4 GEMM for very few activation rows (M <= 16, decode-like shapes) on the CUDA cores.  Included by
// gemm_i4.cu inside namespace qb.
//
// With so few rows the layer is a stream over the packed weights (N * K / 2 bytes, read once) and the tensor-core
// kernels spend most of their time on set-up and on walking K serially.  Here every warp owns C weight rows (output
// columns) at a time and splits K over its lanes: a lane loads 16 packed bytes (32 codes) per weight row and step,
// unpacks them to two int8x4 groups with the same "times sixteen" trick as the tensor-core path
// ((w << 4) & 0xF0F0F0F0 and w & 0xF0F0F0F0: sixteen times the low / high nibble codes, no sign extension needed),
// and multiplies them with dp4a against the activation rows, which the block has staged - packed - in shared memory.
// Both operands carry the factor 16, so the sums carry exactly 256 and are shifted back after the warp reduction
// (redux.sync); the fused epilogue is the same exact expression as everywhere else.
//
// Replaces, for these shapes, gemm-quest/quest/matmul_kernel.cu:8-63 and fused_matmul_dequantize_kernel.cu:4-57.
#pragma once

namespace gemv {
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxStageBytes = 112 * 1024;  // packed activations of all rows must fit in shared memory
}  // namespace gemv

__device__ __forceinline__ int redux_add(int v) {
    int r;
    asm volatile("redux.sync.add.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}

// MR: activation rows held (M <= MR; missing rows are zero).  C: weight rows per warp step (MR * C <= 32).
template <int MR, int C, bool FUSED>
__global__ void __launch_bounds__(gemv::kThreads)
gemv_i4_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B, const EpilogueParams ep, const int M,
               const int N, const int K) {
    extern __shared__ uint4 gemv_sA[];  // [MR][K / 32] chunks of 16 packed bytes
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = K >> 5;          // 32 codes = 16 bytes per chunk
    const size_t row_bytes = (size_t)(K >> 1);
    const int groups = (N + C - 1) / C;
    const int steps = (chunks + 31) >> 5;

    auto load_weights = [&](uint4 (&w)[C], int n0, int ch) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const bool in = ch < chunks && n0 + c < N;
            w[c] = in ? ld_stream16(B + (size_t)(n0 + c) * row_bytes + (size_t)ch * 16) : make_uint4(0, 0, 0, 0);
        }
    };

    // The first weights are requested before the activations are staged: both latencies overlap.
    int group = blockIdx.x * gemv::kWarps + warp;
    uint4 wcur[C];
    load_weights(wcur, group * C, group < groups ? lane : chunks);
    // Launched with a programmatic dependency on the kernel that quantises the activations (fused layer call), this
    // grid starts while that kernel still runs: everything up to here touches only the weights.  Now wait for it.
    wait_for_preceding_grid();
    for (int i = threadIdx.x; i < MR * chunks; i += gemv::kThreads) {
        const int r = i / chunks, ch = i - r * chunks;
        gemv_sA[i] = r < M ? *reinterpret_cast<const uint4*>(A + (size_t)r * row_bytes + (size_t)ch * 16) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();

    for (; group < groups; group += gridDim.x * gemv::kWarps) {
        const int n0 = group * C;
        int acc[MR][C];
#pragma unroll
        for (int m = 0; m < MR; ++m)
#pragma unroll
            for (int c = 0; c < C; ++c) acc[m][c] = 0;
        for (int j = 0; j < steps; ++j) {
            const int ch = lane + 32 * j;
            uint4 wnext[C];
            if (j + 1 < steps) {
                load_weights(wnext, n0, ch + 32);
            } else {  // the first step of this warp's next group
                const int g2 = group + gridDim.x * gemv::kWarps;
                load_weights(wnext, g2 * C, g2 < groups ? lane : chunks);
            }
            uint32_t wl[C][4], wh[C][4];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const uint32_t w4[4] = {wcur[c].x, wcur[c].y, wcur[c].z, wcur[c].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    wl[c][i] = (w4[i] << 4) & 0xF0F0F0F0u;
                    wh[c][i] = w4[i] & 0xF0F0F0F0u;
                }
            }
            if (ch < chunks) {
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const uint4 a = gemv_sA[m * chunks + ch];
                    const uint32_t a4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int al = (int)((a4[i] << 4) & 0xF0F0F0F0u), ah = (int)(a4[i] & 0xF0F0F0F0u);
#pragma unroll
                        for (int c = 0; c < C; ++c) {
                            acc[m][c] = __dp4a(al, (int)wl[c][i], acc[m][c]);
                            acc[m][c] = __dp4a(ah, (int)wh[c][i], acc[m][c]);
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < C; ++c) wcur[c] = wnext[c];
        }
        // warp totals; lane o keeps output (row o / C, column o % C)
        int mine = 0;
#pragma unroll
        for (int m = 0; m < MR; ++m)
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int t = redux_add(acc[m][c]);
                if (lane == m * C + c) mine = t;
            }
        const int m = lane / C, n = n0 + lane % C;
        if (lane < MR * C && m < M && n < N) {
            const int v = mine >> 8;  // exact: both operands carried the factor 16
            if (FUSED) {
                const float f = (float)(2 * v + ep.a_add[m] + ep.b_add[n]) * (0.5f * bf16_to_f32(ep.a_mul[m]) * bf16_to_f32(ep.b_mul[n]));
                static_cast<__nv_bfloat16*>(ep.out)[(size_t)m * ep.ld + n] = __float2bfloat16_rn(f);
            } else {
                static_cast<int32_t*>(ep.out)[(size_t)m * ep.ld + n] = v;
            }
        }
    }
}

// dp4a runs at half the CUDA-core rate, so the kernel is compute-bound from a few rows on: it is used while the whole
// product stays below 2^28 multiply-adds (~7 us of dp4a), beyond that the tensor-core kernels win (measured).
static bool gemv_eligible(int M, int K, int N, int n_peer) {
    if (M < 1 || M > 16 || n_peer != 0) return false;
    if ((long long)M * N * K > (1ll << 28)) return false;
    const int mr = M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : (M <= 8 ? 8 : 16)));
    return (size_t)mr * (size_t)(K / 2) <= (size_t)gemv::kMaxStageBytes;
}

template <int MR, int C, bool FUSED>
static int launch_gemv(const EpilogueParams& ep, const void* a, const void* b, int M, int K, int N, int sms, int dev,
                       cudaStream_t stream) {
    static bool attr_set[64] = {false};
    auto kernel = gemv_i4_kernel<MR, C, FUSED>;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemv::kMaxStageBytes) != cudaSuccess) {
            cudaGetLastError();
            return QB200_ERR_CUDA;
        }
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const size_t smem = (size_t)MR * (size_t)(K / 2);
    const int groups = (N + C - 1) / C;
    int grid = (groups + gemv::kWarps - 1) / gemv::kWarps;
    const int per_sm = smem > 100 * 1024 ? 1 : (smem > 48 * 1024 ? 2 : 4);
    if (grid > sms * per_sm) grid = sms * per_sm;
    if (launch_kernel(kernel, grid, gemv::kThreads, smem, stream, static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), ep, M, N, K) != cudaSuccess) {
        cudaGetLastError();
        return QB200_ERR_CUDA;
    }
    return launch_status();
}

template <bool FUSED>
static int run_gemv(const EpilogueParams& ep, const void* a, const void* b, int M, int K, int N, int sms, int dev,
                    cudaStream_t stream) {
    if (M <= 1) return launch_gemv<1, 4, FUSED>(ep, a, b, M, K, N, sms, dev, stream);
    if (M <= 2) return launch_gemv<2, 4, FUSED>(ep, a, b, M, K, N, sms, dev, stream);
    if (M <= 4) return launch_gemv<4, 4, FUSED>(ep, a, b, M, K, N, sms, dev, stream);
    if (M <= 8) return launch_gemv<8, 4, FUSED>(ep, a, b, M, K, N, sms, dev, stream);
    return launch_gemv<16, 2, FUSED>(ep, a, b, M, K, N, sms, dev, stream);
}
