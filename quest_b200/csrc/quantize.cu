// Row-wise kernels of the W4A4 linear path for sm_100a:
//   - fused block-Hadamard + RMS scale + int4 quantise + pack + row-sum (one pass over x),
//   - the reference's unfused find_scale_int4 / quantize_int4 (same kernel, other template arms),
//   - add_mul_vv (the exact dequantising epilogue as a standalone kernel).
//
// All of them are HBM-bandwidth bound.  One thread block owns one row; every lane owns runs of 32
// contiguous elements (four 16-byte loads, one 16-byte packed store), a "unit" being the 1024
// elements a warp covers at once.  The whole row stays in registers (as bf16 pairs) between the
// sum-of-squares pass and the quantise pass, so x is read from HBM exactly once.
//
// Numerics follow gemm-quest/quest/quantize_kernel.cu and gemm-quest/benchmarks/utils.py:
//   two rounding points decide the codes - the Hadamard output is rounded to bf16 before anything
//   else looks at it, and the scale is rounded to bf16 before the divide.
#include "common.cuh"
#include "tcgen05.cuh"

namespace qb {

thread_local bool qb_tl_dependent_quantiser = false;
thread_local int qb_tl_quantiser_kernel = 0;

struct RowParams {
    const __nv_bfloat16* x;        // [M,K] input
    __nv_bfloat16* x_out;          // optional [M,K] output (transformed or dequantised values)
    const __nv_bfloat16* scale_in; // optional [M] scale to quantise with
    __nv_bfloat16* scale_out;      // optional [M] computed scale
    int8_t* q_dense;               // optional [M,K]
    uint8_t* q_packed;             // optional [M,K/2]
    uint8_t* q_a8;                 // optional [M,K]: sixteen times the codes as int8, in the GEMM's operand order (tcgen05 kernel only)
    int32_t* row_sum;              // optional [M]
    int K;
    int M;
    const __nv_bfloat16* x2;       // producer-fused kernels: second input [M,K] (the "up" branch of SiLU(gate) * up)
    const __nv_bfloat16* norm_w;   // producer-fused kernels: RMSNorm weight [K]
    float norm_eps;                // RMSNorm epsilon
    float had_scale;               // Hadamard normalisation constant
    int x_out_mode;                // 0 none, 1 transformed values, 2 dequantised values
    int quantize;                  // 0: stop after the scale (find_scale / transform only)
};

constexpr int kUnit = 1024;        // elements per warp-unit
constexpr int kMaxVectorK = 64 * kUnit;  // 16 warps x 4 units; longer rows take the scalar kernel
constexpr float kFloorMagic = 12582912.0f;  // 1.5 * 2^23: adding it (round-down) leaves floor(y) in the low mantissa bits
constexpr int kFloorMagicBits = 0x4B400000;

// floor(x / s) for bf16-valued x and s, without a divide.
//
// x / s is an exact integer for about 1 % of the elements, so a plain x * (1/s) mis-floors.  For
// bf16 operands every non-integer quotient of magnitude <= 8 is at least 2^-9 away from an integer,
// while x * rcp(s) is within 2^-22 relative of the true quotient; nudging the product by
// |y| * 2^-13 towards +inf therefore lands exact integers on or above themselves and moves nothing
// else across an integer (and keeps the sign of tiny quotients, so -tiny still floors to -1).
// Verified exhaustively over all pairs of bf16 mantissas and the exponent differences that matter.
// Returns floor as an int; out-of-range quotients keep their sign and saturate later.
__device__ __forceinline__ int floor_quotient(float x, float inv_s) {
    const float y = x * inv_s;
    const float y2 = fmaf(fabsf(y), 1.220703125e-4f, y);
    return __float_as_int(__fadd_rd(y2, kFloorMagic)) - kFloorMagicBits;
}

// Same as floor_quotient but returns the raw bits of the magic-number sum: for |x/s| < 2^22 the low bits are
// floor(x/s) in two's complement, so for a pre-clamped x the low nibble is the int4 code.
__device__ __forceinline__ uint32_t floor_quotient_bits(float x, float inv_s) {
    const float y = x * inv_s;
    const float y2 = fmaf(fabsf(y), 1.220703125e-4f, y);
    return __float_as_uint(__fadd_rd(y2, kFloorMagic));
}

// Element-wise clamp of a bf16 pair to [lo, hi] (both given as bf16 pairs).
__device__ __forceinline__ uint32_t clamp_bf16x2(uint32_t v, uint32_t lo, uint32_t hi) {
    uint32_t r;
    asm("{\n\t.reg .b32 t;\n\tmax.bf16x2 t, %1, %2;\n\tmin.bf16x2 %0, t, %3;\n\t}" : "=r"(r) : "r"(v), "r"(lo), "r"(hi));
    return r;
}

// (sat4(a) << 4 | sat4(b)) | (c << 8): saturating pack of two int32 to signed nibbles.
__device__ __forceinline__ uint32_t pack_sat_s4(int hi, int lo, uint32_t c) {
    uint32_t d;
    asm("cvt.pack.sat.s4.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(c));
    return d;
}

// Sum of the eight signed nibbles of w, times 16, accumulated into acc.
__device__ __forceinline__ int nibble_sum16(uint32_t w, int acc) {
    const uint32_t lo = (w << 4) & 0xF0F0F0F0u;
    const uint32_t hi = w & 0xF0F0F0F0u;
    acc = __dp4a((int)lo, 0x01010101, acc);
    acc = __dp4a((int)hi, 0x01010101, acc);
    return acc;
}

template <int HB>
__device__ __forceinline__ void hadamard32(float (&f)[32], int lane) {
    // Index bits 0..4 live in registers.
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if ((i & s) == 0) {
                const float a = f[i], b = f[i + s];
                f[i] = a + b;
                f[i + s] = a - b;
            }
        }
    }
    // The remaining log2(HB/32) index bits are lane bits: butterfly through warp shuffles.
#pragma unroll
    for (int m = 1; m < HB / 32; m <<= 1) {
        const float sgn = (lane & m) ? -1.f : 1.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float p = __shfl_xor_sync(0xffffffffu, f[i], m);
            f[i] = fmaf(f[i], sgn, p);  // lower lane: a + b, upper lane: a - b
        }
    }
}

// HB: Hadamard block (0 = none).  UNITS: 1024-element units per warp.  EXTRAS: compile the rarely
// used outputs (dense int8 codes, transformed / dequantised bf16 values).
template <int HB, int UNITS, bool EXTRAS>
__global__ void __launch_bounds__(UNITS == 1 ? 256 : 512) row_kernel(const RowParams p) {
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int K = p.K;
    const __nv_bfloat16* xr = p.x + (size_t)row * K;

    __shared__ double red_f[32];
    __shared__ int red_i[32];

    uint32_t v[UNITS][16];  // the lane's elements as bf16 pairs, after the transform
    float ssq = 0.f;

    // Issue every load of the row before touching the data.
    uint4 raw[UNITS][4];
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int e0 = (u * nwarps + warp) * kUnit + lane * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            raw[u][j] = make_uint4(0, 0, 0, 0);
            if (e0 + 8 * j < K) {
                // The EXTRAS arms may write x in place, so they use ordinary (coherent) loads.
                if (EXTRAS) raw[u][j] = *reinterpret_cast<const uint4*>(xr + e0 + 8 * j);
                else raw[u][j] = ld_stream16(xr + e0 + 8 * j);
            }
        }
    }

#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw[u][0]);
        if (HB > 0) {
            float f[32];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                f[2 * i] = bf16lo_to_f32(w[i]);
                f[2 * i + 1] = bf16hi_to_f32(w[i]);
            }
            hadamard32<HB>(f, lane);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[u][i] = pack_bf16x2(f[2 * i] * p.had_scale, f[2 * i + 1] * p.had_scale);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[u][i] = w[i];
        }
        if (p.scale_in == nullptr) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float a = bf16lo_to_f32(v[u][i]), b = bf16hi_to_f32(v[u][i]);
                ssq = fmaf(a, a, ssq);
                ssq = fmaf(b, b, ssq);
            }
        }
    }

    // ---- scale ----
    float s;
    if (p.scale_in != nullptr) {
        s = bf16_to_f32(p.scale_in[row]);
    } else {
        double t = (double)ssq;
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
        if (lane == 0) red_f[warp] = t;
        __syncthreads();
        double tot = 0.0;
        for (int i = 0; i < nwarps; ++i) tot += red_f[i];
        const float mean_sq = (float)(tot / (double)K);
        const __nv_bfloat16 sb = __float2bfloat16_rn(quest_scale_from_mean_square(mean_sq));
        if (threadIdx.x == 0 && p.scale_out != nullptr) p.scale_out[row] = sb;
        s = bf16_to_f32(sb);
    }

    if (EXTRAS && p.x_out_mode == 1) {
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const int e0 = (u * nwarps + warp) * kUnit + lane * 32;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (e0 + 8 * j < K)
                    *reinterpret_cast<uint4*>(p.x_out + (size_t)row * K + e0 + 8 * j) =
                        make_uint4(v[u][4 * j], v[u][4 * j + 1], v[u][4 * j + 2], v[u][4 * j + 3]);
        }
    }
    if (!p.quantize) return;

    // ---- quantise, pack, row sum ----
    const float inv_s = __frcp_rn(s);
    const bool vec_store = (K & 31) == 0;
    int rs16 = 0;
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int e0 = (u * nwarps + warp) * kUnit + lane * 32;
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int q[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q[2 * i] = floor_quotient(bf16lo_to_f32(v[u][4 * j + i]), inv_s);
                q[2 * i + 1] = floor_quotient(bf16hi_to_f32(v[u][4 * j + i]), inv_s);
            }
            uint32_t d = pack_sat_s4(q[7], q[6], 0u);
            d = pack_sat_s4(q[5], q[4], d);
            d = pack_sat_s4(q[3], q[2], d);
            d = pack_sat_s4(q[1], q[0], d);
            pk[j] = d;
            rs16 = nibble_sum16(d, rs16);  // padding lanes hold zeros: code 0, adds nothing

            if (EXTRAS && e0 + 8 * j < K) {
                if (p.q_dense != nullptr) {
                    uint32_t lo = 0, hi = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        lo |= (uint32_t)(min(max(q[i], -8), 7) & 0xFF) << (8 * i);
                        hi |= (uint32_t)(min(max(q[4 + i], -8), 7) & 0xFF) << (8 * i);
                    }
                    *reinterpret_cast<uint2*>(p.q_dense + (size_t)row * K + e0 + 8 * j) = make_uint2(lo, hi);
                }
                if (p.x_out_mode == 2) {
                    uint32_t o[4];
                    const float half_s = s * 0.5f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float a = fmaf((float)min(max(q[2 * i], -8), 7), s, half_s);
                        const float b = fmaf((float)min(max(q[2 * i + 1], -8), 7), s, half_s);
                        o[i] = pack_bf16x2(a, b);
                    }
                    *reinterpret_cast<uint4*>(p.x_out + (size_t)row * K + e0 + 8 * j) =
                        make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        }
        if (p.q_packed != nullptr) {
            uint8_t* dst = p.q_packed + (size_t)row * (K >> 1) + (e0 >> 1);
            if (vec_store) {
                if (e0 < K) *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (e0 + 8 * j < K) *reinterpret_cast<uint32_t*>(dst + 4 * j) = pk[j];
            }
        }
    }
    if (p.row_sum != nullptr) {
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) rs16 += __shfl_xor_sync(0xffffffffu, rs16, m);
        if (lane == 0) red_i[warp] = rs16;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int i = 0; i < nwarps; ++i) tot += red_i[i];
            p.row_sum[row] = tot >> 4;  // exact: every term is a multiple of 16
        }
    }
}

// -------------------------------------------------------------------------------------------------
// The hot path: fused Hadamard + scale + quantise + pack + row sum, tensor-core assisted.
//
// The shuffle-butterfly kernel above spends ~26 instructions per element and is issue-bound at well
// under half of the HBM bandwidth.  Here the block transform is factored as H_block = H_a (x) H_16:
// the 16-point factor over the low four index bits is a tiny bf16 MMA (mma.sync m16n8k16, A = sixteen
// contiguous activations per row, B = +-bf16(block^-0.5) Sylvester signs, fp32 accumulate - the same
// "x times Hadamard matrix" product the reference hands to cuBLAS), and the factor over the high index
// bits is a butterfly over values a thread already holds.  Data path per warp and 1024 elements:
//   cp.async 16 B/lane global -> warp-private shared memory (blocks padded to 272 B: conflict-free)
//   ldmatrix x4  -> A fragments, 8 MMAs -> 32 fp32 values per thread (8 high-index rows x 4 columns)
//   butterflies, round to bf16 pairs (kept in registers until the row's scale is known)
//   quantise -> 2-byte pieces -> warp-private shared staging -> one coalesced 16-byte store per lane.
// -------------------------------------------------------------------------------------------------
constexpr int kBlkPitch = 272;              // 256-byte block of 128 bf16 + 16 bytes of padding
constexpr int kStepIn = 8 * kBlkPitch;      // eight blocks per warp step
constexpr int kOutPitch = 80;               // 64 packed bytes per block + 16 bytes of padding
constexpr int kMaxDynSmem = 220 * 1024;  // leaves room for the static reduction arrays under the 227 KB limit
constexpr int kStepBytes = 2 * kStepIn;  // two input buffers (the next row is prefetched); the packed codes are
                                         // staged in the buffer that has just been consumed

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// Thread-block shape: G row groups x W warps.  The W warps of a group share one row (UNITS 1024-element
// units per warp); the block walks over batches of G rows.  Everything that is per row rather than per
// element (summing the partial sums, sqrt, rounding the scale, its reciprocal, the clamp bounds) is a short
// float chain that every warp evaluates for its own row right after the one barrier that publishes the partial
// sums; the final row sums are written one batch later by warp 0.
#ifdef QB200_TRACE
// Tuning builds only: earliest block start, latest start, earliest end and latest end (globaltimer, ns) of the last launch.
__device__ unsigned long long g_hq_trace[6] = {~0ull, 0ull, ~0ull, 0ull, ~0ull, 0ull};  // [4], [5]: first accumulator ready (tcgen05 kernel)
__device__ __forceinline__ unsigned long long hq_gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#endif

// Packed fp32 pairs (sm_100 executes add/sub/mul/fma on two floats per instruction).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpk2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { f32x2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 add2_rd(f32x2 a, f32x2 b) { f32x2 r; asm("add.rm.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }

// PRO: what produces the rows that are transformed and quantised.
//   0  the input itself.
//   1  RMSNorm of the input:  y = bf16( bf16(x * rsqrt(mean(x^2) + eps)) * w )   (src/models/llama.py:64-76: the
//      normalised value is cast back to the activation type before the weight multiplies it).
//   2  SwiGLU gate:           y = bf16( bf16(silu(x)) * x2 ),  silu(x) = x / (1 + exp(-x)) in fp32
//      (src/models/llama.py:118, torch's silu for bf16 inputs).
// The producer rewrites the row in shared memory, in place, between the copy and the tensor-core stage; everything
// after it is unchanged.  It saves the producer's own kernel(s), one write and one read of [M, K] bf16.
constexpr int kProNone = 0, kProRmsNorm = 1, kProSiluMul = 2;

template <int HB, int UNITS, int PRO = kProNone>
__global__ void __launch_bounds__(256, UNITS == 1 ? 4 : (UNITS == 2 ? 3 : 2))
hadamard_quant_mma_kernel(const RowParams p, const int W, const int G, const int nbuf) {
    extern __shared__ __align__(16) uint8_t hq_smem[];
    __shared__ float part_ssq[2][8];  // indexed by batch parity: one barrier per batch is enough
    __shared__ int part_rs[2][8];
    __shared__ float part_norm[8];    // PRO == kProRmsNorm: the warps' partial sums of squares of the raw row

#ifdef QB200_TRACE
    if (threadIdx.x == 0) {
        const unsigned long long t = hq_gtime();
        atomicMin(&g_hq_trace[0], t);
        atomicMax(&g_hq_trace[1], t);
    }
#endif
    // A kernel launched behind this one with a programmatic dependency (the small-M GEMM of the fused layer call) may
    // start its own prologue now; it waits for this grid's results itself.  Without such a dependent this does nothing.
    let_dependents_launch();
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int grp = warp / W;      // row group of this warp
    const int wig = warp - grp * W;  // warp index within the group
    const int g = lane >> 2, tig = lane & 3;
    const int K = p.K, M = p.M;
    // nbuf = 2: the next row's copies are in flight while this row is processed.  nbuf = 1 (every row batch of the
    // launch is resident at once, nothing to prefetch): half the shared memory, twice the blocks per SM.
    const int step_bytes = nbuf * kStepIn;
    const uint32_t smem_w = (uint32_t)__cvta_generic_to_shared(hq_smem) + warp * (UNITS * step_bytes);
    const int num_batches = (M + G - 1) / G;

    // Copies of this warp's units of one row into input buffer `buf` (16 bytes per lane and instruction).
    auto issue_row = [&](int row, int buf) {
        if (row < M) {
            const __nv_bfloat16* xr = p.x + (size_t)row * K;
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int unit = u * W + wig;
                const uint32_t in_base = smem_w + u * step_bytes + buf * kStepIn;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = j * 32 + lane;  // 16-byte chunk within the unit
                    const int e = unit * kUnit + c * 8;
                    const bool valid = e < K;
                    cp_async16_zfill(in_base + (c >> 4) * kBlkPitch + (c & 15) * 16,
                                     valid ? (const void*)(xr + e) : (const void*)xr, valid);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    int batch = blockIdx.x;
    if (batch < num_batches) issue_row(batch * G + grp, 0);

    // ---- B fragments: h * H16[k][o], MMA column n of tile nu is output o = 4*(n>>1) + 2*nu + (n&1) ----
    uint32_t bfrag[2][2];
    {
        const uint32_t hb = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(p.had_scale));
#pragma unroll
        for (int nu = 0; nu < 2; ++nu) {
            const int o = 4 * (g >> 1) + 2 * nu + (g & 1);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int k0 = 2 * tig + 8 * half;
                const uint32_t lo = hb | ((__popc(k0 & o) & 1) ? 0x8000u : 0u);
                const uint32_t hi = hb | ((__popc((k0 + 1) & o) & 1) ? 0x8000u : 0u);
                bfrag[nu][half] = lo | (hi << 16);
            }
        }
    }

    int prev_batch = -1, last_par = 0;
    for (int it = 0; batch < num_batches; batch += gridDim.x, ++it) {
        const int buf = nbuf == 2 ? (it & 1) : 0;
        const int row = batch * G + grp;
        const int next = batch + gridDim.x;
        if (nbuf == 2 && next < num_batches) {
            issue_row(next * G + grp, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            if (nbuf == 1 && it > 0) issue_row(row, 0);  // single buffer: fetch this row now (the staging reads are done)
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();

        if (PRO != kProNone) {
            // Each lane owns the 16-byte chunks it copied itself (chunk c = 32 j + lane of every unit).
            float rinv = 0.f;
            if (PRO == kProRmsNorm) {
                float nsq = 0.f;
#pragma unroll
                for (int u = 0; u < UNITS; ++u) {
                    const uint32_t in_base = smem_w + u * step_bytes + buf * kStepIn;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int c = j * 32 + lane;
                        const uint4 q = lds128(in_base + (c >> 4) * kBlkPitch + (c & 15) * 16);  // zero beyond K
                        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float a = bf16lo_to_f32(w4[i]), b = bf16hi_to_f32(w4[i]);
                            nsq = fmaf(a, a, nsq);
                            nsq = fmaf(b, b, nsq);
                        }
                    }
                }
#pragma unroll
                for (int m2 = 16; m2 > 0; m2 >>= 1) nsq += __shfl_xor_sync(0xffffffffu, nsq, m2);
                if (W > 1) {  // block-uniform: the row is spread over W warps
                    if (lane == 0) part_norm[warp] = nsq;
                    __syncthreads();
                    nsq = 0.f;
                    for (int i = 0; i < W; ++i) nsq += part_norm[grp * W + i];
                    __syncthreads();  // part_norm is rewritten for the next batch
                }
                rinv = rsqrtf(__fdiv_rn(nsq, (float)K) + p.norm_eps);
            }
            const int row_p = batch * G + grp;
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int unit = u * W + wig;
                const uint32_t in_base = smem_w + u * step_bytes + buf * kStepIn;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = j * 32 + lane;
                    const int e = unit * kUnit + c * 8;
                    if (e >= K || row_p >= M) continue;
                    const uint32_t addr = in_base + (c >> 4) * kBlkPitch + (c & 15) * 16;
                    const uint4 q = lds128(addr);
                    const uint4 o = PRO == kProRmsNorm ? __ldg(reinterpret_cast<const uint4*>(p.norm_w + e))
                                                       : ld_stream16(p.x2 + (size_t)row_p * K + e);
                    const uint32_t w4[4] = {q.x, q.y, q.z, q.w}, o4[4] = {o.x, o.y, o.z, o.w};
                    uint32_t y4[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float a = bf16lo_to_f32(w4[i]), b = bf16hi_to_f32(w4[i]);
                        if (PRO == kProRmsNorm) {
                            a *= rinv;
                            b *= rinv;
                        } else {
                            a = __fdiv_rn(a, 1.f + expf(-a));
                            b = __fdiv_rn(b, 1.f + expf(-b));
                        }
                        const uint32_t t = pack_bf16x2(a, b);  // the producer's first rounding to the activation type
                        y4[i] = pack_bf16x2(bf16lo_to_f32(t) * bf16lo_to_f32(o4[i]), bf16hi_to_f32(t) * bf16hi_to_f32(o4[i]));
                    }
                    sts128(addr, make_uint4(y4[0], y4[1], y4[2], y4[3]));
                }
            }
            __syncwarp();  // ldmatrix below reads chunks written by other lanes of this warp
        }

        uint32_t v[UNITS][16];  // v[u][2a + nu]: elements 16a + 4tig + 2nu (+1) of block g of the unit
        f32x2 ssq2 = 0ull;
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const uint32_t in_base = smem_w + u * step_bytes + buf * kStepIn;
            f32x2 f[8][2];  // f[a][h]: elements 16a + 4tig + 2h, +1 of block g, as packed float pairs
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                uint32_t a[4];
                ldmatrix_x4(in_base + (lane & 7) * kBlkPitch + (2 * t + ((lane >> 3) & 1)) * 32 + (lane >> 4) * 16, a);
#pragma unroll
                for (int nu = 0; nu < 2; ++nu) {
                    float d[4];
                    mma_bf16_16816(d, a, bfrag[nu][0], bfrag[nu][1]);
                    f[2 * t][nu] = pk2(d[0], d[1]);
                    f[2 * t + 1][nu] = pk2(d[2], d[3]);
                }
            }
            // remaining index bits 4.. of the block: butterflies over the row index a (in registers)
#pragma unroll
            for (int s = 1; s < 8 && s < HB / 16; s <<= 1) {
#pragma unroll
                for (int a = 0; a < 8; ++a) {
                    if ((a & s) == 0) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const f32x2 x0 = f[a][h], x1 = f[a + s][h];
                            f[a][h] = add2(x0, x1);
                            f[a + s][h] = sub2(x0, x1);
                        }
                    }
                }
            }
            if (HB == 256) {  // index bit 7 pairs neighbouring 128-element halves: lanes g and g ^ 1
                const float sgn = (g & 1) ? -1.f : 1.f;
#pragma unroll
                for (int a = 0; a < 8; ++a)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float x0, x1;
                        unpk2(f[a][h], x0, x1);
                        const float p0 = __shfl_xor_sync(0xffffffffu, x0, 4);
                        const float p1 = __shfl_xor_sync(0xffffffffu, x1, 4);
                        f[a][h] = pk2(fmaf(x0, sgn, p0), fmaf(x1, sgn, p1));
                    }
            }
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float x0, x1;
                    unpk2(f[a][h], x0, x1);
                    v[u][2 * a + h] = pack_bf16x2(x0, x1);
                }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const f32x2 xx = pk2(bf16lo_to_f32(v[u][i]), bf16hi_to_f32(v[u][i]));
                ssq2 = fma2(xx, xx, ssq2);
            }
        }
        float ssq;
        {
            float s0, s1;
            unpk2(ssq2, s0, s1);
            ssq = s0 + s1;
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, m);
        const int par = it & 1;
        if (lane == 0) part_ssq[par][warp] = ssq;
        __syncthreads();  // the partial sums of this batch (and the row-sum partials of the previous one) are in place

        // Every warp derives its row's constants itself (a short float chain, W partial sums): no second barrier
        // and nobody waits for a designated warp.  Warp 0 additionally publishes the scales and finishes the row
        // sums of the previous batch, off everyone's critical path.
        double tot = 0.0;
        for (int i = 0; i < W; ++i) tot += (double)part_ssq[par][grp * W + i];
        const __nv_bfloat16 sb = __float2bfloat16_rn(quest_scale_from_mean_square(__fdiv_rn((float)tot, (float)K)));
        const float s_f = bf16_to_f32(sb);
        const float inv_s = __frcp_rn(s_f);
        // Saturation is done on the bf16 pairs before the divide: x is clamped to [-8s, ~7.5s], both bounds
        // exact or safely inside [7s, 8s), so floor(x/s) lands in [-8, 7] without integer min/max, and the
        // code is simply the low nibble of the magic-number sum.
        const uint32_t lo1 = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(-8.f * s_f));
        const uint32_t hi1 = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(7.5f * s_f));
        const uint32_t lo2 = lo1 | (lo1 << 16), hi2 = hi1 | (hi1 << 16);
        const f32x2 inv_s2 = pk2(inv_s, inv_s), magic2 = pk2(kFloorMagic, kFloorMagic);
        if (wig == 0 && lane == 0 && row < M) p.scale_out[row] = sb;
        if (warp == 0 && lane < G && prev_batch >= 0 && p.row_sum != nullptr) {
            const int pr = prev_batch * G + lane;
            if (pr < M) {
                int t2 = 0;
                for (int i = 0; i < W; ++i) t2 += part_rs[par ^ 1][lane * W + i];
                p.row_sum[pr] = t2 >> 4;  // exact: every term is a multiple of 16
            }
        }

        // ---- quantise, stage, store ----
        const bool vec_store = (K & 31) == 0;
        int rs16 = 0;
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
            const int unit = u * W + wig;
            const uint32_t out_base = smem_w + u * step_bytes + buf * kStepIn;  // input already consumed
#pragma unroll
            for (int pr = 0; pr < 4; ++pr) {  // rows a = 2pr and 2pr + 1: eight codes -> one 32-bit word
                uint32_t ub[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t c = clamp_bf16x2(v[u][4 * pr + i], lo2, hi2);
                    float y0, y1;
                    unpk2(mul2(pk2(bf16lo_to_f32(c), bf16hi_to_f32(c)), inv_s2), y0, y1);
                    // nudge towards +inf by |y| * 2^-13 (see floor_quotient), then floor through the magic-number sum
                    const f32x2 fl = add2_rd(pk2(fmaf(fabsf(y0), 1.220703125e-4f, y0), fmaf(fabsf(y1), 1.220703125e-4f, y1)), magic2);
                    float u0, u1;
                    unpk2(fl, u0, u1);
                    ub[2 * i] = __float_as_uint(u0);
                    ub[2 * i + 1] = __float_as_uint(u1);
                }
                // ub[0..3] = row 2pr elements 0..3, ub[4..7] = row 2pr+1 elements 0..3; code = low nibble
                const uint32_t ev = __byte_perm(__byte_perm(ub[0], ub[2], 0x0040), __byte_perm(ub[4], ub[6], 0x0040), 0x5410);
                const uint32_t od = __byte_perm(__byte_perm(ub[1], ub[3], 0x0040), __byte_perm(ub[5], ub[7], 0x0040), 0x5410);
                const uint32_t word = (ev & 0x0F0F0F0Fu) | ((od << 4) & 0xF0F0F0F0u);
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(out_base + g * kOutPitch + pr * 16 + tig * 4), "r"(word) : "memory");
            }
            __syncwarp();
            uint4 t4;  // lane reads rows (2c, 2c+1) of block lane>>2, c = lane&3: one word per source thread tig
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(t4.x), "=r"(t4.y), "=r"(t4.z), "=r"(t4.w) : "r"(out_base + (lane >> 2) * kOutPitch + (lane & 3) * 16));
            __syncwarp();  // the staging area is rewritten for the next row
            uint4 w;   // low halves are row 2c (bytes 2tig, 2tig+1), high halves row 2c+1
            w.x = __byte_perm(t4.x, t4.y, 0x5410);
            w.y = __byte_perm(t4.z, t4.w, 0x5410);
            w.z = __byte_perm(t4.x, t4.y, 0x7632);
            w.w = __byte_perm(t4.z, t4.w, 0x7632);
            rs16 = nibble_sum16(w.x, rs16);
            rs16 = nibble_sum16(w.y, rs16);
            rs16 = nibble_sum16(w.z, rs16);
            rs16 = nibble_sum16(w.w, rs16);
            const int e0 = unit * kUnit + lane * 32;
            if (row < M) {
                uint8_t* dst = p.q_packed + (size_t)row * (K >> 1) + (e0 >> 1);
                if (vec_store) {
                    if (e0 < K) *reinterpret_cast<uint4*>(dst) = w;
                } else {
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (e0 + 8 * j < K) *reinterpret_cast<uint32_t*>(dst + 4 * j) = ww[j];
                }
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) rs16 += __shfl_xor_sync(0xffffffffu, rs16, m);
        if (lane == 0) part_rs[par][warp] = rs16;
        prev_batch = batch;
        last_par = par;
    }
    // row sums of the last batch
    __syncthreads();
#ifdef QB200_TRACE
    if (threadIdx.x == 0) {
        const unsigned long long t = hq_gtime();
        atomicMin(&g_hq_trace[2], t);
        atomicMax(&g_hq_trace[3], t);
    }
#endif
    if (warp == 0 && lane < G && prev_batch >= 0 && p.row_sum != nullptr) {
        const int pr = prev_batch * G + lane;
        if (pr < M) {
            int t2 = 0;
            for (int i = 0; i < W; ++i) t2 += part_rs[last_par][lane * W + i];
            p.row_sum[pr] = t2 >> 4;
        }
    }
}

template <int HB, bool EXTRAS>
static int launch_row(const RowParams& p, cudaStream_t stream);

template <int HB, int PRO = kProNone>
static int launch_hq_mma(const RowParams& p, cudaStream_t stream) {
    const int units = (p.K + kUnit - 1) / kUnit;
    // units per warp, warps per row, rows per block (at most 16 warps per block)
    int per = units >= 2 ? 2 : 1;  // two units per warp amortise the per-row work best (measured)
    if (per > units) per = units;
    if (per != 1 && per != 2 && per != 4) per = 2;
    int W = (units + per - 1) / per;
    if (W > 8 && per < 4) { per = 4; W = (units + per - 1) / per; }
    if (W > 8) return PRO != kProNone ? QB200_ERR_UNSUPPORTED : launch_row<HB, false>(p, stream);  // very long rows: shuffle-butterfly kernel
    // Rows per block: up to 8 warps per block, but few rows overall want small blocks so that every SM ends
    // at the same time (a block is the unit the rows are dealt out in).
    int G = 8 / W;
    if (G < 1) G = 1;
    while (G > 1 && (long long)p.M < 96LL * 148 * G) G >>= 1;
    if (G > p.M) G = p.M;
    const int warps = W * G;
    const long long batches = ((long long)p.M + G - 1) / G;
    if ((size_t)warps * per * kStepBytes > kMaxDynSmem) return PRO != kProNone ? QB200_ERR_UNSUPPORTED : launch_row<HB, false>(p, stream);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return QB200_ERR_CUDA;
    {
        static int cached[64] = {0};
        if (dev >= 0 && dev < 64 && cached[dev] > 0) sms = cached[dev];
        else if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) {
            if (dev >= 0 && dev < 64) cached[dev] = sms;
        } else sms = 148;
    }
    // Persistent grid: as many blocks as fit on the device at once (bounded by the number of row batches).
    // The caches are per kernel instantiation (index `which`) and per device.
    static bool attr_done[3][64] = {{false}};
    static int occ_cache[3][64][9][2] = {{{{0}}}};
    auto launch = [&](auto kernel, int which) -> int {
        const bool dev_ok = dev >= 0 && dev < 64;
        if (!(dev_ok && attr_done[which][dev])) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) != cudaSuccess) {
                cudaGetLastError();  // reported through the return value; do not leave it pending
                return QB200_ERR_CUDA;
            }
            if (dev_ok) attr_done[which][dev] = true;
        }
        auto occupancy = [&](int nb) {
            int occ = dev_ok ? occ_cache[which][dev][warps][nb - 1] : 0;
            if (occ <= 0) {
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, 32 * warps, (size_t)warps * per * nb * kStepIn) != cudaSuccess || occ <= 0) {
                    cudaGetLastError();
                    occ = 1;
                }
                if (dev_ok) occ_cache[which][dev][warps][nb - 1] = occ;
            }
            return occ;
        };
        // If every row batch fits on the device at once there is nothing to prefetch: use one input buffer.
        int nbuf = 2;
        long long grid = (long long)sms * occupancy(2);
        if (batches > grid && batches <= (long long)sms * occupancy(1)) {
            nbuf = 1;
            grid = (long long)sms * occupancy(1);
        }
        if (grid > batches) grid = batches;
        // Always an ordinary launch: behind a programmatic dependency this small kernel measured slower (M = 16, K = N =
        // 4096, layers back to back: 16.6 instead of 13.5 us per layer); only the tcgen05 kernel is launched that way.
        if (launch_kernel_dep(false, kernel, grid, 32 * warps, (size_t)warps * per * nbuf * kStepIn, stream, p, W, G, nbuf) != cudaSuccess) {
            cudaGetLastError();
            return QB200_ERR_CUDA;
        }
        return launch_status();
    };
    if (per == 1) return launch(hadamard_quant_mma_kernel<HB, 1, PRO>, 0);
    if (per == 2) return launch(hadamard_quant_mma_kernel<HB, 2, PRO>, 1);
    return launch(hadamard_quant_mma_kernel<HB, 4, PRO>, 2);
}

// Any K, any alignment, no Hadamard: one block per row, scalar accesses.  Only used for shapes the
// vector kernel does not cover (K not a multiple of 8, misaligned base pointers, K > 65536).
__global__ void __launch_bounds__(256) row_kernel_generic(const RowParams p) {
    const int row = blockIdx.x;
    const int K = p.K;
    const __nv_bfloat16* xr = p.x + (size_t)row * K;
    __shared__ double red_f[8];
    __shared__ int red_i[8];
    __shared__ float s_sh;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float s;
    if (p.scale_in != nullptr) {
        s = bf16_to_f32(p.scale_in[row]);
    } else {
        double t = 0.0;
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
            const float a = bf16_to_f32(xr[k]);
            t += (double)(a * a);
        }
        for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
        if (lane == 0) red_f[warp] = t;
        __syncthreads();
        if (threadIdx.x == 0) {
            double tot = 0.0;
            for (int i = 0; i < 8; ++i) tot += red_f[i];
            const __nv_bfloat16 sb = __float2bfloat16_rn(quest_scale_from_mean_square((float)(tot / (double)K)));
            if (p.scale_out != nullptr) p.scale_out[row] = sb;
            s_sh = bf16_to_f32(sb);
        }
        __syncthreads();
        s = s_sh;
    }
    if (!p.quantize) return;
    const float inv_s = __frcp_rn(s);
    int rs = 0;
    // Each thread owns pairs of columns so that it can emit whole packed bytes.
    for (int k = 2 * threadIdx.x; k < K; k += 2 * blockDim.x) {
        int q[2] = {0, 0};
        for (int i = 0; i < 2; ++i) {
            if (k + i < K) {
                q[i] = min(max(floor_quotient(bf16_to_f32(xr[k + i]), inv_s), -8), 7);
                rs += q[i];
                if (p.q_dense != nullptr) p.q_dense[(size_t)row * K + k + i] = (int8_t)q[i];
                if (p.x_out_mode == 2)
                    p.x_out[(size_t)row * K + k + i] = __float2bfloat16_rn(fmaf((float)q[i], s, s * 0.5f));
            }
        }
        if (p.q_packed != nullptr && k + 1 < K)
            p.q_packed[(size_t)row * (K >> 1) + (k >> 1)] = (uint8_t)((q[1] << 4) | (q[0] & 0xF));
    }
    if (p.row_sum != nullptr) {
        for (int m = 16; m > 0; m >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, m);
        if (lane == 0) red_i[warp] = rs;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int i = 0; i < 8; ++i) tot += red_i[i];
            p.row_sum[row] = tot;
        }
    }
}

template <int HB, bool EXTRAS>
static int launch_row(const RowParams& p, cudaStream_t stream) {
    const int units = (p.K + kUnit - 1) / kUnit;
    const dim3 grid((unsigned)p.M);
    if (units <= 8) {
        row_kernel<HB, 1, EXTRAS><<<grid, 32 * units, 0, stream>>>(p);
    } else if (units <= 32) {
        row_kernel<HB, 2, EXTRAS><<<grid, 32 * ((units + 1) / 2), 0, stream>>>(p);
    } else if (units <= 64) {
        row_kernel<HB, 4, EXTRAS><<<grid, 32 * ((units + 3) / 4), 0, stream>>>(p);
    } else {
        return QB200_ERR_UNSUPPORTED;
    }
    return launch_status();
}

#include "hadamard_quant_tc.cuh"

int hq_tc_fetch_and_clear_device_status(int* out) { return fetch_and_clear_device_status(out); }

bool hq_tc_shape_ok(int K) {
    int T, P;
    return K % 128 == 0 && hq_tc_tiling(K, &T, &P);
}

static bool vector_path_ok(const RowParams& p) {
    if (p.K % 8 != 0 || p.K > kMaxVectorK) return false;
    if (!aligned16(p.x)) return false;
    if (p.x_out != nullptr && !aligned16(p.x_out)) return false;
    if (p.q_dense != nullptr && (reinterpret_cast<uintptr_t>(p.q_dense) & 7u)) return false;
    if (p.q_packed != nullptr && !aligned16(p.q_packed)) return false;
    return true;
}

static int run_rows(const RowParams& p, int block, bool extras, cudaStream_t stream) {
    if (p.M == 0 || p.K == 0) return QB200_OK;
    if (!vector_path_ok(p)) {
        if (block != 0) return QB200_ERR_UNSUPPORTED;
        row_kernel_generic<<<(unsigned)p.M, 256, 0, stream>>>(p);
        return launch_status();
    }
    switch (block) {
        case 0: return extras ? launch_row<0, true>(p, stream) : launch_row<0, false>(p, stream);
        case 64: return extras ? launch_row<64, true>(p, stream) : launch_row<64, false>(p, stream);
        case 128: return extras ? launch_row<128, true>(p, stream) : launch_row<128, false>(p, stream);
        case 256: return extras ? launch_row<256, true>(p, stream) : launch_row<256, false>(p, stream);
        default: return QB200_ERR_UNSUPPORTED;
    }
}

// -------------------------------------------------------------------------------------------------
// add_mul_vv: D = bf16( float(2C + a_add[m] + b_add[n]) * (0.5f * a_mul[m] * b_mul[n]) )
// 6 bytes per element of HBM traffic; eight columns per thread when N allows 16-byte accesses.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ float dequant_one(int c, int a_add, int b_add, float a_mul, float b_mul) {
    const float lhs = (float)(c * 2 + a_add + b_add);
    const float rhs = 0.5f * a_mul * b_mul;
    return lhs * rhs;
}

__global__ void __launch_bounds__(256) add_mul_vv_vec8_kernel(__nv_bfloat16* __restrict__ d,
                                                              const int32_t* __restrict__ a_add,
                                                              const __nv_bfloat16* __restrict__ a_mul,
                                                              const int32_t* __restrict__ b_add,
                                                              const __nv_bfloat16* __restrict__ b_mul,
                                                              const int32_t* __restrict__ c, int M, int N) {
    const int groups_per_row = N >> 3;
    const long long total = (long long)M * groups_per_row;
    for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < total;
         g += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(g / groups_per_row);
        const int col = (int)(g - (long long)row * groups_per_row) << 3;
        const int aa = a_add[row];
        const float am = bf16_to_f32(a_mul[row]);
        const int4 c0 = *reinterpret_cast<const int4*>(c + (size_t)row * N + col);
        const int4 c1 = *reinterpret_cast<const int4*>(c + (size_t)row * N + col + 4);
        const int4 b0 = *reinterpret_cast<const int4*>(b_add + col);
        const int4 b1 = *reinterpret_cast<const int4*>(b_add + col + 4);
        const uint4 bm = *reinterpret_cast<const uint4*>(b_mul + col);
        uint4 o;
        o.x = pack_bf16x2(dequant_one(c0.x, aa, b0.x, am, bf16lo_to_f32(bm.x)),
                          dequant_one(c0.y, aa, b0.y, am, bf16hi_to_f32(bm.x)));
        o.y = pack_bf16x2(dequant_one(c0.z, aa, b0.z, am, bf16lo_to_f32(bm.y)),
                          dequant_one(c0.w, aa, b0.w, am, bf16hi_to_f32(bm.y)));
        o.z = pack_bf16x2(dequant_one(c1.x, aa, b1.x, am, bf16lo_to_f32(bm.z)),
                          dequant_one(c1.y, aa, b1.y, am, bf16hi_to_f32(bm.z)));
        o.w = pack_bf16x2(dequant_one(c1.z, aa, b1.z, am, bf16lo_to_f32(bm.w)),
                          dequant_one(c1.w, aa, b1.w, am, bf16hi_to_f32(bm.w)));
        *reinterpret_cast<uint4*>(d + (size_t)row * N + col) = o;
    }
}

__global__ void __launch_bounds__(256) add_mul_vv_scalar_kernel(__nv_bfloat16* __restrict__ d,
                                                                const int32_t* __restrict__ a_add,
                                                                const __nv_bfloat16* __restrict__ a_mul,
                                                                const int32_t* __restrict__ b_add,
                                                                const __nv_bfloat16* __restrict__ b_mul,
                                                                const int32_t* __restrict__ c, int M, int N) {
    const long long total = (long long)M * N;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / N);
        const int col = (int)(i - (long long)row * N);
        d[i] = __float2bfloat16_rn(
            dequant_one(c[i], a_add[row], b_add[col], bf16_to_f32(a_mul[row]), bf16_to_f32(b_mul[col])));
    }
}

// One block of bf16 [rows, cols] (row stride ld_bytes in every buffer) copied from src to n_dst destinations with one
// launch: the small-M exchange of the column-sharded layer (the block a rank has computed goes into every peer's
// output, which is mapped into this address space: plain 16-byte peer stores).
struct CopyDsts {
    void* p[7];
};

__global__ void copy_block_kernel(const uint8_t* __restrict__ src, const CopyDsts dsts, const int n_dst, const int rows,
                                  const int chunks, const long long ld_bytes) {
    const int total = rows * chunks;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int r = idx / chunks, c = idx - r * chunks;
        const long long off = (long long)r * ld_bytes + (long long)c * 16;
        const uint4 v = *reinterpret_cast<const uint4*>(src + off);
        for (int d = 0; d < n_dst; ++d) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(dsts.p[d]) + off) = v;
    }
}

}  // namespace qb

// -------------------------------------------------------------------------------------------------
// C ABI
// -------------------------------------------------------------------------------------------------
using namespace qb;

#ifdef QB200_TRACE
extern "C" int quest_b200_hq_trace(unsigned long long* out) {
    if (cudaDeviceSynchronize() != cudaSuccess) return QB200_ERR_CUDA;
    if (cudaMemcpyFromSymbol(out, g_hq_trace, sizeof(unsigned long long) * 6) != cudaSuccess) return QB200_ERR_CUDA;
    const unsigned long long init[6] = {~0ull, 0ull, ~0ull, 0ull, ~0ull, 0ull};
    return cuda_status(cudaMemcpyToSymbol(g_hq_trace, init, sizeof(init)));
}
#endif

extern "C" int find_scale_int4_cuda_bf16(void* scale_ptr, const void* x_ptr, int group_size, int batch_size,
                                         cudaStream_t stream) {
    if (group_size < 0 || batch_size < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (batch_size == 0) return QB200_OK;
    if (scale_ptr == nullptr || x_ptr == nullptr || group_size == 0) return QB200_ERR_INVALID_ARGUMENT;
    RowParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x_ptr);
    p.scale_out = static_cast<__nv_bfloat16*>(scale_ptr);
    p.K = group_size;
    p.M = batch_size;
    p.quantize = 0;
    return run_rows(p, 0, false, stream);
}

extern "C" int quantize_int4_cuda_bf16(void* x_ptr, const void* scale_ptr, void* x_int_ptr, void* x_int_packed_ptr,
                                       void* x_int_row_sum_ptr, int group_size, int batch_size, int do_dequantize,
                                       cudaStream_t stream) {
    if (group_size < 0 || batch_size < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (batch_size == 0 || group_size == 0) return QB200_OK;
    if (x_ptr == nullptr || scale_ptr == nullptr) return QB200_ERR_INVALID_ARGUMENT;
    if (x_int_packed_ptr != nullptr && (group_size & 1)) return QB200_ERR_INVALID_ARGUMENT;
    RowParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x_ptr);
    p.scale_in = static_cast<const __nv_bfloat16*>(scale_ptr);
    p.q_dense = static_cast<int8_t*>(x_int_ptr);
    p.q_packed = static_cast<uint8_t*>(x_int_packed_ptr);
    p.row_sum = static_cast<int32_t*>(x_int_row_sum_ptr);
    p.K = group_size;
    p.M = batch_size;
    p.quantize = 1;
    if (do_dequantize) {
        p.x_out = static_cast<__nv_bfloat16*>(x_ptr);
        p.x_out_mode = 2;
    }
    const bool extras = do_dequantize || x_int_ptr != nullptr;
    return run_rows(p, 0, extras, stream);
}

extern "C" int hadamard_quantize_int4_cuda_bf16(void* x_int_packed_ptr, void* scale_ptr, void* x_int_row_sum_ptr,
                                                const void* x_ptr, int group_size, int batch_size, int block,
                                                cudaStream_t stream) {
    if (group_size < 0 || batch_size < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (block != 64 && block != 128 && block != 256) return QB200_ERR_UNSUPPORTED;
    if (batch_size == 0) return QB200_OK;
    if (x_int_packed_ptr == nullptr || scale_ptr == nullptr || x_ptr == nullptr || group_size == 0)
        return QB200_ERR_INVALID_ARGUMENT;
    if (group_size % block != 0) return QB200_ERR_INVALID_ARGUMENT;
    RowParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x_ptr);
    p.scale_out = static_cast<__nv_bfloat16*>(scale_ptr);
    p.q_packed = static_cast<uint8_t*>(x_int_packed_ptr);
    p.row_sum = static_cast<int32_t*>(x_int_row_sum_ptr);
    p.K = group_size;
    p.M = batch_size;
    p.quantize = 1;
    p.had_scale = __bfloat162float(__float2bfloat16_rn((float)(1.0 / sqrt((double)block))));
    if (!vector_path_ok(p)) return QB200_ERR_UNSUPPORTED;
    // Tensor-core kernel where the shape fits its tiling; QB200_HQ_KERNEL=mma|tc forces one (tests, tuning).
    const char* force = getenv("QB200_HQ_KERNEL");
    // Measured crossover: below ~12 M elements the launch is one short wave and the CUDA-core kernel's smaller
    // set-up wins by about a microsecond.  Inside the one-call layer the crossover is 3 M elements: there the tcgen05
    // kernel and the GEMM behind it are launched with programmatic dependencies, which gains more than that
    // microsecond (M = 1024, K = N = 4096: 27.2 against 28.2 us per layer), while a GEMM launched that way behind
    // the CUDA-core kernel measured slower from 4 M elements on (29.5 us).
    const long long tc_from = qb_tl_dependent_quantiser ? 3ll * 1024 * 1024 : 12ll * 1024 * 1024;
    const bool want_tc = force != nullptr ? (force[0] == 't') : ((long long)p.M * p.K >= tc_from);
    if (want_tc && hq_tc_eligible(p, block)) {
        qb_tl_quantiser_kernel = kQuantiserTc;
        switch (block) {
            case 64: return launch_hq_tc<64>(p, stream);
            case 128: return launch_hq_tc<128>(p, stream);
            default: return launch_hq_tc<256>(p, stream);
        }
    }
    if (force != nullptr && force[0] == 't') return QB200_ERR_UNSUPPORTED;
    qb_tl_quantiser_kernel = kQuantiserMma;
    switch (block) {
        case 64: return launch_hq_mma<64>(p, stream);
        case 128: return launch_hq_mma<128>(p, stream);
        default: return launch_hq_mma<256>(p, stream);
    }
}

// Producer-fused variants: the rows that are transformed and quantised are RMSNorm(x) * w, or SiLU(gate) * up, computed
// on the fly from the kernel's inputs (see hadamard_quant_mma_kernel).
static int run_producer_hq(RowParams& p, int block, int pro, cudaStream_t stream) {
    p.quantize = 1;
    p.had_scale = __bfloat162float(__float2bfloat16_rn((float)(1.0 / sqrt((double)block))));
    if (!vector_path_ok(p)) return QB200_ERR_UNSUPPORTED;
    if (pro == kProRmsNorm) {
        if (!aligned16(p.norm_w)) return QB200_ERR_UNSUPPORTED;
        switch (block) {
            case 64: return launch_hq_mma<64, kProRmsNorm>(p, stream);
            case 128: return launch_hq_mma<128, kProRmsNorm>(p, stream);
            default: return launch_hq_mma<256, kProRmsNorm>(p, stream);
        }
    }
    if (!aligned16(p.x2)) return QB200_ERR_UNSUPPORTED;
    switch (block) {
        case 64: return launch_hq_mma<64, kProSiluMul>(p, stream);
        case 128: return launch_hq_mma<128, kProSiluMul>(p, stream);
        default: return launch_hq_mma<256, kProSiluMul>(p, stream);
    }
}

extern "C" int rmsnorm_hadamard_quantize_int4_cuda_bf16(void* x_int_packed_ptr, void* scale_ptr, void* x_int_row_sum_ptr,
                                                        const void* x_ptr, const void* norm_weight_ptr, float eps,
                                                        int group_size, int batch_size, int block, cudaStream_t stream) {
    if (group_size < 0 || batch_size < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (block != 64 && block != 128 && block != 256) return QB200_ERR_UNSUPPORTED;
    if (batch_size == 0) return QB200_OK;
    if (!x_int_packed_ptr || !scale_ptr || !x_ptr || !norm_weight_ptr || group_size == 0 || group_size % block != 0)
        return QB200_ERR_INVALID_ARGUMENT;
    RowParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x_ptr);
    p.norm_w = static_cast<const __nv_bfloat16*>(norm_weight_ptr);
    p.norm_eps = eps;
    p.scale_out = static_cast<__nv_bfloat16*>(scale_ptr);
    p.q_packed = static_cast<uint8_t*>(x_int_packed_ptr);
    p.row_sum = static_cast<int32_t*>(x_int_row_sum_ptr);
    p.K = group_size;
    p.M = batch_size;
    return run_producer_hq(p, block, kProRmsNorm, stream);
}

extern "C" int silu_mul_hadamard_quantize_int4_cuda_bf16(void* x_int_packed_ptr, void* scale_ptr, void* x_int_row_sum_ptr,
                                                         const void* gate_ptr, const void* up_ptr, int group_size,
                                                         int batch_size, int block, cudaStream_t stream) {
    if (group_size < 0 || batch_size < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (block != 64 && block != 128 && block != 256) return QB200_ERR_UNSUPPORTED;
    if (batch_size == 0) return QB200_OK;
    if (!x_int_packed_ptr || !scale_ptr || !gate_ptr || !up_ptr || group_size == 0 || group_size % block != 0)
        return QB200_ERR_INVALID_ARGUMENT;
    RowParams p{};
    p.x = static_cast<const __nv_bfloat16*>(gate_ptr);
    p.x2 = static_cast<const __nv_bfloat16*>(up_ptr);
    p.scale_out = static_cast<__nv_bfloat16*>(scale_ptr);
    p.q_packed = static_cast<uint8_t*>(x_int_packed_ptr);
    p.row_sum = static_cast<int32_t*>(x_int_row_sum_ptr);
    p.K = group_size;
    p.M = batch_size;
    return run_producer_hq(p, block, kProSiluMul, stream);
}

extern "C" int hadamard_quantize_a8_cuda_bf16(void* a8_ptr, void* scale_ptr, void* x_int_row_sum_ptr, const void* x_ptr,
                                              int group_size, int batch_size, int block, cudaStream_t stream) {
    if (group_size < 0 || batch_size < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (block != 64 && block != 128 && block != 256) return QB200_ERR_UNSUPPORTED;
    if (batch_size == 0) return QB200_OK;
    if (a8_ptr == nullptr || scale_ptr == nullptr || x_ptr == nullptr || group_size == 0) return QB200_ERR_INVALID_ARGUMENT;
    if (group_size % block != 0) return QB200_ERR_INVALID_ARGUMENT;
    RowParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x_ptr);
    p.scale_out = static_cast<__nv_bfloat16*>(scale_ptr);
    p.q_a8 = static_cast<uint8_t*>(a8_ptr);
    p.row_sum = static_cast<int32_t*>(x_int_row_sum_ptr);
    p.K = group_size;
    p.M = batch_size;
    p.quantize = 1;
    p.had_scale = __bfloat162float(__float2bfloat16_rn((float)(1.0 / sqrt((double)block))));
    if (!hq_tc_eligible(p, block)) return QB200_ERR_UNSUPPORTED;  // only the tcgen05 kernel writes this format
    switch (block) {
        case 64: return launch_hq_tc<64>(p, stream);
        case 128: return launch_hq_tc<128>(p, stream);
        default: return launch_hq_tc<256>(p, stream);
    }
}

extern "C" int hadamard_transform_cuda_bf16(void* out_ptr, const void* x_ptr, int group_size, int batch_size,
                                            int block, int weight_side, cudaStream_t stream) {
    if (group_size < 0 || batch_size < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (block != 64 && block != 128 && block != 256) return QB200_ERR_UNSUPPORTED;
    if (batch_size == 0) return QB200_OK;
    if (out_ptr == nullptr || x_ptr == nullptr || group_size == 0 || group_size % block != 0)
        return QB200_ERR_INVALID_ARGUMENT;
    RowParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x_ptr);
    p.x_out = static_cast<__nv_bfloat16*>(out_ptr);
    p.x_out_mode = 1;
    p.K = group_size;
    p.M = batch_size;
    p.quantize = 0;
    const float exact = (float)(1.0 / sqrt((double)block));  // fp32 rounding of block^-0.5
    p.had_scale = weight_side ? exact : __bfloat162float(__float2bfloat16_rn(exact));
    return run_rows(p, block, true, stream);
}

extern "C" int add_mul_vv_cuda_bf16(void* mat_d, const void* vec_a_add, const void* vec_a_mul, const void* vec_b_add,
                                    const void* vec_b_mul, const void* mat_c, int size_a, int size_b,
                                    cudaStream_t stream) {
    if (size_a < 0 || size_b < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (size_a == 0 || size_b == 0) return QB200_OK;
    if (!mat_d || !vec_a_add || !vec_a_mul || !vec_b_add || !vec_b_mul || !mat_c) return QB200_ERR_INVALID_ARGUMENT;
    auto* d = static_cast<__nv_bfloat16*>(mat_d);
    auto* aa = static_cast<const int32_t*>(vec_a_add);
    auto* am = static_cast<const __nv_bfloat16*>(vec_a_mul);
    auto* ba = static_cast<const int32_t*>(vec_b_add);
    auto* bm = static_cast<const __nv_bfloat16*>(vec_b_mul);
    auto* c = static_cast<const int32_t*>(mat_c);
    const long long total = (long long)size_a * size_b;
    const bool vec = (size_b % 8 == 0) && aligned16(d) && aligned16(c) && aligned16(ba) && aligned16(bm);
    const long long work = vec ? total / 8 : total;
    long long blocks = (work + 255) / 256;
    const long long cap = 148LL * 8 * 4;  // grid-stride beyond a few waves of the 148 SMs
    if (blocks > cap) blocks = cap;
    if (vec)
        add_mul_vv_vec8_kernel<<<(unsigned)blocks, 256, 0, stream>>>(d, aa, am, ba, bm, c, size_a, size_b);
    else
        add_mul_vv_scalar_kernel<<<(unsigned)blocks, 256, 0, stream>>>(d, aa, am, ba, bm, c, size_a, size_b);
    return launch_status();
}

extern "C" int quest_b200_copy_block_to_peers_cuda(const void* src, void* const* dsts, int n_dst, int rows, int cols,
                                                   long long ld, cudaStream_t stream) {
    if (rows < 0 || cols < 0 || n_dst < 0 || n_dst > 7 || ld < cols) return QB200_ERR_INVALID_ARGUMENT;
    if (rows == 0 || cols == 0 || n_dst == 0) return QB200_OK;
    if (!src || !dsts) return QB200_ERR_INVALID_ARGUMENT;
    if (cols % 8 != 0 || ld % 8 != 0 || !aligned16(src)) return QB200_ERR_UNSUPPORTED;  // whole 16-byte pieces only
    CopyDsts d{};
    for (int i = 0; i < n_dst; ++i) {
        if (!dsts[i]) return QB200_ERR_INVALID_ARGUMENT;
        if (!aligned16(dsts[i])) return QB200_ERR_UNSUPPORTED;
        d.p[i] = dsts[i];
    }
    const int chunks = cols / 8;
    const long long total = (long long)rows * chunks;
    if (total > (1ll << 30)) return QB200_ERR_UNSUPPORTED;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    copy_block_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(src), d, n_dst, rows, chunks, ld * 2);
    return launch_status();
}
