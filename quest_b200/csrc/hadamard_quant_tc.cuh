// Fused block-Hadamard + scale + int4 quantise + pack + row sum with the transform on the 5th-generation tensor
// core (tcgen05, accumulators in tensor memory).  Included by quantize.cu inside namespace qb.
//
// The activation matrix [M, K] is viewed as a matrix of 128-element blocks, X2[M*K/128, 128]; the block transform
// of every row of X2 is one GEMM with the 128 x 128 matrix H (entries +-bf16(block^-0.5), Sylvester order; two
// 64 x 64 blocks on the diagonal for block 64; block 256 adds one add/subtract between neighbouring rows):
//
//   TMA (cp.async.bulk.tensor.2d, 128-byte swizzle)   128 rows of X2 (32 KB)  global -> shared      producer warp
//   tcgen05.mma kind::f16, M128 N128 K16, 8 per tile  X2 tile . H -> 128 x 128 fp32 in tensor memory one thread
//   tcgen05.ld / tcgen05.st 32x32b                    thread = one row of X2 (one 128-element block)  16 drain warps
//   pass 1: round to bf16 pairs (written back into tensor memory), sum of squares, per-token reduction, scale;
//   pass 2: saturate, divide-free floor, nibble pack, 16-byte stores, row sums.
//
// This is the same "x times Hadamard matrix" product the reference hands to cuBLAS (gemm-quest/benchmarks/utils.py:
// 17, 89-90); it moves the butterflies off the instruction-issue-bound CUDA cores, which is what limits
// hadamard_quant_mma_kernel.  A tile holds T whole tokens (T * K/128 <= 128 rows; leftover lanes idle) or, for
// K > 16384, one half or quarter of a token; every per-token reduction stays inside one CTA.  Every mbarrier wait is
// bounded (see mbar_wait).
#pragma once

#include "tcgen05.cuh"

namespace tc {
constexpr int STAGES = 4;                 // input ring: 4 x 32 KB
constexpr int TILE_ROWS = 128;
constexpr int TILE_BYTES = TILE_ROWS * 256;
constexpr int HALF_BYTES = TILE_BYTES / 2;  // K halves 0..63 and 64..127: one 128-byte-swizzled region each
constexpr int NUM_ACC = 4;                // accumulator buffers in tensor memory (4 x 128 columns)
constexpr int kDrainWarps = 16, kFirstDrain = 2;
constexpr int kThreads = (kFirstDrain + kDrainWarps) * 32;
constexpr int PART_FLOATS = 64;          // per drain group: the partial sums its warps exchange
constexpr int NUM_BARS = 2 * STAGES + 2 * NUM_ACC + NUM_ACC + 1;
constexpr int SMEM_BYTES = 1024 + STAGES * TILE_BYTES + TILE_BYTES /*H*/ + 2 * PART_FLOATS * 4 + NUM_BARS * 8 + 16;
// instruction descriptor: D = f32, A = B = bf16, both K-major, N = 128, M = 128
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}  // namespace tc

// Block 256: index bit 7 pairs neighbouring rows of X2 (the two 128-element halves of a 256 block): lanes l, l ^ 1.
__device__ __forceinline__ void pair_rows(uint32_t (&r)[16], int lane) {
    const float sgn = (lane & 1) ? -1.f : 1.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float x = __uint_as_float(r[i]);
        const float o = __shfl_xor_sync(0xffffffffu, x, 1);
        r[i] = __float_as_uint(fmaf(x, sgn, o));  // even row: first half + second half; odd row: first - second
    }
}

// nb: 128-element blocks per token (K / 128).  A unit is what a reduction needs together: T whole tokens in one tile
// (P = 1, T * nb <= 128 rows), or one token spread over P = 2 or 4 consecutive tiles of nb / P rows (K > 16384), which
// P neighbouring drain groups then process side by side.
// A8: instead of packed int4, write the operand the GEMM's tensor cores consume, so that the GEMM need not unpack A:
// int8 = 16 x code, [M, K] row-major, and inside every group of 32 consecutive K positions the 16 even positions
// first, then the 16 odd ones - the order in which the GEMM's own unpack lays out the codes of a 16-byte packed piece.
template <int HB, bool A8>
__global__ void __launch_bounds__(tc::kThreads, 1)
hadamard_quant_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const RowParams p, const int nb, const int T,
                         const int P, const int num_units) {
    using namespace tc;
    extern __shared__ uint8_t tc_smem_raw[];
    const uint32_t raw_base = smem_u32(tc_smem_raw);
    const uint32_t smem_base = (raw_base + 1023u) & ~1023u;
    const uint32_t a_base = smem_base;
    const uint32_t h_base = a_base + STAGES * TILE_BYTES;
    const uint32_t part_base = h_base + TILE_BYTES;
    const uint32_t bar_base = part_base + 2 * PART_FLOATS * 4;
    const uint32_t full = bar_base;
    const uint32_t empty = full + 8 * STAGES;
    const uint32_t tmem_full = empty + 8 * STAGES;
    const uint32_t tmem_empty = tmem_full + 8 * NUM_ACC;
    const uint32_t part_bar = tmem_empty + 8 * NUM_ACC;
    const uint32_t mma_done = part_bar + 8 * NUM_ACC;
    const uint32_t tmem_slot = mma_done + 8;
    uint8_t* const smem_gen = tc_smem_raw + (smem_base - raw_base);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tc_smem_raw + (tmem_slot - raw_base));
    float* const part_f = reinterpret_cast<float*>(smem_gen + (part_base - smem_base));
    int* const part_i = reinterpret_cast<int*>(part_f + PART_FLOATS);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
#ifdef QB200_TRACE
    if (threadIdx.x == 0) {
        const unsigned long long t = hq_gtime();
        atomicMin(&g_hq_trace[0], t);
        atomicMax(&g_hq_trace[1], t);
    }
#endif

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(full + 8 * i, 1);
            mbar_init(empty + 8 * i, 1);
        }
        for (int i = 0; i < NUM_ACC; ++i) {
            mbar_init(tmem_full + 8 * i, 1);
            mbar_init(tmem_empty + 8 * i, 4);
            mbar_init(part_bar + 8 * i, 4 * P);  // the warps of the P groups that share a token
        }
        mbar_init(mma_done, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot_ptr;
    // A GEMM launched behind this kernel with a programmatic dependency may be scheduled as soon as every block of this
    // grid has got here (it waits on the device for this grid's end before it touches anything written here).  Only now
    // that tensor memory is allocated: a dependent block that took it first on a shared SM would wait for this grid
    // while this block waits for the allocation.
    let_dependents_launch();
    const int rows_per_tile = P == 1 ? T * nb : nb / P;
    const int unit_rows = P == 1 ? T * nb : nb;  // rows of X2 per unit

    if (warp != 0) {
        // The Hadamard operand, built while the producer warp already fetches the first tiles:
        // H[o][k] = h * (-1)^popc(o & k), K-major rows of 128 bytes per K half, 128-byte swizzle (16-byte chunk
        // index XOR (row & 7)), exactly the layout TMA gives the activation tile.
        const uint32_t hb = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(p.had_scale));
        for (int item = threadIdx.x - 32; item < 128 * 16; item += kThreads - 32) {
            const int o = item >> 4, ch = item & 15;  // row, 16-byte chunk of the 256-byte row
            const int half = ch >> 3, c = ch & 7;
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t pair = 0;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int k = half * 64 + c * 8 + 2 * j + e;
                    uint32_t v = hb | ((__popc(o & k & (HB == 64 ? 63 : 127)) & 1) ? 0x8000u : 0u);
                    if (HB == 64 && ((o ^ k) & 64)) v = 0;  // block 64: two independent 64-point transforms
                    pair |= v << (16 * e);
                }
                w[j] = pair;
            }
            sts128(h_base + half * HALF_BYTES + o * 128 + ((c ^ (o & 7)) << 4), make_uint4(w[0], w[1], w[2], w[3]));
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, %0;" ::"n"(kThreads - 32) : "memory");
        wait_for_preceding_grid();  // the outputs may still be read by the kernel before this one (the producer thread waits too)
    }

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_x);
            wait_for_preceding_grid();  // launched with a programmatic dependency: the input may still be being written
            uint32_t it = 0;
            bool ok = true;
            for (;; ++it) {  // tile `it` of this CTA: part it % P of unit blockIdx.x + (it / P) * gridDim.x
                const int unit = blockIdx.x + (int)(it / P) * gridDim.x;
                if (unit >= num_units) break;
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                if (!(ok = mbar_wait(empty + 8 * s, ph ^ 1u, 21))) break;
                mbar_arrive_expect_tx(full + 8 * s, TILE_BYTES);
                const uint32_t dst = a_base + s * TILE_BYTES;
                const int row0 = unit * unit_rows + (int)(it % P) * rows_per_tile;
                tma_load_2d(dst, &tmap_x, 0, row0, full + 8 * s);
                tma_load_2d(dst + HALF_BYTES, &tmap_x, 64, row0, full + 8 * s);
            }
            const uint32_t pending = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
            for (uint32_t j = 0; j < pending; ++j) {  // do not leave while a copy may still land in shared memory
                const uint32_t i2 = it - 1 - j;
                mbar_wait(full + 8 * (i2 % STAGES), (i2 / STAGES) & 1u, 22);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (;; ++it) {
                if (blockIdx.x + (int)(it / P) * gridDim.x >= num_units) break;
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                const uint32_t acc = it % NUM_ACC, acc_ph = (it / NUM_ACC) & 1u;
                if (!(ok = mbar_wait(tmem_empty + 8 * acc, acc_ph ^ 1u, 23))) break;
                if (!(ok = mbar_wait(full + 8 * s, ph, 24))) break;
                tc_fence_after();
                const uint32_t a_addr = a_base + s * TILE_BYTES;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        umma_bf16(tmem_acc + acc * 128, make_smem_desc(a_addr + half * HALF_BYTES + 32 * j),
                                  make_smem_desc(h_base + half * HALF_BYTES + 32 * j), IDESC, (half | j) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(empty + 8 * s);        // the input stage is free once these MMAs have read it
                umma_commit(tmem_full + 8 * acc);  // and the accumulators are complete
            }
            umma_commit(mma_done);
            mbar_wait(mma_done, 0, 25);
        }
    } else {
        // ------------------------------ drain warps ------------------------------
        // Four groups of four warps; group g owns accumulator buffer g and every fourth tile of this CTA, so up to
        // four tiles are in different phases at once.  Inside a group a warp owns a lane quadrant (32 rows of the
        // tile) and each thread one row of X2: the 128 transformed values of one block, read from tensor memory in
        // four pieces of 32, twice (sum of squares, then quantise) - nothing but the row's scale lives across the passes.
        const int quad = warp & 3;                    // tensor-memory lane quadrant this warp may read
        const int grp = (warp - kFirstDrain) >> 2;    // drain group = accumulator buffer
        const int row = quad * 32 + lane;             // row of the tile = lane of tensor memory
        const int g_rows = nb < 32 ? nb : 32;         // rows of one token inside this warp (a power of two, or all 32)
        const int part = grp % P;                     // which tile of its token this group processes (0 if P == 1)
        const int set0 = grp - part;                  // first group of the set that shares a token
        const int tok_in_tile = P == 1 ? row / nb : 0;
        const int blk = P == 1 ? row - tok_in_tile * nb : part * rows_per_tile + row;  // which block of its token this row is
        const bool row_in_tile = row < rows_per_tile;
        const bool cross = nb > 32;                   // a token spans several warps: exchange through shared memory
        const int K = p.K;
        float* const xf = part_f + set0 * 4;          // [group of the set][quadrant]: partial sums of squares ...
        int* const xi = part_i + set0 * 4;            // ... and row sums
        const uint32_t grp_bar = part_bar + 8 * set0;
        const int q0 = P == 1 ? tok_in_tile * (nb >> 5) : 0;         // first partial of this row's token
        const int nq = P == 1 ? (nb + 31) >> 5 : 4 * P;              // and how many there are
        const uint32_t t_row = tmem_acc + ((uint32_t)(quad * 32) << 16) + grp * 128;
        uint32_t jt = 0;  // tiles this group has done
        bool ok = true;
        for (;; ++jt) {  // this group's tiles are it = grp + 4 jt
            const int unit = blockIdx.x + (int)((grp + NUM_ACC * jt) / P) * gridDim.x;
            if (unit >= num_units) break;
            const int token = P == 1 ? unit * T + tok_in_tile : unit;
            const bool valid = row_in_tile && token < p.M;
            ok = mbar_wait(tmem_full + 8 * grp, jt & 1u, 26);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
#ifdef QB200_TRACE
            if (jt == 0 && grp == 0 && quad == 0 && lane == 0) {
                const unsigned long long t = hq_gtime();
                atomicMin(&g_hq_trace[4], t);
                atomicMax(&g_hq_trace[5], t);
            }
#endif

            // ---- pass 1: sum of squares of the bf16-rounded transform ----
            // Tensor memory is read in pieces of 16 columns into two register sets: the next piece is in flight
            // while the current one is processed.
            uint32_t ra[16], rb[16];
            f32x2 ssq2 = 0ull;
            // Each piece is rounded to bf16 pairs once; the pairs go back into the columns of the accumulator that
            // have already been read (piece c -> columns 8c .. 8c+7), so pass 2 neither re-rounds nor re-pairs.
            auto square_sum = [&](uint32_t (&r)[16], int c) {
                if (HB == 256) pair_rows(r, lane);
                uint32_t v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                    const f32x2 xx = pk2(bf16lo_to_f32(v[i]), bf16hi_to_f32(v[i]));
                    ssq2 = fma2(xx, xx, ssq2);
                }
                tmem_st8(t_row + 8 * c, v);
            };
            tmem_ld16(t_row, ra);
#pragma unroll
            for (int c = 0; c < 8; c += 2) {
                tmem_ld_wait16(ra);
                tmem_ld16(t_row + 16 * (c + 1), rb);
                square_sum(ra, c);
                tmem_ld_wait16(rb);
                if (c + 2 < 8) tmem_ld16(t_row + 16 * (c + 2), ra);
                square_sum(rb, c + 1);
            }
            tmem_st_wait();
            tmem_ld16(t_row, ra);  // the first 32 rounded values for pass 2, in flight during the scale computation
            float ssq;
            {
                float s0, s1;
                unpk2(ssq2, s0, s1);
                ssq = valid ? s0 + s1 : 0.f;
            }
            for (int m = g_rows >> 1; m > 0; m >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, m);
            float tot = ssq;
            if (cross) {  // warp-uniform
                if (lane == 0) xf[part * 4 + quad] = ssq;
                __syncwarp();
                if (lane == 0) mbar_arrive(grp_bar);
                ok = mbar_wait(grp_bar, 0u, 27);  // two rendezvous per tile: phases 2 jt and 2 jt + 1
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                double t2 = 0.0;
                for (int q = 0; q < nq; ++q) t2 += (double)xf[(q0 + q) & 15];
                tot = (float)t2;
            }
            const __nv_bfloat16 sb = __float2bfloat16_rn(quest_scale_from_mean_square(__fdiv_rn(tot, (float)K)));
            const float s_f = bf16_to_f32(sb);
            const float inv_s = __frcp_rn(s_f);
            const uint32_t lo1 = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(-8.f * s_f));
            const uint32_t hi1 = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(7.5f * s_f));
            const uint32_t lo2 = lo1 | (lo1 << 16), hi2 = hi1 | (hi1 << 16);
            const f32x2 inv_s2 = pk2(inv_s, inv_s), magic2 = pk2(kFloorMagic, kFloorMagic);
            if (valid && blk == 0) p.scale_out[token] = sb;

            // ---- pass 2: quantise and pack; a piece is 16 columns of bf16 pairs = 32 elements = 16 packed bytes ----
            uint8_t* const dst = A8 ? p.q_a8 + (size_t)token * K + blk * 128 : p.q_packed + (size_t)token * (K >> 1) + blk * 64;
            int rs16 = 0;
            auto quantise32 = [&](const uint32_t (&v)[16], int piece) {
                uint32_t w[4], wo[4];
#pragma unroll
                for (int q8 = 0; q8 < 4; ++q8) {  // eight elements -> one 32-bit word
                    uint32_t ub[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t c = clamp_bf16x2(v[4 * q8 + i], lo2, hi2);
                        float y0, y1;
                        unpk2(mul2(pk2(bf16lo_to_f32(c), bf16hi_to_f32(c)), inv_s2), y0, y1);
                        const f32x2 fl = add2_rd(pk2(fmaf(fabsf(y0), 1.220703125e-4f, y0), fmaf(fabsf(y1), 1.220703125e-4f, y1)), magic2);
                        float u0, u1;
                        unpk2(fl, u0, u1);
                        ub[2 * i] = __float_as_uint(u0);
                        ub[2 * i + 1] = __float_as_uint(u1);
                    }
                    // byte j of the word = (code[2j+1] << 4) | code[2j]
                    const uint32_t ev = __byte_perm(__byte_perm(ub[0], ub[2], 0x0040), __byte_perm(ub[4], ub[6], 0x0040), 0x5410);
                    const uint32_t od = __byte_perm(__byte_perm(ub[1], ub[3], 0x0040), __byte_perm(ub[5], ub[7], 0x0040), 0x5410);
                    if (A8) {
                        w[q8] = (ev << 4) & 0xF0F0F0F0u;   // 16 x the codes at even positions
                        wo[q8] = (od << 4) & 0xF0F0F0F0u;  // 16 x the codes at odd positions
                    } else {
                        w[q8] = (ev & 0x0F0F0F0Fu) | ((od << 4) & 0xF0F0F0F0u);
                    }
                }
                if (valid) {
                    if (A8) {
#pragma unroll
                        for (int q8 = 0; q8 < 4; ++q8)
                            rs16 = __dp4a((int)wo[q8], 0x01010101, __dp4a((int)w[q8], 0x01010101, rs16));
                        *reinterpret_cast<uint4*>(dst + 32 * piece) = make_uint4(w[0], w[1], w[2], w[3]);
                        *reinterpret_cast<uint4*>(dst + 32 * piece + 16) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
                    } else {
#pragma unroll
                        for (int q8 = 0; q8 < 4; ++q8) rs16 = nibble_sum16(w[q8], rs16);
                        *reinterpret_cast<uint4*>(dst + 16 * piece) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            };
#pragma unroll
            for (int pc = 0; pc < 4; pc += 2) {
                tmem_ld_wait16(ra);
                tmem_ld16(t_row + 16 * (pc + 1), rb);
                quantise32(ra, pc);
                tmem_ld_wait16(rb);
                if (pc + 2 < 4) tmem_ld16(t_row + 16 * (pc + 2), ra);
                quantise32(rb, pc + 1);
            }
            // the accumulator buffer has been read for the last time
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty + 8 * grp);

            // ---- row sums ----
            for (int m = g_rows >> 1; m > 0; m >>= 1) rs16 += __shfl_xor_sync(0xffffffffu, rs16, m);
            if (cross) {
                if (lane == 0) xi[part * 4 + quad] = rs16;
                __syncwarp();
                if (lane == 0) mbar_arrive(grp_bar);
                ok = mbar_wait(grp_bar, 1u, 28);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                int t2 = 0;
                for (int q = 0; q < nq; ++q) t2 += xi[(q0 + q) & 15];
                rs16 = t2;
            }
            if (valid && blk == 0 && p.row_sum != nullptr) p.row_sum[token] = rs16 >> 4;  // exact: every term is a multiple of 16
        }
        tmem_ld_wait();  // a prefetched piece may still be in flight if a bounded wait gave up
    }

    tc_fence_before();
    __syncthreads();
#ifdef QB200_TRACE
    if (threadIdx.x == 0) {
        const unsigned long long t = hq_gtime();
        atomicMin(&g_hq_trace[2], t);
        atomicMax(&g_hq_trace[3], t);
    }
#endif
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_acc, 512);
    }
}

// X2[M*K/128, 128] bf16, row pitch 256 bytes; box = 64 elements (128 bytes, the swizzle span) x 128 rows.
static int make_block_map(CUtensorMap* map, const void* base, long long rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return QB200_ERR_DRIVER;
    const cuuint64_t dims[2] = {128, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, (cuuint32_t)tc::TILE_ROWS};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QB200_OK : QB200_ERR_DRIVER;
}

// Shapes the tensor-core kernel takes: K a multiple of 128 (256 for block 256) with at least 85 % of the 128 tile
// rows holding whole tokens; everything else stays with hadamard_quant_mma_kernel.
// Tiling of a row length: P tiles per token (1, 2 or 4) and, for P = 1, T tokens per tile.  False if no tiling keeps at
// least 85 % of the 128 tile rows busy.
static bool hq_tc_tiling(int K, int* T_out, int* P_out) {
    const int nb = K / 128;
    int T = 1, P = 1;
    if (nb <= 128) {
        T = 128 / nb;
        if (nb < 32 && (nb & (nb - 1)) != 0) return false;  // several tokens per warp need power-of-two groups
        if (nb >= 32 && T > 1 && nb % 32 != 0) return false;
    } else if (nb % 2 == 0 && nb / 2 <= 128) {
        P = 2;
    } else if (nb % 4 == 0 && nb / 4 <= 128) {
        P = 4;
    } else {
        return false;
    }
    const int rows = P == 1 ? T * nb : nb / P;
    if (rows * 100 < 85 * 128) return false;
    *T_out = T;
    *P_out = P;
    return true;
}

static bool hq_tc_eligible(const RowParams& p, int block) {
    if (p.K % 128 != 0 || (block == 256 && p.K % 256 != 0)) return false;
    int T, P;
    if (!hq_tc_tiling(p.K, &T, &P)) return false;
    if (block == 256 && P > 1 && ((p.K / 128 / P) & 1)) return false;  // a 256 block must not straddle two tiles
    if ((p.q_packed == nullptr) == (p.q_a8 == nullptr) || p.scale_out == nullptr || p.scale_in != nullptr ||
        p.q_dense != nullptr || p.x_out != nullptr || !p.quantize)
        return false;
    if ((long long)p.M * (p.K / 128) >= (1ll << 31)) return false;
    return aligned16(p.x) && aligned16(p.q_packed) && aligned16(p.q_a8);
}

template <int HB, bool A8>
static int launch_hq_tc_impl(const RowParams& p, cudaStream_t stream) {
    static bool attr_set[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return QB200_ERR_CUDA;
    auto kernel = hadamard_quant_tc_kernel<HB, A8>;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES) != cudaSuccess) {
            cudaGetLastError();
            return QB200_ERR_CUDA;
        }
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    int sms = 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const int nb = p.K / 128;
    int T = 1, P = 1;
    if (!hq_tc_tiling(p.K, &T, &P)) return QB200_ERR_UNSUPPORTED;
    const int num_units = P == 1 ? (p.M + T - 1) / T : p.M;
    CUtensorMap map;
    const int st = make_block_map(&map, p.x, (long long)p.M * nb);
    if (st != QB200_OK) return st;
    const int grid = num_units < sms ? num_units : sms;
    if (launch_kernel_dep(qb_tl_dependent_quantiser, kernel, grid, tc::kThreads, tc::SMEM_BYTES, stream, map, p, nb, T, P, num_units) != cudaSuccess) {
        cudaGetLastError();
        return QB200_ERR_CUDA;
    }
    return launch_status();
}

template <int HB>
static int launch_hq_tc(const RowParams& p, cudaStream_t stream) {
    return p.q_a8 != nullptr ? launch_hq_tc_impl<HB, true>(p, stream) : launch_hq_tc_impl<HB, false>(p, stream);
}
