// Dense int4 x int4 -> int32 GEMM for sm_100a (B200), with an optional fused dequantising epilogue.
//
//   C[M,N] = A[M,K] . B[N,K]^T      A, B packed int4 (two codes per byte, K contiguous)
//
// sm_100 tensor cores have no int4 MMA, so the kernel unpacks to int8 on the fly:
//
//   TMA (cp.async.bulk.tensor.2d)  : packed tiles  global -> shared      (producer warp)
//   unpack warps                   : packed shared -> int8 shared tile in the canonical K-major
//                                    128-byte-swizzled UMMA layout
//   tcgen05.mma kind::i8           : int8 x int8 -> int32 accumulators in tensor memory (one thread)
//   epilogue warps                 : tcgen05.ld accumulators -> registers -> int32 or bf16 -> global
//
// The unpack uses the "times sixteen" form: for a 32-bit word w holding eight codes,
//   (w << 4) & 0xF0F0F0F0  holds 16 * (codes in the low nibbles)   as four int8
//    w       & 0xF0F0F0F0  holds 16 * (codes in the high nibbles)  as four int8
// which needs no per-nibble sign extension.  Both operands are scaled by 16, so every product and
// hence the accumulator is scaled by exactly 256 and the epilogue shifts it back (exact: the sum is
// a multiple of 256; |acc| * 256 <= 2^14 * K < 2^31 for K < 2^17).  The unpack also permutes K
// inside a 32-element group (even columns first, then odd); A and B are permuted identically, so
// each dot product is unchanged and the accumulators are bit-exact.
//
// The kernel is persistent (one CTA per SM, static round-robin over output tiles), uses two
// accumulator buffers in tensor memory so that the epilogue of tile i overlaps the main loop of
// tile i+1, and bounds every mbarrier wait: on a timeout it records an error code in a device
// status word, drains its copies, frees tensor memory and returns.
//
// Replaces gemm-quest/quest/matmul_kernel.cu:8-63 and gemm-quest/quest/fused_matmul_dequantize_kernel.cu
// with gemm-quest/include/symmetric/** (CUTLASS 2.x Sm80 mma.sync kernels).
#include <string.h>
#include <type_traits>

#include "tcgen05.cuh"

// Set (per host thread) by the one-call layer entry points around their GEMM call: the GEMM kernel is then launched
// with a programmatic dependency on the preceding kernel of the stream (the quantiser of its activations) instead of a
// full one.  Its blocks are scheduled as soon as the quantiser's blocks have left the SMs, set up their barriers and
// tensor memory and request the weights; every thread that touches what the quantiser writes (the A operand, the row
// sums and scales) first executes griddepcontrol.wait, which returns when the quantiser's grid has completed and its
// writes are visible.  Without the launch attribute that instruction returns at once.
static thread_local bool tl_dependent_launch = false;

template <typename Kernel, typename... Args>
static cudaError_t launch_kernel(Kernel kernel, int grid, int threads, size_t smem, cudaStream_t stream, Args... args) {
    return qb::launch_kernel_dep(tl_dependent_launch, kernel, grid, threads, smem, stream, args...);
}

namespace qb {

#ifdef QB200_TRACE
// Timeline probes for tuning builds (python -m quest_b200.build --trace): per CTA, globaltimer (ns) at kernel entry,
// first MMA issue, last MMA retired, last epilogue store.  Read back with quest_b200_trace().
__device__ unsigned long long g_trace[256][4];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define QB_TRACE(slot) do { if (blockIdx.x < 256) g_trace[blockIdx.x][slot] = gtime(); } while (0)
#else
#define QB_TRACE(slot) do { } while (0)
#endif

// ---------------------------------------------------------------------------------------------
// Tile configuration
// ---------------------------------------------------------------------------------------------
constexpr int BM = 128;       // rows of A per tile = UMMA M
constexpr int BK = 128;       // K elements per pipeline stage: 64 packed bytes, 128 int8 bytes (one swizzle row)
constexpr int PK_ROW = BK / 2;  // packed bytes per row per stage
constexpr int U8_ROW = BK;      // unpacked bytes per row per stage

constexpr int kNumUnpackWarps = 8;
constexpr int kNumEpilogueWarps = 4;
constexpr int kFirstEpilogueWarp = 2;
constexpr int kFirstUnpackWarp = kFirstEpilogueWarp + kNumEpilogueWarps;
constexpr int kFirstPushWarp = kFirstUnpackWarp + kNumUnpackWarps;
constexpr int kNumPushWarps = 2;  // copy finished tiles to the other GPUs' outputs (idle on one GPU)
constexpr int kNumWarps = kFirstPushWarp + kNumPushWarps;
constexpr int kNumThreads = kNumWarps * 32;

template <int BN>
struct Cfg {
    static constexpr int ROWS = BM + BN;                 // A rows then B rows, contiguous in shared memory
    static constexpr int P_STAGES = (BN == 256) ? 3 : 4; // packed ring  (TMA -> unpack)
    static constexpr int U_STAGES = 3;                   // int8 ring    (unpack -> MMA)
    static constexpr int P_BYTES = ROWS * PK_ROW;
    static constexpr int U_BYTES = ROWS * U8_ROW;
    static constexpr int TMEM_COLS = (2 * BN > 256) ? 512 : 256;  // two accumulator buffers, power of two
    static constexpr int NUM_BARS = 2 * P_STAGES + 2 * U_STAGES + 4 + 1 + 4;
    static constexpr int VEC_STRIDE = BN * 8;            // per accumulator buffer: b_add (int32) and b_mul (fp32) of the tile
    static constexpr int VEC_BYTES = 2 * VEC_STRIDE;
    static constexpr int SMEM_BYTES = 1024 /*alignment slack*/ + U_STAGES * U_BYTES + P_STAGES * P_BYTES + VEC_BYTES + NUM_BARS * 8 + 16;
    // instruction descriptor: D=s32, A=B=s8, both K-major, N and M of the MMA
    static constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
};

struct EpilogueParams {
    void* out;              // int32 [M, ld] or bf16 [M, ld]
    long long ld;           // leading dimension of out, in elements
    const int32_t* a_add;   // [M]   (fused only)
    const int32_t* b_add;   // [N]
    const __nv_bfloat16* a_mul;  // [M]
    const __nv_bfloat16* b_mul;  // [N]
    int vec_ok;             // 1: 16-byte stores are aligned for every (row, 16-byte column group); 2: 32-byte ones too
    int n_peer;             // fused only: the tile is also stored into n_peer further matrices of the same shape
    void* peer_out[7];      // (buffers of other GPUs mapped into this address space: plain peer stores)
    // split-K (few output tiles, long K): every tile is computed by `splits` CTAs over disjoint K ranges
    int splits;             // 1 = off
    int32_t* scratch;       // [tile * splits + range][slab_rows][256 columns] int32 partial sums
    int slab_ints;          // slab_rows * 256: a slab holds only the rows a tile can have (M rounded up to 8, at most 128)
    int* counters;          // one per output tile, all zero between launches
    int tma_store;          // 256 x 256 kernel, fused: the output tensor map is valid (the last tile leaves as bulk tensor stores)
    int tma_store16;        // int8-operand variant: the 16-column output map is valid too (earlier tiles leave as small bulk stores)
    int test_skip_producer; // tests only: the TMA producer issues nothing, so that every bounded wait of the launch runs out
    // 256-row kernel: the N range is cut into col_count tile columns whose widths are multiples of 16, at most 256; the
    // first col_rem of them are (col_units + 1) * 16 wide, the others col_units * 16 (col_units = 16, col_rem = 0: all 256)
    int col_count, col_units, col_rem;
};


// Converts and stores 32 consecutive accumulators of one output row (columns col0 .. col0+31, clipped to N).
// The accumulators carry the factor 256 of the unpack; FUSED applies the exact dequantising expression
//   D = bf16( float(2*acc + a_add[m] + b_add[n]) * (0.5f * a_mul[m] * b_mul[n]) ),
// otherwise the int32 accumulators are written.  sb_add / sb_mul point at the 32 per-column values of this
// chunk, staged in shared memory by the epilogue warps while the tile was still being accumulated.
__device__ __forceinline__ void stg256(void* p, const uint32_t* w) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

// The dequantising expression for 32 consecutive accumulators of one output row, as 16 bf16 pairs:
//   D = bf16( float(2*acc + a_add[m] + b_add[n]) * (0.5f * a_mul[m] * b_mul[n]) )
// (A variant that replaced the int-to-float conversion by a magic-number addition in packed f32x2 arithmetic measured 1-4 %
// slower per launch: the conversion is not what limits the epilogue.)
__device__ __forceinline__ void dequant_chunk(const uint32_t (&r)[32], int a_add, float half_a_mul, const int* sb_add,
                                              const float* sb_mul, uint32_t (&w)[16]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int4 b0 = *reinterpret_cast<const int4*>(sb_add + 8 * g);
        const int4 b1 = *reinterpret_cast<const int4*>(sb_add + 8 * g + 4);
        const float4 m0 = *reinterpret_cast<const float4*>(sb_mul + 8 * g);
        const float4 m1 = *reinterpret_cast<const float4*>(sb_mul + 8 * g + 4);
        const int ba[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const float bm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)  // acc >> 7 == 2 * (acc >> 8): the accumulator is a multiple of 256
            v[i] = (float)(((int)r[8 * g + i] >> 7) + a_add + ba[i]) * (half_a_mul * bm[i]);
#pragma unroll
        for (int i = 0; i < 4; ++i) w[4 * g + i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
    }
}

template <bool FUSED>
__device__ __forceinline__ void epilogue_store_chunk(const uint32_t (&r)[32], const EpilogueParams& ep, int row, int col0,
                                                     int N, int a_add, float half_a_mul, const int* sb_add,
                                                     const float* sb_mul) {
    if (FUSED) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(ep.out) + (size_t)row * ep.ld + col0;
        uint32_t w[16];  // the 32 results as bf16 pairs
        dequant_chunk(r, a_add, half_a_mul, sb_add, sb_mul, w);
        if (ep.vec_ok == 2 && col0 + 32 <= N) {
            stg256(out, w);
            stg256(out + 16, w + 8);
        } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const int col = col0 + 8 * g;
                if (ep.vec_ok && col + 8 <= N) {
                    *reinterpret_cast<uint4*>(out + 8 * g) = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (col + i < N)
                            reinterpret_cast<uint16_t*>(out)[8 * g + i] = (uint16_t)(w[4 * g + i / 2] >> (16 * (i & 1)));
                }
            }
        }
    } else {
        int32_t* out = static_cast<int32_t*>(ep.out) + (size_t)row * ep.ld + col0;
        if (ep.vec_ok == 2 && col0 + 32 <= N) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = (uint32_t)((int)r[8 * g + i] >> 8);
                stg256(out + 8 * g, w);
            }
            return;
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const int col = col0 + 4 * g;
            if (ep.vec_ok && col + 4 <= N) {
                *reinterpret_cast<int4*>(out + 4 * g) =
                    make_int4((int)r[4 * g] >> 8, (int)r[4 * g + 1] >> 8, (int)r[4 * g + 2] >> 8, (int)r[4 * g + 3] >> 8);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (col + i < N) out[4 * g + i] = (int)r[4 * g + i] >> 8;
            }
        }
    }
}

// The 16 bytes (32 codes) pk unpacked to the two 16-byte int8 chunks of the "times sixteen" form.
__device__ __forceinline__ void unpack_x16(const uint4& pk, uint4& lo, uint4& hi) {
    lo.x = (pk.x << 4) & 0xF0F0F0F0u; hi.x = pk.x & 0xF0F0F0F0u;
    lo.y = (pk.y << 4) & 0xF0F0F0F0u; hi.y = pk.y & 0xF0F0F0F0u;
    lo.z = (pk.z << 4) & 0xF0F0F0F0u; hi.z = pk.z & 0xF0F0F0F0u;
    lo.w = (pk.w << 4) & 0xF0F0F0F0u; hi.w = pk.w & 0xF0F0F0F0u;
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
// SPLIT: a work item is (output tile, K range).  The epilogue writes its shifted int32 partial sums to the item's own
// slab of ep.scratch (plain stores, nothing to zero); the CTA that completes a tile (a counter per tile tells) sums the
// tile's slabs, applies the normal epilogue and resets the counter for the next launch.
template <int BN, bool FUSED, bool SPLIT = false>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_i4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const EpilogueParams ep, const int M, const int N, const int K) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t u_base = smem_base;                                   // int8 ring, 1024-byte aligned stages
    const uint32_t p_base = u_base + C::U_STAGES * C::U_BYTES;           // packed ring
    const uint32_t vec_base = p_base + C::P_STAGES * C::P_BYTES;         // per-column epilogue vectors (16-byte aligned)
    const uint32_t bar_base = vec_base + C::VEC_BYTES;                   // mbarriers (8-byte aligned)
    const uint32_t full_p = bar_base;
    const uint32_t empty_p = full_p + 8 * C::P_STAGES;
    const uint32_t full_u = empty_p + 8 * C::P_STAGES;
    const uint32_t empty_u = full_u + 8 * C::U_STAGES;
    const uint32_t tmem_full = empty_u + 8 * C::U_STAGES;
    const uint32_t tmem_empty = tmem_full + 16;
    const uint32_t mma_done = tmem_empty + 16;
    const uint32_t out_ready = mma_done + 8;   // [2] epilogue -> push warps: the tile is in the local output
    const uint32_t push_free = out_ready + 16; // [2] push warps -> epilogue
    const uint32_t tmem_slot = push_free + 16;
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    // Set by an epilogue warp whose bounded wait gave up; read by all of them behind the named barrier every one of
    // them still reaches, so that they leave the tile loop together (none is left waiting at a later named barrier).
    volatile int* epi_abort = reinterpret_cast<volatile int*>(smem_raw + (tmem_slot + 12 - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int tiles_m = (M + BM - 1) / BM;
    const int tiles_n = (N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + BK - 1) / BK;
    // work items: output tiles, or (tile, K range) pairs with split-K
    const int S = SPLIT ? ep.splits : 1;
    const int num_items = num_tiles * S;
    auto tile_of = [&](int item) { return SPLIT ? item / S : item; };
    auto kb_first = [&](int item) { return SPLIT ? (int)((long long)(item % S) * num_kb / S) : 0; };
    auto kb_last = [&](int item) { return SPLIT ? (int)((long long)(item % S + 1) * num_kb / S) : num_kb; };

    if (threadIdx.x == 0) {
        QB_TRACE(0);
        for (int i = 0; i < C::P_STAGES; ++i) {
            mbar_init(full_p + 8 * i, 1);
            mbar_init(empty_p + 8 * i, kNumUnpackWarps);
        }
        for (int i = 0; i < C::U_STAGES; ++i) {
            mbar_init(full_u + 8 * i, kNumUnpackWarps);
            mbar_init(empty_u + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tmem_full + 8 * i, 1);
            mbar_init(tmem_empty + 8 * i, kNumEpilogueWarps);
        }
        mbar_init(mma_done, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(out_ready + 8 * i, kNumEpilogueWarps);
            mbar_init(push_free + 8 * i, kNumPushWarps);
        }
        fence_barrier_init();
        *epi_abort = 0;
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot_ptr;
    // Tensor memory is allocated: a kernel launched behind this one with a programmatic dependency (the next layer's
    // quantiser, which waits on the device) may be scheduled from now on.  Not earlier: a dependent block that shared
    // the SM and took the tensor memory first would wait for this grid while this block waits for the allocation.
    let_dependents_launch();
    wait_for_preceding_grid();  // barriers and tensor memory are set up; everything from here on may touch the A operand

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            uint32_t it = 0;
            bool ok = ep.test_skip_producer == 0;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
                const int tile = tile_of(item);
                const int m0 = (tile % tiles_m) * BM;
                const int n0 = (tile / tiles_m) * BN;
                for (int kb = kb_first(item), kb1 = kb_last(item); kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % C::P_STAGES, ph = (it / C::P_STAGES) & 1u;
                    if (!(ok = mbar_wait(empty_p + 8 * s, ph ^ 1u, 1))) break;
                    mbar_arrive_expect_tx(full_p + 8 * s, C::P_BYTES);
                    const uint32_t dst = p_base + s * C::P_BYTES;
                    tma_load_2d(dst, &tmap_a, kb * PK_ROW, m0, full_p + 8 * s);
                    tma_load_2d(dst + BM * PK_ROW, &tmap_b, kb * PK_ROW, n0, full_p + 8 * s);
                }
            }
            // Do not leave while a copy of ours may still land in this CTA's shared memory.
            const uint32_t pending = it < (uint32_t)C::P_STAGES ? it : (uint32_t)C::P_STAGES;
            for (uint32_t j = 0; j < pending; ++j) {
                const uint32_t i2 = it - 1 - j;
                mbar_wait(full_p + 8 * (i2 % C::P_STAGES), (i2 / C::P_STAGES) & 1u, 2);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local_tile) {
                const uint32_t acc = local_tile & 1u, acc_ph = (local_tile >> 1) & 1u;
                if (!(ok = mbar_wait(tmem_empty + 8 * acc, acc_ph ^ 1u, 3))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_acc + acc * BN;
                const int kb0 = kb_first(item);
                for (int kb = kb0, kb1 = kb_last(item); kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % C::U_STAGES, ph = (it / C::U_STAGES) & 1u;
                    if (!(ok = mbar_wait(full_u + 8 * s, ph, 4))) break;
                    tc_fence_after();
                    if (it == 0) QB_TRACE(1);
                    const uint32_t a_addr = u_base + s * C::U_BYTES;
                    const uint32_t b_addr = a_addr + BM * U8_ROW;
#pragma unroll
                    for (int j = 0; j < BK / 32; ++j) {
                        umma_i8(d_tmem, make_smem_desc(a_addr + 32 * j), make_smem_desc(b_addr + 32 * j), C::IDESC,
                                (kb != kb0 || j != 0) ? 1u : 0u);
                    }
                    umma_commit(empty_u + 8 * s);  // frees the int8 stage once these MMAs have read it
                }
                if (ok) umma_commit(tmem_full + 8 * acc);
            }
            // Everything issued so far must have completed before tensor memory is released.
            umma_commit(mma_done);
            mbar_wait(mma_done, 0, 5);
            QB_TRACE(2);
        }
    } else if (warp < kFirstUnpackWarp) {
        // ------------------------------ epilogue ------------------------------
        const int quad = warp & 3;  // tensor-memory lane quadrant this warp may read
        const int et = threadIdx.x - kFirstEpilogueWarp * 32;  // 0 .. 127
        uint8_t* vec_ptr = smem_raw + (vec_base - smem_u32(smem_raw));
        uint32_t local_tile = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local_tile) {
            const int tile = tile_of(item);
            const int m0 = (tile % tiles_m) * BM;
            const int n0 = (tile / tiles_m) * BN;
            const uint32_t acc = local_tile & 1u, acc_ph = (local_tile >> 1) & 1u;
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < M;
            int a_add = 0;
            float half_a_mul = 0.f;
            int* sb_add = reinterpret_cast<int*>(vec_ptr + acc * C::VEC_STRIDE);
            float* sb_mul = reinterpret_cast<float*>(vec_ptr + acc * C::VEC_STRIDE + BN * 4);
            if (FUSED) {
                // Everything the epilogue needs besides the accumulators is fetched while the tile is still being
                // accumulated: this tile's per-column vectors go to shared memory, the per-row pair to registers.
                for (int c = et; c < BN; c += kNumEpilogueWarps * 32) {
                    const bool in = n0 + c < N;
                    sb_add[c] = in ? ep.b_add[n0 + c] : 0;
                    sb_mul[c] = in ? bf16_to_f32(ep.b_mul[n0 + c]) : 0.f;
                }
                if (row_ok) {
                    a_add = ep.a_add[row];
                    half_a_mul = 0.5f * bf16_to_f32(ep.a_mul[row]);
                }
            }
            ok = mbar_wait(tmem_full + 8 * acc, acc_ph, 6);
            if (!ok) *epi_abort = 1;
            // the staged vectors are visible, and the give-up decision is the same for every epilogue warp
            asm volatile("bar.sync 1, %0;" ::"n"(kNumEpilogueWarps * 32) : "memory");
            if (*epi_abort) break;
            tc_fence_after();
            const uint32_t t_row = tmem_acc + ((uint32_t)(quad * 32) << 16) + acc * BN;
            if (SPLIT) {
                // This K range's partial sums -> the work item's own slab of scratch, [row of the tile][column],
                // plain 32-byte stores (rows inside M only).  No atomics, and nothing has to be zeroed.
                const int rows_valid = min(BM, M - m0);
                int32_t* slab = ep.scratch + (size_t)item * ep.slab_ints;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (n0 + c0 >= N) break;  // warp-uniform
                    uint32_t r0[32];
                    tmem_ld32(t_row + c0, r0);
                    tmem_ld_wait();
                    if (row_ok) {
                        int32_t* dst = slab + (quad * 32 + lane) * BN + c0;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) w[i] = (uint32_t)((int)r0[8 * g + i] >> 8);
                            stg256(dst + 8 * g, w);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty + 8 * acc);
                // which CTA completes the tile?  The one whose increment of the tile's counter finds splits - 1.
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(kNumEpilogueWarps * 32) : "memory");
                int* flag = reinterpret_cast<int*>(smem_raw + (tmem_slot + 8 - smem_u32(smem_raw)));
                if (et == 0) *flag = (atomicAdd(ep.counters + tile, 1) == S - 1) ? 1 : 0;
                asm volatile("bar.sync 1, %0;" ::"n"(kNumEpilogueWarps * 32) : "memory");
                if (*flag) {
                    // Sum the S slabs of the tile and apply the epilogue.  The (row, 8-column group) pieces are dealt
                    // out over all 128 epilogue threads, so that few valid rows still mean many loads in flight.
                    __threadfence();
                    const int32_t* tile_slabs = ep.scratch + (size_t)tile * S * ep.slab_ints;
                    const int groups = BN / 8;
                    for (int piece = et; piece < rows_valid * groups; piece += kNumEpilogueWarps * 32) {
                        const int pr = piece / groups, pc = (piece - pr * groups) * 8;
                        if (n0 + pc >= N) continue;
                        int acc8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        const int4* src = reinterpret_cast<const int4*>(tile_slabs + pr * BN + pc);
                        const int kSlabInt4 = ep.slab_ints / 4;
                        for (int sp = 0; sp < S; sp += 4) {  // four slabs' loads are in flight before the first add
                            int4 v[4][2];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const bool in = sp + u < S;
                                v[u][0] = in ? __ldcg(src + (size_t)(sp + u) * kSlabInt4) : make_int4(0, 0, 0, 0);
                                v[u][1] = in ? __ldcg(src + (size_t)(sp + u) * kSlabInt4 + 1) : make_int4(0, 0, 0, 0);
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                acc8[0] += v[u][0].x; acc8[1] += v[u][0].y; acc8[2] += v[u][0].z; acc8[3] += v[u][0].w;
                                acc8[4] += v[u][1].x; acc8[5] += v[u][1].y; acc8[6] += v[u][1].z; acc8[7] += v[u][1].w;
                            }
                        }
                        const int prow = m0 + pr;
                        if (FUSED) {
                            const int pa = ep.a_add[prow];
                            const float pm = 0.5f * bf16_to_f32(ep.a_mul[prow]);
                            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(ep.out) + (size_t)prow * ep.ld + n0 + pc;
                            uint32_t w[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float v0 = (float)(2 * acc8[2 * i] + pa + sb_add[pc + 2 * i]) * (pm * sb_mul[pc + 2 * i]);
                                const float v1 = (float)(2 * acc8[2 * i + 1] + pa + sb_add[pc + 2 * i + 1]) * (pm * sb_mul[pc + 2 * i + 1]);
                                w[i] = pack_bf16x2(v0, v1);
                            }
                            if (ep.vec_ok && n0 + pc + 8 <= N) {
                                *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (n0 + pc + i < N) reinterpret_cast<uint16_t*>(out)[i] = (uint16_t)(w[i / 2] >> (16 * (i & 1)));
                            }
                        } else {
                            int32_t* out = static_cast<int32_t*>(ep.out) + (size_t)prow * ep.ld + n0 + pc;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (n0 + pc + i < N) out[i] = acc8[i];
                        }
                    }
                    if (et == 0) ep.counters[tile] = 0;  // ready for the next launch
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kNumEpilogueWarps * 32) : "memory");  // the flag is reused by the next item
            }
#pragma unroll 1
            for (int c0 = 0; !SPLIT && c0 < BN; c0 += 64) {
                if (n0 + c0 >= N) break;  // warp-uniform
                uint32_t r0[32], r1[32];
                tmem_ld32(t_row + c0, r0);
                tmem_ld32(t_row + c0 + 32, r1);
                tmem_ld_wait();
                if (!row_ok) continue;
                epilogue_store_chunk<FUSED>(r0, ep, row, n0 + c0, N, a_add, half_a_mul, sb_add + c0, sb_mul + c0);
                if (n0 + c0 + 32 < N)
                    epilogue_store_chunk<FUSED>(r1, ep, row, n0 + c0 + 32, N, a_add, half_a_mul, sb_add + c0 + 32, sb_mul + c0 + 32);
            }
            if (!SPLIT) {  // this warp has finished reading the accumulator buffer
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty + 8 * acc);
            }
            if (warp == kFirstEpilogueWarp && lane == 0) QB_TRACE(3);
            if (!SPLIT && FUSED && ep.n_peer > 0) {
                // Hand the tile (now in the local output) to the push warps; at most two tiles may be pending.
                if (!mbar_wait(push_free + 8 * acc, acc_ph ^ 1u, 11)) *epi_abort = 1;  // all warps leave at the next tile's barrier
                __threadfence_block();
                __syncwarp();
                if (lane == 0) mbar_arrive(out_ready + 8 * acc);
            }
        }
    } else if (warp >= kFirstPushWarp) {
        // ------------------------------ push warps (multi-GPU only) ------------------------------
        // Re-read each finished tile from the local output (L2) one whole row segment per warp instruction and
        // store it to the same place of every peer buffer: 512-byte contiguous peer stores, which NVLink moves
        // far better than the 16-byte-per-row pieces the epilogue threads own.
        if (FUSED && ep.n_peer > 0) {
            const int pw = warp - kFirstPushWarp;
            uint32_t local_tile = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local_tile) {
                const int tile = tile_of(item);
                const int m0 = (tile % tiles_m) * BM;
                const int n0 = (tile / tiles_m) * BN;
                const uint32_t acc = local_tile & 1u, acc_ph = (local_tile >> 1) & 1u;
                ok = mbar_wait(out_ready + 8 * acc, acc_ph, 12);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const int rows = min(BM, M - m0);
                const int cols = min(BN, N - n0);  // multiple of 8 on this path (checked on the host)
                // eight rows per pass: all loads of a pass are in flight before the first store is issued
                for (int r0 = pw * 8; r0 < rows; r0 += kNumPushWarps * 8) {
                    for (int c = lane * 8; c < cols; c += 256) {
                        uint4 v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (r0 + j < rows) {
                                const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(ep.out) + (size_t)(m0 + r0 + j) * ep.ld + n0 + c;
                                asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                                             : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w) : "l"(src));
                            }
                        }
                        for (int pi = 0; pi < ep.n_peer; ++pi) {
                            __nv_bfloat16* dstp = static_cast<__nv_bfloat16*>(ep.peer_out[pi]) + (size_t)(m0 + r0) * ep.ld + n0 + c;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (r0 + j < rows) *reinterpret_cast<uint4*>(dstp + (size_t)j * ep.ld) = v[j];
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(push_free + 8 * acc);
            }
        }
    } else {
        // ------------------------------ unpack warps ------------------------------
        const int t = threadIdx.x - kFirstUnpackWarp * 32;  // 0 .. 255
        uint32_t it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            for (int kb = kb_first(item), kb1 = kb_last(item); kb < kb1; ++kb, ++it) {
                const uint32_t ps = it % C::P_STAGES, pph = (it / C::P_STAGES) & 1u;
                const uint32_t us = it % C::U_STAGES, uph = (it / C::U_STAGES) & 1u;
                ok = mbar_wait(full_p + 8 * ps, pph, 7) && mbar_wait(empty_u + 8 * us, uph ^ 1u, 8);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t src = p_base + ps * C::P_BYTES;
                const uint32_t dst = u_base + us * C::U_BYTES;
                constexpr int ITEMS = C::ROWS * 4 / (kNumUnpackWarps * 32);
                uint4 pk[ITEMS];
#pragma unroll
                for (int i = 0; i < ITEMS; ++i) {
                    const int item = t + i * kNumUnpackWarps * 32;
                    pk[i] = lds128(src + (item >> 2) * PK_ROW + (item & 3) * 16);
                }
#pragma unroll
                for (int i = 0; i < ITEMS; ++i) {
                    const int item = t + i * kNumUnpackWarps * 32;
                    const int r = item >> 2, c = item & 3;
                    uint4 lo, hi;
                    lo.x = (pk[i].x << 4) & 0xF0F0F0F0u; hi.x = pk[i].x & 0xF0F0F0F0u;
                    lo.y = (pk[i].y << 4) & 0xF0F0F0F0u; hi.y = pk[i].y & 0xF0F0F0F0u;
                    lo.z = (pk[i].z << 4) & 0xF0F0F0F0u; hi.z = pk[i].z & 0xF0F0F0F0u;
                    lo.w = (pk[i].w << 4) & 0xF0F0F0F0u; hi.w = pk[i].w & 0xF0F0F0F0u;
                    // 16-byte chunk index is XORed with (row & 7): the 128-byte swizzle of the UMMA layout.
                    const uint32_t rowaddr = dst + r * U8_ROW;
                    sts128(rowaddr + (((2 * c) ^ (r & 7)) << 4), lo);
                    sts128(rowaddr + (((2 * c + 1) ^ (r & 7)) << 4), hi);
                }
                fence_proxy_async_smem();  // make the generic-proxy stores visible to the tensor core
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_u + 8 * us);
                    mbar_arrive(empty_p + 8 * ps);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_acc, C::TMEM_COLS);
    }
}


// ---------------------------------------------------------------------------------------------
// The 256 x 256 tile kernel
// ---------------------------------------------------------------------------------------------
// The kernel above is bound by shared-memory traffic, not by the tensor core: per 128-K stage every operand row
// costs a TMA write, a 64-byte read, a 128-byte int8 write and the MMA's own reads.  A 256 x 256 output tile
// (two 128-row accumulators that share the B operand) halves the B traffic per unit of work.  Its price: the two
// accumulators fill all 512 columns of tensor memory, so the epilogue of a tile cannot overlap the MMAs of the
// next one (its TMA and unpack still do), and shared memory holds only two int8 stages.  The host picks this
// kernel where the estimated time is shorter (large M and N).
namespace wide {
constexpr int TM = 256, TN = 256;
constexpr int P_STAGES = 3, U_STAGES = 2;
constexpr int P_BYTES = (TM + TN) * PK_ROW;   // 32 KB packed per stage
constexpr int U_BYTES = (TM + TN) * U8_ROW;   // 64 KB int8 per stage
constexpr int kEpiWarps = 8, kFirstEpi = 2;
constexpr int kUnpackWarps = 8, kFirstUnpack = kFirstEpi + kEpiWarps;
constexpr int kPushWarps = 2, kFirstPush = kFirstUnpack + kUnpackWarps;
constexpr int kWarps = kFirstPush + kPushWarps;
constexpr int kThreads = kWarps * 32;
constexpr int VEC_BYTES = TN * 8;
constexpr int A_STAGES = 3;  // A8 variant: ring of the int8 A tiles (two in the A halves of the int8 stages, one behind the packed B ring)
constexpr int NUM_BARS = 2 * P_STAGES + 2 * U_STAGES + 2 + 1 + 4 + 2 * A_STAGES;
constexpr int LAYOUT_BYTES = U_STAGES * U_BYTES + P_STAGES * P_BYTES + VEC_BYTES + NUM_BARS * 8 + 16;
constexpr int SMEM_BYTES = 232448;  // all the shared memory one CTA can have; the layout needs a 1024-byte aligned start
static_assert(LAYOUT_BYTES <= SMEM_BYTES, "layout does not fit");
constexpr uint32_t IDESC_BASE = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 4) << 24);  // + (tile width >> 3) << 17
// First output column and width of tile column `col` (see EpilogueParams::col_count).
__device__ __forceinline__ void column_range(const EpilogueParams& ep, int col, int& n0, int& bn) {
    const int wider = col < ep.col_rem ? col : ep.col_rem;
    n0 = (col * ep.col_units + wider) << 4;
    bn = (ep.col_units + (col < ep.col_rem ? 1 : 0)) << 4;
}
}  // namespace wide

// Copies this warp's share of a finished tile (rows part*8 .. +7, then every parts*8 further) from the local output
// to the same place of every peer buffer: eight rows are loaded (L2) before the first 512-byte row segment is stored.
__device__ __noinline__ void push_tile_rows(const EpilogueParams& ep, int m0, int n0, int rows, int cols, int part,
                                            int parts, int lane) {
    for (int r0 = part * 8; r0 < rows; r0 += parts * 8) {
        for (int c = lane * 8; c < cols; c += 256) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (r0 + j < rows) {
                    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(ep.out) + (size_t)(m0 + r0 + j) * ep.ld + n0 + c;
                    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w) : "l"(src));
                }
            }
            for (int pi = 0; pi < ep.n_peer; ++pi) {
                __nv_bfloat16* dstp = static_cast<__nv_bfloat16*>(ep.peer_out[pi]) + (size_t)(m0 + r0) * ep.ld + n0 + c;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (r0 + j < rows) *reinterpret_cast<uint4*>(dstp + (size_t)j * ep.ld) = v[j];
            }
        }
    }
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the bulk stores issued by this thread have read their shared-memory source (their global writes complete
// on their own, at the latest when the grid ends): enough to let the CTA go.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// At most the newest bulk group of this thread may still be reading its shared-memory source.
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// One warp's share of a 256 x 256 tile: its 32 rows (tensor-memory lanes) x the columns [c_begin, c_end), in pieces of 64.
// stage_base == 0: every thread stores its row's results itself (32-byte pieces).  stage_base != 0 (fused output, the
// CTA's last tile, when the shared-memory rings are no longer needed): the warp writes each 32 x 64 piece as bf16 into
// its own 4 KB slab of shared memory in the 128-byte-swizzled layout and one bulk tensor store moves the slab to the
// output as whole 128-byte lines; rows and columns outside the matrix are clipped by the tensor map.  Per-thread
// 32-byte stores to 32 different rows per instruction cost the store path about 3 us per tile; the bulk stores do not.
// Tensor maps of the same output matrix in the memory of the other GPUs (multi-GPU variant only): the staged pieces of a
// CTA's last tile are stored to them with the same bulk tensor stores as to the local output - plain stores over NVLink,
// no multicast, issued by the copy engine of the SM instead of by push warps.
template <bool PUSH>
struct PeerMaps {
    CUtensorMap m[PUSH ? 7 : 1];
};

template <bool FUSED>
__device__ __forceinline__ void wide_convert_columns(const EpilogueParams& ep, const CUtensorMap* tmap_d,
                                                     const CUtensorMap* peer_maps, int n_peer_maps, uint32_t t_row,
                                                     int row, bool row_ok, int a_add, float half_a_mul, const int* sb_add,
                                                     const float* sb_mul, int n0, int N, int c_begin, int c_end,
                                                     uint32_t stage_base, int warp_row0, int lane,
                                                     const CUtensorMap* tmap_d16 = nullptr, uint32_t mini_base = 0,
                                                     uint32_t* mini_count = nullptr) {
    if (FUSED && mini_base != 0) {
        // A tile that is not the CTA's last one (int8-operand variant): the rings belong to the next tile already, but
        // 16 KB of shared memory are free there - two 1 KB slabs per epilogue warp.  The warp writes 32 rows x 16
        // columns of bf16 (dense rows of 32 bytes) into one slab while the bulk store of the other is still being
        // read, so the stores leave through the copy engine behind the arithmetic instead of occupying the warp's store
        // path (about 3 us per tile), and tensor memory is released for the next tile's MMAs as soon as it has been
        // read.  Rows and columns outside the matrix are clipped by the tensor map.
        uint32_t piece = *mini_count;
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 64) {
            if (n0 + c0 >= N) break;  // warp-uniform
            uint32_t r0[32], r1[32];
            tmem_ld32(t_row + c0, r0);
            tmem_ld32(t_row + c0 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (c0 + 32 * h >= c_end) break;  // widths are multiples of 16: a tile may end inside a chunk
                uint32_t w[16];
                dequant_chunk(h == 0 ? r0 : r1, a_add, half_a_mul, sb_add + c0 + 32 * h, sb_mul + c0 + 32 * h, w);
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int c = c0 + 32 * h + 16 * q;
                    if (c >= c_end) break;
                    const uint32_t slab = mini_base + (piece & 1u) * 1024u;
                    if (lane == 0) bulk_wait_read_but_one();  // the store that used this slab two pieces ago has read it
                    __syncwarp();
                    sts128(slab + lane * 32, make_uint4(w[8 * q], w[8 * q + 1], w[8 * q + 2], w[8 * q + 3]));
                    sts128(slab + lane * 32 + 16, make_uint4(w[8 * q + 4], w[8 * q + 5], w[8 * q + 6], w[8 * q + 7]));
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(tmap_d16, slab, n0 + c, warp_row0);
                        bulk_commit_group();
                    }
                    ++piece;
                }
            }
        }
        *mini_count = piece;
        return;
    }
#pragma unroll 1
    for (int cx = c_begin; cx < c_end; cx += 64) {
        // a tile width that is no multiple of 64: the last piece starts earlier and rewrites columns of the one before
        // it (with the same values) instead of reaching into the next tile
        const int c0 = cx + 64 <= c_end ? cx : c_end - 64;
        if (n0 + c0 >= N) break;  // warp-uniform
        uint32_t r0[32], r1[32];
        tmem_ld32(t_row + c0, r0);
        tmem_ld32(t_row + c0 + 32, r1);
        tmem_ld_wait();
        if (FUSED && stage_base != 0) {
            const uint32_t slab = stage_base + (uint32_t)(cx >> 6) * 4096u;
            if (row_ok) {
                const uint32_t rowaddr = slab + lane * 128;
                uint32_t w[16];
                dequant_chunk(r0, a_add, half_a_mul, sb_add + c0, sb_mul + c0, w);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    sts128(rowaddr + ((j ^ (lane & 7)) << 4), make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
                dequant_chunk(r1, a_add, half_a_mul, sb_add + c0 + 32, sb_mul + c0 + 32, w);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    sts128(rowaddr + (((4 + j) ^ (lane & 7)) << 4), make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(tmap_d, slab, n0 + c0, warp_row0);
                for (int pi = 0; pi < n_peer_maps; ++pi) tma_store_2d(peer_maps + pi, slab, n0 + c0, warp_row0);
                bulk_commit_group();
            }
            continue;
        }
        if (!row_ok) continue;
        epilogue_store_chunk<FUSED>(r0, ep, row, n0 + c0, N, a_add, half_a_mul, sb_add + c0, sb_mul + c0);
        if (n0 + c0 + 32 < N)
            epilogue_store_chunk<FUSED>(r1, ep, row, n0 + c0 + 32, N, a_add, half_a_mul, sb_add + c0 + 32, sb_mul + c0 + 32);
    }
    if (FUSED && stage_base != 0 && lane == 0) {
        if (n_peer_maps > 0) bulk_wait_all();  // stores to other GPUs: complete before this thread goes on
        else bulk_wait_read_all();             // the slabs have been read before the CTA ends
    }
}

// PUSH: the multi-GPU variant (two more warps that copy finished tiles to the peers, helped by the epilogue warps on
// a CTA's last tile); the single-GPU instantiation carries none of that code and is launched without those warps.
// A8 (single GPU only): the A operand arrives already as int8 in operand order (see hadamard_quant_tc_kernel<HB, true>):
// one more warp copies its tiles with TMA (128-byte swizzle) straight into the int8 ring, the unpack warps handle
// only B, and the main loop is bound by the MMAs instead of the unpack.
template <bool FUSED, bool PUSH, bool A8 = false, bool CLIP = A8>
__global__ void __launch_bounds__(PUSH ? wide::kThreads : (A8 ? wide::kThreads - 32 : wide::kThreads - 32 * wide::kPushWarps), 1)
gemm_i4_wide_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ CUtensorMap tmap_d16,
                    const __grid_constant__ PeerMaps<PUSH> peers, const __grid_constant__ EpilogueParams ep, const int M,
                    const int N, const int K) {
    using namespace wide;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_base = smem_u32(smem_raw);
    const uint32_t smem_base = (raw_base + 1023u) & ~1023u;
    if (smem_base - raw_base + LAYOUT_BYTES > SMEM_BYTES) {  // uniform over the CTA: nothing has been set up yet
        if (threadIdx.x == 0) atomicCAS(&g_device_status, 0, (13 << 8) | QB200_ERR_DEVICE_TIMEOUT);
        return;
    }
    const uint32_t u_base = smem_base;
    const uint32_t p_base = u_base + U_STAGES * U_BYTES;
    const uint32_t vec_base = p_base + P_STAGES * P_BYTES;
    const uint32_t bar_base = vec_base + VEC_BYTES;
    const uint32_t full_p = bar_base;
    const uint32_t empty_p = full_p + 8 * P_STAGES;
    const uint32_t full_u = empty_p + 8 * P_STAGES;
    const uint32_t empty_u = full_u + 8 * U_STAGES;
    const uint32_t tmem_full = empty_u + 8 * U_STAGES;
    const uint32_t tmem_empty = tmem_full + 8;
    const uint32_t mma_done = tmem_empty + 8;
    const uint32_t out_ready = mma_done + 8;    // [2]
    const uint32_t push_free = out_ready + 16;  // [2]
    const uint32_t full_a = push_free + 16;      // [A_STAGES] A8 only
    const uint32_t empty_a = full_a + 8 * A_STAGES;
    const uint32_t tmem_slot = empty_a + 8 * A_STAGES;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw_base));
    volatile int* epi_abort = reinterpret_cast<volatile int*>(smem_raw + (tmem_slot + 12 - raw_base));  // see gemm_i4_kernel
    // A8: packed B stages are compact (TN * 64 bytes each), which leaves room for a third A slot behind them
    constexpr int PB_BYTES = A8 ? TN * PK_ROW : P_BYTES;
    auto a_slot = [&](uint32_t sa) { return sa < 2 ? u_base + sa * U_BYTES : p_base + P_STAGES * (TN * PK_ROW); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = (M + TM - 1) / TM;
    const int num_tiles = tiles_m * ep.col_count;
    const int num_kb = (K + BK - 1) / BK;
    uint32_t pre_issued = 0;  // producer thread: copies already issued before the CTA-wide synchronisation

    if (threadIdx.x == 0) {
        QB_TRACE(0);
        for (int i = 0; i < P_STAGES; ++i) {
            mbar_init(full_p + 8 * i, 1);
            mbar_init(empty_p + 8 * i, kUnpackWarps);
        }
        for (int i = 0; i < U_STAGES; ++i) {
            mbar_init(full_u + 8 * i, kUnpackWarps);
            mbar_init(empty_u + 8 * i, 1);
        }
        for (int i = 0; i < A_STAGES; ++i) {
            mbar_init(full_a + 8 * i, 1);
            mbar_init(empty_a + 8 * i, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, kEpiWarps);
        mbar_init(mma_done, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(out_ready + 8 * i, kEpiWarps);
            mbar_init(push_free + 8 * i, kPushWarps);
        }
        fence_barrier_init();
        *epi_abort = 0;
        // The first copies of the CTA's first tile leave before tensor memory is allocated and the CTA has synchronised:
        // they need nothing but the barriers initialised above (this thread is also the producer thread below).
        if (ep.test_skip_producer == 0 && (int)blockIdx.x < num_tiles) {
            if (!A8) wait_for_preceding_grid();  // these copies include A tiles
            if (!A8) tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            const int m0 = ((int)blockIdx.x % tiles_m) * TM;
            int n0, bn;
            column_range(ep, (int)blockIdx.x / tiles_m, n0, bn);
            for (; pre_issued < (uint32_t)P_STAGES && (int)pre_issued < num_kb; ++pre_issued) {
                mbar_arrive_expect_tx(full_p + 8 * pre_issued, PB_BYTES);
                const uint32_t dst = p_base + pre_issued * PB_BYTES;
                if (!A8) tma_load_2d(dst, &tmap_a, (int)pre_issued * PK_ROW, m0, full_p + 8 * pre_issued);
                tma_load_2d(A8 ? dst : dst + TM * PK_ROW, &tmap_b, (int)pre_issued * PK_ROW, n0, full_p + 8 * pre_issued);
            }
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot_ptr;
    let_dependents_launch();  // only now that tensor memory is allocated (see gemm_i4_kernel)
    // The packed variants load A from the first copy on: every thread waits here.  A8: only the warps that touch the
    // quantiser's outputs wait (A producer, epilogue), the weights are requested, copied and unpacked before.
    if (!A8) wait_for_preceding_grid();

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = ep.test_skip_producer == 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TM;
                int n0, bn;
                column_range(ep, tile / tiles_m, n0, bn);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    if (it < pre_issued) continue;  // left before the CTA synchronised
                    const uint32_t s = it % P_STAGES, ph = (it / P_STAGES) & 1u;
                    if (!(ok = mbar_wait(empty_p + 8 * s, ph ^ 1u, 1))) break;
                    mbar_arrive_expect_tx(full_p + 8 * s, PB_BYTES);
                    const uint32_t dst = p_base + s * PB_BYTES;
                    if (!A8) tma_load_2d(dst, &tmap_a, kb * PK_ROW, m0, full_p + 8 * s);
                    tma_load_2d(A8 ? dst : dst + TM * PK_ROW, &tmap_b, kb * PK_ROW, n0, full_p + 8 * s);
                }
            }
            const uint32_t pending = it < (uint32_t)P_STAGES ? it : (uint32_t)P_STAGES;
            for (uint32_t j = 0; j < pending; ++j) {
                const uint32_t i2 = it - 1 - j;
                mbar_wait(full_p + 8 * (i2 % P_STAGES), (i2 / P_STAGES) & 1u, 2);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
                const int m0 = (tile % tiles_m) * TM;
                const int halves = (m0 + 128 < M) ? 2 : 1;  // the lower accumulator is skipped when its rows are all outside M
                int n0, bn;
                column_range(ep, tile / tiles_m, n0, bn);
                const uint32_t idesc = IDESC_BASE | ((uint32_t)(bn >> 3) << 17);
                if (!(ok = mbar_wait(tmem_empty, (local_tile & 1u) ^ 1u, 3))) break;
                tc_fence_after();
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % U_STAGES, ph = (it / U_STAGES) & 1u;
                    if (!(ok = mbar_wait(full_u + 8 * s, ph, 4))) break;
                    tc_fence_after();
                    if (it == 0) QB_TRACE(1);
                    const uint32_t sa = it % A_STAGES;
                    if (A8) {
                        if (!(ok = mbar_wait(full_a + 8 * sa, (it / A_STAGES) & 1u, 21))) break;
                        tc_fence_after();
                    }
                    const uint32_t a_addr = A8 ? a_slot(sa) : u_base + s * U_BYTES;
                    const uint32_t b_addr = u_base + s * U_BYTES + TM * U8_ROW;
#pragma unroll
                    for (int j = 0; j < BK / 32; ++j) {
                        const uint64_t db = make_smem_desc(b_addr + 32 * j);
                        umma_i8(tmem_acc, make_smem_desc(a_addr + 32 * j), db, idesc, (kb | j) != 0 ? 1u : 0u);
                        if (halves == 2)
                            umma_i8(tmem_acc + TN, make_smem_desc(a_addr + 128 * U8_ROW + 32 * j), db, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_u + 8 * s);
                    if (A8) umma_commit(empty_a + 8 * sa);
                }
                if (ok) umma_commit(tmem_full);
            }
            umma_commit(mma_done);
            mbar_wait(mma_done, 0, 5);
            QB_TRACE(2);
        }
    } else if (warp < kFirstUnpack) {
        // ------------------------------ epilogue ------------------------------
        const int quad = warp & 3;                  // tensor-memory lane quadrant this warp may read
        const int half = (warp - kFirstEpi) >> 2;   // which accumulator (rows 0-127 or 128-255 of the tile)
        const int et = threadIdx.x - kFirstEpi * 32;  // 0 .. 255
        uint8_t* vec_ptr = smem_raw + (vec_base - raw_base);
        int* sb_add = reinterpret_cast<int*>(vec_ptr);
        float* sb_mul = reinterpret_cast<float*>(vec_ptr + TN * 4);
        uint32_t local_tile = 0, mini_pieces = 0;
        bool ok = true;
        if (A8) wait_for_preceding_grid();  // the row sums and scales come from the quantiser
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
            const int m0 = (tile % tiles_m) * TM;
            int n0, bn;
            column_range(ep, tile / tiles_m, n0, bn);
            const uint32_t slot = local_tile & 1u, slot_ph = (local_tile >> 1) & 1u;
            const int row = m0 + half * 128 + quad * 32 + lane;
            const bool row_ok = row < M;
            int a_add = 0;
            float half_a_mul = 0.f;
            if (FUSED) {
                // all epilogue warps are done with the previous tile's vectors before they are overwritten
                asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
                {
                    const bool in = et < bn && n0 + et < N;
                    sb_add[et] = in ? ep.b_add[n0 + et] : 0;
                    sb_mul[et] = in ? bf16_to_f32(ep.b_mul[n0 + et]) : 0.f;
                }
                if (row_ok) {
                    a_add = ep.a_add[row];
                    half_a_mul = 0.5f * bf16_to_f32(ep.a_mul[row]);
                }
            }
            ok = mbar_wait(tmem_full, local_tile & 1u, 6);
            if (!ok) *epi_abort = 1;
            asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * 32) : "memory");  // vectors staged; uniform give-up decision
            if (*epi_abort) break;
            tc_fence_after();
            const uint32_t t_row = tmem_acc + ((uint32_t)(quad * 32) << 16) + half * TN;
            // The CTA's last tile leaves through shared memory: the int8 ring is free once the tile's MMAs have completed.
            // In the multi-GPU variant the same staged pieces are stored to every peer's output as well, so that tile
            // needs neither the local round trip nor the push warps.
            const bool last = tile + (int)gridDim.x >= num_tiles;
            const bool staged = FUSED && last && ep.tma_store;
            const uint32_t stage_base = staged ? u_base + (uint32_t)(half * 4 + quad) * 16384u : 0u;
            // int8-operand variant, earlier tiles: the 16 KB behind the third A slot hold two 1 KB slabs per epilogue warp
            const uint32_t mini_base = (A8 && FUSED && !staged && ep.tma_store16)
                                           ? p_base + (uint32_t)(P_STAGES * (TN * PK_ROW) + TM * U8_ROW) + (uint32_t)(warp - kFirstEpi) * 2048u
                                           : 0u;
            if (m0 + half * 128 < M)  // warp-uniform: otherwise this accumulator was not computed
                wide_convert_columns<FUSED>(ep, &tmap_d, peers.m, PUSH ? ep.n_peer : 0, t_row, row, row_ok, a_add, half_a_mul,
                                            sb_add, sb_mul, n0, N, 0, bn, stage_base, m0 + half * 128 + quad * 32, lane,
                                            &tmap_d16, mini_base, &mini_pieces);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty);
            if (warp == kFirstEpi && lane == 0) QB_TRACE(3);
            if (PUSH && !staged) {
                if (!mbar_wait(push_free + 8 * slot, slot_ph ^ 1u, 11)) *epi_abort = 1;  // all warps leave at the next tile's barrier
                __threadfence_block();
                __syncwarp();
                if (lane == 0) mbar_arrive(out_ready + 8 * slot);
                if (tile + (int)gridDim.x >= num_tiles) {  // last tile: wait until all of it is in the local output, then help
                    ok = mbar_wait(out_ready + 8 * slot, slot_ph, 18);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;  // no named barrier follows the last tile
                    push_tile_rows(ep, m0, n0, min(TM, M - m0), min(bn, N - n0), kPushWarps + (warp - kFirstEpi),
                                   kPushWarps + kEpiWarps, lane);
                }
            }
        }
    } else if (A8 && warp == kFirstPush) {
        // ------------------------------ A operand producer (A8 only; there are no push warps then) -----------
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            wait_for_preceding_grid();  // the A operand is the quantiser's output
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TM;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t sa = it % A_STAGES, aph = (it / A_STAGES) & 1u;
                    if (!(ok = mbar_wait(empty_a + 8 * sa, aph ^ 1u, 19))) break;
                    mbar_arrive_expect_tx(full_a + 8 * sa, TM * U8_ROW);
                    tma_load_2d(a_slot(sa), &tmap_a, kb * U8_ROW, m0, full_a + 8 * sa);
                }
            }
            const uint32_t pending = it < (uint32_t)A_STAGES ? it : (uint32_t)A_STAGES;
            for (uint32_t j = 0; j < pending; ++j) {  // do not leave while a copy of ours may still land
                const uint32_t i2 = it - 1 - j;
                mbar_wait(full_a + 8 * (i2 % A_STAGES), (i2 / A_STAGES) & 1u, 20);
            }
        }
    } else if (warp >= kFirstPush) {
        // ------------------------------ push warps (multi-GPU only) ------------------------------
        if (PUSH) {
            const int pw = warp - kFirstPush;
            uint32_t local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
                if (FUSED && ep.tma_store && tile + (int)gridDim.x >= num_tiles) break;  // the epilogue warps send the last tile
                const int m0 = (tile % tiles_m) * TM;
                int n0, bn;
                column_range(ep, tile / tiles_m, n0, bn);
                const uint32_t slot = local_tile & 1u, slot_ph = (local_tile >> 1) & 1u;
                ok = mbar_wait(out_ready + 8 * slot, slot_ph, 12);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const int rows = min(TM, M - m0);
                const int cols = min(bn, N - n0);
                // the CTA's last tile: the epilogue warps have nothing left to do and push as well
                const bool last = tile + (int)gridDim.x >= num_tiles;
                push_tile_rows(ep, m0, n0, rows, cols, pw, last ? kPushWarps + kEpiWarps : kPushWarps, lane);
                __syncwarp();
                if (lane == 0) mbar_arrive(push_free + 8 * slot);
            }
        }
    } else {
        // ------------------------------ unpack warps ------------------------------
        const int t = threadIdx.x - kFirstUnpack * 32;  // 0 .. 255
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            // CLIP (a launch with tile columns narrower than 256): B rows beyond the tile's width (a multiple of 16, so the
            // test is warp-uniform) are not unpacked.  A template parameter, not a run-time test: inside the plain loop the
            // tests cost the packed variant 2-7 %.
            int b_end = TM + TN;
            if (CLIP) {
                int n0, bn;
                column_range(ep, tile / tiles_m, n0, bn);
                b_end = TM + bn;
            }
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const uint32_t ps = it % P_STAGES, pph = (it / P_STAGES) & 1u;
                const uint32_t us = it % U_STAGES, uph = (it / U_STAGES) & 1u;
                ok = mbar_wait(full_p + 8 * ps, pph, 7) && mbar_wait(empty_u + 8 * us, uph ^ 1u, 8);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t src = A8 ? p_base + ps * PB_BYTES - TM * PK_ROW : p_base + ps * P_BYTES;  // rows are numbered from the A rows on
                const uint32_t dst = u_base + us * U_BYTES;
                constexpr int ITEMS = (TM + TN) * 4 / (kUnpackWarps * 32);  // 8
#pragma unroll
                for (int h = A8 ? 1 : 0; h < 2; ++h) {  // the first half of the items are the A rows
                    uint4 pk[ITEMS / 2];
#pragma unroll
                    for (int i = 0; i < ITEMS / 2; ++i) {
                        const int item = t + (h * (ITEMS / 2) + i) * kUnpackWarps * 32;
                        if (!CLIP || (item >> 2) < b_end) pk[i] = lds128(src + (item >> 2) * PK_ROW + (item & 3) * 16);
                    }
#pragma unroll
                    for (int i = 0; i < ITEMS / 2; ++i) {
                        const int item = t + (h * (ITEMS / 2) + i) * kUnpackWarps * 32;
                        const int r = item >> 2, c = item & 3;
                        if (CLIP && r >= b_end) continue;
                        uint4 lo, hi;
                        unpack_x16(pk[i], lo, hi);
                        const uint32_t rowaddr = dst + r * U8_ROW;
                        sts128(rowaddr + (((2 * c) ^ (r & 7)) << 4), lo);
                        sts128(rowaddr + (((2 * c + 1) ^ (r & 7)) << 4), hi);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_u + 8 * us);
                    mbar_arrive(empty_p + 8 * ps);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_acc, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
// Packed operand [rows, K/2] bytes, row-major; box = 64 bytes x box_rows, no swizzle, zero fill outside.
static int make_packed_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return QB200_ERR_DRIVER;
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    const cuuint32_t box[2] = {(cuuint32_t)PK_ROW, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QB200_OK : QB200_ERR_DRIVER;
}

static int sm_count_of_current_device(int* dev_out) {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev_out) *dev_out = dev;
    if (dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

template <int BN, bool FUSED, bool SPLIT = false>
static int launch_gemm(const EpilogueParams& ep, const void* a, const void* b, int M, int K, int N, int sms, int dev,
                       cudaStream_t stream) {
    using C = Cfg<BN>;
    static bool attr_set[64] = {false};
    auto kernel = gemm_i4_kernel<BN, FUSED, SPLIT>;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
            return QB200_ERR_CUDA;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    CUtensorMap ma, mb;
    int st = make_packed_map(&ma, a, M, K, BM);
    if (st != QB200_OK) return st;
    st = make_packed_map(&mb, b, N, K, BN);
    if (st != QB200_OK) return st;
    const int items = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * (SPLIT ? ep.splits : 1);
    const int grid = items < sms ? items : sms;
    // the two push warps are the last ones of the block: without peers they are simply not launched
    const int threads = ep.n_peer > 0 ? kNumThreads : kNumThreads - 32 * kNumPushWarps;
    if (launch_kernel(kernel, grid, threads, C::SMEM_BYTES, stream, ma, mb, ep, M, N, K) != cudaSuccess) {
        cudaGetLastError();
        return QB200_ERR_CUDA;
    }
    return launch_status();
}

// ---- split-K scratch --------------------------------------------------------------------------------------------
// Split-K needs a rows x 256 int32 slab per work item (tile, K range) and one counter per output tile; the counters are
// zero between launches (the kernel leaves them so; reset_split_counters() restores that after a kernel reported a
// timeout), the slabs need no initialisation.  The ordinary entry points keep ONE such buffer per device.  It has a
// fixed size - kSplitSlabs slabs of 128 x 256 int32 (21 MB) and kSplitTiles counters, enough for every split the
// library chooses itself (tiles x ranges <= number of SMs) - is allocated on the first launch that wants it and is
// never freed, grown or moved afterwards: a CUDA graph that captured a split-K launch keeps valid pointers for the
// life of the process.  It is not allocated while the stream is being captured; a request that does not fit (only a
// forced split count can ask for that) or cannot be served runs the kernels without split-K instead.  One split-K
// launch per device may be in flight at a time (launches on one stream are).
struct SplitScratch {
    int32_t* sums = nullptr;
    int* counters = nullptr;
    size_t ints = 0;
    int tiles = 0;
};
constexpr size_t kSplitSlabs = 160;
constexpr size_t kSplitInts = kSplitSlabs * 128 * 256;
constexpr int kSplitTiles = 4096;
static SplitScratch g_split_scratch[64];
static std::mutex g_split_mutex;

static bool get_split_scratch(int dev, cudaStream_t stream, size_t need_ints, int need_tiles, SplitScratch* out) {
    if (dev < 0 || dev >= 64) return false;
    if (need_ints > kSplitInts || need_tiles > kSplitTiles) return false;
    std::lock_guard<std::mutex> lock(g_split_mutex);
    SplitScratch& ws = g_split_scratch[dev];
    if (ws.sums == nullptr) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            return false;
        }
        void* ptr = nullptr;
        if (cudaMalloc(&ptr, (kSplitInts + (size_t)kSplitTiles) * sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        int* counters = reinterpret_cast<int*>(static_cast<int32_t*>(ptr) + kSplitInts);
        if (cudaMemset(counters, 0, (size_t)kSplitTiles * sizeof(int)) != cudaSuccess) {  // synchronous: done before any launch
            cudaFree(ptr);
            cudaGetLastError();
            return false;
        }
        ws.sums = static_cast<int32_t*>(ptr);
        ws.counters = counters;
        ws.ints = kSplitInts;
        ws.tiles = kSplitTiles;
    }
    *out = ws;
    return true;
}

// The same scratch as a fixed array in device memory, for the entry point that must not allocate: 2 Mi int32
// (8 MiB) of slabs - work items x rows per slab <= 8192 - and 1024 tile counters.  Static storage is zero at module
// load and the kernel leaves the counters zero, so nothing ever has to initialise it.
constexpr size_t kStaticScratchInts = (size_t)2 << 20;
constexpr int kStaticScratchTiles = 1024;
static __device__ __align__(256) int g_static_scratch[kStaticScratchInts + kStaticScratchTiles];

static bool get_static_scratch(int dev, SplitScratch* out) {
    static int32_t* cached[64] = {nullptr};  // the symbol's address, looked up once per device
    if (dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(g_split_mutex);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return false;
        }
        cached[dev] = static_cast<int32_t*>(ptr);
    }
    out->sums = cached[dev];
    out->counters = reinterpret_cast<int*>(cached[dev] + kStaticScratchInts);
    out->ints = kStaticScratchInts;
    out->tiles = kStaticScratchTiles;
    return true;
}

// Zeroes the tile counters of both scratch buffers of the current device.  A launch that ended through a bounded-wait
// timeout may have left counters half way; without this every later split-K launch on the device would complete its
// tiles too early or never.  Called (after a device synchronisation) when a non-zero device status is fetched.
static void reset_split_counters() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    int* allocated = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_split_mutex);
        allocated = g_split_scratch[dev].counters;
    }
    if (allocated != nullptr) cudaMemset(allocated, 0, (size_t)kSplitTiles * sizeof(int));
    SplitScratch st;
    if (get_static_scratch(dev, &st)) cudaMemset(st.counters, 0, (size_t)kStaticScratchTiles * sizeof(int));
    cudaGetLastError();
}

// Number of K ranges for the 128 x 256 kernel, or 1.  Split-K pays when the output has so few tiles that most SMs
// would idle while each busy one walks the whole K serially (small M: the MMA issue rate, ~154 cycles per K=32 step
// whatever the tile width, makes a CTA need ~10 us for K = 4096).
static int pick_splits(int M, int N, int K, int sms) {
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
    const int num_kb = (K + BK - 1) / BK;
    long long s = sms / tiles;
    if (s > num_kb / 2) s = num_kb / 2;
    if (s > 16) s = 16;
    return s >= 2 ? (int)s : 1;
}

// Fused output D as bf16 [M, N] with row pitch ld: box = 64 columns (128 bytes, the swizzle span) x 32 rows, the piece one
// warp of the 256 x 256 kernel stores at a time; the same for every peer output of the multi-GPU variant.  Leaves
// ep->tma_store 0 where a tensor map cannot describe an output: the kernel then keeps to per-thread stores (and push
// warps).  QB200_GEMM_TMA_STORE=0 switches the bulk stores off.
static int encode_output_map(CUtensorMap* map, void* base, long long ld, int M, int N) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return QB200_ERR_DRIVER;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, 32};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? QB200_OK : QB200_ERR_DRIVER;
}

// The same output as 32-row x 16-column boxes of dense 32-byte rows (no swizzle): what an epilogue warp of the
// int8-operand variant stores per piece of a tile that is not its CTA's last one.
static int encode_output_map16(CUtensorMap* map, void* base, long long ld, int M, int N) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return QB200_ERR_DRIVER;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {16, 32};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? QB200_OK : QB200_ERR_DRIVER;
}

template <bool PUSH>
static void make_output_maps(CUtensorMap* map, PeerMaps<PUSH>* peers, EpilogueParams* ep, int M, int N) {
    memset(map, 0, sizeof(*map));
    memset(peers, 0, sizeof(*peers));
    ep->tma_store = 0;
    if (!aligned16(ep->out) || ep->ld % 8 != 0) return;
    if (const char* e = getenv("QB200_GEMM_TMA_STORE"))
        if (e[0] == '0') return;
    if (PUSH != (ep->n_peer > 0)) return;
    if (encode_output_map(map, ep->out, ep->ld, M, N) != QB200_OK) return;
    for (int i = 0; PUSH && i < ep->n_peer; ++i)
        if (!aligned16(ep->peer_out[i]) || encode_output_map(&peers->m[i], ep->peer_out[i], ep->ld, M, N) != QB200_OK) return;
    ep->tma_store = 1;
}

// A operand as int8 [rows, K] row-major; box = 128 bytes (one K stage, the swizzle span) x 256 rows.
static int make_a8_map(CUtensorMap* map, const void* base, int rows, int K) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return QB200_ERR_DRIVER;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K};
    const cuuint32_t box[2] = {(cuuint32_t)U8_ROW, (cuuint32_t)wide::TM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QB200_OK : QB200_ERR_DRIVER;
}

// Tile columns of the 256-row kernel.  All 256 wide by default.  With `balance`, where more, narrower columns fill the
// same number of waves over the SMs (M = 2048, N = 4096 on 148 SMs: 8 x 16 = 128 tiles leave 20 SMs idle; 8 x 18 tiles
// of 224 or 240 columns use 144 and every CTA finishes 1/16 earlier), N is cut into that many columns instead.
static void wide_columns(EpilogueParams* ep, int M, int N, int sms, bool balance, int min_units = 12, int max_units = 15,
                         int align_units = 1) {
    const int tiles_m = (M + wide::TM - 1) / wide::TM;
    ep->col_count = (N + wide::TN - 1) / wide::TN;
    ep->col_units = wide::TN / 16;
    ep->col_rem = 0;
    if (const char* e = getenv("QB200_GEMM_BALANCE"))
        if (e[0] == '0') balance = false;
    if (!balance || sms <= 0) return;
    const int units = (N + 15) / 16;
    const long long waves = ((long long)tiles_m * ep->col_count + sms - 1) / sms;
    const int most = (int)(waves * sms / tiles_m);  // the most columns that still fit these waves
    if (most <= ep->col_count) return;
    int widest = (units + most - 1) / most;
    if (align_units > 1) {
        // Every column equally wide, a multiple of align_units * 16 (64 columns = 128 bytes of bf16): what the multi-GPU
        // variant needs, whose 64-column bulk stores to the peers should cover whole 128-byte lines and no column twice.
        widest = (widest + align_units - 1) / align_units * align_units;
        if (widest > max_units || widest < min_units) return;
        ep->col_count = (units + widest - 1) / widest;
        ep->col_units = widest;
        ep->col_rem = 0;
        return;
    }
    if (widest > max_units || widest < min_units) return;  // nothing gained / tiles too narrow for this variant
    ep->col_count = most;
    ep->col_units = units / most;
    ep->col_rem = units % most;
}

static int launch_gemm_wide_a8(const EpilogueParams& ep_in, const void* a8, const void* b, int M, int K, int N, int sms,
                               int dev, cudaStream_t stream) {
    EpilogueParams ep = ep_in;
    static bool attr_set[64] = {false};
    auto kernel = gemm_i4_wide_kernel<true, false, true>;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide::SMEM_BYTES) != cudaSuccess)
            return QB200_ERR_CUDA;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    CUtensorMap ma, mb;
    int st = make_a8_map(&ma, a8, M, K);
    if (st != QB200_OK) return st;
    st = make_packed_map(&mb, b, N, K, wide::TN);
    if (st != QB200_OK) return st;
    CUtensorMap md;
    PeerMaps<false> peers;
    make_output_maps<false>(&md, &peers, &ep, M, N);
    CUtensorMap md16;
    memset(&md16, 0, sizeof(md16));
    ep.tma_store16 = 0;
    if (ep.tma_store && encode_output_map16(&md16, ep.out, ep.ld, M, N) == QB200_OK) ep.tma_store16 = 1;
    if (const char* e = getenv("QB200_GEMM_TMA_STORE"))
        if (e[0] == '1') ep.tma_store16 = 0;  // 1: only the last tile of a CTA leaves through shared memory
    wide_columns(&ep, M, N, sms, true);
    const int tiles = ((M + wide::TM - 1) / wide::TM) * ep.col_count;
    const int grid = tiles < sms ? tiles : sms;
    if (launch_kernel(kernel, grid, wide::kThreads - 32, wide::SMEM_BYTES, stream, ma, mb, md, md16, peers, ep, M, N, K) != cudaSuccess) {
        cudaGetLastError();
        return QB200_ERR_CUDA;
    }
    return launch_status();
}

template <bool FUSED, bool PUSH>
static int launch_gemm_wide_impl(const EpilogueParams& ep_in, const void* a, const void* b, int M, int K, int N, int sms,
                                 int dev, cudaStream_t stream) {
    EpilogueParams ep = ep_in;
    // The unpack of both operands bounds this variant (about 3 cycles per operand row and K stage): a narrower tile saves
    // its share of the B rows only, so widths of 224 and 240 gain nothing (measured: +1 %), but A comes packed (half the
    // bytes of the int8 operand), so tiles of 128 ... 208 columns pay where they fill idle SMs or save a wave (K = 8192,
    // M = 2048: N = 2560 -15 %, N = 5120 -17 %, N = 14336 -12 %).  The fused variants only.  With peers the widths are
    // multiples of 64 columns: with 144-column tiles the last, overlapping 64-column piece sent 48 columns a second time
    // and no piece covered whole 128-byte lines, and the exchange of a 4-GPU step grew from 51 to 91 us.  With a single
    // peer the narrower tiles won all the same (2 GPUs, M = 2048, K = 8192, N = 14336 per rank: step 262 -> 242 us).
    wide_columns(&ep, M, N, sms, FUSED, 8, 13, PUSH && ep.n_peer > 1 ? 4 : 1);
    const bool clip = ep.col_units < wide::TN / 16;
    static bool attr_set[2][64] = {{false}};
    auto kernel = clip ? gemm_i4_wide_kernel<FUSED, PUSH, false, FUSED> : gemm_i4_wide_kernel<FUSED, PUSH, false, false>;
    if (dev < 0 || dev >= 64 || !attr_set[clip][dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wide::SMEM_BYTES) != cudaSuccess)
            return QB200_ERR_CUDA;
        if (dev >= 0 && dev < 64) attr_set[clip][dev] = true;
    }
    CUtensorMap ma, mb;
    int st = make_packed_map(&ma, a, M, K, wide::TM);
    if (st != QB200_OK) return st;
    st = make_packed_map(&mb, b, N, K, wide::TN);
    if (st != QB200_OK) return st;
    const int tiles = ((M + wide::TM - 1) / wide::TM) * ep.col_count;
    const int grid = tiles < sms ? tiles : sms;
    const int threads = PUSH ? wide::kThreads : wide::kThreads - 32 * wide::kPushWarps;
    CUtensorMap md;
    PeerMaps<PUSH> peers;
    if (FUSED) {
        make_output_maps<PUSH>(&md, &peers, &ep, M, N);
    } else {
        memset(&md, 0, sizeof(md));
        memset(&peers, 0, sizeof(peers));
    }
    if (launch_kernel(kernel, grid, threads, wide::SMEM_BYTES, stream, ma, mb, md, md, peers, ep, M, N, K) != cudaSuccess) {
        cudaGetLastError();
        return QB200_ERR_CUDA;
    }
    return launch_status();
}

template <bool FUSED>
static int launch_gemm_wide(const EpilogueParams& ep, const void* a, const void* b, int M, int K, int N, int sms, int dev,
                            cudaStream_t stream) {
    if (FUSED && ep.n_peer > 0) return launch_gemm_wide_impl<FUSED, FUSED>(ep, a, b, M, K, N, sms, dev, stream);
    return launch_gemm_wide_impl<FUSED, false>(ep, a, b, M, K, N, sms, dev, stream);
}

#include "gemv_i4.cuh"

// Tile shapes: 64, 128, 256 = gemm_i4_kernel<BN> (128-row tiles); kWideTile = gemm_i4_wide_kernel (256 x 256).
constexpr int kWideTile = 512;

static int pick_tile(int M, int N, int K, int sms, long long* est_cycles) {
    // Estimated cycles.  Per 128-K stage a CTA of the 128-row kernel needs about max(616, 3 * (128 + BN)) cycles:
    // the four MMAs take ~616 cycles whatever N is, the unpack moves 3 shared-memory wavefronts per operand row.
    // Wide tiles amortise the A rows; narrow ones fill more SMs when there are few tiles (small M).  The 256 x 256
    // kernel shares B between two accumulators (3 * 512 cycles for twice the work) but exposes one epilogue per tile.
    // QB200_GEMM_TILE = 64 | 128 | 256 | 512 in the environment forces a shape (tests and tuning).
    if (const char* e = getenv("QB200_GEMM_TILE")) {
        const int v = atoi(e);
        if (v == 64 || v == 128 || v == 256 || v == kWideTile) {
            *est_cycles = 0;  // forced: no split-K either
            return v;
        }
    }
    const long long kb = (K + BK - 1) / BK;
    int best = 256;
    long long best_t = -1;
    for (int bn : {256, 128, 64}) {
        const long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
        const long long waves = (tiles + sms - 1) / sms;
        const long long per_stage = 3 * (128 + bn) > 616 ? 3 * (128 + bn) : 616;
        const long long t = waves * kb * per_stage + 24 * bn;  // + the last tile's epilogue
        if (best_t < 0 || t < best_t) { best_t = t; best = bn; }
    }
    {
        EpilogueParams cols{};
        wide_columns(&cols, M, N, sms, true, 8, 13);  // the tile columns the 256-row kernel would use
        const long long width = 16ll * (cols.col_units + (cols.col_rem > 0 ? 1 : 0));
        const long long tiles = (long long)((M + wide::TM - 1) / wide::TM) * cols.col_count;
        const long long waves = (tiles + sms - 1) / sms;
        const long long t = waves * (kb * 3 * (wide::TM + width) + 7000 * width / wide::TN);
        // narrow balanced tiles must beat the 128-row kernel clearly: at an estimated tie they measured 5 % slower
        const bool clear = width == wide::TN || t * 21 < best_t * 20;
        if (t < best_t && clear) { best_t = t; best = kWideTile; }
    }
    *est_cycles = best_t;
    return best;
}

// static_splits < 0: the ordinary entry points (split-K scratch from the per-device buffer).  static_splits >= 0: the
// entry point that allocates nothing (scratch in the static array; 0 = the library's choice of K ranges, n = n ranges).
static int run_gemm_impl(bool fused, const EpilogueParams& ep_in, const void* a, const void* b, int M, int K, int N,
                         cudaStream_t stream, int static_splits) {
    if (M < 0 || N < 0 || K < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (M == 0 || N == 0) return QB200_OK;
    if (ep_in.out == nullptr || a == nullptr || b == nullptr) return QB200_ERR_INVALID_ARGUMENT;
    if (K == 0 || K % 32 != 0 || K >= (1 << 17)) return QB200_ERR_UNSUPPORTED;
    if (!aligned16(a) || !aligned16(b)) return QB200_ERR_INVALID_ARGUMENT;
    EpilogueParams ep = ep_in;
    const int elem = fused ? 2 : 4;
    const int vec_elems = 16 / elem;
    ep.vec_ok = aligned16(ep.out) && (ep.ld % vec_elems == 0);
    if (ep.vec_ok && (reinterpret_cast<uintptr_t>(ep.out) & 31u) == 0 && ep.ld % (2 * vec_elems) == 0) ep.vec_ok = 2;
    for (int i = 0; i < ep.n_peer; ++i) {
        if (ep.peer_out[i] == nullptr) return QB200_ERR_INVALID_ARGUMENT;
        if (!aligned16(ep.peer_out[i])) ep.vec_ok = 0;
    }
    if (ep.n_peer > 0 && (!ep.vec_ok || N % 8 != 0)) return QB200_ERR_UNSUPPORTED;  // the push path moves 16-byte pieces
    int dev = 0;
    const int sms = sm_count_of_current_device(&dev);
    if (sms <= 0) return QB200_ERR_CUDA;
    // Up to 16 rows: the CUDA-core kernel that streams the weights once (QB200_GEMM_GEMV=0 switches it off; a forced
    // tile shape or split count also means the tensor-core kernels are wanted).
    {
        const char* g = getenv("QB200_GEMM_GEMV");
        const bool forced_tc = getenv("QB200_GEMM_TILE") != nullptr || getenv("QB200_GEMM_SPLITS") != nullptr;
        if (static_splits <= 0 && !forced_tc && !(g != nullptr && g[0] == '0') && gemv_eligible(M, K, N, ep.n_peer))
            return fused ? run_gemv<true>(ep, a, b, M, K, N, sms, dev, stream)
                         : run_gemv<false>(ep, a, b, M, K, N, sms, dev, stream);
    }
    long long est = 0;
    const int bn = pick_tile(M, N, K, sms, &est);
    // Split-K (128 x 256 tiles over several K ranges) when that is estimated to be faster and its scratch is there.
    // QB200_GEMM_SPLITS = n in the environment forces n ranges (1 = never split).
    int splits = 1;
    if (ep.n_peer == 0) {
        const int smax = pick_splits(M, N, K, sms);
        if (const char* e = getenv("QB200_GEMM_SPLITS")) {
            const int v = atoi(e);
            const int num_kb = (K + BK - 1) / BK;
            splits = v < 1 ? 1 : (v > num_kb ? num_kb : (v > 64 ? 64 : v));
        } else if (smax >= 2 && est > 0) {
            // K stages of the 128 x 256 kernel at ~1152 cycles, plus the completing CTA's reduction: it reads
            // rows x splits KB through 128 threads (~40 cycles per row and range, measured), plus fixed costs.
            const long long num_kb = (K + BK - 1) / BK;
            const long long rows = M < BM ? M : BM;
            long long best = est;
            for (int sp = 2; sp <= smax; ++sp) {
                const long long t = ((num_kb + sp - 1) / sp) * 1152 + rows * sp * 40 + 24 * 256 + 3000;
                if (t < best) { best = t; splits = sp; }
            }
        }
    }
    if (static_splits > 0) {
        const int num_kb = (K + BK - 1) / BK;
        splits = static_splits > num_kb ? num_kb : static_splits;
    }
    if (splits >= 2) {
        const int tiles = ((M + BM - 1) / BM) * ((N + 255) / 256);
        const int slab_rows = M >= BM ? BM : (M + 7) / 8 * 8;
        ep.slab_ints = slab_rows * 256;
        if (static_splits == 0) {
            // The library's own choice must never be refused: use as many K ranges as the static array holds
            // (down to 1 = the kernels without scratch).  Only an explicit request (static_splits >= 2) can fail.
            while (splits >= 2 && ((size_t)tiles * splits * ep.slab_ints > kStaticScratchInts || tiles > kStaticScratchTiles))
                --splits;
        }
    }
    if (splits >= 2) {
        const int tiles = ((M + BM - 1) / BM) * ((N + 255) / 256);
        const size_t need = (size_t)tiles * splits * ep.slab_ints;
        SplitScratch ws;
        bool have;
        if (static_splits >= 0) {
            if (need > kStaticScratchInts || tiles > kStaticScratchTiles) return QB200_ERR_SCRATCH_LIMIT;
            have = get_static_scratch(dev, &ws);
            if (!have) return QB200_ERR_CUDA;
        } else {
            have = get_split_scratch(dev, stream, need, tiles, &ws);
        }
        if (have) {
            ep.splits = splits;
            ep.scratch = ws.sums;
            ep.counters = ws.counters;
            return fused ? launch_gemm<256, true, true>(ep, a, b, M, K, N, sms, dev, stream)
                         : launch_gemm<256, false, true>(ep, a, b, M, K, N, sms, dev, stream);
        }
    }
    if (bn == kWideTile)
        return fused ? launch_gemm_wide<true>(ep, a, b, M, K, N, sms, dev, stream)
                     : launch_gemm_wide<false>(ep, a, b, M, K, N, sms, dev, stream);
    if (fused) {
        if (bn == 256) return launch_gemm<256, true>(ep, a, b, M, K, N, sms, dev, stream);
        if (bn == 128) return launch_gemm<128, true>(ep, a, b, M, K, N, sms, dev, stream);
        return launch_gemm<64, true>(ep, a, b, M, K, N, sms, dev, stream);
    }
    if (bn == 256) return launch_gemm<256, false>(ep, a, b, M, K, N, sms, dev, stream);
    if (bn == 128) return launch_gemm<128, false>(ep, a, b, M, K, N, sms, dev, stream);
    return launch_gemm<64, false>(ep, a, b, M, K, N, sms, dev, stream);
}

}  // namespace qb

using namespace qb;


// ---- layer mode ---------------------------------------------------------------------------------------------------
// Between quest_b200_begin_layer and quest_b200_end_layer (host-thread state; the one-call layer entry points use the
// same two calls) the Hadamard+quantise entry point and the fused GEMM entry points launch their kernels as one layer:
// which of the two kernels carries a programmatic dependency follows what was measured (layers back to back, 20 in a
// CUDA graph):
//  * from 3 M activation elements on the quantiser is the tcgen05 kernel where it can tile K, launched behind whatever
//    kernel precedes the layer (it executes griddepcontrol.wait before its first access to global memory, so this is
//    safe behind any kernel; behind one of this library's GEMMs its blocks are scheduled as the GEMM's leave), and the
//    GEMM is launched behind it: -1 ... -2 us per layer;
//  * below that the quantiser is the small CUDA-core kernel in plain stream order and only the GEMM is dependent (its
//    set-up and first weight requests overlap the quantiser): -1.5 us per layer at M = 64 ... 512, K = 4096;
//  * a GEMM launched that way behind the CUDA-core quantiser of a large input measured slower (+1 ... +10 us at 4 M
//    elements and more), so where the tcgen05 kernel cannot tile K both launches stay plain.
// QB200_DEPENDENT_LAUNCH in the environment (tests, tuning) forces the launches instead: bit 0 = the GEMM, bit 1 = the
// quantiser is launched with a programmatic dependency; 0 = both in plain stream order.
static thread_local bool tl_layer_mode = false;

static int dependent_launch_mask() {
    const char* e = getenv("QB200_DEPENDENT_LAUNCH");
    return e == nullptr ? -1 : atoi(e);
}

static int run_gemm(bool fused, const EpilogueParams& ep, const void* a, const void* b, int M, int K, int N,
                    cudaStream_t stream, int static_splits = -1) {
    if (tl_layer_mode) {  // the kernel before this GEMM in the stream is the layer's quantiser
        const int mask = dependent_launch_mask();
        const bool small = (long long)M * K < 3ll * 1024 * 1024;
        tl_dependent_launch = mask >= 0 ? (mask & 1) != 0
                                        : (qb_tl_quantiser_kernel == kQuantiserTc || (qb_tl_quantiser_kernel == kQuantiserMma && small));
        qb_tl_quantiser_kernel = 0;  // consumed: a second GEMM of the layer follows a GEMM, not the quantiser
    }
    const int st = run_gemm_impl(fused, ep, a, b, M, K, N, stream, static_splits);
    tl_dependent_launch = false;
    return st;
}

extern "C" int matmul_int4_int4t_int32_cuda(void* mat_c, const void* mat_a, const void* mat_b, int M, int K, int N,
                                            cudaStream_t stream) {
    EpilogueParams ep{};
    ep.out = mat_c;
    ep.ld = N;
    return run_gemm(false, ep, mat_a, mat_b, M, K, N, stream);
}

extern "C" int fused_matmul_dequantize_int4_int4t_bf16_strided_cuda(void* mat_d, long long ld_d, const void* mat_a,
                                                                    const void* mat_b, const void* vec_a_add,
                                                                    const void* vec_b_add, const void* vec_a_mul,
                                                                    const void* vec_b_mul, int M, int K, int N,
                                                                    cudaStream_t stream) {
    if (M > 0 && N > 0 && (!vec_a_add || !vec_b_add || !vec_a_mul || !vec_b_mul)) return QB200_ERR_INVALID_ARGUMENT;
    if (ld_d < N) return QB200_ERR_INVALID_ARGUMENT;
    EpilogueParams ep{};
    ep.out = mat_d;
    ep.ld = ld_d;
    ep.a_add = static_cast<const int32_t*>(vec_a_add);
    ep.b_add = static_cast<const int32_t*>(vec_b_add);
    ep.a_mul = static_cast<const __nv_bfloat16*>(vec_a_mul);
    ep.b_mul = static_cast<const __nv_bfloat16*>(vec_b_mul);
    return run_gemm(true, ep, mat_a, mat_b, M, K, N, stream);
}

extern "C" int fused_matmul_dequantize_int4_int4t_bf16_push_cuda(void* const* mat_d_list, int n_dst, long long ld_d,
                                                                 const void* mat_a, const void* mat_b,
                                                                 const void* vec_a_add, const void* vec_b_add,
                                                                 const void* vec_a_mul, const void* vec_b_mul, int M, int K,
                                                                 int N, cudaStream_t stream) {
    if (mat_d_list == nullptr || n_dst < 1 || n_dst > 8) return QB200_ERR_INVALID_ARGUMENT;
    if (M > 0 && N > 0 && (!vec_a_add || !vec_b_add || !vec_a_mul || !vec_b_mul)) return QB200_ERR_INVALID_ARGUMENT;
    if (ld_d < N) return QB200_ERR_INVALID_ARGUMENT;
    EpilogueParams ep{};
    ep.out = mat_d_list[0];
    ep.n_peer = n_dst - 1;
    for (int i = 1; i < n_dst; ++i) ep.peer_out[i - 1] = mat_d_list[i];
    ep.ld = ld_d;
    ep.a_add = static_cast<const int32_t*>(vec_a_add);
    ep.b_add = static_cast<const int32_t*>(vec_b_add);
    ep.a_mul = static_cast<const __nv_bfloat16*>(vec_a_mul);
    ep.b_mul = static_cast<const __nv_bfloat16*>(vec_b_mul);
    return run_gemm(true, ep, mat_a, mat_b, M, K, N, stream);
}

extern "C" int fused_matmul_dequantize_a8_int4t_bf16_cuda(void* mat_d, const void* mat_a8, const void* mat_b,
                                                          const void* vec_a_add, const void* vec_b_add,
                                                          const void* vec_a_mul, const void* vec_b_mul, int M, int K,
                                                          int N, cudaStream_t stream) {
    if (M < 0 || N < 0 || K < 0) return QB200_ERR_INVALID_ARGUMENT;
    if (M == 0 || N == 0) return QB200_OK;
    if (!mat_d || !mat_a8 || !mat_b || !vec_a_add || !vec_b_add || !vec_a_mul || !vec_b_mul) return QB200_ERR_INVALID_ARGUMENT;
    if (K == 0 || K % 128 != 0 || K >= (1 << 17)) return QB200_ERR_UNSUPPORTED;
    if (!aligned16(mat_a8) || !aligned16(mat_b)) return QB200_ERR_INVALID_ARGUMENT;
    EpilogueParams ep{};
    ep.out = mat_d;
    ep.ld = N;
    ep.a_add = static_cast<const int32_t*>(vec_a_add);
    ep.b_add = static_cast<const int32_t*>(vec_b_add);
    ep.a_mul = static_cast<const __nv_bfloat16*>(vec_a_mul);
    ep.b_mul = static_cast<const __nv_bfloat16*>(vec_b_mul);
    ep.vec_ok = aligned16(mat_d) && (N % 8 == 0);
    if (ep.vec_ok && (reinterpret_cast<uintptr_t>(mat_d) & 31u) == 0 && N % 16 == 0) ep.vec_ok = 2;
    int dev = 0;
    const int sms = sm_count_of_current_device(&dev);
    if (sms <= 0) return QB200_ERR_CUDA;
    if (tl_layer_mode) {  // behind the layer's tcgen05 quantiser: dependent unless the environment says otherwise
        const int mask = dependent_launch_mask();
        tl_dependent_launch = mask < 0 || (mask & 1) != 0;
        qb_tl_quantiser_kernel = 0;
    }
    const int st = launch_gemm_wide_a8(ep, mat_a8, mat_b, M, K, N, sms, dev, stream);
    tl_dependent_launch = false;
    return st;
}

constexpr bool kA8ByDefault = true;  // measured faster wherever the 256 x 256 kernel and the tcgen05 quantiser both apply (QB200_A8=0 switches it off)

// 1 if, for this layer shape, the int8-operand route (hadamard_quantize_a8_cuda_bf16 + the GEMM above) is the faster one:
// the 256 x 256 kernel would be chosen anyway and the quantiser's tcgen05 kernel can tile K.
extern "C" int quest_b200_prefers_a8(int M, int K, int N) {
    if (M <= 0 || K <= 0 || N <= 0 || K % 128 != 0 || K >= (1 << 17)) return 0;
    if (getenv("QB200_GEMM_TILE") != nullptr || getenv("QB200_GEMM_SPLITS") != nullptr) return 0;
    if (const char* e = getenv("QB200_A8")) return e[0] != '0';
    if (!kA8ByDefault) return 0;
    int dev = 0;
    const int sms = sm_count_of_current_device(&dev);
    long long est = 0;
    if (sms <= 0 || pick_tile(M, N, K, sms, &est) != kWideTile) return 0;
    // The int8 operand is twice the packed one.  Up to 32 MB (M = 8192, K = 4096) the route measured 1-5 % faster, at
    // 64 MB the same, beyond that slower (M = 65536, K = 4096: 889 against 791 us): the operand no longer stays in L2
    // between the CTAs that share its rows.
    if ((long long)M * K > (48ll << 20)) return 0;
    return hq_tc_shape_ok(K) ? 1 : 0;
}

extern "C" int fused_matmul_dequantize_int4_int4t_bf16_noalloc_cuda(void* mat_d, const void* mat_a, const void* mat_b,
                                                                    const void* vec_a_add, const void* vec_b_add,
                                                                    const void* vec_a_mul, const void* vec_b_mul, int M,
                                                                    int K, int N, int splits, cudaStream_t stream) {
    if (M > 0 && N > 0 && (!vec_a_add || !vec_b_add || !vec_a_mul || !vec_b_mul)) return QB200_ERR_INVALID_ARGUMENT;
    if (splits < 0) return QB200_ERR_INVALID_ARGUMENT;
    EpilogueParams ep{};
    ep.out = mat_d;
    ep.ld = N;
    ep.a_add = static_cast<const int32_t*>(vec_a_add);
    ep.b_add = static_cast<const int32_t*>(vec_b_add);
    ep.a_mul = static_cast<const __nv_bfloat16*>(vec_a_mul);
    ep.b_mul = static_cast<const __nv_bfloat16*>(vec_b_mul);
    return run_gemm(true, ep, mat_a, mat_b, M, K, N, stream, splits);
}

extern "C" int fused_matmul_dequantize_int4_int4t_bf16_cuda(void* mat_d, const void* mat_a, const void* mat_b,
                                                            const void* vec_a_add, const void* vec_b_add,
                                                            const void* vec_a_mul, const void* vec_b_mul, int M, int K,
                                                            int N, cudaStream_t stream) {
    return fused_matmul_dequantize_int4_int4t_bf16_strided_cuda(mat_d, (long long)N, mat_a, mat_b, vec_a_add, vec_b_add,
                                                                vec_a_mul, vec_b_mul, M, K, N, stream);
}

extern "C" int hadamard_quantize_int4_cuda_bf16(void*, void*, void*, const void*, int, int, int, cudaStream_t);

extern "C" int quest_b200_begin_layer(void) {
    const int mask = dependent_launch_mask();
    tl_layer_mode = true;
    qb_tl_dependent_quantiser = mask < 0 || (mask & 2) != 0;
    qb_tl_quantiser_kernel = 0;
    return QB200_OK;
}

extern "C" int quest_b200_end_layer(void) {
    tl_layer_mode = false;
    qb_tl_dependent_quantiser = false;
    qb_tl_quantiser_kernel = 0;
    tl_dependent_launch = false;
    return QB200_OK;
}

extern "C" int w4a4_linear_hadamard_bf16_cuda(void* mat_d, const void* x, const void* w_int_packed, const void* w_add,
                                              const void* w_scale, void* a_int_packed, void* a_scale, void* a_int_row_sum,
                                              int M, int K, int N, int block, cudaStream_t stream) {
    if (!a_int_row_sum) return QB200_ERR_INVALID_ARGUMENT;
    quest_b200_begin_layer();
    int st = hadamard_quantize_int4_cuda_bf16(a_int_packed, a_scale, a_int_row_sum, x, K, M, block, stream);
    if (st == QB200_OK)
        st = fused_matmul_dequantize_int4_int4t_bf16_cuda(mat_d, a_int_packed, w_int_packed, a_int_row_sum, w_add, a_scale,
                                                          w_scale, M, K, N, stream);
    quest_b200_end_layer();
    return st;
}

extern "C" int hadamard_quantize_a8_cuda_bf16(void*, void*, void*, const void*, int, int, int, cudaStream_t);

extern "C" int w4a4_linear_hadamard_a8_bf16_cuda(void* mat_d, const void* x, const void* w_int_packed, const void* w_add,
                                                 const void* w_scale, void* a_int8, void* a_scale, void* a_int_row_sum,
                                                 int M, int K, int N, int block, cudaStream_t stream) {
    if (!a_int_row_sum) return QB200_ERR_INVALID_ARGUMENT;
    quest_b200_begin_layer();  // the quantiser of this route is always the tcgen05 kernel: both launches dependent
    int st = hadamard_quantize_a8_cuda_bf16(a_int8, a_scale, a_int_row_sum, x, K, M, block, stream);
    if (st == QB200_OK)
        st = fused_matmul_dequantize_a8_int4t_bf16_cuda(mat_d, a_int8, w_int_packed, a_int_row_sum, w_add, a_scale, w_scale,
                                                        M, K, N, stream);
    quest_b200_end_layer();
    return st;
}

extern "C" int quest_b200_test_bounded_wait_cuda(void* mat_d, const void* mat_a, const void* mat_b, const void* vec_a_add,
                                                 const void* vec_b_add, const void* vec_a_mul, const void* vec_b_mul, int M,
                                                 int K, int N, long long wait_limit_cycles, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || !vec_a_add || !vec_b_add || !vec_a_mul || !vec_b_mul) return QB200_ERR_INVALID_ARGUMENT;
    if (wait_limit_cycles < kWaitLimitFloor || wait_limit_cycles > kWaitLimitCycles) return QB200_ERR_INVALID_ARGUMENT;
    if (cudaDeviceSynchronize() != cudaSuccess) return QB200_ERR_CUDA;
    int st = set_wait_limit_cycles(wait_limit_cycles);
    if (st != QB200_OK) return st;
    EpilogueParams ep{};
    ep.out = mat_d;
    ep.ld = N;
    ep.a_add = static_cast<const int32_t*>(vec_a_add);
    ep.b_add = static_cast<const int32_t*>(vec_b_add);
    ep.a_mul = static_cast<const __nv_bfloat16*>(vec_a_mul);
    ep.b_mul = static_cast<const __nv_bfloat16*>(vec_b_mul);
    ep.test_skip_producer = 1;
    st = run_gemm(true, ep, mat_a, mat_b, M, K, N, stream, /*static_splits=*/1);  // tensor-core kernels, no split-K, no dp4a kernel
    const bool synced = cudaStreamSynchronize(stream) == cudaSuccess;
    const int st2 = set_wait_limit_cycles(kWaitLimitCycles);
    if (st != QB200_OK) return st;
    return synced ? st2 : QB200_ERR_CUDA;
}

extern "C" int quest_b200_device_status(int* status) {
    if (status == nullptr) return QB200_ERR_INVALID_ARGUMENT;
    if (cudaDeviceSynchronize() != cudaSuccess) return QB200_ERR_CUDA;
    int v = 0, v2 = 0;
    int st = fetch_and_clear_device_status(&v);
    if (st != QB200_OK) return st;
    st = hq_tc_fetch_and_clear_device_status(&v2);  // the tensor-core quantiser keeps its own status word
    if (st != QB200_OK) return st;
    if (v != 0) reset_split_counters();  // a GEMM that gave up may have left split-K tile counters half way
    *status = v != 0 ? v : v2;
    return QB200_OK;
}

extern "C" const char* quest_b200_error_string(int status) {
    switch (status & 0xFF) {
        case QB200_OK: return "ok";
        case QB200_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, negative size or misaligned buffer)";
        case QB200_ERR_UNSUPPORTED: return "shape not supported by the sm_100a kernels";
        case QB200_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
        case QB200_ERR_DRIVER: return "cuTensorMapEncodeTiled unavailable or failed";
        case QB200_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel timed out";
        case QB200_ERR_SCRATCH_LIMIT:
            return "split-K scratch would exceed the 8 MiB static buffer (tiles x splits x rows per tile must be <= 8192)";
        default: return "unknown status";
    }
}

extern "C" int quest_b200_version(void) { return 100; }

#ifdef QB200_TRACE
extern "C" int quest_b200_trace(unsigned long long* out, int n_ctas) {
    if (cudaDeviceSynchronize() != cudaSuccess) return QB200_ERR_CUDA;
    return cuda_status(cudaMemcpyFromSymbol(out, g_trace, sizeof(unsigned long long) * 4 * (n_ctas < 256 ? n_ctas : 256)));
}
#endif
