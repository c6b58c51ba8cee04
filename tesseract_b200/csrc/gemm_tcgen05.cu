// bfloat16 matrix product on the fifth-generation tensor cores: C[M,N] = A[M,K] . W[N,K]^T, 32-bit accumulation.
//
// The Blackwell-native path for prompt-sized batches.  A persistent CTA per SM computes 128 x 256 tiles of C, two
// accumulators in tensor memory so that one tile's epilogue runs under the next tile's products:
//   * warp 0, one elected lane: TMA producer.  Tiles of A (128 x 64) and W (256 x 64) are brought into a
//     four-stage ring in shared memory by cp.async.bulk.tensor with the 128-byte swizzle; completion is
//     signalled on an mbarrier per stage (no multicast: every CTA issues its own loads).
//   * warp 1, one elected lane: issues tcgen05.mma (M128 x N256 x K16, operands from shared memory through
//     64-bit matrix descriptors, accumulator in tensor memory) and hands each stage back with tcgen05.commit.
//   * warps 4..7: epilogue.  Each warp reads its 32 lanes of the accumulator with tcgen05.ld, 32 columns at
//     a time, and stores bfloat16 (or 32-bit) rows, or applies SwiGLU to a weight whose rows interleave eight
//     gate rows and their eight up rows: out[m, j] = round(silu(gate_j) * up_j) on the unrounded accumulators
//     (the reference multiplies rounded projections, src/cuda/kernels.rs:191-208; here one rounding fewer).
// Products of more than 128 rows take the pair form further down: two CTAs of a cluster on one 256 x 256 tile
// (tcgen05.mma.cta_group::2), each bringing half of the operands.
// Rows of A beyond M, rows of W beyond N and columns beyond K are zero-filled by the TMA unit and never stored.
// Every wait on an mbarrier is bounded: a wait that runs out sets *error, tells the other roles to stop, and the
// CTA still frees its tensor memory before it returns.
#include "umma.cuh"

namespace {

using namespace tbtma;
using namespace tbumma;

constexpr int BM = 128, BK = 64;
// Tiles of 128 x 256 with a four-stage ring; products of at most 128 rows (one row of tiles) take 128 x 128 tiles
// with six stages instead, so that twice as many SMs stream the weights.
template <int BN>
constexpr int kStages = BN == 256 ? 4 : 6;
constexpr int kThreads = 256;
constexpr uint32_t kATileBytes = BM * BK * 2;   // 16 KiB
template <int BN>
constexpr uint32_t kStageBytes = kATileBytes + BN * BK * 2;
template <int BN>
constexpr uint32_t kTmemColumns = 2 * BN;   // two accumulators of BN columns

enum Epilogue : int { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_F32 = 2 };

// smem_u32, the mbarrier helpers (every wait bounded) and the tensor-map encoder come from tma.cuh; descriptors,
// products, commits and tensor-memory loads from umma.cuh

struct GemmParams {
    void* out;
    int64_t out_stride;
    int M, N, K;
    int* error;
};

// One 32-column chunk of an accumulator row: to memory as the epilogue asks.
template <int EPI>
__device__ __forceinline__ void store_chunk(const GemmParams& p, int row, int col0, const uint32_t (&acc)[32]) {
    if (row >= p.M || col0 >= p.N) return;
    if (EPI == EPI_F32) {
        float* dst = reinterpret_cast<float*>(p.out) + (int64_t)row * p.out_stride + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            if (col0 + j < p.N)
                *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]),
                                                                  __uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3]));
    } else if (EPI == EPI_BF16) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.out_stride + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            if (col0 + j >= p.N) break;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(acc[j + e]);
            Packet<__nv_bfloat16>::store(dst + j, v);
        }
    } else {
        // columns come in blocks of sixteen: eight gates, then their eight up projections
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)row * p.out_stride + col0 / 2;
#pragma unroll
        for (int j = 0; j < 32; j += 16) {
            if (col0 + j >= p.N) break;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float gate = __uint_as_float(acc[j + e]), up = __uint_as_float(acc[j + 8 + e]);
                v[e] = gate * __fdividef(1.0f, 1.0f + __expf(-gate)) * up;   // 32-bit, fast reciprocal and exponential
            }
            Packet<__nv_bfloat16>::store(dst + j / 2, v);
        }
    }
}

// Persistent: a CTA per SM walks over the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (tiles that are
// neighbours in time share a panel of W and the rows of A, which then come from L2).  Two accumulators of 256
// columns in tensor memory: while the epilogue warps drain one tile, the products of the next fill the other.
template <int EPI, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    constexpr int STAGES = kStages<BN>;
    constexpr uint32_t kStageBytes = ::kStageBytes<BN>;
    constexpr uint32_t kTmemColumns = ::kTmemColumns<BN>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (p.K + BK - 1) / BK;
    const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]), acc_empty0 = acc_full0 + 16;
    const uint32_t tiles = smem_u32(smem);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);      // one arrival per epilogue warp
        }
        mbar_fence_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    // barriers and tensor memory were set up while the kernel before this one drained; its results (the rows of
    // A) are read from here on
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        int s = 0;
        uint32_t parity = 1;                                     // fresh barriers pass a wait for parity 1
        for (int t = blockIdx.x; t < total_tiles && !abort_flag; t += gridDim.x) {
            const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(empty0 + 8 * s, parity, &abort_flag)) {
                    abort_flag = 1;
                    atomicExch(p.error, 1);
                    break;
                }
                mbar_expect_tx(full0 + 8 * s, kStageBytes);
                const uint32_t a_dst = tiles + s * kStageBytes;
                tma_load_2d(a_dst, &map_a, full0 + 8 * s, kb * BK, m0);
                tma_load_2d(a_dst + kATileBytes, &map_b, full0 + 8 * s, kb * BK, n0);
                if (++s == STAGES) {
                    s = 0;
                    parity ^= 1;
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
        // the descriptors of stage 0; those of the other stages and K steps are sums (see umma_desc_advance)
        const uint64_t desc_a0 = umma_desc_k_sw128(tiles), desc_b0 = umma_desc_k_sw128(tiles + kATileBytes);
        int s = 0, i = 0;
        uint32_t parity = 0;                                      // of the wait for a stage: flips with every turn of the ring
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++i) {
            const int buf = i & 1;
            // the epilogue must have drained this accumulator's previous tile
            if (!mbar_wait(acc_empty0 + 8 * buf, ((i >> 1) & 1) ^ 1, &abort_flag)) {
                abort_flag = 1;
                atomicExch(p.error, 4);
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + buf * BN;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(full0 + 8 * s, parity, &abort_flag)) {
                    abort_flag = 1;
                    atomicExch(p.error, 2);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t desc_a = umma_desc_advance(desc_a0, s * kStageBytes);
                const uint64_t desc_b = umma_desc_advance(desc_b0, s * kStageBytes);
                // inside the 128-byte swizzle atom a step of 16 elements along K is 32 bytes of start address
                umma_bf16(acc, desc_a, desc_b, idesc, kb != 0);
#pragma unroll
                for (int kk = 1; kk < BK / 16; ++kk)
                    umma_bf16_add(acc, umma_desc_advance(desc_a, kk * 32), umma_desc_advance(desc_b, kk * 32), idesc);
                umma_commit(empty0 + 8 * s);          // the stage is free once these products have read it
                if (++s == STAGES) {
                    s = 0;
                    parity ^= 1;
                }
            }
            if (ok) umma_commit(acc_full0 + 8 * buf); // the accumulator is complete once all products are done
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;             // a warp may touch tensor-memory lanes 32*(warp % 4) .. +31
        int i = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++i) {
            const int buf = i & 1;
            const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            if (!mbar_wait(acc_full0 + 8 * buf, (i >> 1) & 1, &abort_flag)) {
                abort_flag = 1;
                atomicExch(p.error, 3);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lanes = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c += 2) {
                uint32_t acc0[32], acc1[32];      // two chunks in flight: the second loads while the first is stored
                tmem_load_32(lanes + c * 32, acc0);
                tmem_load_32(lanes + c * 32 + 32, acc1);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                store_chunk<EPI>(p, row, n0 + c * 32, acc0);
                store_chunk<EPI>(p, row, n0 + c * 32 + 32, acc1);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The pair form for products of more than 128 rows: two CTAs on neighbouring SMs (a cluster of two) compute one
// tile of 256 rows with tcgen05.mma.cta_group::2.  Each CTA brings its own 128 rows of A and its own half of the
// tile's rows of W (at a tile width of 256, 32 KiB a stage instead of 48: a third less traffic from L2 per product,
// which is what bounds the single-CTA form at this size) and holds its 128 rows of the accumulators in its own
// tensor memory; one thread of the even CTA issues the products for both and its commits arrive in both CTAs.
//   full[s]       in the even CTA only: its producer announces both CTAs' bytes, both CTAs' copies count on it
//   empty[s]      in each CTA (commit to both): that CTA's producer may refill the stage
//   acc_full[b]   in each CTA (commit to both): that CTA's epilogue warps may read accumulator b
//   acc_empty[b]  in the even CTA only: eight arrivals, one per epilogue warp of either CTA
// No CTA leaves before both are done (the even CTA's products read the odd CTA's shared memory, the odd CTA's
// warps arrive on the even CTA's barriers).
// Two tile widths.  256: one product per K step, two accumulators that take turns (a tile's epilogue under the
// next tile's products).  448: two products of 224 columns into ONE accumulator, the W rows of a CTA in two blocks
// (the hardware gives the first half of each product's columns to the even CTA); it is the choice where its
// tiles fill the 74 pairs in fewer rounds (512 x 16,384: one round of 74 tiles instead of two of 128).  (The width
// as a kernel argument, tried from 96 to 512 in steps of 32, cost the issuing thread 3-5 % at every width and won
// nowhere else.)
constexpr int kPairMaxStages = 6;
constexpr uint32_t kPairSmemBudget = 196 * 1024;
constexpr uint32_t kPairTmemColumns = 512;

template <int BN>
struct PairShape {
    static constexpr int n_product = BN > 256 ? BN / 2 : BN;        // columns of one product
    static constexpr int products = BN / n_product;                  // per K step
    static constexpr int accumulators = BN > 256 ? 1 : 2;
    static constexpr uint32_t stage_bytes = kATileBytes + (BN / 2) * 128;   // this CTA's A rows and W rows
    static constexpr int stages = (int)(kPairSmemBudget / stage_bytes) < kPairMaxStages
                                      ? (int)(kPairSmemBudget / stage_bytes) : kPairMaxStages;
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 512, "tile width");
};

template <int EPI, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p) {
    constexpr int PM = 256;
    using Shape = PairShape<BN>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // every CTA's dynamic shared memory starts at the same offset, so the rounded-up tiles do too in both CTAs
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bars[2 * kPairMaxStages + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();                     // 0: issues the products; 1: its partner
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    constexpr int STAGES = Shape::stages, NP = Shape::n_product, products = Shape::products;
    constexpr uint32_t stage_bytes = Shape::stage_bytes;
    const int k_blocks = (p.K + BK - 1) / BK;
    const int m_tiles = (p.M + PM - 1) / PM, n_tiles = (p.N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kPairMaxStages]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * kPairMaxStages]), acc_empty0 = acc_full0 + 16;
    const uint32_t tiles = smem_u32(smem);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 8);      // one arrival per epilogue warp of both CTAs
        }
        mbar_fence_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) tmem_pair_alloc(smem_u32(&tmem_base_slot), kPairTmemColumns);
    tc_fence_before();
    __syncthreads();
    cluster_barrier_all();                          // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer (one in each CTA)
        const uint32_t full_in_even = cluster_shared_address(full0, 0);
        constexpr int half = NP / 2;                              // W rows of one product in this CTA
        int s = 0;
        uint32_t parity = 1;
        for (int t = pair; t < total_tiles && !abort_flag; t += pairs) {
            const int m0 = (t % m_tiles) * PM + (int)rank * BM, n0 = (t / m_tiles) * BN + (int)rank * half;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(empty0 + 8 * s, parity, &abort_flag)) {
                    abort_flag = 1;
                    atomicExch(p.error, 11);
                    break;
                }
                if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * stage_bytes);
                const uint32_t a_dst = tiles + s * stage_bytes;
                tma_load_2d_pair(a_dst, &map_a, full_in_even + 8 * s, kb * BK, m0);
#pragma unroll
                for (int q = 0; q < products; ++q)
                    tma_load_2d_pair(a_dst + kATileBytes + q * half * 128, &map_b, full_in_even + 8 * s, kb * BK,
                                     n0 + q * NP);
                if (++s == STAGES) {
                    s = 0;
                    parity ^= 1;
                }
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------------------------------------------------------- MMA issuer (the even CTA's, for both)
        constexpr uint32_t idesc = umma_idesc_bf16(PM, NP);
        const uint64_t desc_a0 = umma_desc_k_sw128(tiles), desc_b0 = umma_desc_k_sw128(tiles + kATileBytes);
        constexpr uint32_t second = (uint32_t)(NP / 2) * 128;     // the second product's W rows in a stage
        constexpr int bufs = Shape::accumulators;
        int s = 0, i = 0;
        uint32_t parity = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles && ok; t += pairs, ++i) {
            const int buf = bufs == 2 ? (i & 1) : 0;
            const uint32_t turn = bufs == 2 ? (uint32_t)(i >> 1) : (uint32_t)i;
            if (!mbar_wait(acc_empty0 + 8 * buf, (turn & 1) ^ 1, &abort_flag)) {
                abort_flag = 1;
                atomicExch(p.error, 14);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * 256;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(full0 + 8 * s, parity, &abort_flag)) {
                    abort_flag = 1;
                    atomicExch(p.error, 12);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint64_t desc_a = umma_desc_advance(desc_a0, s * stage_bytes);
                const uint64_t desc_b = umma_desc_advance(desc_b0, s * stage_bytes);
                if (products == 1) {
                    umma_pair_bf16(acc, desc_a, desc_b, idesc, kb != 0);
#pragma unroll
                    for (int kk = 1; kk < BK / 16; ++kk)
                        umma_pair_bf16_add(acc, umma_desc_advance(desc_a, kk * 32), umma_desc_advance(desc_b, kk * 32), idesc);
                } else {
                    const uint64_t desc_b2 = umma_desc_advance(desc_b, second);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        umma_pair_bf16(acc, umma_desc_advance(desc_a, kk * 32), umma_desc_advance(desc_b, kk * 32), idesc,
                                       (kb | kk) != 0);
                        umma_pair_bf16(acc + NP, umma_desc_advance(desc_a, kk * 32), umma_desc_advance(desc_b2, kk * 32),
                                       idesc, (kb | kk) != 0);
                    }
                }
                umma_pair_commit(empty0 + 8 * s, 3);      // both CTAs' stage s is free once these products have read it
                if (++s == STAGES) {
                    s = 0;
                    parity ^= 1;
                }
            }
            if (ok) umma_pair_commit(acc_full0 + 8 * buf, 3);
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- epilogue (this CTA's 128 rows)
        const int quarter = warp & 3;
        const uint32_t acc_empty_in_even = cluster_shared_address(acc_empty0, 0);
        constexpr int bufs = Shape::accumulators;
        int i = 0;
        for (int t = pair; t < total_tiles; t += pairs, ++i) {
            const int buf = bufs == 2 ? (i & 1) : 0;
            const uint32_t turn = bufs == 2 ? (uint32_t)(i >> 1) : (uint32_t)i;
            const int m0 = (t % m_tiles) * PM + (int)rank * BM, n0 = (t / m_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            if (!mbar_wait(acc_full0 + 8 * buf, turn & 1, &abort_flag)) {
                abort_flag = 1;
                atomicExch(p.error, 13);
                break;
            }
            tc_fence_after();
            const uint32_t lanes = tmem_base + buf * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c += 2) {
                uint32_t acc0[32], acc1[32];
                tmem_load_32(lanes + c * 32, acc0);
                if (c + 1 < BN / 32) tmem_load_32(lanes + c * 32 + 32, acc1);
                tmem_wait_ld();
                store_chunk<EPI>(p, row, n0 + c * 32, acc0);
                if (c + 1 < BN / 32) store_chunk<EPI>(p, row, n0 + c * 32 + 32, acc1);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_in_even + 8 * buf);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_barrier_all();                          // both CTAs are done with each other's memory and barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_pair_dealloc(tmem_base, kPairTmemColumns);
    }
}

// The tile width for an M x N product on `pairs` CTA pairs: the one whose rounds cost less, a round costing its
// width plus a share for what is not overlapped (a tile's first loads and, with one accumulator, its epilogue).
inline int pair_tile_width(int M, int N, int pairs) {
    const int m_tiles = (M + 255) / 256;
    const int rounds_256 = (m_tiles * ((N + 255) / 256) + pairs - 1) / pairs;
    const int rounds_448 = (m_tiles * ((N + 447) / 448) + pairs - 1) / pairs;
    return rounds_448 * (448 + 48) < rounds_256 * (256 + 16) ? 448 : 256;
}

}  // namespace

// 1 if the kernel takes these sizes.  K and the row strides must be multiples of 8 (16-byte TMA strides), N of 8
// (16 for the SwiGLU epilogue).
TB_EXPORT int tb_gemm_tcgen05_supported(int M, int N, int K, int epilogue) {
    if (M < 1 || N < 8 || K < 8 || K % 8 != 0 || N % 8 != 0) return 0;
    if (epilogue == EPI_SWIGLU && N % 16 != 0) return 0;
    return 1;
}

// error: device int, set non-zero if a bounded wait ran out (the result is then unusable).
TB_EXPORT int tb_gemm_tcgen05(const void* a, int64_t a_stride, const void* w, int64_t w_stride, void* out,
                              int64_t out_stride, int M, int N, int K, int epilogue, int* error,
                              cudaStream_t stream) {
    if (!tb_gemm_tcgen05_supported(M, N, K, epilogue)) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)out) % 16 != 0 || a_stride % 8 != 0 || w_stride % 8 != 0 ||
        out_stride % 8 != 0)
        return TB_ERR_BAD_ALIGN;
    // one row of tiles: narrower tiles, so that twice as many SMs stream the weights
    const int bn = M <= BM ? 128 : 256;
    CUtensorMap map_a, map_b;
    if (int status = make_map_2d(&map_a, a, (uint64_t)M, (uint64_t)K, (uint64_t)a_stride, BM)) return status;
    if (int status = make_map_2d(&map_b, w, (uint64_t)N, (uint64_t)K, (uint64_t)w_stride, bn)) return status;
    GemmParams p;
    p.out = out;
    p.out_stride = out_stride;
    p.M = M;
    p.N = N;
    p.K = K;
    p.error = error;
    const int total_tiles = ((N + bn - 1) / bn) * ((M + BM - 1) / BM);
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 1;
    }
    dim3 grid(total_tiles < sms ? total_tiles : sms);
#define TB_LAUNCH_BN(E, W)                                                                                    \
    {                                                                                                         \
        const size_t smem = (size_t)kStages<W> * kStageBytes<W> + 1024;                                       \
        cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<E, W>,                                     \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        if (err != cudaSuccess) return (int)err;                                                              \
        err = tb_launch_pdl(gemm_tcgen05_kernel<E, W>, grid, dim3(kThreads), smem, stream, map_a, map_b, p);  \
        if (err != cudaSuccess) return (int)err;                                                              \
    }
#define TB_LAUNCH(E)                                                                                          \
    {                                                                                                         \
        if (bn == 128) TB_LAUNCH_BN(E, 128) else TB_LAUNCH_BN(E, 256)                                         \
    }
    if (epilogue == EPI_BF16) TB_LAUNCH(EPI_BF16)
    else if (epilogue == EPI_SWIGLU) TB_LAUNCH(EPI_SWIGLU)
    else if (epilogue == EPI_F32) TB_LAUNCH(EPI_F32)
    else return TB_ERR_BAD_SIZE;
#undef TB_LAUNCH
#undef TB_LAUNCH_BN
    return tb_launch_status();
}

// The pair form (see gemm_pair_tcgen05_kernel): the same contract, for M > 128.  n_tile: the tile's width (256 or
// 448), or 0 for the width that pair_tile_width picks.
TB_EXPORT int tb_gemm_pair_tcgen05_width(int M, int N) {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 1) sms = 2;
    }
    return pair_tile_width(M, N, sms / 2);
}

TB_EXPORT int tb_gemm_pair_tcgen05(const void* a, int64_t a_stride, const void* w, int64_t w_stride, void* out,
                                   int64_t out_stride, int M, int N, int K, int epilogue, int n_tile, int* error,
                                   cudaStream_t stream) {
    if (!tb_gemm_tcgen05_supported(M, N, K, epilogue)) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)out) % 16 != 0 || a_stride % 8 != 0 || w_stride % 8 != 0 ||
        out_stride % 8 != 0)
        return TB_ERR_BAD_ALIGN;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 1) sms = 2;
    }
    if (n_tile == 0) n_tile = pair_tile_width(M, N, sms / 2);
    if (n_tile != 256 && n_tile != 448) return TB_ERR_BAD_SIZE;
    const int w_rows = n_tile == 256 ? PairShape<256>::n_product / 2 : PairShape<448>::n_product / 2;
    CUtensorMap map_a, map_b;
    if (int status = make_map_2d(&map_a, a, (uint64_t)M, (uint64_t)K, (uint64_t)a_stride, BM)) return status;
    if (int status = make_map_2d(&map_b, w, (uint64_t)N, (uint64_t)K, (uint64_t)w_stride, w_rows)) return status;
    GemmParams p;
    p.out = out;
    p.out_stride = out_stride;
    p.M = M;
    p.N = N;
    p.K = K;
    p.error = error;
    const int total_tiles = ((N + n_tile - 1) / n_tile) * ((M + 255) / 256);
    const int pairs = total_tiles < sms / 2 ? total_tiles : sms / 2;
    dim3 grid(2 * pairs);
#define TB_LAUNCH_PAIR_W(E, W)                                                                                \
    {                                                                                                         \
        const size_t smem = (size_t)PairShape<W>::stages * PairShape<W>::stage_bytes + 1024;                  \
        static bool allowed = false;                                                                          \
        if (!allowed) {                                                                                       \
            cudaError_t err = cudaFuncSetAttribute(gemm_pair_tcgen05_kernel<E, W>,                            \
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
            if (err != cudaSuccess) return (int)err;                                                          \
            allowed = true;                                                                                   \
        }                                                                                                     \
        cudaError_t err = tb_launch_pdl(gemm_pair_tcgen05_kernel<E, W>, grid, dim3(kThreads), smem, stream,   \
                                        map_a, map_b, p);                                                     \
        if (err != cudaSuccess) return (int)err;                                                              \
    }
#define TB_LAUNCH_PAIR(E)                                                                                     \
    {                                                                                                         \
        if (n_tile == 256) TB_LAUNCH_PAIR_W(E, 256) else TB_LAUNCH_PAIR_W(E, 448)                             \
    }
    if (epilogue == EPI_BF16) TB_LAUNCH_PAIR(EPI_BF16)
    else if (epilogue == EPI_SWIGLU) TB_LAUNCH_PAIR(EPI_SWIGLU)
    else if (epilogue == EPI_F32) TB_LAUNCH_PAIR(EPI_F32)
    else return TB_ERR_BAD_SIZE;
#undef TB_LAUNCH_PAIR
#undef TB_LAUNCH_PAIR_W
    return tb_launch_status();
}
