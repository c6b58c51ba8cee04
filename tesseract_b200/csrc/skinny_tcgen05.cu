// Matrix products over a few dozen rows (17 to 128: decode steps of many sequences, short prompt portions) on the
// fifth-generation tensor cores, bfloat16 weights streamed once from HBM:
//
//   y[M, N] = X[M, K] . W[N, K]^T          with M <= 128, 32-bit accumulation
//
// The operands are swapped against the usual GEMM: 128 rows of W (output features) are the 128-row operand of
// tcgen05.mma, the M batch rows (rounded up to a multiple of 16) its narrow one, so that the tensor cores see
// full-height tiles however few rows there are; the accumulator [128 features x M rows] sits in tensor memory
// with one feature per lane.  What bounds such a product is the one thread that issues it: a product of
// 128 x 64 x 16 takes 46 cycles, a commit as much, and a wait on an mbarrier that is already complete 200; so a
// stage of the ring is two K blocks of 64 (eight products per wait), descriptors are built once and moved by
// additions, and a CTA then takes weights in at about 50 bytes a cycle.  Per CTA:
//   * warp 0, one lane: sets up the barriers and is the TMA producer.  A stage holds two tiles of W (128 x 64) and
//     two of X (M x 64), 128-byte swizzle, one mbarrier, no multicast.  The weights of the first stages do not
//     depend on the kernel in front: they are asked for before anything else, ahead even of the tensor-memory
//     allocation and of the dependency wait of the programmatic launch.
//   * warp 1, one lane: issues tcgen05.mma (M128 x N(rows) x K16), hands stages back with tcgen05.commit.
//   * warps 2..9: epilogue.  They copy the accumulator to shared memory as [row][feature] (two warps share a
//     quarter of the tensor-memory lanes and take every other chunk of columns); then a warp takes a batch row
//     at a time, a lane four neighbouring features of it, so that what goes to memory is contiguous.
// A product with fewer feature tiles than SMs is also split along K, the splits of a tile being one thread-block
// cluster: as many splits (up to 8) as let all clusters run at once (a cluster lies inside one GPC, so fewer fit
// than SMs / splits: 15 of 8 and 22 of 6 on a B200).  After a cluster barrier split r takes the batch rows r,
// r + S, ... and adds the splits' partial sums in ascending order of the splits, whichever finished first, through
// distributed shared memory (all of a row pair's loads are in flight at once: a load from a peer's shared memory
// takes about a microsecond).  A CTA with several tiles (the head) alternates between two accumulators, so that
// one tile's epilogue runs under the next tile's products.
//
// Epilogues: bfloat16 or 32-bit store; SwiGLU (src/cuda/kernels.rs:191-208) for a weight whose rows interleave
// eight gate rows and their eight up rows; and EPI_ADD_NORM, the work of the addition and RMSNorm that FOLLOW the
// product (src/cuda/kernels.rs:59-103): with o = round(y), c = res + o in 32 bits, it stores res_out = round(c),
// xw = round(c * w) and per tile of 128 features and batch row the sum of c^2.  SCALED is the other half: X is
// such an xw, and y = s * sum_k xw_k W_k with s = rsqrt(sum of the tiles' sums / K + eps): the same single
// rounding of the operand and the same 32-bit statistics as the norm in front would have, the per-row scale
// applied to the 32-bit sums.
// Every wait on an mbarrier is bounded: a wait that runs out sets *error and tells the other roles to stop; the
// CTA still meets its cluster barriers and frees its tensor memory.
#include "umma.cuh"

#include <atomic>

namespace {

using namespace tbtma;
using namespace tbumma;

constexpr int BF = 128;                 // output features per tile: the 128-row operand
constexpr int BK = 64;                  // K elements of one TMA box (128 bytes)
constexpr int kBlocksPerStage = 2;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kMaxStages = 8;
constexpr int kMaxSplits = 8;           // the portable limit of a thread-block cluster
constexpr int kSumsStride = 128;        // floats per tile in the sums-of-squares array
constexpr uint32_t kWBlockBytes = BF * BK * 2;     // 16 KiB
constexpr size_t kSmemBudget = 208 * 1024;

enum Epilogue : int { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_F32 = 2, EPI_ADD_NORM = 3 };

struct SkinnyParams {
    void* out;
    int64_t out_stride;
    int M, MP, N, K;               // MP: M rounded up to a multiple of 16
    int splits, stages;
    uint32_t tmem_columns;
    uint32_t red_offset;           // where in shared memory the copy of the accumulator lies (0: over the ring)
    float eps;
    const float* ss_in;            // SCALED: [ss_tiles][kSumsStride]
    int ss_tiles;
    const __nv_bfloat16* epi_res;  // EPI_ADD_NORM: residual [M, N], the following norm's weights [N] and the
    const float* epi_norm_w;       // outputs: new residual [M, N], round(c * w) [M, N], sums [tiles][kSumsStride]
    __nv_bfloat16* epi_res_out;
    __nv_bfloat16* epi_xw;
    float* epi_ss;
    int* error;
};

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// A generic pointer to the same place in the shared memory of CTA `rank` of the cluster: loads through it are
// ordinary loads to the compiler, which asks for all of them before it uses the first.
__device__ __forceinline__ const float* map_to_rank(const float* local, uint32_t rank) {
    uint64_t remote;
    asm volatile("mapa.u64 %0, %1, %2;\n" : "=l"(remote) : "l"((uint64_t)local), "r"(rank));
    return reinterpret_cast<const float*>(remote);
}
__device__ __forceinline__ void epilogue_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");
}

__device__ __forceinline__ uint2 pack4_bf16(float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// The epilogue of features n .. n + 3 (n a multiple of 4; a lane's four) of batch row m < M.  All lanes of a warp
// call it together with the same m.  Returns (EPI_ADD_NORM) the warp's sum of c^2 over the row's 128 features.
template <int EPI, bool SCALED>
__device__ __forceinline__ float epilogue_row(const SkinnyParams& p, float4 v, int m, int n, int lane, float scale) {
    if (SCALED) {
        v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    }
    const bool whole = n + 3 < p.N;
    if (EPI == EPI_F32) {
        float* dst = reinterpret_cast<float*>(p.out) + (int64_t)m * p.out_stride + n;
        if (whole && ((uintptr_t)dst & 15) == 0) {
            *reinterpret_cast<float4*>(dst) = v;
        } else {
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n + i < p.N) dst[i] = e[i];
        }
    } else if (EPI == EPI_BF16) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)m * p.out_stride + n;
        if (whole && ((uintptr_t)dst & 7) == 0) {
            *reinterpret_cast<uint2*>(dst) = pack4_bf16(v.x, v.y, v.z, v.w);
        } else {
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n + i < p.N) dst[i] = __float2bfloat16_rn(e[i]);
        }
    } else if (EPI == EPI_SWIGLU) {
        // of every sixteen features (four lanes) the first eight are gates, the last eight the matching up
        // projections: a gate lane takes its four up values from the lane two further on (N is a multiple of 16,
        // so a group of sixteen is whole or absent)
        const float ux = __shfl_down_sync(0xffffffffu, v.x, 2), uy = __shfl_down_sync(0xffffffffu, v.y, 2);
        const float uz = __shfl_down_sync(0xffffffffu, v.z, 2), uw = __shfl_down_sync(0xffffffffu, v.w, 2);
        if ((lane & 2) == 0 && n < p.N) {
            auto act = [](float gate, float up) { return gate * __fdividef(1.0f, 1.0f + __expf(-gate)) * up; };
            // gate feature n + i of the tile's group (n >> 4) is activation column (n >> 4) * 8 + (n & 7) + i
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)m * p.out_stride + (n >> 4) * 8 + (n & 7);
            const float a0 = act(v.x, ux), a1 = act(v.y, uy), a2 = act(v.z, uz), a3 = act(v.w, uw);
            if (((uintptr_t)dst & 7) == 0) {
                *reinterpret_cast<uint2*>(dst) = pack4_bf16(a0, a1, a2, a3);
            } else {
                dst[0] = __float2bfloat16_rn(a0);
                dst[1] = __float2bfloat16_rn(a1);
                dst[2] = __float2bfloat16_rn(a2);
                dst[3] = __float2bfloat16_rn(a3);
            }
        }
    } else {
        const int64_t at = (int64_t)m * p.N + n;
        const float e[4] = {v.x, v.y, v.z, v.w};
        float r[4] = {0.0f, 0.0f, 0.0f, 0.0f}, w[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c[4], x[4];
        const bool vector = whole && (p.N & 3) == 0;      // rows of N elements from 16-byte aligned bases
        if (vector) {
            const uint2 raw = *reinterpret_cast<const uint2*>(p.epi_res + at);
            r[0] = __uint_as_float(raw.x << 16); r[1] = __uint_as_float(raw.x & 0xffff0000u);
            r[2] = __uint_as_float(raw.y << 16); r[3] = __uint_as_float(raw.y & 0xffff0000u);
            const float4 w4 = *reinterpret_cast<const float4*>(p.epi_norm_w + n);
            w[0] = w4.x; w[1] = w4.y; w[2] = w4.z; w[3] = w4.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n + i < p.N) {
                    r[i] = __bfloat162float(p.epi_res[at + i]);
                    w[i] = p.epi_norm_w[n + i];
                }
        }
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float o = __bfloat162float(__float2bfloat16_rn(e[i]));
            c[i] = r[i] + o;
            x[i] = c[i] * w[i];
            if (n + i < p.N) ss = fmaf(c[i], c[i], ss);
        }
        if (vector) {
            *reinterpret_cast<uint2*>(p.epi_res_out + at) = pack4_bf16(c[0], c[1], c[2], c[3]);
            *reinterpret_cast<uint2*>(p.epi_xw + at) = pack4_bf16(x[0], x[1], x[2], x[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (n + i < p.N) {
                    p.epi_res_out[at + i] = __float2bfloat16_rn(c[i]);
                    p.epi_xw[at + i] = __float2bfloat16_rn(x[i]);
                }
        }
        return warp_sum(ss);
    }
    return 0.0f;
}

template <int EPI, bool SCALED>
__global__ void __launch_bounds__(kThreads, 1)
skinny_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const SkinnyParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // barriers: full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2]
    __shared__ __align__(8) uint64_t bars[2 * kMaxStages + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ float scale_s[BF];            // SCALED: the batch rows' reciprocal root mean squares

    pdl_trigger();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.splits, stages = p.stages;
    const int rank = S > 1 ? (int)cluster_rank() : 0;
    const int clusters = (int)gridDim.x / S, cluster_id = (int)blockIdx.x / S;
    const int k_pairs = ((p.K + BK - 1) / BK + kBlocksPerStage - 1) / kBlocksPerStage;
    const int kp0 = rank * k_pairs / S, my_pairs = (rank + 1) * k_pairs / S - kp0;
    const int tiles = (p.N + BF - 1) / BF;
    const int my_tiles = (tiles - cluster_id + clusters - 1) / clusters;
    const uint32_t x_block_bytes = (uint32_t)p.MP * 128u;
    const uint32_t stage_bytes = kBlocksPerStage * (kWBlockBytes + x_block_bytes);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kMaxStages]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * kMaxStages]), acc_empty0 = acc_full0 + 16;
    const uint32_t ring = smem_u32(smem);
    // [MP][BF] the accumulator as 32-bit rows.  It lies over the ring where a CTA has one tile (when that tile's
    // accumulator is complete every copy into the ring has landed and every product has read it), else behind it.
    float* red = reinterpret_cast<float*>(smem + p.red_offset);

    // the producer's cursors: tile row, K pair, ring slot and its barrier, for the weight and for the row loads
    const int total = my_tiles * my_pairs;
    const int pre = total < stages ? total : stages;
    int w_row = cluster_id * BF, w_kp = kp0, x_kp = kp0;
    uint32_t w_dst = ring, w_bar = full0, x_dst = ring + kBlocksPerStage * kWBlockBytes, x_bar = full0;
    int w_slot = 0, x_slot = 0;
    auto load_w = [&]() {
        tma_load_2d(w_dst, &map_w, w_bar, w_kp * (kBlocksPerStage * BK), w_row);
        tma_load_2d(w_dst + kWBlockBytes, &map_w, w_bar, w_kp * (kBlocksPerStage * BK) + BK, w_row);
        if (++w_kp == kp0 + my_pairs) { w_kp = kp0; w_row += clusters * BF; }
        if (++w_slot == stages) { w_slot = 0; w_dst = ring; w_bar = full0; }
        else { w_dst += stage_bytes; w_bar += 8; }
    };
    auto load_x = [&]() {
        tma_load_2d(x_dst, &map_x, x_bar, x_kp * (kBlocksPerStage * BK), 0);
        tma_load_2d(x_dst + x_block_bytes, &map_x, x_bar, x_kp * (kBlocksPerStage * BK) + BK, 0);
        if (++x_kp == kp0 + my_pairs) x_kp = kp0;
        if (++x_slot == stages) { x_slot = 0; x_dst = ring + kBlocksPerStage * kWBlockBytes; x_bar = full0; }
        else { x_dst += stage_bytes; x_bar += 8; }
    };
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, kEpilogueWarps);      // one arrival per epilogue warp
        }
        mbar_fence_init();
        // weights do not depend on the kernel in front, nor on anything the other warps set up
        for (int g = 0; g < pre; ++g) {
            mbar_expect_tx(full0 + 8 * g, stage_bytes);
            load_w();
        }
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), p.tmem_columns);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ------------------------------------------------------------ TMA producer
            pdl_wait();
            for (int g = 0; g < pre; ++g) load_x();
            uint32_t parity = 0;                  // of the wait for a slot's products: flips with every turn of the ring
            for (int g = pre; g < total && !abort_flag; ++g) {
                if (!mbar_wait(empty0 + 8 * w_slot, parity, &abort_flag)) {
                    abort_flag = 1;
                    atomicExch(p.error, 1);
                    break;
                }
                if (w_slot == stages - 1) parity ^= 1;
                mbar_expect_tx(w_bar, stage_bytes);
                load_w();
                load_x();
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            const uint32_t idesc = umma_idesc_bf16(BF, p.MP);
            // the descriptors of stage 0; those of the other stages, blocks and K steps are sums (umma_desc_advance)
            const uint64_t desc_w0 = umma_desc_k_sw128(ring);
            const uint64_t desc_x0 = umma_desc_k_sw128(ring + kBlocksPerStage * kWBlockBytes);
            int s = 0;
            uint32_t parity = 0;                  // of the wait for a stage: flips with every turn of the ring
            uint32_t stage_at = 0;                // s * stage_bytes
            bool ok = true;
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int buf = i & 1;
                if (!mbar_wait(acc_empty0 + 8 * buf, ((i >> 1) & 1) ^ 1, &abort_flag)) {
                    abort_flag = 1;
                    atomicExch(p.error, 4);
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + buf * p.MP;
                for (int j = 0; j < my_pairs; ++j) {
                    if (!mbar_wait(full0 + 8 * s, parity, &abort_flag)) {
                        abort_flag = 1;
                        atomicExch(p.error, 2);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t desc_w = umma_desc_advance(desc_w0, stage_at), desc_x = umma_desc_advance(desc_x0, stage_at);
                    umma_bf16(acc, desc_w, desc_x, idesc, j != 0);
#pragma unroll
                    for (int kk = 1; kk < BK / 16; ++kk)
                        umma_bf16_add(acc, umma_desc_advance(desc_w, kk * 32), umma_desc_advance(desc_x, kk * 32), idesc);
                    const uint64_t desc_w1 = umma_desc_advance(desc_w, kWBlockBytes);
                    const uint64_t desc_x1 = umma_desc_advance(desc_x, x_block_bytes);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)
                        umma_bf16_add(acc, umma_desc_advance(desc_w1, kk * 32), umma_desc_advance(desc_x1, kk * 32), idesc);
                    umma_commit(empty0 + 8 * s);
                    stage_at += stage_bytes;
                    if (++s == stages) {
                        s = 0;
                        stage_at = 0;
                        parity ^= 1;
                    }
                }
                if (ok) umma_commit(acc_full0 + 8 * buf);
            }
        }
        __syncwarp();
    } else {
        pdl_wait();
        if (SCALED) {
            const int e = (int)threadIdx.x - 64;
            if (e < p.M) {
                float total_ss = 0.0f;
                for (int t = 0; t < p.ss_tiles; ++t) total_ss += __ldcg(p.ss_in + (int64_t)t * kSumsStride + e);
                scale_s[e] = 1.0f / sqrtf(total_ss / (float)p.K + p.eps);
            }
            epilogue_barrier();
        }
    }

    // ---------------------------------------------------------------- epilogue (warps 2..9), tile by tile
    const int quarter = warp & 3;                 // a warp may touch tensor-memory lanes 32 * (warp % 4) .. + 31
    const int f = quarter * 32 + lane;            // the feature whose accumulator lane this thread copies
    const float* peer[kMaxSplits];
#pragma unroll
    for (int q = 0; q < kMaxSplits; ++q) peer[q] = S > 1 ? map_to_rank(red, q < S ? q : 0) : red;
    for (int i = 0; i < my_tiles; ++i) {
        const int buf = i & 1;
        const int tile = cluster_id + i * clusters;
        const int n0 = tile * BF;
        bool ok = true;
        if (warp >= 2) {
            ok = mbar_wait(acc_full0 + 8 * buf, (i >> 1) & 1, &abort_flag);
            if (!ok) {
                abort_flag = 1;
                atomicExch(p.error, 3);
            }
            tc_fence_after();
            const uint32_t lanes = tmem_base + buf * p.MP + ((uint32_t)(quarter * 32) << 16);
            if (ok) {
                for (int c0 = ((warp - 2) >> 2) * 16; c0 < p.MP; c0 += 32) {
                    uint32_t raw[16];
                    tmem_load_16(lanes + c0, raw);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) red[(c0 + j) * BF + f] = __uint_as_float(raw[j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
        }
        // every split's partial sums (or, unsplit, the four warps' quarters) are in shared memory
        if (S > 1) cluster_sync();
        else if (warp >= 2) epilogue_barrier();
        if (warp >= 2 && ok && !abort_flag) {
            // split r takes the batch rows r, r + S, ...; of those, warp w every eighth; two rows at a time, so
            // that 2 S loads are in flight (a load from a peer's shared memory takes about a microsecond)
            const int w = warp - 2;
            const int n = n0 + 4 * lane;
            for (int m = rank + w * S; m < p.M; m += 2 * kEpilogueWarps * S) {
                const int m2 = m + kEpilogueWarps * S;
                const bool second = m2 < p.M;
                float4 part[2][kMaxSplits];
#pragma unroll
                for (int q = 0; q < kMaxSplits; ++q) {
                    if (q < S) {
                        part[0][q] = *reinterpret_cast<const float4*>(peer[q] + m * BF + 4 * lane);
                        part[1][q] = *reinterpret_cast<const float4*>(peer[q] + (second ? m2 : m) * BF + 4 * lane);
                    }
                }
                float4 v0 = part[0][0], v1 = part[1][0];
#pragma unroll
                for (int q = 1; q < kMaxSplits; ++q) {
                    if (q < S) {
                        v0.x += part[0][q].x; v0.y += part[0][q].y; v0.z += part[0][q].z; v0.w += part[0][q].w;
                        v1.x += part[1][q].x; v1.y += part[1][q].y; v1.z += part[1][q].z; v1.w += part[1][q].w;
                    }
                }
                const float ss0 = epilogue_row<EPI, SCALED>(p, v0, m, n, lane, SCALED ? scale_s[m] : 1.0f);
                if (EPI == EPI_ADD_NORM && lane == 0) p.epi_ss[(int64_t)tile * kSumsStride + m] = ss0;
                if (second) {
                    const float ss1 = epilogue_row<EPI, SCALED>(p, v1, m2, n, lane, SCALED ? scale_s[m2] : 1.0f);
                    if (EPI == EPI_ADD_NORM && lane == 0) p.epi_ss[(int64_t)tile * kSumsStride + m2] = ss1;
                }
            }
        }
        // nobody overwrites (or leaves with) sums that somebody may still read
        if (S > 1) cluster_sync();
        else if (warp >= 2 && i + 1 < my_tiles) epilogue_barrier();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_columns);
    }
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 1;
    }
    return sms;
}

struct Shape {
    int mp, tiles, splits, clusters, stages;
    uint32_t tmem_columns, red_offset;
    size_t smem;
};

// Ring depth and shared memory of a CTA with these rows, tiles and K pairs.
void fit(Shape& s, int my_tiles, int my_pairs) {
    const size_t stage = (size_t)kBlocksPerStage * (kWBlockBytes + (size_t)s.mp * 128);
    const size_t red = (size_t)s.mp * BF * sizeof(float);
    const bool red_apart = my_tiles > 1;          // the next tile's loads are in the ring while this one's sums are read
    int stages = (int)((kSmemBudget - (red_apart ? red : 0)) / stage);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > my_tiles * my_pairs) stages = my_tiles * my_pairs;
    s.stages = stages;
    const size_t ring = (size_t)stages * stage;
    s.red_offset = red_apart ? (uint32_t)ring : 0;
    s.smem = (red_apart ? ring + red : (ring > red ? ring : red)) + 1024;
}

// How many clusters of `splits` CTAs with this much shared memory the GPU runs at once (a cluster needs its SMs
// inside one GPC, so this is less than SMs / splits: 15 clusters of 8 and 22 of 6 on a B200 with a CTA per SM).
int clusters_at_once(int splits, size_t smem) {
    static std::mutex lock;
    static int known[kMaxSplits + 1] = {0};       // by cluster size, for the largest shared memory asked so far
    static size_t known_smem[kMaxSplits + 1] = {0};
    std::lock_guard<std::mutex> guard(lock);
    if (known[splits] != 0 && smem <= known_smem[splits]) return known[splits];
    auto kernel = skinny_tcgen05_kernel<EPI_BF16, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kSmemBudget + 1024)) != cudaSuccess)
        return 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(splits * sm_count());
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = splits;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    int count = 0;
    if (cudaOccupancyMaxActiveClusters(&count, kernel, &config) != cudaSuccess) {
        cudaGetLastError();
        count = 0;
    }
    known[splits] = count;
    known_smem[splits] = smem;
    return count;
}

// How a product of these sizes is cut: as many K splits (up to 8, one cluster per tile) as let all clusters run at
// once, so that about every SM streams weights; ring depth by what fits.
Shape shape_for(int M, int N, int K) {
    Shape s;
    s.mp = (M + 15) / 16 * 16;
    s.tiles = (N + BF - 1) / BF;
    s.tmem_columns = 32;
    while ((int)s.tmem_columns < 2 * s.mp) s.tmem_columns *= 2;
    const int k_pairs = ((K + BK - 1) / BK + kBlocksPerStage - 1) / kBlocksPerStage;
    const int sms = sm_count();
    int splits = sms / s.tiles;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits > k_pairs) splits = k_pairs;
    for (; splits > 1; --splits) {
        s.splits = splits;
        s.clusters = s.tiles;                     // a split CTA has exactly one tile
        fit(s, 1, (k_pairs + splits - 1) / splits);
        if (clusters_at_once(splits, s.smem) >= s.tiles) return s;
    }
    s.splits = 1;
    s.clusters = s.tiles < sms ? s.tiles : sms;
    fit(s, (s.tiles + s.clusters - 1) / s.clusters, k_pairs);
    return s;
}

template <int EPI, bool SCALED>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const SkinnyParams& p, const Shape& s,
           cudaStream_t stream) {
    auto kernel = skinny_tcgen05_kernel<EPI, SCALED>;
    static std::atomic<bool> allowed{false};      // this instantiation may use as much shared memory as any shape asks
    cudaError_t err = cudaSuccess;
    if (!allowed.load(std::memory_order_acquire)) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kSmemBudget + 1024));
        if (err != cudaSuccess) return (int)err;
        allowed.store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(s.clusters * s.splits);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = s.smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = 1;
    config.numAttrs = 1;
    if (s.splits > 1) {
        attributes[1].id = cudaLaunchAttributeClusterDimension;
        attributes[1].val.clusterDim.x = s.splits;
        attributes[1].val.clusterDim.y = 1;
        attributes[1].val.clusterDim.z = 1;
        config.numAttrs = 2;
    }
    config.attrs = attributes;
    err = cudaLaunchKernelEx(&config, kernel, map_w, map_x, p);
    return err == cudaSuccess ? tb_launch_status() : (int)err;
}

}  // namespace

// 1 if the kernel takes these sizes.  K and the row strides must be multiples of 8 (16-byte TMA strides); the
// SwiGLU epilogue needs N to be a multiple of 16.
TB_EXPORT int tb_skinny_tcgen05_supported(int M, int N, int K, int epilogue) {
    if (M < 1 || M > BF || N < 1 || K < 8 || K % 8 != 0) return 0;
    if (epilogue == EPI_SWIGLU && N % 16 != 0) return 0;
    if (epilogue < EPI_BF16 || epilogue > EPI_ADD_NORM) return 0;
    return shape_for(M, N, K).stages >= 1;
}

// Floats per tile and the number of tiles in the sums-of-squares array that EPI_ADD_NORM leaves for a product of
// N output features.
TB_EXPORT int tb_skinny_tcgen05_sums_stride() { return kSumsStride; }
TB_EXPORT int tb_skinny_tcgen05_sums_tiles(int N) { return (N + BF - 1) / BF; }

// x [M, K] (row stride x_stride), w [N, K] (row stride w_stride), out [M, N] ([M, N / 2] for SwiGLU; out_stride in
// elements of the output type; not written by EPI_ADD_NORM).
// ss_in (or null): sums of squares [ss_tiles][128] that an EPI_ADD_NORM product left; the product is then scaled
//   per row by rsqrt(sum / K + eps).
// EPI_ADD_NORM: epi_res [M, N] residual, epi_norm_w [N], and the outputs epi_res_out [M, N], epi_xw [M, N],
//   epi_ss [tb_skinny_tcgen05_sums_tiles(N)][128].
// error: device int, set non-zero if a bounded wait ran out (the result is then unusable).
TB_EXPORT int tb_skinny_tcgen05(const void* x, int64_t x_stride, const void* w, int64_t w_stride, void* out,
                                int64_t out_stride, int M, int N, int K, int epilogue, const float* ss_in,
                                int ss_tiles, float eps, const void* epi_res, const float* epi_norm_w,
                                void* epi_res_out, void* epi_xw, float* epi_ss, int* error, cudaStream_t stream) {
    if (!tb_skinny_tcgen05_supported(M, N, K, epilogue)) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)x | (uintptr_t)w) % 16 != 0 || x_stride % 8 != 0 || w_stride % 8 != 0 || error == nullptr)
        return TB_ERR_BAD_ALIGN;
    if (epilogue == EPI_ADD_NORM) {
        if (ss_in != nullptr || epi_res == nullptr || epi_norm_w == nullptr || epi_res_out == nullptr ||
            epi_xw == nullptr || epi_ss == nullptr || epi_res_out == epi_res ||
            ((uintptr_t)epi_res | (uintptr_t)epi_res_out | (uintptr_t)epi_xw | (uintptr_t)epi_norm_w) % 16 != 0)
            return TB_ERR_BAD_ALIGN;
    } else if (out == nullptr) {
        return TB_ERR_BAD_ALIGN;
    }
    if (ss_in != nullptr && ss_tiles < 1) return TB_ERR_BAD_ALIGN;
    const Shape s = shape_for(M, N, K);
    const CUtensorMap* cached_w = cached_map_2d(w, (uint64_t)N, (uint64_t)K, (uint64_t)w_stride, BF);
    if (cached_w == nullptr) return TB_ERR_BAD_SIZE;
    const CUtensorMap map_w = *cached_w;
    const CUtensorMap* cached_x = cached_map_2d(x, (uint64_t)M, (uint64_t)K, (uint64_t)x_stride, (uint32_t)s.mp);
    if (cached_x == nullptr) return TB_ERR_BAD_SIZE;
    const CUtensorMap map_x = *cached_x;
    SkinnyParams p;
    p.out = out;
    p.out_stride = out_stride;
    p.M = M;
    p.MP = s.mp;
    p.N = N;
    p.K = K;
    p.splits = s.splits;
    p.stages = s.stages;
    p.tmem_columns = s.tmem_columns;
    p.red_offset = s.red_offset;
    p.eps = eps;
    p.ss_in = ss_in;
    p.ss_tiles = ss_tiles;
    p.epi_res = (const __nv_bfloat16*)epi_res;
    p.epi_norm_w = epi_norm_w;
    p.epi_res_out = (__nv_bfloat16*)epi_res_out;
    p.epi_xw = (__nv_bfloat16*)epi_xw;
    p.epi_ss = epi_ss;
    p.error = error;
    const bool scaled = ss_in != nullptr;
    switch (epilogue) {
        case EPI_BF16:
            return scaled ? launch<EPI_BF16, true>(map_w, map_x, p, s, stream) : launch<EPI_BF16, false>(map_w, map_x, p, s, stream);
        case EPI_SWIGLU:
            return scaled ? launch<EPI_SWIGLU, true>(map_w, map_x, p, s, stream) : launch<EPI_SWIGLU, false>(map_w, map_x, p, s, stream);
        case EPI_F32:
            return scaled ? launch<EPI_F32, true>(map_w, map_x, p, s, stream) : launch<EPI_F32, false>(map_w, map_x, p, s, stream);
        case EPI_ADD_NORM:
            return launch<EPI_ADD_NORM, false>(map_w, map_x, p, s, stream);
    }
    return TB_ERR_BAD_SIZE;
}
