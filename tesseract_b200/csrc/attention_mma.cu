// Tensor-core paged attention for bfloat16: prompt portions (tiles of query rows) and decode
// (split over the keys), over the same block tables and cache pages.
//
// Math per query row, as in the plain kernel and the reference (src/cuda/kernels.rs:447-562):
//   s_j = (q . k_j) * scale for keys j in [max(0, p - window + 1), p], streaming softmax in
//   32-bit, probabilities rounded to bfloat16 for P.V, 32-bit accumulator, out = acc / max(l, 1e-8).
//
// Layout of the work.  The G = num_heads / num_kv_heads query heads that share a kv head are
// folded into the row dimension of a tile: row r of a sequence's tile space is query position
// r / G, head (kv_head * G + r % G), so one pass over a kv head's keys serves the whole group.
//   tb_attention_tiles   : one CTA per (128-row tile, kv head, sequence); its 8 warps own 16 rows
//                          each and share every K/V tile.  For sequences with more than 16 rows.
//   tb_attention_decode  : sequences with at most 16 rows (decode, and tiny portions); one CTA per
//                          (key split, kv head, sequence); its 8 warps (4 for the widest heads) share the 16
//                          rows, each streams every eighth tile of 16 keys through a ring of its own, they are
//                          merged in shared memory, and the splits are merged through the shared memory of a
//                          thread-block cluster (up to 8 splits) or by the split that finishes last from 32-bit
//                          partials in scratch memory.
// K/V tiles come in through cp.async (16-byte chunks, XOR-swizzled in shared memory, rings of three
// stages); the products are mma.sync.m16n8k16 bf16 with fragments from ldmatrix.
// head_dim may be any multiple of 16 up to 256: tiles are zero-padded to 32/64/128/256 columns.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMasked = -1.0e30f;
// split decode kernel: keys per warp tile, warps per CTA and depth of each warp's ring, chosen so that two CTAs
// share an SM up to a padded head size of 128: eight warps of three stages at 64 (96 KiB), six warps of two stages
// at 128 (96 KiB; at batch 64 that reads keys and values at 6.0 TB/s, eight warps of three stages, one CTA per SM,
// at 4.1), four warps of three stages above (192 KiB, one CTA per SM).  Deeper rings measured no faster: a lone
// warp is bound by its own instruction chain.
constexpr int kDecodeKeys = 16;
template <int D>
constexpr int kDecodeWarps = D <= 64 ? 8 : D <= 128 ? 6 : 4;
constexpr int kMaxClusterSplits = 8;  // the portable limit of a thread-block cluster
template <int D>
constexpr int kDecodeStages = D > 64 && D <= 128 ? 2 : 3;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (relative error about 2^-22, far below bfloat16's rounding of P).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Thread-block clusters: a barrier over all CTAs of the cluster and a load from a peer CTA's shared memory.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] bf16 tile, XOR-swizzled so that the
// eight rows an ldmatrix reads fall into distinct bank groups.
template <int D>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
    constexpr int CH = D / 8;
    const int key = (CH >= 8) ? (row & 7) : ((row >> 1) & (CH - 1));
    return (uint32_t)(row * (D * 2) + ((chunk ^ key) << 4));
}

struct AttnParams {
    const __nv_bfloat16* q;      // [rows, num_heads*head_dim], row stride q_stride
    __nv_bfloat16* out;          // [rows, num_heads*head_dim], row stride out_stride
    const __nv_bfloat16* cache;  // [page][K|V][kv_head][page_size][head_dim]
    const int* row_start;        // [R+1]
    const int* seq_begin;        // [R] position of the sequence's first new row
    const int* block_table;      // [R, bt_stride]
    float* part_o;               // [splits][num_seqs][num_kv_heads][16 folded rows][D]   (decode, > 8 splits only)
    float* part_ml;              // [splits][num_seqs][num_kv_heads][16 folded rows][2]
    int* counters;               // [num_seqs][num_kv_heads] arrival counts of the splits; zero between launches
    int64_t q_stride, out_stride;
    int bt_stride, total_rows;
    int num_heads, num_kv_heads, group, head_dim, page_shift, page_size, window, splits;
    int cluster;                 // decode: the splits of a (sequence, kv head) are one thread-block cluster
    // decode with the rotation fused in (every sequence brings exactly one row): q is read unrotated from the
    // packed projection rows [q heads | k heads | v heads], rotated here, and the CTA whose keys include the new
    // position rotates the new key and (write_kv) stores it and the new value into their cache page.
    const __nv_bfloat16* qkv;    // null: q holds rotated queries and the cache already holds the new keys
    const float* inv_freq;       // [head_dim / 2] or null (no rotation)
    int64_t qkv_stride;
    int write_kv;
    float scale_log2;            // scale * log2(e): scores are kept in the base-2 domain
};

// Copies rows [key0, key0 + ROWS) of one kv head's K (which = 0) or V (which = 1) into a swizzled tile.
template <int D, int ROWS, int NT = kThreads>
__device__ __forceinline__ void load_kv_tile(uint32_t tile, const AttnParams& p, const int* table, int kv_head,
                                             int which, int key0, int key_lo, int key_hi) {
    constexpr int CH = D / 8;
    const int64_t head_block = (int64_t)p.page_size * p.head_dim;
    const int64_t page_block = 2 * (int64_t)p.num_kv_heads * head_block;
    const __nv_bfloat16* base = p.cache + ((int64_t)which * p.num_kv_heads + kv_head) * head_block;
    for (int idx = threadIdx.x; idx < ROWS * CH; idx += NT) {
        const int r = idx / CH, c = idx % CH;
        const int key = key0 + r;
        const bool ok = key >= key_lo && key <= key_hi && c * 8 < p.head_dim;
        const __nv_bfloat16* src = base;
        if (ok) {
            const int page = table[key >> p.page_shift];
            src = base + (int64_t)page * page_block + (int64_t)(key & (p.page_size - 1)) * p.head_dim + c * 8;
        }
        cp_async16(tile + tile_offset<D>(r, c), src, ok);
    }
}

// Copies ROWS folded query rows starting at tile-space row r0 of a sequence into a swizzled tile.
template <int D, int ROWS, int NT = kThreads>
__device__ __forceinline__ void load_q_tile(uint32_t tile, const AttnParams& p, int first_row, int kv_head, int r0,
                                            int n_rows) {
    constexpr int CH = D / 8;
    for (int idx = threadIdx.x; idx < ROWS * CH; idx += NT) {
        const int r = idx / CH, c = idx % CH;
        const int fr = r0 + r;
        const bool ok = fr < n_rows && c * 8 < p.head_dim;
        const __nv_bfloat16* src = p.q;
        if (ok) {
            const int qpos = fr / p.group, g = fr - qpos * p.group;
            src = p.q + (int64_t)(first_row + qpos) * p.q_stride + (int64_t)(kv_head * p.group + g) * p.head_dim + c * 8;
        }
        cp_async16(tile + tile_offset<D>(r, c), src, ok);
    }
}

// One warp: 16 query rows (tile rows qrow0..qrow0+15) against NK keys (tile rows krow0..krow0+NK-1, absolute
// keys key_base..).  Updates the running maximum m, the per-thread partial sum l and the accumulator o of the
// thread's two rows (lane/4 and lane/4 + 8).  pos[i] is the absolute position of row i (-1: no such row) and
// lo[i] its first visible key.
// QREG: the Q fragments are already in registers (qf); MASK: some (row, key) pairs of this block are invisible.
template <int D, int NK, bool QREG = false, bool MASK = true>
__device__ __forceinline__ void warp_attend(uint32_t q_tile, int qrow0, uint32_t k_tile, uint32_t v_tile, int krow0,
                                            int key_base, const int (&pos)[2], const int (&lo)[2], float scale_log2,
                                            float (&o)[D / 8][4], float (&m)[2], float (&l)[2],
                                            const uint32_t (*qf)[4] = nullptr) {
    const int lane = threadIdx.x & 31;
    float s[NK / 8][4];
#pragma unroll
    for (int nt = 0; nt < NK / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;

#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a[4];
        if (QREG) {
#pragma unroll
            for (int e = 0; e < 4; ++e) a[e] = qf[ks][e];
        } else {
            ldmatrix_x4(a, q_tile + tile_offset<D>(qrow0 + (lane & 15), ks * 2 + (lane >> 4)));
        }
#pragma unroll
        for (int np = 0; np < NK / 16; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, k_tile + tile_offset<D>(krow0 + np * 16 + (lane & 7) + ((lane >> 4) << 3),
                                                   ks * 2 + ((lane >> 3) & 1)));
            mma_bf16(s[2 * np], a, b[0], b[1]);
            mma_bf16(s[2 * np + 1], a, b[2], b[3]);
        }
    }

    // scale, mask, running maximum
    float block_max[2] = {kMasked, kMasked};
#pragma unroll
    for (int nt = 0; nt < NK / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = e >> 1;
            const int key = key_base + nt * 8 + 2 * (lane & 3) + (e & 1);
            const bool valid = !MASK || (key >= lo[i] && key <= pos[i]);
            s[nt][e] = valid ? s[nt][e] * scale_log2 : kMasked;
            block_max[i] = fmaxf(block_max[i], s[nt][e]);
        }
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        block_max[i] = fmaxf(block_max[i], __shfl_xor_sync(0xffffffffu, block_max[i], 1));
        block_max[i] = fmaxf(block_max[i], __shfl_xor_sync(0xffffffffu, block_max[i], 2));
        const float m_new = fmaxf(m[i], block_max[i]);
        corr[i] = fast_exp2(m[i] - m_new);
        m[i] = m_new;
        l[i] *= corr[i];
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        o[dt][0] *= corr[0];
        o[dt][1] *= corr[0];
        o[dt][2] *= corr[1];
        o[dt][3] *= corr[1];
    }
    // probabilities (masked lanes are exactly zero), 32-bit row sums, bfloat16 P fragments
    uint32_t pa[NK / 16][4];
#pragma unroll
    for (int nt = 0; nt < NK / 8; ++nt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = e >> 1;
            pv[e] = (!MASK || s[nt][e] > 0.5f * kMasked) ? fast_exp2(s[nt][e] - m[i]) : 0.0f;
            l[i] += pv[e];
        }
        pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(pv[0], pv[1]);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
    }
    // O += P . V
#pragma unroll
    for (int kk = 0; kk < NK / 16; ++kk) {
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_tile + tile_offset<D>(krow0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3),
                                                         dp * 2 + (lane >> 4)));
            mma_bf16(o[2 * dp], pa[kk], b[0], b[1]);
            mma_bf16(o[2 * dp + 1], pa[kk], b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Prompt portions: one CTA per (BM-row tile, kv head, sequence); WARPS warps of 16 rows each share every K/V
// tile, which arrive through a STAGES-deep cp.async pipeline.
template <int D, int BN, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, (D <= 64 ? 2 : 1)) attention_tiles_kernel(const AttnParams p) {
    constexpr int BM = WARPS * 16;
    constexpr int NT = WARPS * 32;
    constexpr bool QREG = D <= 128;  // Q fragments live in registers unless the head is very wide
    extern __shared__ __align__(128) unsigned char smem[];
    // blockIdx.x runs over (tile rank, kv head), the kv head fastest: CTAs start in index order, so the heavy
    // tiles (late rows see the most keys) of all heads start first and the light ones fill the gaps
    const int seq = blockIdx.z, kv_head = blockIdx.x % p.num_kv_heads, tile_rank = blockIdx.x / p.num_kv_heads;
    const int first_row = p.row_start[seq];
    const int q_len = p.row_start[seq + 1] - first_row;
    const int n_rows = q_len * p.group;
    const int n_tiles = (n_rows + BM - 1) / BM;
    if (n_rows <= 16 || tile_rank >= n_tiles) return;  // short sequences belong to the decode kernel
    const int r0 = (n_tiles - 1 - tile_rank) * BM;
    const int begin = p.seq_begin[seq];
    const int* table = p.block_table + (int64_t)seq * p.bt_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t q_tile = smem_u32(smem);
    const uint32_t kv_tiles = q_tile + BM * D * 2;  // [stage][K|V][BN][D]
    constexpr uint32_t kTileBytes = BN * D * 2;

    const int last_row = min(n_rows, r0 + BM) - 1;
    const int key_hi = begin + last_row / p.group;
    const int key_lo = p.window > 0 ? max(0, begin + r0 / p.group - p.window + 1) : 0;
    const int kb_first = key_lo / BN, kb_last = key_hi / BN;
    const int n_blocks = kb_last - kb_first + 1;

    load_q_tile<D, BM, NT>(q_tile, p, first_row, kv_head, r0, n_rows);
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < n_blocks) {
            const uint32_t dst = kv_tiles + st * 2 * kTileBytes;
            load_kv_tile<D, BN, NT>(dst, p, table, kv_head, 0, (kb_first + st) * BN, key_lo, key_hi);
            load_kv_tile<D, BN, NT>(dst + kTileBytes, p, table, kv_head, 1, (kb_first + st) * BN, key_lo, key_hi);
        }
        cp_async_commit();  // one group per stage, empty or not, keeps the wait count fixed
    }

    int pos[2], lo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int fr = r0 + warp * 16 + (lane >> 2) + i * 8;
        pos[i] = fr < n_rows ? begin + fr / p.group : -1;
        lo[i] = p.window > 0 ? max(0, pos[i] - p.window + 1) : 0;
    }
    float o[D / 8][4], m[2] = {kMasked, kMasked}, l[2] = {0.0f, 0.0f};
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
    const int warp_first = r0 + warp * 16;
    const bool warp_active = warp_first < n_rows;
    const int warp_rows_end = min(n_rows, warp_first + 16);
    const int warp_hi_key = begin + (warp_rows_end - 1) / p.group;   // last key any row of this warp sees
    const int warp_lo_pos = begin + warp_first / p.group;            // every row of this warp sees keys up to here
    const bool all_rows = warp_first + 16 <= n_rows;

    uint32_t qf[QREG ? D / 16 : 1][4];
    for (int it = 0; it < n_blocks; ++it) {
        const int kb = kb_first + it;
        // prefetch block it + STAGES - 1 into the stage that was consumed in the previous iteration
        if (it + STAGES - 1 < n_blocks) {
            const uint32_t dst = kv_tiles + ((it + STAGES - 1) % STAGES) * 2 * kTileBytes;
            load_kv_tile<D, BN, NT>(dst, p, table, kv_head, 0, (kb + STAGES - 1) * BN, key_lo, key_hi);
            load_kv_tile<D, BN, NT>(dst + kTileBytes, p, table, kv_head, 1, (kb + STAGES - 1) * BN, key_lo, key_hi);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (QREG && it == 0) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(qf[ks], q_tile + tile_offset<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
        }
        if (warp_active && kb * BN <= warp_hi_key) {
            const uint32_t cur = kv_tiles + (it % STAGES) * 2 * kTileBytes;
            // no mask when every key of the block is visible to every row of the warp
            const bool full = all_rows && p.window <= 0 && kb * BN + BN - 1 <= warp_lo_pos;
            if (full)
                warp_attend<D, BN, QREG, false>(q_tile, warp * 16, cur, cur + kTileBytes, 0, kb * BN, pos, lo,
                                                p.scale_log2, o, m, l, qf);
            else
                warp_attend<D, BN, QREG, true>(q_tile, warp * 16, cur, cur + kTileBytes, 0, kb * BN, pos, lo,
                                               p.scale_log2, o, m, l, qf);
        }
        __syncthreads();  // everyone is done with this stage before the next prefetch overwrites it
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        if (pos[i] < 0) continue;
        const int fr = r0 + warp * 16 + (lane >> 2) + i * 8;
        const int qpos = fr / p.group, g = fr - qpos * p.group;
        const float inv = 1.0f / fmaxf(l[i], 1.0e-8f);
        __nv_bfloat16* dst = p.out + (int64_t)(first_row + qpos) * p.out_stride +
                             (int64_t)(kv_head * p.group + g) * p.head_dim;
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            const int col = dt * 8 + 2 * (lane & 3);
            if (col < p.head_dim)
                *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[dt][2 * i] * inv, o[dt][2 * i + 1] * inv);
        }
    }
}

// Tail of the decode kernel: merges the CTA's four warps (each saw some of the split's keys) through shared
// memory and then the splits, in ascending order whichever way they meet: as a thread-block cluster the splits
// leave their partial results in shared memory and the first CTA reads them from its peers; otherwise they go
// to scratch memory and the split that finishes last merges them.
template <int D, int WARPS>
__device__ __forceinline__ void decode_finish(const AttnParams& p, unsigned char* smem, int split, int kv_head, int seq,
                                              int first_row, int n_rows, float (&o)[D / 8][4], float (&m)[2],
                                              float (&l)[2]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // merge the four warps (each saw a quarter of the keys) through shared memory
    // rows of the accumulators are D + 8 floats apart: the eight rows that a warp's lanes store at once then fall
    // on different banks (64-bit stores, conflict-free by half-warp)
    constexpr int P = D + 8;
    float* sm_m = reinterpret_cast<float*>(smem);             // [warps][16]
    float* sm_l = sm_m + WARPS * 16;                         // [warps][16]
    float* sm_o = sm_l + WARPS * 16;                         // [warps][16][P]
    float* x_ml = sm_o + WARPS * 16 * P;                     // [2][16]  this split's maximum and sum (cluster merge)
    float* x_acc = x_ml + 32;                                 // [16][D]  this split's accumulator
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        const int r = (lane >> 2) + i * 8;
        if ((lane & 3) == 0) {
            sm_m[warp * 16 + r] = m[i];
            sm_l[warp * 16 + r] = l[i];
        }
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            const int col = dt * 8 + 2 * (lane & 3);
            *reinterpret_cast<float2*>(sm_o + (warp * 16 + r) * P + col) = make_float2(o[dt][2 * i], o[dt][2 * i + 1]);
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_rows * D; idx += (WARPS * 32)) {
        const int r = idx / D, col = idx - r * D;
        float big = kMasked;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) big = fmaxf(big, sm_m[w * 16 + r]);
        float acc = 0.0f, sum = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float wgt = exp2f(sm_m[w * 16 + r] - big);
            acc += wgt * sm_o[(w * 16 + r) * P + col];
            sum += wgt * sm_l[w * 16 + r];
        }
        const int qpos = r / p.group, g = r - qpos * p.group;
        const int head = kv_head * p.group + g;
        const int row = first_row + qpos;
        if (p.splits == 1) {
            if (col < p.head_dim)
                p.out[(int64_t)row * p.out_stride + (int64_t)head * p.head_dim + col] =
                    __float2bfloat16_rn(acc / fmaxf(sum, 1.0e-8f));
        } else if (p.cluster) {
            x_acc[idx] = acc;
            if (col == 0) {
                x_ml[r] = sum > 0.0f ? big : kMasked;
                x_ml[16 + r] = sum;
            }
        } else {
            // a slot per (split, sequence, kv head, folded row): the scratch is sized by the sequences of the
            // step, never by its rows (a prompt portion beside the decode rows costs nothing here)
            const int64_t slot = ((((int64_t)split * gridDim.z + seq) * p.num_kv_heads + kv_head) << 4) + r;
            p.part_o[slot * D + col] = acc;
            if (col == 0) {
                p.part_ml[slot * 2] = big;
                p.part_ml[slot * 2 + 1] = sum;
            }
        }
    }
    if (p.splits == 1) return;
    if (p.cluster) {
        cluster_sync();  // every split's partial result is in its shared memory
        if (cluster_rank() == 0) {
            for (int idx = threadIdx.x; idx < n_rows * D; idx += (WARPS * 32)) {
                const int r = idx / D, col = idx - r * D;
                if (col >= p.head_dim) continue;
                // every split's maximum, sum and accumulator at once: the remote loads are independent of each
                // other, so their latencies overlap (one after the other they cost a round trip per split)
                float m_s[kMaxClusterSplits], l_s[kMaxClusterSplits], a_s[kMaxClusterSplits];
#pragma unroll
                for (int s = 0; s < kMaxClusterSplits; ++s) {
                    const bool have = s < p.splits;
                    m_s[s] = have ? ld_cluster_f32(x_ml + r, s) : kMasked;
                    l_s[s] = have ? ld_cluster_f32(x_ml + 16 + r, s) : 0.0f;
                    a_s[s] = have ? ld_cluster_f32(x_acc + idx, s) : 0.0f;
                }
                float big = kMasked;
#pragma unroll
                for (int s = 0; s < kMaxClusterSplits; ++s) big = fmaxf(big, m_s[s]);
                float acc = 0.0f, sum = 0.0f;
#pragma unroll
                for (int s = 0; s < kMaxClusterSplits; ++s) {
                    const float w = l_s[s] > 0.0f ? exp2f(m_s[s] - big) : 0.0f;
                    sum += w * l_s[s];
                    acc += w * a_s[s];
                }
                const int qpos = r / p.group, g = r - qpos * p.group;
                p.out[(int64_t)(first_row + qpos) * p.out_stride + (int64_t)(kv_head * p.group + g) * p.head_dim + col] =
                    __float2bfloat16_rn(acc / fmaxf(sum, 1.0e-8f));
            }
        }
        cluster_sync();  // no CTA leaves while a peer may still read its shared memory
        return;
    }

    // The split that arrives last merges all of them (a fixed order over the splits, so the result does not
    // depend on which one that is) and leaves the counter at zero for the next launch.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = p.counters + seq * p.num_kv_heads + kv_head;
        const int ticket = atomicAdd(counter, 1);
        is_last = ticket == p.splits - 1;
        if (is_last) *counter = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // weights of the splits per row, computed side by side: wgt[s][r] = 2^(m_s - max m) (0 for an empty split)
    float* wgt = reinterpret_cast<float*>(smem);              // [splits][16]
    float* row_big = wgt + p.splits * 16;                     // [16]
    float* row_sum = row_big + 16;                            // [16]
    for (int idx = threadIdx.x; idx < p.splits * n_rows; idx += (WARPS * 32)) {
        const int s = idx / n_rows, r = idx - s * n_rows;
        const int64_t slot = ((((int64_t)s * gridDim.z + seq) * p.num_kv_heads + kv_head) << 4) + r;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + slot * 2));
        wgt[s * 16 + r] = ml.y > 0.0f ? ml.x : kMasked;        // the maximum for now
        wgt[(p.splits + 2 + s) * 16 + r] = ml.y;               // the sums, parked behind row_big / row_sum
    }
    __syncthreads();
    if (threadIdx.x < n_rows) {
        const int r = threadIdx.x;
        float big = kMasked;
        for (int s = 0; s < p.splits; ++s) big = fmaxf(big, wgt[s * 16 + r]);
        float sum = 0.0f;
        for (int s = 0; s < p.splits; ++s) {
            const float l_s = wgt[(p.splits + 2 + s) * 16 + r];
            const float w = l_s > 0.0f ? exp2f(wgt[s * 16 + r] - big) : 0.0f;
            wgt[s * 16 + r] = w;
            sum += w * l_s;
        }
        row_sum[r] = sum;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_rows * D; idx += (WARPS * 32)) {
        const int r = idx / D, col = idx - r * D;
        if (col >= p.head_dim) continue;
        const int qpos = r / p.group, g = r - qpos * p.group;
        const int head = kv_head * p.group + g;
        const int row = first_row + qpos;
        const float* src = p.part_o + ((((int64_t)seq * p.num_kv_heads + kv_head) << 4) + r) * D + col;
        const int64_t split_stride = (int64_t)gridDim.z * p.num_kv_heads * 16 * D;
        float acc = 0.0f;
#pragma unroll 8
        for (int s = 0; s < p.splits; ++s) acc += wgt[s * 16 + r] * __ldcg(src + s * split_stride);
        p.out[(int64_t)row * p.out_stride + (int64_t)head * p.head_dim + col] =
            __float2bfloat16_rn(acc / fmaxf(row_sum[r], 1.0e-8f));
    }
}

// One warp copies NK keys of one kv head's K and V (keys key0.. of the sequence) into its own swizzled tiles, in
// passes of 32 sixteen-byte chunks.  The page of a lane's key in each pass comes from the block table: a load that
// the copy depends on, so the kernel below looks the pages of a tile up one tile ahead (warp_pages) and copies
// with them later (warp_copy_kv); warp_load_kv does both at once.
template <int D, int NK>
__device__ __forceinline__ void warp_pages(const AttnParams& p, const int* table, int key0, int key_lo, int key_hi,
                                           int (&pages)[NK * (D / 8) / 32]) {
    constexpr int CH = D / 8;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int pass = 0; pass < NK * CH / 32; ++pass) {
        const int key = key0 + (pass * 32 + lane) / CH;
        pages[pass] = key >= key_lo && key <= key_hi ? table[key >> p.page_shift] : 0;
    }
}

template <int D, int NK>
__device__ __forceinline__ void warp_copy_kv(uint32_t k_tile, uint32_t v_tile, const AttnParams& p, int kv_head,
                                             int key0, int key_lo, int key_hi, const int (&pages)[NK * (D / 8) / 32]) {
    constexpr int CH = D / 8;
    static_assert((NK * CH) % 32 == 0, "a warp copies whole passes of 32 chunks");
    const int lane = threadIdx.x & 31;
    const int64_t head_block = (int64_t)p.page_size * p.head_dim;
    const int64_t page_block = 2 * (int64_t)p.num_kv_heads * head_block;
    const int64_t v_offset = (int64_t)p.num_kv_heads * head_block;
    const __nv_bfloat16* base = p.cache + (int64_t)kv_head * head_block;
#pragma unroll
    for (int pass = 0; pass < NK * CH / 32; ++pass) {
        const int idx = pass * 32 + lane;
        const int r = idx / CH, c = idx % CH;
        const int key = key0 + r;
        const bool ok = key >= key_lo && key <= key_hi && c * 8 < p.head_dim;
        const __nv_bfloat16* src = base;
        if (ok)
            src = base + (int64_t)pages[pass] * page_block + (int64_t)(key & (p.page_size - 1)) * p.head_dim + c * 8;
        const uint32_t offset = tile_offset<D>(r, c);
        cp_async16(k_tile + offset, src, ok);
        cp_async16(v_tile + offset, src + v_offset, ok);
    }
}

template <int D, int NK>
__device__ __forceinline__ void warp_load_kv(uint32_t k_tile, uint32_t v_tile, const AttnParams& p, const int* table,
                                             int kv_head, int key0, int key_lo, int key_hi) {
    int pages[NK * (D / 8) / 32];
    warp_pages<D, NK>(p, table, key0, key_lo, key_hi, pages);
    warp_copy_kv<D, NK>(k_tile, v_tile, p, kv_head, key0, key_lo, key_hi, pages);
}

// ------------------------------------------------------------------------------------------------
// Decode and tiny portions (at most 16 folded rows): one CTA per (key split, kv head, sequence).  The split's
// keys are cut into tiles of NK keys; warp w takes every WARPS-th tile and streams its tiles through a ring of its
// own (cp.async groups, waits and __syncwarp only), so no warp ever waits for another inside the loop and each
// keeps STAGES - 1 tiles in flight.
template <int D, int WARPS, int NK>
__global__ void __launch_bounds__(WARPS * 32) attention_decode_kernel(const AttnParams p) {
    constexpr int STAGES = kDecodeStages<D>;
    constexpr bool QREG = D <= 128;
    constexpr uint32_t kTileBytes = NK * D * 2;
    constexpr uint32_t kStageBytes = 2 * kTileBytes;
    extern __shared__ __align__(128) unsigned char smem[];
    // The kernel before this one in the stream wrote this step's queries and keys.  Sequence metadata, block
    // tables and the keys of earlier steps do not depend on it and are fetched before waiting for it.
    pdl_trigger();
    const int split = blockIdx.x, kv_head = blockIdx.y, seq = blockIdx.z;
    const int first_row = p.row_start[seq];
    const int q_len = p.row_start[seq + 1] - first_row;
    const int n_rows = q_len * p.group;
    if (n_rows > 16 || n_rows == 0 || (p.qkv != nullptr && q_len != 1)) {
        pdl_wait();
        return;
    }
    const int begin = p.seq_begin[seq];
    const int* table = p.block_table + (int64_t)seq * p.bt_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t q_tile = smem_u32(smem);
    const uint32_t ring = q_tile + 16 * D * 2 + warp * (STAGES * kStageBytes);
    float* trig = reinterpret_cast<float*>(smem + 16 * D * 2 + WARPS * STAGES * kStageBytes);   // [D] (fused rotation)
    __nv_bfloat16* new_kv = reinterpret_cast<__nv_bfloat16*>(trig + D);                          // [2][D]

    const int key_hi = begin + q_len - 1;
    const int key_lo = p.window > 0 ? max(0, begin - p.window + 1) : 0;
    const int lo_max = p.window > 0 ? max(0, key_hi - p.window + 1) : 0;  // first key that every row sees
    const int kb_first = key_lo / NK, kb_end = key_hi / NK + 1;
    const int per_split = (kb_end - kb_first + p.splits - 1) / p.splits;
    const int b0 = kb_first + split * per_split;
    const int b1 = min(kb_end, b0 + per_split);
    const int kb_new = begin / NK;                       // fused rotation: the tile of the new key
    const bool owns_new = p.qkv != nullptr && kb_new >= b0 && kb_new < b1;

    int pos[2], lo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int fr = (lane >> 2) + i * 8;
        pos[i] = fr < n_rows ? begin + fr / p.group : -1;
        lo[i] = p.window > 0 ? max(0, pos[i] - p.window + 1) : 0;
    }
    float o[D / 8][4], m[2] = {kMasked, kMasked}, l[2] = {0.0f, 0.0f};
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;

    bool waited = false;
    int next_pages[NK * (D / 8) / 32];
    if (b0 < b1) {
        if (p.qkv != nullptr) {
            // angles of the one new position: angle_i = float(position) * inv_freq[i], 32-bit, accurate functions
            const int half = p.head_dim >> 1;
            for (int i = threadIdx.x; i < half; i += WARPS * 32) {
                float c = 1.0f, s = 0.0f;
                if (p.inv_freq != nullptr) {
                    const float angle = (float)begin * p.inv_freq[i];
                    sincosf(angle, &s, &c);     // (the same call as in rope_cache.cu: a key is the same bits whichever wrote it)
                }
                trig[i] = c;
                trig[half + i] = s;
            }
            __syncthreads();
        }
        int kb_load = b0 + warp;
#pragma unroll
        for (int st = 0; st < STAGES - 1; ++st) {
            if (kb_load < b1) {
                if (!waited && (kb_load + 1) * NK > begin) {  // the tile holds keys of this step
                    pdl_wait();
                    waited = true;
                }
                warp_load_kv<D, NK>(ring + st * kStageBytes, ring + st * kStageBytes + kTileBytes, p, table, kv_head,
                                    kb_load * NK, key_lo, key_hi);
            }
            cp_async_commit();  // one group per stage, empty or not, keeps the wait count fixed
            kb_load += WARPS;
        }
        // the pages of the tile that the loop fetches first, looked up a tile ahead from here on
        if (kb_load < b1) warp_pages<D, NK>(p, table, kb_load * NK, key_lo, key_hi, next_pages);
        if (!waited) {
            pdl_wait();
            waited = true;
        }
        if (p.qkv == nullptr) {
            load_q_tile<D, 16, WARPS * 32>(q_tile, p, first_row, kv_head, 0, n_rows);
        } else {
            // rotate-half on the way in (src/cuda/kernels.rs:210-282), a pair (x[i], x[half + i]) at a time; the
            // columns beyond head_dim and the rows beyond the group are zero
            const int half = p.head_dim >> 1;
            const __nv_bfloat16* row = p.qkv + (int64_t)first_row * p.qkv_stride;
            auto put = [&](unsigned char* tile_or_null, __nv_bfloat16* linear, int r, int col, float v) {
                const __nv_bfloat16 b = __float2bfloat16_rn(v);
                if (tile_or_null != nullptr)
                    *reinterpret_cast<__nv_bfloat16*>(tile_or_null + tile_offset<D>(r, col >> 3) + (col & 7) * 2) = b;
                else
                    linear[col] = b;
                return b;
            };
            auto pair_columns = [&](int i, int& c0, int& c1) {
                if (i < half) { c0 = i; c1 = half + i; }
                else { c0 = p.head_dim + 2 * (i - half); c1 = c0 + 1; }
            };
#pragma unroll 2
            for (int idx = threadIdx.x; idx < 16 * (D / 2); idx += WARPS * 32) {
                const int r = idx / (D / 2), i = idx - r * (D / 2);
                int c0, c1;
                pair_columns(i, c0, c1);
                float a = 0.0f, b = 0.0f;
                if (r < n_rows && i < half) {
                    const __nv_bfloat16* x = row + (int64_t)(kv_head * p.group + r) * p.head_dim;
                    const float lo = __bfloat162float(x[i]), hi = __bfloat162float(x[half + i]);
                    const float c = trig[i], s = trig[half + i];
                    a = lo * c - hi * s;
                    b = hi * c + lo * s;
                }
                put(smem, nullptr, r, c0, a);
                put(smem, nullptr, r, c1, b);
            }
            if (owns_new && p.write_kv) {
                // the new key (rotated) and value of this kv head: to the staging rows and to the cache page
                const __nv_bfloat16* k = row + (int64_t)(p.num_heads + kv_head) * p.head_dim;
                const __nv_bfloat16* v = k + (int64_t)p.num_kv_heads * p.head_dim;
                const int64_t head_block = (int64_t)p.page_size * p.head_dim;
                __nv_bfloat16* kdst = const_cast<__nv_bfloat16*>(p.cache) +
                                      ((int64_t)table[begin >> p.page_shift] * 2 * p.num_kv_heads + kv_head) * head_block +
                                      (int64_t)(begin & (p.page_size - 1)) * p.head_dim;
                __nv_bfloat16* vdst = kdst + (int64_t)p.num_kv_heads * head_block;
                for (int i = threadIdx.x; i < D / 2; i += WARPS * 32) {
                    int c0, c1;
                    pair_columns(i, c0, c1);
                    float a = 0.0f, b = 0.0f;
                    __nv_bfloat16 v0 = __float2bfloat16_rn(0.0f), v1 = v0;
                    if (i < half) {
                        const float lo = __bfloat162float(k[i]), hi = __bfloat162float(k[half + i]);
                        const float c = trig[i], s = trig[half + i];
                        a = lo * c - hi * s;
                        b = hi * c + lo * s;
                        v0 = v[c0];
                        v1 = v[c1];
                    }
                    const __nv_bfloat16 k0 = put(nullptr, new_kv, 0, c0, a), k1 = put(nullptr, new_kv, 0, c1, b);
                    new_kv[D + c0] = v0;
                    new_kv[D + c1] = v1;
                    if (i < half) {
                        kdst[c0] = k0;
                        kdst[c1] = k1;
                        vdst[c0] = v0;
                        vdst[c1] = v1;
                    }
                }
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        uint32_t qf[QREG ? D / 16 : 1][4];
        if (QREG) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(qf[ks], q_tile + tile_offset<D>(lane & 15, ks * 2 + (lane >> 4)));
        }
        int it = 0;
        for (int kb = b0 + warp; kb < b1; kb += WARPS, ++it) {
            if (kb_load < b1) {
                const uint32_t dst = ring + ((it + STAGES - 1) % STAGES) * kStageBytes;
                warp_copy_kv<D, NK>(dst, dst + kTileBytes, p, kv_head, kb_load * NK, key_lo, key_hi, next_pages);
            }
            cp_async_commit();
            kb_load += WARPS;
            if (kb_load < b1) warp_pages<D, NK>(p, table, kb_load * NK, key_lo, key_hi, next_pages);
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            const uint32_t cur = ring + (it % STAGES) * kStageBytes;
            if (owns_new && p.write_kv && kb == kb_new) {
                // the copy may have read the page before this CTA's store reached it: take the staged rows
                if (lane < D / 8) {
                    const uint32_t off = tile_offset<D>(begin - kb_new * NK, lane);
                    const uint4* staged = reinterpret_cast<const uint4*>(new_kv);
                    *reinterpret_cast<uint4*>(smem + (cur - q_tile) + off) = staged[lane];
                    *reinterpret_cast<uint4*>(smem + (cur - q_tile) + kTileBytes + off) = staged[D / 8 + lane];
                }
                __syncwarp();
            }
            // no mask when every row sees every key of the tile
            const bool full = kb * NK >= lo_max && kb * NK + NK - 1 <= begin;
            if (full)
                warp_attend<D, NK, QREG, false>(q_tile, 0, cur, cur + kTileBytes, 0, kb * NK, pos, lo, p.scale_log2,
                                                o, m, l, qf);
            else
                warp_attend<D, NK, QREG, true>(q_tile, 0, cur, cur + kTileBytes, 0, kb * NK, pos, lo, p.scale_log2,
                                               o, m, l, qf);
            __syncwarp();  // every lane is done with this stage before the next copy overwrites it
        }
        cp_async_wait<0>();
    }
    if (!waited) pdl_wait();
    __syncthreads();  // the rings become the merge area
    decode_finish<D, WARPS>(p, smem, split, kv_head, seq, first_row, n_rows, o, m, l);
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

template <int D, int warps>
int launch_decode(const AttnParams& p, int num_seqs, cudaStream_t stream) {
    const size_t merge_a = (size_t)(2 * warps * 16 + warps * 16 * (D + 8) + 32 + 16 * D) * sizeof(float);
    const size_t merge_b = (size_t)(2 * p.splits + 2) * 16 * sizeof(float);
    const size_t merge = merge_a > merge_b ? merge_a : merge_b;
    const size_t tiles = (size_t)16 * D * 2 + (size_t)warps * kDecodeStages<D> * 2 * kDecodeKeys * D * 2 +
                         (size_t)D * sizeof(float) + (size_t)2 * D * 2;   // + rotation angles, staged new key/value
    const size_t smem = tiles > merge ? tiles : merge;
    auto kernel = attention_decode_kernel<D, warps, kDecodeKeys>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    // programmatic dependent launch; the splits of a (sequence, kv head) as one cluster when they fit one
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(p.splits, p.num_kv_heads, num_seqs);
    config.blockDim = dim3(warps * 32);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = 1;
    config.numAttrs = 1;
    if (p.cluster) {
        attributes[1].id = cudaLaunchAttributeClusterDimension;
        attributes[1].val.clusterDim.x = p.splits;
        attributes[1].val.clusterDim.y = 1;
        attributes[1].val.clusterDim.z = 1;
        config.numAttrs = 2;
    }
    config.attrs = attributes;
    if (cudaError_t err = cudaLaunchKernelEx(&config, kernel, p)) return (int)err;
    return tb_launch_status();
}

template <int D>
int launch_all(const AttnParams& p, int num_seqs, int max_rows_per_seq, int run_tiles, int run_decode,
               cudaStream_t stream) {
    constexpr int BN = D <= 128 ? 64 : 32;
    constexpr int WARPS = D <= 128 ? 8 : 4;
    constexpr int STAGES = D <= 64 ? 3 : 2;
    if (run_tiles) {
        constexpr int BM = WARPS * 16;
        const size_t smem = (size_t)BM * D * 2 + (size_t)STAGES * 2 * BN * D * 2;
        auto kernel = attention_tiles_kernel<D, BN, WARPS, STAGES>;
        if (smem > 48 * 1024) {
            cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (err != cudaSuccess) return (int)err;
        }
        dim3 grid(((max_rows_per_seq + BM - 1) / BM) * p.num_kv_heads, 1, num_seqs);
        kernel<<<grid, WARPS * 32, smem, stream>>>(p);
        if (int status = tb_launch_status()) return status;
    }
    if (run_decode) {
        // Many sequences and no splits: CTAs of four warps, of which an SM holds twice as many, so that the launch
        // stays one wave (head size 64 at batch 64: 45.8 against 50.3 us; fewer CTAs are faster with eight warps).
        if constexpr (D <= 64) {
            if (p.splits == 1 && (int64_t)num_seqs * p.num_kv_heads > 2 * (int64_t)sm_count())
                return launch_decode<D, 4>(p, num_seqs, stream);
        }
        return launch_decode<D, kDecodeWarps<D>>(p, num_seqs, stream);
    }
    return 0;
}

}  // namespace

// Column count of the zero-padded tiles (and of the partial accumulators) for a head size.
TB_EXPORT int tb_attention_mma_padded_dim(int head_dim) {
    if (head_dim <= 0 || head_dim > 256 || head_dim % 16 != 0) return TB_ERR_BAD_SIZE;
    return head_dim <= 32 ? 32 : head_dim <= 64 ? 64 : head_dim <= 128 ? 128 : 256;
}

// Attention of every row of a packed batch over its sequence's cached keys (bfloat16).
//   run_tiles  : launch the tile kernel (sequences with more than 16 folded rows)
//   run_decode : launch the split kernel (sequences with at most 16 folded rows) with `splits` key splits;
//                2 to 8 splits meet as a thread-block cluster and use no scratch; more than 8 need
//                part_o float[splits * num_seqs * num_kv_heads * 16 * padded_dim] and
//                part_ml float[splits * num_seqs * num_kv_heads * 16 * 2] (a slot per folded row of a (split,
//                sequence, kv head), whatever the step's row count); scratch_floats is the capacity of part_o;
//                counters int[num_seqs * num_kv_heads], all zero before the first launch (each launch leaves
//                them zero again).
static int attention_entry(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                           const int* row_start, const int* seq_begin, const int* block_table, int bt_stride,
                           int num_seqs, int total_rows, int max_rows_per_seq, int num_heads, int num_kv_heads,
                           int head_dim, int page_size, int window, float scale, int run_tiles, int run_decode,
                           int splits, float* part_o, float* part_ml, int64_t scratch_floats, int* counters,
                           const void* qkv, int64_t qkv_stride, const float* inv_freq, int write_kv,
                           cudaStream_t stream) {
    if (num_seqs == 0 || total_rows == 0) return 0;
    const int padded = tb_attention_mma_padded_dim(head_dim);
    if (padded < 0) return padded;
    if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return TB_ERR_BAD_SIZE;
    if (page_size < 8 || (page_size & (page_size - 1)) != 0) return TB_ERR_BAD_SIZE;
    if (num_seqs > 65535 || num_kv_heads > 65535 || num_heads > 65535) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache | (uintptr_t)qkv) % 16 != 0 || (q_stride % 8) != 0)
        return TB_ERR_BAD_ALIGN;
    if (splits < 1) splits = 1;
    const int cluster = splits >= 2 && splits <= kMaxClusterSplits;
    if (run_decode && splits > 1 && !cluster) {
        const int64_t need = (int64_t)splits * num_seqs * num_kv_heads * 16 * padded;
        if (part_o == nullptr || part_ml == nullptr || counters == nullptr || need > scratch_floats) return -5;
    }
    AttnParams p;
    p.q = (const __nv_bfloat16*)q;
    p.out = (__nv_bfloat16*)out;
    p.cache = (const __nv_bfloat16*)cache;
    p.row_start = row_start;
    p.seq_begin = seq_begin;
    p.block_table = block_table;
    p.part_o = part_o;
    p.part_ml = part_ml;
    p.counters = counters;
    p.q_stride = q_stride;
    p.out_stride = out_stride;
    p.bt_stride = bt_stride;
    p.total_rows = total_rows;
    p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads;
    p.group = num_heads / num_kv_heads;
    p.head_dim = head_dim;
    p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window;
    p.splits = splits;
    p.cluster = cluster;
    p.qkv = (const __nv_bfloat16*)qkv;
    p.qkv_stride = qkv_stride;
    p.inv_freq = inv_freq;
    p.write_kv = write_kv;
    p.scale_log2 = scale * kLog2e;
    const int max_folded = max_rows_per_seq * p.group;
    switch (padded) {
        case 32: return launch_all<32>(p, num_seqs, max_folded, run_tiles, run_decode, stream);
        case 64: return launch_all<64>(p, num_seqs, max_folded, run_tiles, run_decode, stream);
        case 128: return launch_all<128>(p, num_seqs, max_folded, run_tiles, run_decode, stream);
        default: return launch_all<256>(p, num_seqs, max_folded, run_tiles, run_decode, stream);
    }
}

TB_EXPORT int tb_attention_mma(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                               const int* row_start, const int* seq_begin, const int* block_table, int bt_stride,
                               int num_seqs, int total_rows, int max_rows_per_seq, int num_heads, int num_kv_heads,
                               int head_dim, int page_size, int window, float scale, int run_tiles, int run_decode,
                               int splits, float* part_o, float* part_ml, int64_t scratch_floats,
                               int* counters, cudaStream_t stream) {
    return attention_entry(q, q_stride, out, out_stride, cache, row_start, seq_begin, block_table, bt_stride, num_seqs,
                           total_rows, max_rows_per_seq, num_heads, num_kv_heads, head_dim, page_size, window, scale,
                           run_tiles, run_decode, splits, part_o, part_ml, scratch_floats, counters, nullptr, 0,
                           nullptr, 0, stream);
}

// Decode step with the position encoding and the cache write folded in: every sequence brings exactly one row.
// qkv holds the packed projection rows [q heads | k heads | v heads] (unrotated, row stride qkv_stride); queries
// and the new key are rotated by angle_i = float(position) * inv_freq[i] (inv_freq null: no rotation), and with
// write_kv the new key and value are stored into the cache page of their position (cache is written here).
// Scratch arguments as for tb_attention_mma.
TB_EXPORT int tb_attention_decode_rope(const void* qkv, int64_t qkv_stride, void* out, int64_t out_stride, void* cache,
                                       const int* row_start, const int* seq_begin, const int* block_table,
                                       int bt_stride, int num_seqs, int num_heads, int num_kv_heads, int head_dim,
                                       int page_size, int window, float scale, const float* inv_freq, int write_kv,
                                       int splits, float* part_o, float* part_ml, int64_t scratch_floats,
                                       int* counters, cudaStream_t stream) {
    if (qkv == nullptr || qkv_stride % 8 != 0 || (head_dim & 1)) return TB_ERR_BAD_ALIGN;
    return attention_entry(qkv, qkv_stride, out, out_stride, cache, row_start, seq_begin, block_table, bt_stride,
                           num_seqs, num_seqs, 1, num_heads, num_kv_heads, head_dim, page_size, window, scale,
                           /*run_tiles=*/0, /*run_decode=*/1, splits, part_o, part_ml, scratch_floats, counters, qkv,
                           qkv_stride, inv_freq, write_kv, stream);
}
