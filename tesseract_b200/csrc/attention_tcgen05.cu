// Prompt-portion attention on the fifth-generation tensor cores (bfloat16, head_dim 64 or 128), over cache pages.
//
// Same mathematics and the same folding of grouped query heads into tile rows as attention_mma.cu (which see):
// one CTA owns 128 folded rows (query position x head of the group) of one sequence and one kv head, and
// walks over the sequence's keys in blocks of BN (128 for head_dim 64, 64 for head_dim 128).  Per block, for
// head_dim 64 (head_dim 128: N64 x K128 and N128 x K64, operands cut into 64-element slices along the head size):
//   S = Q . K^T        tcgen05.mma, M128 x N128 x K64, both operands in shared memory (K-major, 128-byte swizzle),
//                      accumulator in tensor memory (128 columns)
//   softmax            four warps, one thread per row: tcgen05.ld of the row, scale, mask, running maximum,
//                      2^x, 32-bit row sum, probabilities rounded to bfloat16 into a swizzled P tile in shared memory
//                      (a block that needs no mask is read once, against the maximum that earlier blocks left; the
//                      row is read twice, maximum first, only where that maximum is exceeded by more than 2^8)
//   O += P . V         tcgen05.mma, M128 x N64 x K128, P K-major, V MN-major (the cache's [key][dim] rows as they
//                      are), accumulating in 64 further columns of tensor memory; when a row's maximum jumps by
//                      more than 2^8 its thread rescales that row of O in place (tcgen05.ld / tcgen05.st)
// Warps 0-3 are the softmax / correction / epilogue warps (warp w owns tensor-memory lanes 32w..32w+31); one lane
// of warp 5 brings K and V blocks into a ring of shared-memory stages, page by page through the block table, with
// cp.async.bulk.tensor over a five-dimensional tensor map of the cache (no multicast); one lane of warp 4 issues
// the tensor-core instructions.  Roles meet on mbarriers; every wait is bounded, and a wait that
// runs out sets *error, stops the other roles, and the CTA still frees its tensor memory.
// Two CTAs fit on an SM (112 KiB of shared memory and 256 tensor-memory columns each), so one CTA's softmax
// overlaps the other's products.
#include "tma.cuh"

namespace {

using namespace tbtma;

constexpr int BM = 128;          // folded query rows per CTA
// Keys per block for head_dim 64: 128, two CTAs per SM (64 with three CTAs per SM was faster only beyond some 4,000
// tokens of context).  head_dim 128 takes 64 keys per block, which lets two CTAs share an SM (112 KiB of shared
// memory and 256 tensor-memory columns each).
constexpr int kBlockKeys64 = 128;
constexpr int STAGES = 2;        // K/V ring depth
constexpr int kThreads = 192;         // warps 0..3 softmax, warp 4 issuer, warp 5 TMA producer
// A swizzled tile of 128 rows x 64 bfloat16 (128 bytes a row): the unit that Q, P, K and V tiles are made of.  A Q
// tile is D / 64 of them side by side (dims 0..63 | 64..127), a P tile BN / 64 (keys 0..63 | 64..127); K and V
// blocks are D / 64 tiles of BN rows each.
constexpr uint32_t kTileBytes = BM * 128;
template <int D, int BN>
struct Shape {
    static constexpr uint32_t kQBytes = (D / 64) * kTileBytes;
    static constexpr int kPTiles = BN / 64;
    static constexpr uint32_t kKVHalfBytes = BN * 128;               // one 64-dim slice of a K or V block
    static constexpr uint32_t kKVTileBytes = (D / 64) * kKVHalfBytes;   // one K or V block
    static constexpr int kCtasPerSm = D == 64 && BN == 64 ? 3 : 2;
    static constexpr uint32_t kTmemColumns = BN + D <= 128 ? 128 : 256;   // S: columns 0..BN-1, O: the D columns after them
    static constexpr size_t kSmemBytes = (size_t)kQBytes + (size_t)kPTiles * kTileBytes + (size_t)2 * STAGES * kKVTileBytes;
};
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMasked = -1.0e30f;

struct TcAttnParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const __nv_bfloat16* cache;
    const int* row_start;
    const int* seq_begin;
    const int* block_table;
    int* error;
    // key splits (gridDim.y > 1): every split's unnormalised output rows, their maxima and sums, arrival counters
    float* part_o;                 // [tile CTA][split][128 rows][D]
    float* part_ml;                // [tile CTA][split][128 rows][2]
    int* counters;                 // [tile CTA], zero before and after every launch
    int64_t q_stride, out_stride;
    int bt_stride;
    int num_heads, num_kv_heads, group, page_shift, page_size, window;
    float scale_log2;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
// makes this thread's earlier shared-memory writes visible to the tensor core's (asynchronous) reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile of 128-byte rows with the 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// Matrix descriptors for such tiles: version 1, SWIZZLE_128B, 1024 bytes between groups of eight rows.
// lbo: 1 for K-major tiles (the field is not used there); for MN-major tiles the distance between 64-element
// atoms along MN in 16-byte units (one atom here, so it is not used either).
__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr, uint32_t lbo) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)lbo << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D = F32, A = B = BF16; b_mn = 1 when B is MN-major (bit 16); N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_add(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {   // D += A . B
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.eq.u32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_load_32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31,%32};"
        ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(v[8]),
          "f"(v[9]), "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]), "f"(v[16]), "f"(v[17]),
          "f"(v[18]), "f"(v[19]), "f"(v[20]), "f"(v[21]), "f"(v[22]), "f"(v[23]), "f"(v[24]), "f"(v[25]), "f"(v[26]),
          "f"(v[27]), "f"(v[28]), "f"(v[29]), "f"(v[30]), "f"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Blackwell's packed 32-bit pairs (one instruction for two lanes of a 64-bit register pair) and three-input
// maximum: the softmax loop is bound by the number of instructions it issues per score.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {   // each lane: fmaf(a, b, c)
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// 2^x for a pair of lanes on the FMA pipe, for x <= 8 or so (the softmax's exponents): the special-function unit
// gives 16 results a cycle and SM, which bounds the unmasked blocks' loop once two CTAs share an SM, so at head
// size 64 every fourth pair of a row goes this way (2 to 5 % faster; every third or second pair is slower again,
// and so is any share at head size 128, whose blocks have more products per exponential).  x = n + f with n the
// nearest integer (the low mantissa bits of x + 1.5 * 2^23) and f in [-0.5, 0.5]; 2^f by a cubic (largest
// relative error 7.5e-5, far below the rounding of the probabilities to bfloat16); n is added into the exponent
// field.  All of it in 32-bit arithmetic.
template <int D>
constexpr int kPolyEvery = D == 64 ? 4 : 0;
__device__ __forceinline__ void exp2_pair_fma(uint64_t x2, float& p0, float& p1) {
    float x0, x1;
    unpack2(x2, x0, x1);
    const uint64_t x = pack2(fmaxf(x0, -125.0f), fmaxf(x1, -125.0f));
    const uint64_t t = add2(x, pack2(12582912.0f, 12582912.0f));
    const uint64_t n = add2(t, pack2(-12582912.0f, -12582912.0f));
    const uint64_t f = fma2(n, pack2(-1.0f, -1.0f), x);
    uint64_t q = fma2(f, pack2(0.0551716685f, 0.0551716685f), pack2(0.2426111251f, 0.2426111251f));
    q = fma2(q, f, pack2(0.6932609677f, 0.6932609677f));
    q = fma2(q, f, pack2(0.9999280572f, 0.9999280572f));
    float q0, q1, t0, t1;
    unpack2(q, q0, q1);
    unpack2(t, t0, t1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

// SPLIT: tiles shared by gridDim.y CTAs (the code that leaves and adds partial rows costs the unsplit kernel 2-6 %
// of its time through its registers alone, so it is an instantiation of its own).
template <int D, int BN, bool SPLIT>
__global__ void __launch_bounds__(kThreads, (Shape<D, BN>::kCtasPerSm))
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap cache_map, const TcAttnParams p) {
    using Tiles = Shape<D, BN>;
    constexpr uint32_t kKVTileBytes = Tiles::kKVTileBytes, kKVHalfBytes = Tiles::kKVHalfBytes;
    constexpr uint32_t kTmemColumns = Tiles::kTmemColumns;
    constexpr int kPTiles = Tiles::kPTiles;
    extern __shared__ __align__(1024) unsigned char smem[];   // the swizzled tiles need 1024-byte alignment
    // barriers: k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES], s_full, p_ready, o_full, s_free.
    // Keys and values have rings of their own: a key block's stage is free again as soon as its scores are
    // computed, a whole block before its value stage is.
    __shared__ __align__(8) uint64_t bars[4 * STAGES + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ int last_to_arrive;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blockIdx.x runs over (tile rank, kv head) with the kv head fastest: CTAs start in the order of their index,
    // so the heavy tiles (late rows see the most keys) of ALL heads start first and the light ones fill the gaps
    const int seq = blockIdx.z, kv_head = blockIdx.x % p.num_kv_heads, tile_rank = blockIdx.x / p.num_kv_heads;
    const int first_row = p.row_start[seq];
    const int q_len = p.row_start[seq + 1] - first_row;
    const int n_rows = q_len * p.group;
    const int n_tiles = (n_rows + BM - 1) / BM;
    pdl_trigger();
    if (n_rows <= 16 || tile_rank >= n_tiles) {           // short sequences belong to the decode kernel
        pdl_wait();                                             // (no thread leaves before the kernel in front is done)
        return;
    }
    if (smem_u32(smem) & 1023u) {                               // never expected: refuse rather than compute garbage
        if (threadIdx.x == 0) atomicExch(p.error, 99);
        pdl_wait();
        return;
    }
    const int r0 = (n_tiles - 1 - tile_rank) * BM;              // heavy tiles first
    const int begin = p.seq_begin[seq];
    const int* table = p.block_table + (int64_t)seq * p.bt_stride;

    const uint32_t q_tile = smem_u32(smem);
    const uint32_t p_tile = q_tile + Tiles::kQBytes;                // kPTiles tiles of 16 KiB (keys 0..63 | 64..127)
    const uint32_t kv_tiles = p_tile + kPTiles * kTileBytes;    // [stage][K | V]
    const uint32_t k_full = smem_u32(&bars[0]), k_empty = smem_u32(&bars[STAGES]);
    const uint32_t v_full = smem_u32(&bars[2 * STAGES]), v_empty = smem_u32(&bars[3 * STAGES]);
    const uint32_t s_full = smem_u32(&bars[4 * STAGES]), p_ready = s_full + 8, o_full = s_full + 16;
    const uint32_t s_free = s_full + 24;

    const int last_row = min(n_rows, r0 + BM) - 1;
    const int key_hi = begin + last_row / p.group;
    const int key_lo = p.window > 0 ? max(0, begin + r0 / p.group - p.window + 1) : 0;
    // The tile's key blocks, cut into gridDim.y contiguous runs: a step whose tiles are too few to fill the GPU (a
    // 512-token portion late in a long prompt) gives each tile to several CTAs, which leave unnormalised partial
    // rows; the one that finishes last adds them in the order of the runs.  A run may be empty (early tiles).
    const int key_splits = SPLIT ? (int)gridDim.y : 1, key_split = SPLIT ? (int)blockIdx.y : 0;
    const int tile_blocks = key_hi / BN - key_lo / BN + 1;
    const int first_of_run = key_split * tile_blocks / key_splits;
    const int kb_first = key_lo / BN + first_of_run;
    const int n_blocks = (key_split + 1) * tile_blocks / key_splits - first_of_run;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(k_full + 8 * s, 1);
            mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1);
            mbar_init(v_empty + 8 * s, 1);
        }
        mbar_init(s_full, 1);
        mbar_init(p_ready, BM);
        mbar_init(o_full, 1);
        mbar_init(s_free, BM);
        mbar_fence_init();
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // barriers and tensor memory are set up while the kernel before this one drains; its results (the rotated
    // queries, this step's keys and values) are read from here on
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();
    // The Q tile: the threads of warps 0..4 copy their share of the 128 rows x D / 8 chunks, swizzled like the K/V
    // tiles, while warp 5 already brings the first key and value blocks (a tile's first scores used to wait for
    // the two loads one after the other).
    constexpr int kChunks = D / 8;
    if (warp != 5) {
        for (int idx = threadIdx.x; idx < BM * kChunks; idx += kThreads - 32) {
            const int r = idx / kChunks, c = idx % kChunks;
            const int fr = r0 + r;
            const bool ok = fr < n_rows;
            const __nv_bfloat16* src = p.q;
            if (ok) {
                const int qpos = fr / p.group, g = fr - qpos * p.group;
                src = p.q + (int64_t)(first_row + qpos) * p.q_stride + (int64_t)(kv_head * p.group + g) * D + c * 8;
            }
            cp_async16(q_tile + (c >> 3) * kTileBytes + sw128(r, c & 7), src, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_async_smem();
        asm volatile("bar.sync 1, 160;" ::: "memory");            // warps 0..4: the issuer reads Q after this
    }
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + BN;

    if (warp == 5) {
        // ------------------------------------------------------------ TMA producer: K and V blocks, page by page
        // Lane c brings page c of a block (its table entry, one copy); lane 0 waits for the stage and announces
        // the bytes.  Order: K_0 V_0 K_1 V_1 ... (K_{j+STAGES} becomes possible before V_{j+STAGES} does).
        const int rows_per_copy = min(p.page_size, BN);          // keys one bulk copy brings
        const int copies = BN / rows_per_copy;                   // at most 16 (pages of 8 keys or more)
        const int last_page = key_hi >> p.page_shift;            // pages past it hold nothing of this sequence
        bool ok = true;
        for (int it = 0; it < n_blocks && ok; ++it) {
            const int s = it % STAGES;
            const int key0 = (kb_first + it) * BN;
            int page = 0, in_page = 0;
            if (lane < copies) {
                const int key = key0 + lane * rows_per_copy;
                const int logical = key >> p.page_shift;
                // keys past the sequence come from the scratch page: finite values that the mask removes
                page = logical <= last_page ? table[logical] : 0;
                in_page = key & (p.page_size - 1);
            }
            const uint32_t dst = kv_tiles + s * 2 * kKVTileBytes + (uint32_t)(lane * rows_per_copy) * 128;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                const uint32_t full = (which ? v_full : k_full) + 8 * s, empty = (which ? v_empty : k_empty) + 8 * s;
                int go = 1;
                if (lane == 0) {
                    go = mbar_wait(empty, ((it / STAGES) & 1) ^ 1, &abort_flag) ? 1 : 0;
                    if (go) mbar_expect_tx(full, kKVTileBytes);
                }
                go = __shfl_sync(0xffffffffu, go, 0);            // also orders the announcement before the copies
                if (!go) { ok = false; break; }
                if (lane < copies) {
#pragma unroll
                    for (int h = 0; h < D / 64; ++h)
                        tma_load_kv(dst + which * kKVTileBytes + h * kKVHalfBytes, &cache_map, full, h * 64, in_page,
                                    kv_head, which, page);
                }
            }
        }
        if (!ok && lane == 0) {
            abort_flag = 1;
            atomicExch(p.error, 10);
        }
    } else if (warp == 4) {
        // ------------------------------------------------------------ the issuer: one lane feeds the tensor core
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_bf16(BM, BN, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(BM, D, 1);
            // One thread issues every product, and what it executes between two of them is time the tensor core
            // idles (a 128 x 64 x 16 product takes 46 cycles; building two descriptors from addresses takes 100):
            // the descriptors of stage 0 are built once and moved by adding to the start-address field (bytes >> 4;
            // the field holds addresses below 256 KiB, so the sum never carries out of it).
            const uint64_t q_desc = desc_sw128(q_tile, 1), p_desc = desc_sw128(p_tile, 1);
            const uint64_t k_desc0 = desc_sw128(kv_tiles, 1);
            const uint64_t v_desc0 = desc_sw128(kv_tiles + kKVTileBytes, kKVHalfBytes >> 4);
            constexpr uint32_t kStageStep = (2 * kKVTileBytes) >> 4;          // a ring stage further, in the field's units
            // (a wait costs this thread some 200 cycles even on a barrier that is long complete, so the keys and
            // values, which arrive far ahead, are waited for BEFORE the barrier that the softmax warps are about
            // to complete: their answer is then the only one on the path from the softmax to the product)
            auto issue_qk = [&](int s) {
                tc_fence_after();
                const uint64_t k_desc = k_desc0 + (uint32_t)s * kStageStep;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint64_t a = q_desc + (((kk >> 2) * kTileBytes + (kk & 3) * 32) >> 4);
                    const uint64_t b = k_desc + (((kk >> 2) * kKVHalfBytes + (kk & 3) * 32) >> 4);
                    if (kk == 0) umma(tmem_s, a, b, idesc_qk, 0);
                    else umma_add(tmem_s, a, b, idesc_qk);
                }
                umma_commit(s_full);
                umma_commit(k_empty + 8 * s);     // the key stage may be refilled once these products are done
            };
            // ring cursors of the block whose scores are issued (qs, q_parity) and of the one whose P.V is (s, parity)
            int qs = 0, s = 0;
            uint32_t q_parity = 0, parity = 0;
            auto next_q = [&]() { if (++qs == STAGES) { qs = 0; q_parity ^= 1; } };
            bool ok = n_blocks == 0 || mbar_wait(k_full + 8 * qs, q_parity, &abort_flag);
            if (ok && n_blocks > 0) issue_qk(qs);
            next_q();
            for (int j = 0; j < n_blocks && ok; ++j) {
                // as soon as the softmax warps hold S_j in registers the next block's scores may overwrite it
                if (j + 1 < n_blocks) {
                    if (!mbar_wait(k_full + 8 * qs, q_parity, &abort_flag)) { ok = false; break; }
                    if (!mbar_wait(s_free, j & 1, &abort_flag)) { ok = false; break; }
                    issue_qk(qs);
                    next_q();
                }
                // P_j is in shared memory (and O has been rescaled if the maximum jumped): O += P_j V_j
                if (!mbar_wait(v_full + 8 * s, parity, &abort_flag)) { ok = false; break; }
                if (!mbar_wait(p_ready, j & 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t v_desc = v_desc0 + (uint32_t)s * kStageStep;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t a = p_desc + (((kk >> 2) * kTileBytes + (kk & 3) * 32) >> 4);
                    const uint64_t b = v_desc + ((kk * 2048) >> 4);
                    if (kk == 0) umma(tmem_o, a, b, idesc_pv, j != 0);
                    else umma_add(tmem_o, a, b, idesc_pv);
                }
                umma_commit(o_full);
                umma_commit(v_empty + 8 * s);
                if (++s == STAGES) { s = 0; parity ^= 1; }
            }
            if (!ok) {
                abort_flag = 1;
                atomicExch(p.error, 20);
            }
        }
    } else {
        // ------------------------------------------------------------ softmax, correction, epilogue: one thread per row
        const int r = warp * 32 + lane;                 // row of the tile = tensor-memory lane
        const int fr = r0 + r;
        const int pos = fr < n_rows ? begin + fr / p.group : -1;
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        // rows of this warp span positions [warp_lo_pos, ...]: blocks at or below warp_lo_pos need no mask
        const int warp_first = r0 + warp * 32;
        const bool all_rows = warp_first + 32 <= n_rows;
        const int warp_lo_pos = begin + warp_first / p.group;
        const int warp_hi_pos = begin + (warp_first + 31) / p.group;    // (of a warp whose rows are all there)
        // The running output lives in tensor memory (P.V accumulates there).  m is the maximum that the stored
        // probabilities and O are scaled by; it is only raised (and O rescaled) when a block's maximum exceeds it
        // by more than 2^8, which keeps every probability at or below 256 and makes the rescaling rare.
        float m = kMasked, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_blocks; ++j) {
            const int key0 = (kb_first + j) * BN;
            if (!mbar_wait(s_full, j & 1, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            const bool full = all_rows && p.window <= 0 && key0 + BN - 1 <= warp_lo_pos;   // uniform across the warp
            if (full && j > 0) {
                // One pass for a block that needs no mask: its probabilities are computed against the maximum that
                // earlier blocks left, while the block's own maximum is followed on the side.  Only if that exceeds m
                // by more than 2^8 in some row of the warp (rare after a row's first block) is the work thrown away
                // and the block done again by the two passes below, from the scores that are still in tensor memory:
                // either way the probabilities are those of the two passes, bit for bit.  The first chunks wait in
                // registers until the product before this one has read the P tile.
                uint32_t ca[32], cb[32], held[32];
                float mx[4] = {kMasked, kMasked, kMasked, kMasked};
                uint64_t ls[4] = {0, 0, 0, 0};
                const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg_m2 = pack2(-m, -m);
                auto maxima = [&](const uint32_t (&chunk)[32]) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(chunk[i]), __uint_as_float(chunk[i + 1]));
                };
                auto exps = [&](const uint32_t (&chunk)[32], uint32_t* packed) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const uint64_t x2 = fma2(pack2(__uint_as_float(chunk[i]), __uint_as_float(chunk[i + 1])), scale2, neg_m2);
                        float p0, p1;
                        constexpr int kEvery = kPolyEvery<D> > 0 ? kPolyEvery<D> : 1;
                        if (kPolyEvery<D> > 0 && (i >> 1) % kEvery == kEvery - 1) {
                            exp2_pair_fma(x2, p0, p1);
                        } else {
                            float t0, t1;
                            unpack2(x2, t0, t1);
                            p0 = fast_exp2(t0);
                            p1 = fast_exp2(t1);
                        }
                        ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
                        packed[i >> 1] = pack_bf16(p0, p1);
                    }
                };
                auto store = [&](const uint32_t* packed, int c) {
                    unsigned char* dst = smem + Tiles::kQBytes + (c >> 1) * kTileBytes;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        *reinterpret_cast<uint4*>(dst + sw128(r, (c & 1) * 4 + q4)) =
                            make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
                };
                constexpr int kLast = BN / 32 - 1;                 // the chunk whose maxima decide
                tmem_load_32_nowait(tmem_s + lane_base, ca);
                tmem_wait_ld();
                tmem_load_32_nowait(tmem_s + lane_base + 32, cb);
                maxima(ca);
                exps(ca, held);
                tmem_wait_ld();
                if (BN == 128) {
                    tmem_load_32_nowait(tmem_s + lane_base + 64, ca);
                    maxima(cb);
                    exps(cb, held + 16);
                }
                if (!mbar_wait(o_full, (j - 1) & 1, &abort_flag)) { ok = false; break; }
                store(held, 0);
                if (BN == 128) {
                    store(held + 16, 1);
                    tmem_wait_ld();
                    tmem_load_32_nowait(tmem_s + lane_base + 96, cb);
                    maxima(ca);
                    exps(ca, held);
                    store(held, 2);
                    tmem_wait_ld();
                }
                maxima(cb);
                const float seen = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
                if (!__any_sync(0xffffffffu, seen > m + 8.0f)) {
                    tc_fence_before();
                    mbar_arrive(s_free);               // S has been read: the issuer may start the next block's scores
                    exps(cb, held);
                    store(held, kLast);
                    float lo_sum, hi_sum;
                    unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), lo_sum, hi_sum);
                    l += lo_sum + hi_sum;
                    fence_async_smem();
                    tc_fence_before();
                    mbar_arrive(p_ready);
                    continue;
                }
            }
            // The two passes, chunk by chunk.  A warp's rows are a few neighbouring positions, so of the block on the
            // diagonal most 32-key chunks lie wholly before them (no mask needed: the short path) or wholly behind
            // them (no score counts: zeros, nothing computed), and only the chunk or two that the rows' last keys
            // (and, with a window, their first) fall into are masked element by element, which costs four times
            // the instructions: a whole block done that way took as long as three and a half unmasked ones.
            enum { kOpen = 0, kMaskedChunk = 1, kDead = 2 };
            auto chunk_mode = [&](int c) {                          // uniform across the warp
                if (full) return (int)kOpen;
                if (!all_rows) return (int)kMaskedChunk;
                const int first_key = key0 + c * 32, last_key = first_key + 31;
                if (first_key > warp_hi_pos) return (int)kDead;
                if (p.window > 0) {
                    if (last_key < max(0, warp_lo_pos - p.window + 1)) return (int)kDead;
                    if (first_key < max(0, warp_hi_pos - p.window + 1)) return (int)kMaskedChunk;
                }
                return last_key <= warp_lo_pos ? (int)kOpen : (int)kMaskedChunk;
            };
            // Pass 1: the row's maximum over the block, 32 columns at a time (the next chunk is in flight while one
            // is reduced; four partial maxima keep the dependency chains short).
            uint32_t ca[32], cb[32];
            float mx[4] = {kMasked, kMasked, kMasked, kMasked};
            const int lo_col = lo - key0, hi_col = pos - key0;     // this row sees columns lo_col..hi_col of the block
            // (the scale is positive, so the maximum of the raw scores is scaled once at the end; blocks that need
            // no mask take the short path: one instruction per element)
            auto reduce_max = [&](const uint32_t (&chunk)[32], int c) {
                const int mode = chunk_mode(c);
                if (mode == kOpen) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(chunk[i]), __uint_as_float(chunk[i + 1]));
                } else if (mode == kMaskedChunk) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const bool valid = c * 32 + i >= lo_col && c * 32 + i <= hi_col;
                        mx[i & 3] = fmaxf(mx[i & 3], valid ? __uint_as_float(chunk[i]) : kMasked);
                    }
                }
            };
            tmem_load_32_nowait(tmem_s + lane_base, ca);
            tmem_wait_ld();
            tmem_load_32_nowait(tmem_s + lane_base + 32, cb);
            reduce_max(ca, 0);
            tmem_wait_ld();
            if (BN == 128) {
                tmem_load_32_nowait(tmem_s + lane_base + 64, ca);
                reduce_max(cb, 1);
                tmem_wait_ld();
                tmem_load_32_nowait(tmem_s + lane_base + 96, cb);
                reduce_max(ca, 2);
                tmem_wait_ld();
                reduce_max(cb, 3);
            } else {
                reduce_max(cb, 1);
            }
            const float raw_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const float block_max = raw_max > 0.5f * kMasked ? raw_max * p.scale_log2 : kMasked;
            // P_{j-1} V_{j-1} must be complete before the P tile is overwritten (and before O is rescaled)
            if (j > 0 && !mbar_wait(o_full, (j - 1) & 1, &abort_flag)) { ok = false; break; }
            const bool jump = block_max > m + 8.0f;
            if (__any_sync(0xffffffffu, jump)) {
                const float m_new = fmaxf(m, block_max);
                const float corr = fast_exp2(m - m_new);
                m = m_new;
                l *= corr;
                if (j > 0) {
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        float v[32];
                        tmem_load_32(tmem_o + lane_base + c * 32, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] *= corr;
                        tmem_store_32(tmem_o + lane_base + c * 32, v);
                    }
                }
            }
            // Pass 2: probabilities, their 32-bit sum (four partial sums), and the bfloat16 P tile.
            uint64_t ls[4] = {0, 0, 0, 0};   // four pairs of partial sums (0 is the bit pattern of (0.0f, 0.0f))
            auto emit = [&](const uint32_t (&chunk)[32], int c) {
                uint32_t packed[16];
                const float neg_m = -m;
                const int mode = chunk_mode(c);
                if (mode == kDead) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) packed[i] = 0u;
                } else if (mode == kOpen) {
                    const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg_m2 = pack2(neg_m, neg_m);
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float t0, t1;
                        unpack2(fma2(pack2(__uint_as_float(chunk[i]), __uint_as_float(chunk[i + 1])), scale2, neg_m2),
                                t0, t1);
                        const float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
                        ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
                        packed[i >> 1] = pack_bf16(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float pr[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const bool valid = c * 32 + i + e >= lo_col && c * 32 + i + e <= hi_col;
                            pr[e] = valid ? fast_exp2(fmaf(__uint_as_float(chunk[i + e]), p.scale_log2, neg_m)) : 0.0f;
                        }
                        ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(pr[0], pr[1]));
                        packed[i >> 1] = pack_bf16(pr[0], pr[1]);
                    }
                }
                unsigned char* dst = smem + Tiles::kQBytes + (c >> 1) * kTileBytes;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    *reinterpret_cast<uint4*>(dst + sw128(r, (c & 1) * 4 + q4)) =
                        make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
            };
            tmem_load_32_nowait(tmem_s + lane_base, ca);
            tmem_wait_ld();
            tmem_load_32_nowait(tmem_s + lane_base + 32, cb);
            emit(ca, 0);
            tmem_wait_ld();
            if (BN == 128) {
                tmem_load_32_nowait(tmem_s + lane_base + 64, ca);
                emit(cb, 1);
                tmem_wait_ld();
                tmem_load_32_nowait(tmem_s + lane_base + 96, cb);
                emit(ca, 2);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(s_free);                   // S has been read: the issuer may start the next block's scores
                emit(cb, 3);
            } else {
                tc_fence_before();
                mbar_arrive(s_free);
                emit(cb, 1);
            }
            {
                float lo, hi;
                unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), lo, hi);
                l += lo + hi;
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(p_ready);
        }
        if (ok && n_blocks > 0 && !mbar_wait(o_full, (n_blocks - 1) & 1, &abort_flag)) ok = false;
        const int qpos = pos >= 0 ? fr / p.group : 0, g = pos >= 0 ? fr - qpos * p.group : 0;
        __nv_bfloat16* dst = p.out + (int64_t)(first_row + qpos) * p.out_stride + (int64_t)(kv_head * p.group + g) * D;
        if (!SPLIT) {
            if (ok) {
                tc_fence_after();
                const float inv = 1.0f / fmaxf(l, 1.0e-8f);
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    float v[32];
                    tmem_load_32(tmem_o + lane_base + c * 32, v);
                    if (pos >= 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            float w8[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) w8[e] = v[i + e] * inv;
                            Packet<__nv_bfloat16>::store(dst + c * 32 + i, w8);
                        }
                    }
                }
                tc_fence_before();
            }
        } else {
            // this run's rows as they stand (scaled by 2^-m, not yet divided by the sum), its maxima and sums
            const int64_t tile_cta = (int64_t)seq * gridDim.x + blockIdx.x;
            float* my_o = p.part_o + ((tile_cta * key_splits + key_split) * BM + r) * D;
            float* my_ml = p.part_ml + ((tile_cta * key_splits + key_split) * BM + r) * 2;
            if (ok && n_blocks > 0) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    float v[32];
                    tmem_load_32(tmem_o + lane_base + c * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        __stcg(reinterpret_cast<float4*>(my_o + c * 32 + i), make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]));
                }
                tc_fence_before();
            }
            __stcg(reinterpret_cast<float2*>(my_ml), make_float2(n_blocks > 0 ? m : kMasked, n_blocks > 0 ? l : 0.0f));
            __threadfence();
            asm volatile("bar.sync 2, 128;" ::: "memory");            // the four softmax warps
            if (r == 0) {
                const int arrived = atomicAdd(p.counters + tile_cta, 1);
                last_to_arrive = arrived == key_splits - 1;
                if (last_to_arrive) p.counters[tile_cta] = 0;         // every run of the tile has arrived: as found
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (last_to_arrive && ok && pos >= 0) {
                // the runs in ascending order, whichever arrived when: o = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s
                __threadfence();
                const float* runs_o = p.part_o + (tile_cta * key_splits * BM + r) * D;
                const float* runs_ml = p.part_ml + (tile_cta * key_splits * BM + r) * 2;
                float weight[8];
                float big = kMasked, total = 0.0f;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    weight[s] = kMasked;
                    if (s < key_splits) weight[s] = __ldcg(runs_ml + (int64_t)s * BM * 2);
                    big = fmaxf(big, weight[s]);
                }
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    const float sum = s < key_splits ? __ldcg(runs_ml + (int64_t)s * BM * 2 + 1) : 0.0f;
                    weight[s] = sum > 0.0f ? fast_exp2(weight[s] - big) : 0.0f;
                    total = fmaf(sum, weight[s], total);
                }
                const float inv = 1.0f / fmaxf(total, 1.0e-8f);
                // 64 columns at a time, run by run: all of a run's sixteen loads are in flight before the first is
                // used (a loop over the columns with the runs inside waits for L2 once per eight columns)
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 64) {
                    float acc[64];
#pragma unroll
                    for (int e = 0; e < 64; ++e) acc[e] = 0.0f;
#pragma unroll 1
                    for (int s = 0; s < key_splits; ++s) {
                        float w = 0.0f;
#pragma unroll
                        for (int t = 0; t < 8; ++t) w = t == s ? weight[t] : w;
                        if (w > 0.0f) {
                            float4 part[16];
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                part[e] = __ldcg(reinterpret_cast<const float4*>(runs_o + (int64_t)s * BM * D + c0 + 4 * e));
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                acc[4 * e] = fmaf(part[e].x, w, acc[4 * e]);
                                acc[4 * e + 1] = fmaf(part[e].y, w, acc[4 * e + 1]);
                                acc[4 * e + 2] = fmaf(part[e].z, w, acc[4 * e + 2]);
                                acc[4 * e + 3] = fmaf(part[e].w, w, acc[4 * e + 3]);
                            }
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 64; e += 8) {
                        float w8[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) w8[i] = acc[e + i] * inv;
                        Packet<__nv_bfloat16>::store(dst + c0 + e, w8);
                    }
                }
            }
        }
        if (!ok) {
            abort_flag = 1;
            atomicExch(p.error, 30);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
}

}  // namespace

// 1 if this kernel takes the sizes (else the caller uses the mma.sync kernel).
TB_EXPORT int tb_attention_tcgen05_supported(int num_heads, int num_kv_heads, int head_dim, int page_size) {
    if (head_dim != 64 && head_dim != 128) return 0;
    if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return 0;
    if (page_size < 8 || (page_size & (page_size - 1)) != 0) return 0;
    return 1;
}

namespace {

template <int D, int BN>
int launch_attention(const void* cache, int cache_pages, int num_seqs, int max_rows_per_seq, int key_splits,
                     int64_t part_o_floats, int64_t part_ml_floats, int64_t counters_len, const TcAttnParams& p,
                     cudaStream_t stream) {
    const CUtensorMap* map = cache_map_for(cache, cache_pages, p.num_kv_heads, p.page_size, BN, D);
    if (map == nullptr) return TB_ERR_BAD_SIZE;
    auto kernel = key_splits > 1 ? attention_tcgen05_kernel<D, BN, true> : attention_tcgen05_kernel<D, BN, false>;
    const size_t smem = Shape<D, BN>::kSmemBytes;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    const int max_folded = max_rows_per_seq * p.group;
    dim3 grid(((max_folded + BM - 1) / BM) * p.num_kv_heads, key_splits, num_seqs);
    if (key_splits > 1) {
        const int64_t tile_ctas = (int64_t)grid.x * num_seqs;
        if (p.part_o == nullptr || p.part_ml == nullptr || p.counters == nullptr ||
            part_o_floats < tile_ctas * key_splits * BM * D || part_ml_floats < tile_ctas * key_splits * BM * 2 ||
            counters_len < tile_ctas || ((uintptr_t)p.part_o | (uintptr_t)p.part_ml) % 16 != 0)
            return TB_ERR_BAD_SIZE;
    }
    if (cudaError_t launch = tb_launch_pdl(kernel, grid, dim3(kThreads), smem, stream, *map, p)) return (int)launch;
    return tb_launch_status();
}

}  // namespace

// Attention of the sequences with more than 16 folded rows of a packed batch (the others are left to the split
// decode kernel).  Arguments as tb_attention_mma; error: device int, set non-zero if a bounded wait ran out.
// key_splits (1 to 8): CTAs per tile, each over a contiguous run of the tile's key blocks; more than one needs
// part_o (tile CTAs x key_splits x 128 x head_dim floats, 16-byte aligned; tile CTAs = ceil(max_rows_per_seq *
// group / 128) * num_kv_heads * num_seqs), part_ml (tile CTAs x key_splits x 128 x 2 floats) and counters (tile
// CTAs ints, zero before the first launch; every launch leaves them zero).  Launches that share them must be
// ordered on one stream.
TB_EXPORT int tb_attention_tcgen05(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                                   const int* row_start, const int* seq_begin, const int* block_table, int bt_stride,
                                   int num_seqs, int max_rows_per_seq, int num_heads, int num_kv_heads, int head_dim,
                                   int page_size, int cache_pages, int window, float scale, int key_splits,
                                   float* part_o, int64_t part_o_floats, float* part_ml, int64_t part_ml_floats,
                                   int* counters, int64_t counters_len, int* error, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    if (!tb_attention_tcgen05_supported(num_heads, num_kv_heads, head_dim, page_size)) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) % 16 != 0 || q_stride % 8 != 0 || out_stride % 8 != 0)
        return TB_ERR_BAD_ALIGN;
    if (num_seqs > 65535 || num_kv_heads > 65535 || key_splits < 1 || key_splits > 8) return TB_ERR_BAD_SIZE;
    TcAttnParams p;
    p.q = (const __nv_bfloat16*)q;
    p.out = (__nv_bfloat16*)out;
    p.cache = (const __nv_bfloat16*)cache;
    p.row_start = row_start;
    p.seq_begin = seq_begin;
    p.block_table = block_table;
    p.error = error;
    p.part_o = part_o;
    p.part_ml = part_ml;
    p.counters = counters;
    p.q_stride = q_stride;
    p.out_stride = out_stride;
    p.bt_stride = bt_stride;
    p.num_heads = num_heads;
    p.num_kv_heads = num_kv_heads;
    p.group = num_heads / num_kv_heads;
    p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window;
    p.scale_log2 = scale * kLog2e;
    if (head_dim == 128)
        return launch_attention<128, 64>(cache, cache_pages, num_seqs, max_rows_per_seq, key_splits, part_o_floats,
                                         part_ml_floats, counters_len, p, stream);
    return launch_attention<64, kBlockKeys64>(cache, cache_pages, num_seqs, max_rows_per_seq, key_splits, part_o_floats,
                                              part_ml_floats, counters_len, p, stream);
}
