// bfloat16 products over a few dozen rows (decode batches of 9..128 sequences, short prompt portions):
//
//   out[M, N] = X[M, K] . W[N, K]^T          32-bit accumulation, M <= 128
//
// At these sizes the weights are what moves: every byte of W is read once and the kernel has to keep HBM busy.
// The product is computed transposed on the fifth-generation tensor cores: 128 weight rows are the M operand of
// tcgen05.mma, the batch rows (padded to a multiple of 16) the N operand, so a CTA owns a tile of 128 output
// features for all rows and an accumulator of 128 lanes x rows columns in tensor memory.
//   * K is cut into `splits` ranges so that narrow products still give every SM work; the CTAs of a feature
//     tile form a thread-block cluster along K and add their partial tiles through distributed shared memory
//     in rank order (the sum depends on K and the split count alone, never on the batch).
//   * warp 0, one lane: TMA producer (weights 128 x 64 and activations rows x 64 per stage, 128-byte swizzle,
//     four stages; two CTAs fit an SM); warp 1, one lane: issues the products; warps 2..5: epilogue.
//   * epilogues: bfloat16 store, or SwiGLU on a weight whose rows interleave eight gate rows and their eight up
//     rows: out[m, j] = round(silu(gate_j) * up_j) on the unrounded sums (src/cuda/kernels.rs:191-208 multiplies
//     rounded projections; here one rounding fewer, as in the decode kernel).
// No copy uses cluster multicast.  Every wait is bounded: a wait that runs out sets *error, the other roles
// stop, the cluster barriers are still passed, and the CTA frees its tensor memory before it returns.
#include "tma.cuh"

namespace {

using namespace tbtma;

constexpr int BF = 128;          // features per tile (rows of W, the M of the tensor-core instruction)
constexpr int BK = 64;           // K per stage: one 128-byte swizzled row
constexpr int STAGES = 4;
constexpr int kThreads = 192;
constexpr int kMaxSplits = 8;    // the portable cluster size
constexpr uint32_t kWTileBytes = BF * BK * 2;

enum Epilogue : int { EPI_BF16 = 0, EPI_SWIGLU = 1 };

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// K-major tile of 128-byte rows with the 128-byte swizzle: 1024 bytes between groups of eight rows.
__device__ __forceinline__ uint64_t desc_k_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D = F32, A = B = BF16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
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

struct SkinnyParams {
    __nv_bfloat16* out;
    int64_t out_stride;
    int M, N, K;
    int rows_padded;      // M rounded up to a multiple of 16: the N of the tensor-core instruction
    int tmem_columns;     // power of two >= 32 and >= rows_padded
    int splits;
    int* error;
};

__device__ __forceinline__ float silu_mul(float gate, float up) { return gate * (1.0f / (1.0f + expf(-gate))) * up; }

// One output value of feature f0 + f (this thread's) and row r.  SwiGLU: features come in blocks of sixteen, eight
// gates and then their eight up projections; the gate's thread fetches the up value from eight lanes further on.
template <int EPI>
__device__ __forceinline__ void store_value(const SkinnyParams& p, int f0, int f, int r, float v) {
    if (EPI == EPI_SWIGLU) {
        const float up = __shfl_down_sync(0xffffffffu, v, 8);
        if ((f & 15) < 8 && r < p.M && f0 + f + 8 < p.N)
            p.out[(int64_t)r * p.out_stride + ((f0 + f) >> 4) * 8 + (f & 7)] = __float2bfloat16_rn(silu_mul(v, up));
    } else {
        if (r < p.M && f0 + f < p.N) p.out[(int64_t)r * p.out_stride + f0 + f] = __float2bfloat16_rn(v);
    }
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 2)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const SkinnyParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];   // the swizzled tiles need 1024-byte alignment
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * BF, split = blockIdx.y;
    const int kb_total = (p.K + BK - 1) / BK;
    const int per_split = (kb_total + p.splits - 1) / p.splits;
    const int kb0 = split * per_split;
    const int n_kb = max(0, min(kb_total, kb0 + per_split) - kb0);
    const uint32_t x_tile_bytes = (uint32_t)p.rows_padded * BK * 2;
    const uint32_t stage_bytes = kWTileBytes + x_tile_bytes;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]), done_bar = smem_u32(&bars[2 * STAGES]);
    const uint32_t tiles = smem_u32(smem);
    const bool aligned = (tiles & 1023u) == 0;                // never expected otherwise: refuse, do not compute garbage

    if (threadIdx.x == 0) {
        abort_flag = aligned ? 0 : 1;
        if (!aligned) atomicExch(p.error, 99);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(done_bar, 1);
        mbar_fence_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(p.tmem_columns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    float* part = reinterpret_cast<float*>(smem);             // [rows_padded][BF] partial sums, over the drained ring

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        for (int i = 0; i < n_kb && !abort_flag; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(empty0 + 8 * s, ((i / STAGES) & 1) ^ 1, &abort_flag)) {   // a fresh barrier passes parity 1
                abort_flag = 1;
                atomicExch(p.error, 1);
                break;
            }
            mbar_expect_tx(full0 + 8 * s, stage_bytes);
            const uint32_t dst = tiles + s * stage_bytes;
            tma_load_2d(dst, &map_w, full0 + 8 * s, (kb0 + i) * BK, f0);
            tma_load_2d(dst + kWTileBytes, &map_x, full0 + 8 * s, (kb0 + i) * BK, 0);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------------- issuer
        const uint32_t idesc = idesc_bf16(BF, p.rows_padded);
        bool ok = !abort_flag;
        for (int i = 0; i < n_kb && ok; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(full0 + 8 * s, (i / STAGES) & 1, &abort_flag)) {
                abort_flag = 1;
                atomicExch(p.error, 2);
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t w_addr = tiles + s * stage_bytes, x_addr = w_addr + kWTileBytes;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)   // 16 elements along K are 32 bytes of start address in the swizzle atom
                umma(tmem_base, desc_k_sw128(w_addr + kk * 32), desc_k_sw128(x_addr + kk * 32), idesc, (i | kk) != 0);
            umma_commit(empty0 + 8 * s);           // the stage is free once these products have read it
        }
        if (ok) umma_commit(done_bar);             // the accumulator is complete once all products are done
    } else if (warp >= 2) {
        // ---------------------------------------------------------------- epilogue: a thread per feature
        const int quarter = warp & 3;              // a warp may touch tensor-memory lanes 32 * (warp % 4) .. + 31
        const int f = quarter * 32 + lane;
        if (mbar_wait(done_bar, 0, &abort_flag)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int c = 0; c < p.rows_padded / 16; ++c) {
                uint32_t acc[16];
                tmem_load_16(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 16, acc);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int r = c * 16 + j;
                    const float v = n_kb > 0 ? __uint_as_float(acc[j]) : 0.0f;   // a split without work adds zeros
                    if (p.splits == 1) store_value<EPI>(p, f0, f, r, v);
                    else part[r * BF + f] = v;
                }
            }
        } else {
            abort_flag = 1;
            atomicExch(p.error, 3);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (p.splits > 1) {
        cluster_sync();                            // every split's partial tile is in its shared memory
        if (warp >= 2 && !abort_flag) {
            const int f = (warp & 3) * 32 + lane;
            // rows rank, rank + splits, ... of the tile, four at a time: all their loads from the peers are
            // issued before the first sum needs one (a load from a peer takes several hundred cycles)
            for (int r = (int)cluster_rank(); r < p.M; r += 4 * p.splits) {
                float v[4][kMaxSplits];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = min(r + i * p.splits, p.rows_padded - 1);
#pragma unroll
                    for (int s = 0; s < kMaxSplits; ++s)
                        if (s < p.splits) v[i][s] = ld_cluster_f32(part + row * BF + f, s);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float sum = 0.0f;
#pragma unroll
                    for (int s = 0; s < kMaxSplits; ++s)
                        if (s < p.splits) sum += v[i][s];                                        // rank order
                    if (r + i * p.splits < p.M) store_value<EPI>(p, f0, f, r + i * p.splits, sum);
                }
            }
        }
        cluster_sync();                            // no CTA leaves while a peer may still read its shared memory
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_columns) : "memory");
    }
}

// A row-major [rows, cols] bfloat16 matrix with `stride` elements between rows, cut into boxes of box_rows x 64.
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t stride, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return TB_ERR_BAD_SIZE;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {stride * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : TB_ERR_BAD_SIZE;
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

template <int EPI>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const SkinnyParams& p, size_t smem, cudaStream_t stream) {
    auto kernel = skinny_gemm_kernel<EPI>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((p.N + BF - 1) / BF, p.splits, 1);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 1;
    attribute[0].val.clusterDim.y = p.splits;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    err = cudaLaunchKernelEx(&config, kernel, map_w, map_x, p);
    return err == cudaSuccess ? tb_launch_status() : (int)err;
}

}  // namespace

// 1 if the kernel takes these sizes: at most 128 rows, K and the row strides multiples of 8 (16-byte TMA strides),
// N a multiple of 8 (16 for the SwiGLU epilogue).
TB_EXPORT int tb_skinny_gemm_supported(int M, int N, int K, int epilogue) {
    if (M < 1 || M > 128 || N < 8 || K < 8 || K % 8 != 0 || N % 8 != 0) return 0;
    if (epilogue == EPI_SWIGLU && N % 16 != 0) return 0;
    return epilogue == EPI_BF16 || epilogue == EPI_SWIGLU;
}

// How many ranges K is cut into for a product of these sizes: enough CTAs for two per SM, at least four
// 64-wide blocks each, at most a portable cluster.  A function of N and K alone.
TB_EXPORT int tb_skinny_gemm_splits(int N, int K) {
    const int tiles = (N + BF - 1) / BF, blocks = (K + BK - 1) / BK;
    int splits = 2 * sm_count() / tiles;
    if (splits > blocks / 4) splits = blocks / 4;
    if (splits > kMaxSplits) splits = kMaxSplits;
    return splits < 1 ? 1 : splits;
}

// error: device int, set non-zero if a bounded wait ran out (the result is then unusable).
// out: [M, N] bfloat16 (EPI_BF16) or [M, N / 2] (EPI_SWIGLU), out_stride in elements.
TB_EXPORT int tb_skinny_gemm(const void* x, int64_t x_stride, const void* w, int64_t w_stride, void* out,
                             int64_t out_stride, int M, int N, int K, int epilogue, int* error, cudaStream_t stream) {
    if (!tb_skinny_gemm_supported(M, N, K, epilogue)) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)x | (uintptr_t)w) % 16 != 0 || (uintptr_t)out % 2 != 0 || x_stride % 8 != 0 || w_stride % 8 != 0)
        return TB_ERR_BAD_ALIGN;
    SkinnyParams p;
    p.out = (__nv_bfloat16*)out;
    p.out_stride = out_stride;
    p.M = M;
    p.N = N;
    p.K = K;
    p.rows_padded = (M + 15) / 16 * 16;
    p.tmem_columns = p.rows_padded <= 32 ? 32 : p.rows_padded <= 64 ? 64 : 128;
    p.splits = tb_skinny_gemm_splits(N, K);
    p.error = error;
    CUtensorMap map_w, map_x;
    if (int status = make_map(&map_w, w, (uint64_t)N, (uint64_t)K, (uint64_t)w_stride, BF)) return status;
    if (int status = make_map(&map_x, x, (uint64_t)M, (uint64_t)K, (uint64_t)x_stride, (uint32_t)p.rows_padded))
        return status;
    const size_t smem = (size_t)STAGES * (kWTileBytes + (size_t)p.rows_padded * BK * 2);
    if (epilogue == EPI_SWIGLU) return launch<EPI_SWIGLU>(map_w, map_x, p, smem, stream);
    return launch<EPI_BF16>(map_w, map_x, p, smem, stream);
}
