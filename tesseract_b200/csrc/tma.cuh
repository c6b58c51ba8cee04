// Bulk tensor copies (TMA) and mbarriers, shared by the kernels that stream cache pages.
//
// A cache entry [pages][K|V][kv_heads][page_size][head_dim] (bfloat16, head_dim a multiple of 64) is described to the TMA unit
// once by a five-dimensional tensor map; a copy then brings min(page_size, max_rows) consecutive keys of one page
// and one head into shared memory as rows of 128 bytes with the 128-byte swizzle (16-byte chunk index XOR row
// mod 8), the layout that both ldmatrix-fed mma.sync tiles and tcgen05 matrix descriptors read.  No copy uses
// cluster multicast.  Every wait on an mbarrier is bounded.
#pragma once

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace tbtma {

constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// False if the barrier did not flip within the limit, or another thread of the CTA has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255) == 255 && *abort_flag) return false;
    }
    return false;
}

// One box of the cache tensor: dims dim0..dim0+63 (dim0 a multiple of 64, so the copy starts on a 16-byte boundary)
// of keys key_in_page.. of `page`, head `kv_head`, K (which = 0) or V (which = 1).
__device__ __forceinline__ void tma_load_kv(uint32_t dst, const CUtensorMap* map, uint32_t bar, int dim0,
                                            int key_in_page, int kv_head, int which, int page) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(dim0), "r"(key_in_page), "r"(kv_head), "r"(which), "r"(page) : "memory");
}

// One box of a two-dimensional tensor map at element coordinates (c0 along the rows, c1 = the row).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

// The same from a CTA of a pair (cta_group::2): the bytes are counted on `bar`, a shared::cluster address that may lie
// in the other CTA of the pair (the even CTA's barrier, which its issuing thread waits on).  No multicast: each CTA
// brings its own boxes into its own shared memory.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Cluster helpers: this CTA's rank, the shared::cluster address of `local` in CTA `rank`, an arrival on a barrier
// there, and the barrier of all threads of the cluster.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_shared_address(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_barrier_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// A row-major [rows, cols] bfloat16 matrix with `stride` elements between rows, cut into boxes of box_rows rows of
// 64 elements (128 bytes, stored with the 128-byte swizzle).  Rows and columns beyond the matrix read as zero.
// The base address and the stride in bytes must be multiples of 16.
inline int make_map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t stride,
                       uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return TB_ERR_BAD_SIZE;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {stride * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : TB_ERR_BAD_SIZE;
}

// The same, kept per (pointer, geometry): encoding a map costs the host a couple of microseconds, a step launched
// kernel by kernel makes hundreds, and weights (and, through the caching allocator, most activations) come back
// at the same addresses.  A map depends on nothing but the key, so an entry can never go stale; the table is
// emptied when it has grown to 4,096 entries.  The pointer stays valid until the next call from the same thread.
inline const CUtensorMap* cached_map_2d(const void* base, uint64_t rows, uint64_t cols, uint64_t stride,
                                        uint32_t box_rows) {
    static std::mutex lock;
    static std::map<std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t>, CUtensorMap> maps;
    thread_local CUtensorMap mine;
    std::lock_guard<std::mutex> guard(lock);
    const auto key = std::make_tuple(base, rows, cols, stride, box_rows);
    auto found = maps.find(key);
    if (found == maps.end()) {
        CUtensorMap map;
        if (make_map_2d(&map, base, rows, cols, stride, box_rows) != 0) return nullptr;
        if (maps.size() >= 4096) maps.clear();
        found = maps.emplace(key, map).first;
    }
    mine = found->second;
    return &mine;
}

// Tensor map of one cache entry [pages][K|V][kv head][key][head_dim] (head_dim a multiple of 64), boxes of 64 dims
// of min(page_size, max_rows) keys of one head.  Maps are kept per (pointer, geometry): a cache entry lives as long
// as its model.
inline const CUtensorMap* cache_map_for(const void* cache, int pages, int num_kv_heads, int page_size, int max_rows,
                                        int head_dim) {
    static std::mutex lock;
    static std::map<std::tuple<const void*, int, int, int, int, int>, CUtensorMap> maps;
    std::lock_guard<std::mutex> guard(lock);
    const auto key = std::make_tuple(cache, pages, num_kv_heads, page_size, max_rows, head_dim);
    auto found = maps.find(key);
    if (found != maps.end()) return &found->second;
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return nullptr;
    CUtensorMap map;
    const cuuint64_t dims[5] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)num_kv_heads, 2,
                                (cuuint64_t)pages};
    const cuuint64_t row = (cuuint64_t)head_dim * 2;
    const cuuint64_t strides[4] = {row, row * page_size, row * page_size * num_kv_heads,
                                   row * page_size * num_kv_heads * 2};
    const cuuint32_t box[5] = {64, (cuuint32_t)(page_size < max_rows ? page_size : max_rows), 1, 1, 1};
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return nullptr;
    return &maps.emplace(key, map).first->second;
}

}  // namespace tbtma
