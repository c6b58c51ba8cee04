// The allocation-free variant of the split decode attention: same kernels as attention_mma.cu,
// with the per-split partial results in a static device array instead of caller-supplied buffers.
// See attention_noalloc.h for who this is for, the size limit and the rules of use.
#include "attention_mma.cu"
#include "attention_noalloc.h"

namespace {

// Part of the library image: present on every GPU that loads this library, until the process exits.
static __device__ __align__(256) float g_noalloc_scratch[TB_NOALLOC_SCRATCH_FLOATS];
// Arrival counters of the splits, one per (sequence, kv head).  Zero at load; every call leaves them zero.
static __device__ __align__(256) int g_noalloc_counters[TB_NOALLOC_COUNTERS];

constexpr int kMaxDevices = 64;
// Device address of the array, per device.  In host code the name g_noalloc_scratch is only a handle
// for the runtime, not an address a kernel may use, so the address is asked for once per device.
float* g_scratch_address[kMaxDevices] = {};
int* g_counter_address[kMaxDevices] = {};

int scratch_for_current_device(float** ptr, int** counters) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return (int)err;
    if (device < 0 || device >= kMaxDevices) return TB_ERR_BAD_SIZE;
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, g_noalloc_scratch);
        if (err != cudaSuccess) return (int)err;
        void* counter_address = nullptr;
        err = cudaGetSymbolAddress(&counter_address, g_noalloc_counters);
        if (err != cudaSuccess) return (int)err;
        g_counter_address[device] = static_cast<int*>(counter_address);
        g_scratch_address[device] = static_cast<float*>(address);
    }
    *ptr = g_scratch_address[device];
    *counters = g_counter_address[device];
    return 0;
}

int64_t round_up_64(int64_t n) { return (n + 63) / 64 * 64; }

}  // namespace

TB_EXPORT int64_t tb_attention_noalloc_floats_needed(int splits, int num_seqs, int num_kv_heads, int head_dim) {
    const int padded = tb_attention_mma_padded_dim(head_dim);
    if (padded < 0) return padded;
    if (num_seqs < 0 || num_kv_heads <= 0) return TB_ERR_BAD_SIZE;
    if (splits <= kMaxClusterSplits) return 0;   // these meet in a thread-block cluster and never touch the array
    const int64_t slots = (int64_t)splits * num_seqs * num_kv_heads * 16;
    return round_up_64(slots * padded) + slots * 2;
}

TB_EXPORT const char* tb_attention_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "success";
        case TB_ERR_BAD_DTYPE: return "unsupported dtype";
        case TB_ERR_BAD_SIZE: return "unsupported size (head_dim must be a multiple of 16 up to 256, page_size a "
                                     "power of two, num_heads a multiple of num_kv_heads)";
        case TB_ERR_BAD_ALIGN: return "q, out and cache must be 16-byte aligned and q_stride a multiple of 8";
        case TB_NOALLOC_TOO_LARGE: return "with more than 8 splits the call needs more than the 16 MiB static scratch "
                                          "array (splits * num_seqs * num_kv_heads * 16 * (padded_head_dim + 2) "
                                          "floats) or more than 16384 (sequence, kv head) pairs; use at most 8 "
                                          "splits (which need no scratch), fewer sequences, or the entry point "
                                          "that takes scratch buffers";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown refusal code";
    }
}

TB_EXPORT int tb_attention_decode_noalloc(const void* q, int64_t q_stride, void* out, int64_t out_stride,
                                          const void* cache, const int* row_start, const int* seq_begin,
                                          const int* block_table, int bt_stride, int num_seqs, int total_rows,
                                          int max_rows_per_seq, int num_heads, int num_kv_heads, int head_dim,
                                          int page_size, int window, float scale, int splits, cudaStream_t stream) {
    if (splits < 1) splits = 1;
    const int64_t need = tb_attention_noalloc_floats_needed(splits, num_seqs, num_kv_heads, head_dim);
    if (need < 0) return (int)need;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    int* counters = nullptr;
    int64_t part_o_floats = 0;
    if (splits > kMaxClusterSplits) {      // only these use the array and the counters; the limits are theirs alone
        if (need > (int64_t)TB_NOALLOC_SCRATCH_FLOATS) return TB_NOALLOC_TOO_LARGE;
        if ((int64_t)num_seqs * num_kv_heads > (int64_t)TB_NOALLOC_COUNTERS) return TB_NOALLOC_TOO_LARGE;
        float* scratch = nullptr;
        if (int status = scratch_for_current_device(&scratch, &counters)) return status;
        const int padded = tb_attention_mma_padded_dim(head_dim);
        part_o_floats = round_up_64((int64_t)splits * num_seqs * num_kv_heads * 16 * padded);
        part_o = scratch;
        part_ml = scratch + part_o_floats;
    }
    return tb_attention_mma(q, q_stride, out, out_stride, cache, row_start, seq_begin, block_table, bt_stride,
                            num_seqs, total_rows, max_rows_per_seq, num_heads, num_kv_heads, head_dim, page_size,
                            window, scale, /*run_tiles=*/0, /*run_decode=*/1, splits, part_o, part_ml, part_o_floats,
                            counters, stream);
}
