// Plain paged attention: one warp per (query row, query head), keys walked in ascending
// blocks of 32 through the request's block table.  It serves the 32-bit path of every
// model and any size the fast bfloat16 kernels refuse.
//
// For row r at absolute position p of request q, head h (kv head h / group):
//   keys j in [max(0, p - window + 1), p]   (window <= 0: all keys; causal by construction)
//   s_j = (q_r . k_j) * scale ; masked lanes -1e30
//   streaming softmax per block: m' = max(m, max s); p_j = exp(s_j - m');
//   l = l*exp(m - m') + sum p ; acc = acc*exp(m - m') + sum round(p_j) * v_j
//   out = round(acc / max(l, 1e-8))
// as the reference's ragged attention does with blocks of 16 (src/cuda/kernels.rs:447-562).
// Scores, softmax state and the accumulator are 32-bit.  The order of every reduction depends
// only on (p, window, head_dim): not on the batch, the cut of the prompt, or the page ids.
#include "common.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kKeyBlock = 32;

template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <typename T, int NC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attention_rows_kernel(const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t out_stride,
                      const T* __restrict__ cache, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_row, const int* __restrict__ block_table, int bt_stride,
                      int num_heads, int num_kv_heads, int head_dim, int page_size, int window, float scale) {
    extern __shared__ float q_smem[];  // kWarpsPerBlock * head_dim
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    const int head = blockIdx.y * kWarpsPerBlock + warp;
    if (head >= num_heads) return;  // whole warp leaves together; no block-wide barrier below
    const int kv_head = head / (num_heads / num_kv_heads);
    const int pos = positions[row];
    const int seq = seq_of_row[row];
    const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    float* qs = q_smem + warp * head_dim;
    const T* qrow = q + (int64_t)row * q_stride + (int64_t)head * head_dim;
    for (int i = lane; i < head_dim; i += 32) qs[i] = Elem<T>::load(qrow + i);
    __syncwarp();

    const int64_t head_block = (int64_t)page_size * head_dim;
    const int64_t page_block = 2 * (int64_t)num_kv_heads * head_block;
    const T* kbase = cache + (int64_t)kv_head * head_block;
    const T* vbase = kbase + (int64_t)num_kv_heads * head_block;
    const int* table = block_table + (int64_t)seq * bt_stride;

    float m = -1.0e30f, l = 0.0f;
    float acc[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[c] = 0.0f;

    for (int kb = first_key / kKeyBlock; kb * kKeyBlock <= pos; ++kb) {
        const int key = kb * kKeyBlock + lane;
        const bool valid = key >= first_key && key <= pos;
        int64_t key_offset = 0;
        float s = -1.0e30f;
        if (valid) {
            const int page = table[key / page_size];
            key_offset = (int64_t)page * page_block + (int64_t)(key % page_size) * head_dim;
            const T* kp = kbase + key_offset;
            float dot = 0.0f;
            float kv[Vec16<T>::N];
            for (int i = 0; i < head_dim; i += Vec16<T>::N) {
                Vec16<T>::load(kp + i, kv);
#pragma unroll
                for (int e = 0; e < Vec16<T>::N; ++e) dot = fmaf(qs[i + e], kv[e], dot);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[c] *= corr;
        const float p_mma = Elem<T>::round(p);
        const int keys_here = min(kKeyBlock, pos - kb * kKeyBlock + 1);
        for (int j = 0; j < keys_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p_mma, j);
            const int64_t off = __shfl_sync(0xffffffffu, key_offset, j);
            if (pj != 0.0f) {  // uniform across the warp; masked keys contribute nothing
                const T* vp = vbase + off;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int col = c * 32 + lane;
                    if (col < head_dim) acc[c] = fmaf(pj, Elem<T>::load(vp + col), acc[c]);
                }
            }
        }
        m = m_new;
    }
    const float denom = fmaxf(l, 1.0e-8f);
    T* orow = out + (int64_t)row * out_stride + (int64_t)head * head_dim;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const int col = c * 32 + lane;
        if (col < head_dim) Elem<T>::store(orow + col, acc[c] / denom);
    }
}

template <typename T>
int launch(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
           const int* positions, const int* seq_of_row, const int* block_table, int bt_stride, int rows,
           int num_heads, int num_kv_heads, int head_dim, int page_size, int window, float scale,
           cudaStream_t stream) {
    dim3 grid(rows, (num_heads + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const size_t smem = (size_t)kWarpsPerBlock * head_dim * sizeof(float);
#define TB_LAUNCH(NC)                                                                                          \
    attention_rows_kernel<T, NC><<<grid, kWarpsPerBlock * 32, smem, stream>>>(                                 \
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)cache, positions, seq_of_row, block_table,       \
        bt_stride, num_heads, num_kv_heads, head_dim, page_size, window, scale)
    if (head_dim <= 32) TB_LAUNCH(1);
    else if (head_dim <= 64) TB_LAUNCH(2);
    else if (head_dim <= 128) TB_LAUNCH(4);
    else TB_LAUNCH(8);
#undef TB_LAUNCH
    return tb_launch_status();
}

}  // namespace

// q: rows x (num_heads*head_dim) with row stride q_stride (elements); out likewise.
// cache: base of the cache entry, [page][K|V][kv_head][page_size][head_dim].
// head_dim must be a multiple of 8 (16-byte key rows) and at most 256.
TB_EXPORT int tb_attention_rows(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                                const int* positions, const int* seq_of_row, const int* block_table,
                                int bt_stride, int rows, int num_heads, int num_kv_heads, int head_dim,
                                int page_size, int window, float scale, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (head_dim <= 0 || head_dim > 256 || head_dim % 8 != 0) return TB_ERR_BAD_SIZE;
    if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return TB_ERR_BAD_SIZE;
    if ((uintptr_t)cache % 16 != 0) return TB_ERR_BAD_ALIGN;
    if (dtype == TB_F32)
        return launch<float>(q, q_stride, out, out_stride, cache, positions, seq_of_row, block_table, bt_stride,
                             rows, num_heads, num_kv_heads, head_dim, page_size, window, scale, stream);
    if (dtype == TB_BF16)
        return launch<__nv_bfloat16>(q, q_stride, out, out_stride, cache, positions, seq_of_row, block_table,
                                     bt_stride, rows, num_heads, num_kv_heads, head_dim, page_size, window, scale,
                                     stream);
    return TB_ERR_BAD_DTYPE;
}
