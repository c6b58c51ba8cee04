// Rotary position encoding fused with the write of new keys and values into cache pages.
//
// For every new row t (absolute position p = positions[t]) of the packed projection
// qkv[t] = [q heads | k heads | v heads]:
//   q, k:  lo = x[0:d/2], hi = x[d/2:d];  angle_i = float(p) * inv_freq[i]
//          out_lo = round(lo*cos - hi*sin), out_hi = round(hi*cos + lo*sin)   (rotate-half)
//          (src/cuda/kernels.rs:210-242 for Q, :244-282 for K; angles as src/cuda/dense_decoder.rs:1549-1556)
//   q is rotated in place; rotated k and raw v go to the page that the request's block table
//   names for position p (K is cached after rotation, src/cuda/kernels.rs:283-337).
//
// Cache layout of one cache entry: [page][K|V][kv_head][page_size][head_dim].
// Angles, cos and sin are 32-bit with the accurate library functions.
#include "common.cuh"

namespace {

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int64_t qkv_stride, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_row, const int* __restrict__ block_table,
                                     int bt_stride, const float* __restrict__ inv_freq, T* __restrict__ cache,
                                     int num_heads, int num_kv_heads, int head_dim, int page_size, int write_kv) {
    const int row = blockIdx.x;
    const int pos = positions[row];
    const int half = head_dim >> 1;
    T* base = qkv + (int64_t)row * qkv_stride;

    int64_t page = 0;
    int offset = 0;
    if (write_kv) {
        const int seq = seq_of_row[row];
        page = block_table[(int64_t)seq * bt_stride + pos / page_size];
        offset = pos % page_size;
    }
    const int64_t head_block = (int64_t)page_size * head_dim;              // one (page, K|V, head) tile
    const int64_t page_block = 2 * (int64_t)num_kv_heads * head_block;     // one page, K and V
    T* kpage = cache + page * page_block + (int64_t)offset * head_dim;
    T* vpage = kpage + (int64_t)num_kv_heads * head_block;

    const int rot_heads = num_heads + num_kv_heads;
    const int rot_items = rot_heads * half;
    for (int item = threadIdx.x; item < rot_items; item += blockDim.x) {
        const int head = item / half;
        const int i = item - head * half;
        T* x = base + (int64_t)head * head_dim;
        const float lo = Elem<T>::load(x + i);
        const float hi = Elem<T>::load(x + half + i);
        float c = 1.0f, s = 0.0f;
        if (inv_freq != nullptr) {
            const float angle = (float)pos * inv_freq[i];
            c = cosf(angle);
            s = sinf(angle);
        }
        const float out_lo = lo * c - hi * s;
        const float out_hi = hi * c + lo * s;
        if (head < num_heads) {
            Elem<T>::store(x + i, out_lo);
            Elem<T>::store(x + half + i, out_hi);
        } else if (write_kv) {
            T* dst = kpage + (int64_t)(head - num_heads) * head_block;
            Elem<T>::store(dst + i, out_lo);
            Elem<T>::store(dst + half + i, out_hi);
        }
    }
    if (write_kv) {
        const T* v = base + (int64_t)(num_heads + num_kv_heads) * head_dim;
        const int v_items = num_kv_heads * head_dim;
        for (int item = threadIdx.x; item < v_items; item += blockDim.x) {
            const int head = item / head_dim;
            const int i = item - head * head_dim;
            vpage[(int64_t)head * head_block + i] = v[item];
        }
    }
}

}  // namespace

// cache: base of this cache entry, [num_pages][2][num_kv_heads][page_size][head_dim].
// inv_freq may be null (no rotation).  write_kv = 0 rotates q only.
TB_EXPORT int tb_rope_kv_write(void* qkv, int64_t qkv_stride, const int* positions, const int* seq_of_row,
                               const int* block_table, int bt_stride, const float* inv_freq, void* cache,
                               int rows, int num_heads, int num_kv_heads, int head_dim, int page_size,
                               int write_kv, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (head_dim <= 0 || (head_dim & 1)) return TB_ERR_BAD_SIZE;
    const int work = (num_heads + num_kv_heads) * (head_dim / 2);
    int threads = 64;
    while (threads < 512 && threads * 4 < work) threads <<= 1;
    if (dtype == TB_F32)
        rope_kv_write_kernel<float><<<rows, threads, 0, stream>>>(
            (float*)qkv, qkv_stride, positions, seq_of_row, block_table, bt_stride, inv_freq, (float*)cache,
            num_heads, num_kv_heads, head_dim, page_size, write_kv);
    else if (dtype == TB_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<rows, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, qkv_stride, positions, seq_of_row, block_table, bt_stride, inv_freq,
            (__nv_bfloat16*)cache, num_heads, num_kv_heads, head_dim, page_size, write_kv);
    else
        return TB_ERR_BAD_DTYPE;
    return tb_launch_status();
}
