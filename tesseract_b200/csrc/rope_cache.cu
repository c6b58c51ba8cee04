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

template <typename T, bool VEC>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int64_t qkv_stride, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_row, const int* __restrict__ block_table,
                                     int bt_stride, const float* __restrict__ inv_freq, T* __restrict__ cache,
                                     int num_heads, int num_kv_heads, int head_dim, int page_size, int write_kv) {
    extern __shared__ float trig[];  // cos[half] then sin[half] of this row's angles, shared by all heads
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int pos = positions[row];
    const int half = head_dim >> 1;
    T* base = qkv + (int64_t)row * qkv_stride;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float c = 1.0f, s = 0.0f;
        if (inv_freq != nullptr) {
            const float angle = (float)pos * inv_freq[i];
            sincosf(angle, &s, &c);
        }
        trig[i] = c;
        trig[half + i] = s;
    }
    __syncthreads();

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

    constexpr int N = VEC ? Packet<T>::N : 1;
    const int rot_heads = num_heads + num_kv_heads;
    const int per_head = half / N;
    const int rot_items = rot_heads * per_head;
    for (int item = threadIdx.x; item < rot_items; item += blockDim.x) {
        const int head = item / per_head;
        const int i = (item - head * per_head) * N;
        T* x = base + (int64_t)head * head_dim;
        float lo[N], hi[N], out_lo[N], out_hi[N];
        if (VEC) {
            Packet<T>::load(x + i, lo);
            Packet<T>::load(x + half + i, hi);
        } else {
            lo[0] = Elem<T>::load(x + i);
            hi[0] = Elem<T>::load(x + half + i);
        }
#pragma unroll
        for (int e = 0; e < N; ++e) {
            const float c = trig[i + e], s = trig[half + i + e];
            out_lo[e] = lo[e] * c - hi[e] * s;
            out_hi[e] = hi[e] * c + lo[e] * s;
        }
        T* dst = nullptr;
        if (head < num_heads) dst = x;
        else if (write_kv) dst = kpage + (int64_t)(head - num_heads) * head_block;
        if (dst != nullptr) {
            if (VEC) {
                Packet<T>::store(dst + i, out_lo);
                Packet<T>::store(dst + half + i, out_hi);
            } else {
                Elem<T>::store(dst + i, out_lo[0]);
                Elem<T>::store(dst + half + i, out_hi[0]);
            }
        }
    }
    if (write_kv) {
        const T* v = base + (int64_t)(num_heads + num_kv_heads) * head_dim;
        if (VEC) {
            const int per = head_dim / N;
            for (int item = threadIdx.x; item < num_kv_heads * per; item += blockDim.x) {
                const int head = item / per;
                const int i = (item - head * per) * N;
                *reinterpret_cast<uint4*>(vpage + (int64_t)head * head_block + i) =
                    *reinterpret_cast<const uint4*>(v + (int64_t)head * head_dim + i);
            }
        } else {
            const int v_items = num_kv_heads * head_dim;
            for (int item = threadIdx.x; item < v_items; item += blockDim.x) {
                const int head = item / head_dim;
                const int i = item - head * head_dim;
                vpage[(int64_t)head * head_block + i] = v[item];
            }
        }
    }
}

// The same for rows whose work fits two 16-byte items per thread (every Llama size): a thread asks for its
// packets of q, k and v, the row's position and its page before anything is computed, so that one round of loads
// covers the row (the loop above waits for the position, the angles, the page and the data one after the other:
// 11 us for 2,048 rows of the 1B sizes against 6).  The arithmetic and its order are the loop's.
constexpr int kItemsPerThread = 2;
template <typename T>
__global__ void rope_kv_write_preload_kernel(T* __restrict__ qkv, int64_t qkv_stride, const int* __restrict__ positions,
                                             const int* __restrict__ seq_of_row, const int* __restrict__ block_table,
                                             int bt_stride, const float* __restrict__ inv_freq, T* __restrict__ cache,
                                             int num_heads, int num_kv_heads, int head_dim, int page_size,
                                             int write_kv) {
    extern __shared__ float trig[];  // cos[half] then sin[half] of this row's angles, shared by all heads
    constexpr int N = Packet<T>::N;
    pdl_trigger();
    const int half = head_dim >> 1;
    float freq = 0.0f;
    if (inv_freq != nullptr && (int)threadIdx.x < half) freq = inv_freq[threadIdx.x];   // (does not depend on the kernel in front)
    pdl_wait();
    const int row = blockIdx.x;
    const int pos = positions[row];
    const int seq = write_kv ? seq_of_row[row] : 0;
    T* base = qkv + (int64_t)row * qkv_stride;
    const int rot_heads = num_heads + num_kv_heads;
    const int per_head = half / N;
    const int rot_items = rot_heads * per_head;
    const int v_per = head_dim / N;
    const int v_items = write_kv ? num_kv_heads * v_per : 0;
    const T* v = base + (int64_t)rot_heads * head_dim;
    uint4 lo[kItemsPerThread], hi[kItemsPerThread];       // as loaded: converted when they are rotated
    uint4 v_packet[kItemsPerThread];
#pragma unroll
    for (int k = 0; k < kItemsPerThread; ++k) {
        const int item = (int)threadIdx.x + k * (int)blockDim.x;
        if (item < rot_items) {
            const int head = item / per_head;
            const int i = (item - head * per_head) * N;
            lo[k] = *reinterpret_cast<const uint4*>(base + (int64_t)head * head_dim + i);
            hi[k] = *reinterpret_cast<const uint4*>(base + (int64_t)head * head_dim + half + i);
        }
        if (item < v_items) {
            const int head = item / v_per;
            v_packet[k] = *reinterpret_cast<const uint4*>(v + (int64_t)head * head_dim + (item - head * v_per) * N);
        }
    }
    const int64_t page = write_kv ? block_table[(int64_t)seq * bt_stride + pos / page_size] : 0;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float c = 1.0f, s = 0.0f;
        if (inv_freq != nullptr) {
            const float angle = (float)pos * (i == (int)threadIdx.x ? freq : inv_freq[i]);
            sincosf(angle, &s, &c);
        }
        trig[i] = c;
        trig[half + i] = s;
    }
    __syncthreads();
    const int offset = pos % page_size;
    const int64_t head_block = (int64_t)page_size * head_dim;              // one (page, K|V, head) tile
    const int64_t page_block = 2 * (int64_t)num_kv_heads * head_block;     // one page, K and V
    T* kpage = cache + page * page_block + (int64_t)offset * head_dim;
    T* vpage = kpage + (int64_t)num_kv_heads * head_block;
#pragma unroll
    for (int k = 0; k < kItemsPerThread; ++k) {
        const int item = (int)threadIdx.x + k * (int)blockDim.x;
        if (item < rot_items) {
            const int head = item / per_head;
            const int i = (item - head * per_head) * N;
            float in_lo[N], in_hi[N], out_lo[N], out_hi[N];
            Packet<T>::unpack(lo[k], in_lo);
            Packet<T>::unpack(hi[k], in_hi);
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float c = trig[i + e], s = trig[half + i + e];
                out_lo[e] = in_lo[e] * c - in_hi[e] * s;
                out_hi[e] = in_hi[e] * c + in_lo[e] * s;
            }
            T* dst = nullptr;
            if (head < num_heads) dst = base + (int64_t)head * head_dim;
            else if (write_kv) dst = kpage + (int64_t)(head - num_heads) * head_block;
            if (dst != nullptr) {
                Packet<T>::store(dst + i, out_lo);
                Packet<T>::store(dst + half + i, out_hi);
            }
        }
        if (item < v_items) {
            const int head = item / v_per;
            *reinterpret_cast<uint4*>(vpage + (int64_t)head * head_block + (item - head * v_per) * N) = v_packet[k];
        }
    }
}

template <typename T>
int launch(void* qkv, int64_t qkv_stride, const int* positions, const int* seq_of_row, const int* block_table,
           int bt_stride, const float* inv_freq, void* cache, int rows, int num_heads, int num_kv_heads, int head_dim,
           int page_size, int write_kv, cudaStream_t stream) {
    const int half = head_dim / 2;
    const bool vec = (half % Packet<T>::N == 0) && (qkv_stride % Packet<T>::N == 0) &&
                     (((uintptr_t)qkv | (uintptr_t)cache) % 16 == 0);
    const int work = (num_heads + num_kv_heads) * (vec ? half / Packet<T>::N : half);
    int threads = 32;
    while (threads < 128 && threads < work) threads <<= 1;   // small blocks: many rows in flight per SM
    const size_t smem = (size_t)head_dim * sizeof(float);
    cudaError_t err;
    const int v_work = write_kv ? num_kv_heads * (head_dim / Packet<T>::N) : 0;
    const int most = work > v_work ? work : v_work;
    if (vec && most <= kItemsPerThread * 512) {
        // (which kernel runs depends on the sizes alone; both do the same arithmetic in the same order)
        const int few = ((most + kItemsPerThread - 1) / kItemsPerThread + 31) / 32 * 32;
        err = tb_launch_pdl(rope_kv_write_preload_kernel<T>, dim3(rows), dim3(few), smem, stream, (T*)qkv, qkv_stride,
                            positions, seq_of_row, block_table, bt_stride, inv_freq, (T*)cache, num_heads,
                            num_kv_heads, head_dim, page_size, write_kv);
        return err == cudaSuccess ? tb_launch_status() : (int)err;
    }
    if (vec)
        err = tb_launch_pdl(rope_kv_write_kernel<T, true>, dim3(rows), dim3(threads), smem, stream, (T*)qkv, qkv_stride,
                            positions, seq_of_row, block_table, bt_stride, inv_freq, (T*)cache, num_heads,
                            num_kv_heads, head_dim, page_size, write_kv);
    else
        err = tb_launch_pdl(rope_kv_write_kernel<T, false>, dim3(rows), dim3(threads), smem, stream, (T*)qkv,
                            qkv_stride, positions, seq_of_row, block_table, bt_stride, inv_freq, (T*)cache, num_heads,
                            num_kv_heads, head_dim, page_size, write_kv);
    return err == cudaSuccess ? tb_launch_status() : (int)err;
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
    if (dtype == TB_F32)
        return launch<float>(qkv, qkv_stride, positions, seq_of_row, block_table, bt_stride, inv_freq, cache, rows,
                             num_heads, num_kv_heads, head_dim, page_size, write_kv, stream);
    if (dtype == TB_BF16)
        return launch<__nv_bfloat16>(qkv, qkv_stride, positions, seq_of_row, block_table, bt_stride, inv_freq, cache,
                                     rows, num_heads, num_kv_heads, head_dim, page_size, write_kv, stream);
    return TB_ERR_BAD_DTYPE;
}
