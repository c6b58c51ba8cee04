// Row gathers and the SwiGLU activation.
//
//   tb_embedding     out[t, :] = table[token[t], :]           (src/cuda/kernels.rs:10-24)
//   tb_gather_rows   out[s, :] = in[rows[s], :]               (src/cuda/kernels.rs:774-801)
//   tb_silu_mul      out[t, j] = silu(gate[t, j]) * up[t, j]  (src/cuda/kernels.rs:191-208); gate and up lie
//                    either in the two halves of a row or interleaved in blocks of eight columns
//
// The activation is computed in 32-bit: g * (1 / (1 + exp(-g))) * u, rounded once.
#include "common.cuh"

namespace {

// Copies `row_bytes` bytes per row; 16-byte vectors when the row allows it.
template <int VEC_BYTES>
__global__ void gather_rows_kernel(const int* __restrict__ index, const char* __restrict__ src,
                                   char* __restrict__ dst, int64_t row_bytes, int num_src_rows) {
    pdl_trigger();
    pdl_wait();   // the indices (and often the rows) come from the kernel in front
    const int row = blockIdx.x;
    int from = index[row];
    if (from < 0 || from >= num_src_rows) from = 0;  // host validates; never read out of bounds
    const char* s = src + (int64_t)from * row_bytes;
    char* d = dst + (int64_t)row * row_bytes;
    if (VEC_BYTES == 16) {
        const int n = (int)(row_bytes / 16);
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
    } else {
        const int n = (int)(row_bytes / VEC_BYTES);
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            if (VEC_BYTES == 4) reinterpret_cast<uint32_t*>(d)[i] = reinterpret_cast<const uint32_t*>(s)[i];
            else reinterpret_cast<uint16_t*>(d)[i] = reinterpret_cast<const uint16_t*>(s)[i];
        }
    }
}

int gather_rows(const int* index, const void* src, void* dst, int rows, int64_t width, int num_src_rows,
                int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (dtype != TB_F32 && dtype != TB_BF16) return TB_ERR_BAD_DTYPE;
    const int64_t elem = dtype == TB_F32 ? 4 : 2;
    const int64_t row_bytes = width * elem;
    const bool aligned = (row_bytes % 16 == 0) && ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0);
    const int threads = 128;
    cudaError_t launched;
    if (aligned)
        launched = tb_launch_pdl(gather_rows_kernel<16>, dim3(rows), dim3(threads), 0, stream, index, (const char*)src,
                                 (char*)dst, row_bytes, num_src_rows);
    else if (elem == 4)
        launched = tb_launch_pdl(gather_rows_kernel<4>, dim3(rows), dim3(threads), 0, stream, index, (const char*)src,
                                 (char*)dst, row_bytes, num_src_rows);
    else
        launched = tb_launch_pdl(gather_rows_kernel<2>, dim3(rows), dim3(threads), 0, stream, index, (const char*)src,
                                 (char*)dst, row_bytes, num_src_rows);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, int64_t gu_stride,
                                int interleaved) {
    const int row = blockIdx.x;
    const T* g = gu + (int64_t)row * gu_stride;
    T* o = out + (int64_t)row * inter;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < inter; j += gridDim.y * blockDim.x) {
        const int gi = interleaved ? (j >> 3) * 16 + (j & 7) : j;
        const int ui = interleaved ? gi + 8 : inter + j;
        const float gv = Elem<T>::load(g + gi);
        const float uv = Elem<T>::load(g + ui);
        const float act = gv * (1.0f / (1.0f + expf(-gv))) * uv;
        Elem<T>::store(o + j, act);
    }
}

// bfloat16, eight elements (16 bytes) per thread and iteration.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       int inter, int64_t gu_stride, int interleaved) {
    const int row = blockIdx.x;
    const uint4* g = reinterpret_cast<const uint4*>(gu + (int64_t)row * gu_stride);
    uint4* o = reinterpret_cast<uint4*>(out + (int64_t)row * inter);
    const int packets = inter / 8;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < packets; j += gridDim.y * blockDim.x) {
        const uint4 gp = g[interleaved ? 2 * j : j], up = g[interleaved ? 2 * j + 1 : packets + j];
        const uint32_t gw[4] = {gp.x, gp.y, gp.z, gp.w}, uw[4] = {up.x, up.y, up.z, up.w};
        uint32_t ow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float g0 = __uint_as_float(gw[i] << 16), g1 = __uint_as_float(gw[i] & 0xffff0000u);
            const float u0 = __uint_as_float(uw[i] << 16), u1 = __uint_as_float(uw[i] & 0xffff0000u);
            const float a0 = g0 * (1.0f / (1.0f + expf(-g0))) * u0;
            const float a1 = g1 * (1.0f / (1.0f + expf(-g1))) * u1;
            __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1);
            ow[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        o[j] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

}  // namespace

TB_EXPORT int tb_embedding(const int* tokens, const void* table, void* out, int rows, int hidden, int vocab,
                           int dtype, cudaStream_t stream) {
    return gather_rows(tokens, table, out, rows, hidden, vocab, dtype, stream);
}

TB_EXPORT int tb_gather_rows(const int* rows_index, const void* in, void* out, int rows, int width,
                             int num_in_rows, int dtype, cudaStream_t stream) {
    return gather_rows(rows_index, in, out, rows, width, num_in_rows, dtype, stream);
}

// gu: [rows, 2*inter].  interleaved = 0: the gate in columns [0, inter), the up projection in [inter, 2*inter);
// interleaved = 1: blocks of 16 columns hold eight gates then the eight matching up projections.
TB_EXPORT int tb_silu_mul(const void* gu, void* out, int rows, int inter, int interleaved, int dtype,
                          cudaStream_t stream) {
    if (rows == 0 || inter == 0) return 0;
    if (interleaved && inter % 8 != 0) return TB_ERR_BAD_SIZE;
    const int threads = 256;
    int bx = (inter + threads - 1) / threads;
    if (bx > 64) bx = 64;
    dim3 grid(rows, bx);
    if (dtype == TB_F32)
        silu_mul_kernel<float><<<grid, threads, 0, stream>>>((const float*)gu, (float*)out, inter, 2 * (int64_t)inter,
                                                              interleaved);
    else if (dtype == TB_BF16 && inter % 8 == 0 && ((uintptr_t)gu | (uintptr_t)out) % 16 == 0) {
        int by = (inter / 8 + threads - 1) / threads;
        if (by > 64) by = 64;
        silu_mul_bf16x8_kernel<<<dim3(rows, by), threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                                                                      inter, 2 * (int64_t)inter, interleaved);
    } else if (dtype == TB_BF16)
        silu_mul_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                                                                    inter, 2 * (int64_t)inter, interleaved);
    else
        return TB_ERR_BAD_DTYPE;
    return tb_launch_status();
}

namespace {

// out[i] = feed[i] >= 0 ? previous[feed[i]] : tokens[i]: a decode step takes the token of a sequence either from
// the host (its first decoded token) or straight from the row of the previous step's sampler output.
__global__ void select_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ feed,
                                     const int* __restrict__ previous, int* __restrict__ out, int n, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int token = tokens[i];
    const int from = feed[i];
    if (from >= 0) token = previous[from];
    out[i] = (token >= 0 && token < vocab) ? token : 0;   // never index the embedding table out of range
}

}  // namespace

TB_EXPORT int tb_select_tokens(const int* tokens, const int* feed, const int* previous, int* out, int n, int vocab,
                               cudaStream_t stream) {
    if (n <= 0) return 0;
    cudaError_t launched = tb_launch_pdl(select_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, feed,
                                         previous, out, n, vocab);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
