// RMSNorm and the fused residual-add + RMSNorm.
//
//   tb_rms_norm       y = round(x * rsqrt(mean(x^2) + eps) * w)              (src/cuda/kernels.rs:26-57)
//   tb_add_rms_norm   c = res + upd (32-bit, unrounded); res_out = round(c);
//                     y = round(c * rsqrt(mean(c^2) + eps) * w)              (src/cuda/kernels.rs:59-103)
//
// Statistics and products are 32-bit; the weight is multiplied before the single
// rounding.  One block per row: a 16-byte packet per thread where the row has at most 1,024 of them (2,048
// elements of bfloat16: 1.8 us for up to 128 rows, 5.7 us for 2,048 rows, where a warp per row took 5.2 and 8.9),
// else a loop over the row; the kernel and block size are chosen from the width alone, so that a row's result
// does not depend on the batch around it.  The weight vector
// is always 32-bit (a bfloat16 checkpoint vector is widened exactly at load).
#include "common.cuh"

namespace {

// VEC: 16-byte packets (width a multiple of the packet, pointers aligned) or one element at a time.
// Which of the two runs depends on the width and the buffers' alignment only, never on the batch.
template <typename T, bool ADD, bool VEC>
__global__ void rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ upd, const float* __restrict__ w,
                                T* __restrict__ y, T* __restrict__ res_out, int width, float eps) {
    extern __shared__ __align__(16) float row_cache[];  // width floats: the (summed) row, kept between the passes
    __shared__ float scratch[32];
    const int64_t base = (int64_t)blockIdx.x * width;
    float ss = 0.0f;
    if (VEC) {
        constexpr int N = Packet<T>::N;
        for (int j = threadIdx.x * N; j < width; j += blockDim.x * N) {
            float v[N];
            Packet<T>::load(x + base + j, v);
            if (ADD) {
                float u[N];
                Packet<T>::load(upd + base + j, u);
#pragma unroll
                for (int e = 0; e < N; ++e) v[e] += u[e];
                Packet<T>::store(res_out + base + j, v);
            }
#pragma unroll
            for (int e = 0; e < N; ++e) {
                row_cache[j + e] = v[e];
                ss += v[e] * v[e];
            }
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            float v = Elem<T>::load(x + base + j);
            if (ADD) {
                v += Elem<T>::load(upd + base + j);
                Elem<T>::store(res_out + base + j, v);
            }
            row_cache[j] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    if (VEC) {
        constexpr int N = Packet<T>::N;
        for (int j = threadIdx.x * N; j < width; j += blockDim.x * N) {
            float v[N];
#pragma unroll
            for (int e = 0; e < N; ++e) v[e] = row_cache[j + e] * inv * w[j + e];
            Packet<T>::store(y + base + j, v);
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x)
            Elem<T>::store(y + base + j, row_cache[j] * inv * w[j]);
    }
}

// One block per row, a 16-byte packet per thread (rows of up to 1,024 packets): everything a thread needs (its
// packet of the row, of the update and of the weights) is asked for at once, so that a row costs one round of
// loads, a block sum and a store, and many rows per SM overlap each other's loads and stores.  The sum of squares is
// taken per thread over its packet in order, then by block_sum: an order fixed by the width alone.
template <typename T, bool ADD>
__global__ void __launch_bounds__(1024) rms_norm_block_kernel(const T* __restrict__ x, const T* __restrict__ upd,
                                                              const float* __restrict__ w, T* __restrict__ y,
                                                              T* __restrict__ res_out, int width, float eps) {
    constexpr int N = Packet<T>::N;
    __shared__ float scratch[32];
    pdl_trigger();
    const int j = (int)threadIdx.x * N;
    const bool mine = j < width;
    float wv[N];
#pragma unroll
    for (int e = 0; e < N; ++e) wv[e] = 0.0f;
    if (mine) {                                   // the weights do not depend on the kernel in front
        Packet<float>::load(w + j, wv);
        if (N == 8) Packet<float>::load(w + j + 4, wv + 4);
    }
    pdl_wait();
    const int64_t base = (int64_t)blockIdx.x * width;
    float v[N];
#pragma unroll
    for (int e = 0; e < N; ++e) v[e] = 0.0f;
    if (mine) {
        Packet<T>::load(x + base + j, v);
        if (ADD) {
            float u[N];
            Packet<T>::load(upd + base + j, u);
#pragma unroll
            for (int e = 0; e < N; ++e) v[e] += u[e];
            Packet<T>::store(res_out + base + j, v);
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < N; ++e) ss += v[e] * v[e];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    if (mine) {
#pragma unroll
        for (int e = 0; e < N; ++e) v[e] = v[e] * inv * wv[e];
        Packet<T>::store(y + base + j, v);
    }
}

template <typename T, bool ADD>
int launch_block_kernel(const void* x, const void* upd, const float* w, void* y, void* res_out, int rows, int width,
                        float eps, cudaStream_t stream) {
    const int threads = ((width / Packet<T>::N + 31) / 32) * 32;
    cudaError_t err = tb_launch_pdl(rms_norm_block_kernel<T, ADD>, dim3(rows), dim3(threads), 0, stream, (const T*)x,
                                    (const T*)upd, w, (T*)y, (T*)res_out, width, eps);
    return err == cudaSuccess ? tb_launch_status() : (int)err;
}

template <typename T, bool ADD, bool VEC>
int launch_kernel(const void* x, const void* upd, const float* w, void* y, void* res_out, int rows, int width,
                  float eps, cudaStream_t stream) {
    const size_t smem = (size_t)width * sizeof(float);
    const int per_thread = VEC ? Packet<T>::N : 4;
    int threads = 32;
    while (threads < 512 && threads * per_thread < width) threads <<= 1;
    auto kernel = rms_norm_kernel<T, ADD, VEC>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    kernel<<<rows, threads, smem, stream>>>((const T*)x, (const T*)upd, w, (T*)y, (T*)res_out, width, eps);
    return tb_launch_status();
}

template <typename T, bool ADD>
int launch(const void* x, const void* upd, const float* w, void* y, void* res_out, int rows, int width, float eps,
           cudaStream_t stream) {
    if (rows == 0) return 0;
    if ((size_t)width * sizeof(float) > 200 * 1024) return TB_ERR_BAD_SIZE;
    const uintptr_t bits = (uintptr_t)x | (uintptr_t)upd | (uintptr_t)y | (uintptr_t)res_out | (uintptr_t)w;
    const bool vec = (width % Packet<T>::N == 0) && (bits % 16 == 0);
    // which kernel runs depends on the width and the buffers' alignment only, never on the batch
    if (vec && width / Packet<T>::N <= 1024) return launch_block_kernel<T, ADD>(x, upd, w, y, res_out, rows, width, eps, stream);
    if (vec) return launch_kernel<T, ADD, true>(x, upd, w, y, res_out, rows, width, eps, stream);
    return launch_kernel<T, ADD, false>(x, upd, w, y, res_out, rows, width, eps, stream);
}

}  // namespace

TB_EXPORT int tb_rms_norm(const void* x, const float* w, void* y, int rows, int width, float eps, int dtype,
                          cudaStream_t stream) {
    if (dtype == TB_F32) return launch<float, false>(x, nullptr, w, y, nullptr, rows, width, eps, stream);
    if (dtype == TB_BF16) return launch<__nv_bfloat16, false>(x, nullptr, w, y, nullptr, rows, width, eps, stream);
    return TB_ERR_BAD_DTYPE;
}

// res_out may alias res (each element is read and written by the same thread).
TB_EXPORT int tb_add_rms_norm(const void* res, const void* upd, const float* w, void* y, void* res_out, int rows,
                              int width, float eps, int dtype, cudaStream_t stream) {
    if (dtype == TB_F32) return launch<float, true>(res, upd, w, y, res_out, rows, width, eps, stream);
    if (dtype == TB_BF16) return launch<__nv_bfloat16, true>(res, upd, w, y, res_out, rows, width, eps, stream);
    return TB_ERR_BAD_DTYPE;
}
