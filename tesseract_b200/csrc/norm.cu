// RMSNorm and the fused residual-add + RMSNorm.
//
//   tb_rms_norm       y = round(x * rsqrt(mean(x^2) + eps) * w)              (src/cuda/kernels.rs:26-57)
//   tb_add_rms_norm   c = res + upd (32-bit, unrounded); res_out = round(c);
//                     y = round(c * rsqrt(mean(c^2) + eps) * w)              (src/cuda/kernels.rs:59-103)
//
// Statistics and products are 32-bit; the weight is multiplied before the single
// rounding.  One warp per row (rows of up to 8 packets per lane) or one block per row, with the
// kernel and block size chosen from the width alone, so that a row's result does not depend on the
// batch around it.  The weight vector
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

// Narrow rows (up to 8 packets per lane): one warp per row, the row stays in registers between the passes and
// no block barrier is needed; eight rows per block keep many loads in flight.  The sum of squares is taken per
// lane over its packets in order, then by the warp's shuffle tree: an order fixed by the width alone.
template <typename T, bool ADD, int PACKETS>
__global__ void __launch_bounds__(256) rms_norm_warp_kernel(const T* __restrict__ x, const T* __restrict__ upd,
                                                            const float* __restrict__ w, T* __restrict__ y,
                                                            T* __restrict__ res_out, int rows, int width, float eps) {
    constexpr int N = Packet<T>::N;
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int64_t base = (int64_t)row * width;
    float v[PACKETS][N];
#pragma unroll
    for (int k = 0; k < PACKETS; ++k) {
        const int j = (k * 32 + lane) * N;
        if (j < width) {
            Packet<T>::load(x + base + j, v[k]);
        } else {
#pragma unroll
            for (int e = 0; e < N; ++e) v[k][e] = 0.0f;
        }
    }
    if (ADD) {
#pragma unroll
        for (int k = 0; k < PACKETS; ++k) {
            const int j = (k * 32 + lane) * N;
            if (j < width) {
                float u[N];
                Packet<T>::load(upd + base + j, u);
#pragma unroll
                for (int e = 0; e < N; ++e) v[k][e] += u[e];
                Packet<T>::store(res_out + base + j, v[k]);
            }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < PACKETS; ++k)
#pragma unroll
        for (int e = 0; e < N; ++e) ss += v[k][e] * v[k][e];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int k = 0; k < PACKETS; ++k) {
        const int j = (k * 32 + lane) * N;
        if (j < width) {
            float wv[N];
            Packet<float>::load(w + j, wv);
            if (N == 8) Packet<float>::load(w + j + 4, wv + 4);
#pragma unroll
            for (int e = 0; e < N; ++e) v[k][e] = v[k][e] * inv * wv[e];
            Packet<T>::store(y + base + j, v[k]);
        }
    }
}

template <typename T, bool ADD, int PACKETS>
int launch_warp_kernel(const void* x, const void* upd, const float* w, void* y, void* res_out, int rows, int width,
                       float eps, cudaStream_t stream) {
    const int rows_per_block = 8;
    // programmatic dependent launch: the kernel behind this one may set itself up while this one runs
    cudaError_t err = tb_launch_pdl(rms_norm_warp_kernel<T, ADD, PACKETS>, dim3((rows + rows_per_block - 1) / rows_per_block),
                                    dim3(rows_per_block * 32), 0, stream, (const T*)x, (const T*)upd, w, (T*)y,
                                    (T*)res_out, rows, width, eps);
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
    if (vec) {
        // which kernel runs depends on the width and the buffers' alignment only, never on the batch
        const int packets = (width / Packet<T>::N + 31) / 32;   // per lane
        if (packets <= 1) return launch_warp_kernel<T, ADD, 1>(x, upd, w, y, res_out, rows, width, eps, stream);
        if (packets <= 2) return launch_warp_kernel<T, ADD, 2>(x, upd, w, y, res_out, rows, width, eps, stream);
        if (packets <= 4) return launch_warp_kernel<T, ADD, 4>(x, upd, w, y, res_out, rows, width, eps, stream);
        if (packets <= 8) return launch_warp_kernel<T, ADD, 8>(x, upd, w, y, res_out, rows, width, eps, stream);
    }
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
