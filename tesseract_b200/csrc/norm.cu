// RMSNorm and the fused residual-add + RMSNorm.
//
//   tb_rms_norm       y = round(x * rsqrt(mean(x^2) + eps) * w)              (src/cuda/kernels.rs:26-57)
//   tb_add_rms_norm   c = res + upd (32-bit, unrounded); res_out = round(c);
//                     y = round(c * rsqrt(mean(c^2) + eps) * w)              (src/cuda/kernels.rs:59-103)
//
// Statistics and products are 32-bit; the weight is multiplied before the single
// rounding.  One block per row with a block size chosen from the width alone, so
// that a row's result does not depend on the batch around it.  The weight vector
// is always 32-bit (a bfloat16 checkpoint vector is widened exactly at load).
#include "common.cuh"

namespace {

template <typename T, bool ADD>
__global__ void rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ upd, const float* __restrict__ w,
                                T* __restrict__ y, T* __restrict__ res_out, int width, float eps) {
    extern __shared__ float row_cache[];  // width floats: the (summed) row, kept between the two passes
    __shared__ float scratch[32];
    const int64_t base = (int64_t)blockIdx.x * width;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float v = Elem<T>::load(x + base + j);
        if (ADD) {
            v += Elem<T>::load(upd + base + j);
            Elem<T>::store(res_out + base + j, v);
        }
        row_cache[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        Elem<T>::store(y + base + j, row_cache[j] * inv * w[j]);
}

template <typename T, bool ADD>
int launch(const void* x, const void* upd, const float* w, void* y, void* res_out, int rows, int width, float eps,
           cudaStream_t stream) {
    if (rows == 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TB_ERR_BAD_SIZE;
    int threads = 32;
    while (threads < 512 && threads * 4 < width) threads <<= 1;
    auto kernel = rms_norm_kernel<T, ADD>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    kernel<<<rows, threads, smem, stream>>>((const T*)x, (const T*)upd, w, (T*)y, (T*)res_out, width, eps);
    return tb_launch_status();
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
