// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] * W[N,K]^T.
//
// Plain FFMA tiles (no tensor cores, so no reduced-precision matrix mode can slip in).
// Every output element is one K-ordered chain of fused multiply-adds, k = 0, 1, ..., K-1,
// whatever M, N, the tile position or the batch: logits therefore do not depend on how a
// prompt is cut or what shares the step.  The reference runs this product through a library
// in bfloat16 only (src/cuda/cublas.rs:49-92); a 32-bit path has no counterpart there.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool VEC>
__global__ void __launch_bounds__(256)
gemm_f32_nt_kernel(const float* __restrict__ A, int64_t lda, const float* __restrict__ W, int64_t ldw,
                   float* __restrict__ C, int64_t ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;  // thread tile: rows ty*4.., cols tx*4..
    const int load_row = tid / 4;            // 0..63
    const int load_k = (tid % 4) * 4;        // 0,4,8,12

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        const int am = m0 + load_row, wn = n0 + load_row, kk = k0 + load_k;
        if (VEC) {
            if (am < M && kk < K) {
                const float4 v = *reinterpret_cast<const float4*>(A + (int64_t)am * lda + kk);
                a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
            }
            if (wn < N && kk < K) {
                const float4 v = *reinterpret_cast<const float4*>(W + (int64_t)wn * ldw + kk);
                w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (am < M && kk + e < K) a[e] = A[(int64_t)am * lda + kk + e];
                if (wn < N && kk + e < K) w[e] = W[(int64_t)wn * ldw + kk + e];
            }
        }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            As[load_k + e][load_row] = a[e];
            Ws[load_k + e][load_row] = w[e];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float ar[TM], wr[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ar[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wr[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) C[(int64_t)m * ldc + n] = acc[i][j];
        }
    }
}

}  // namespace

// Zero padding inside a K tile adds exact zeros at the end of the chain, which leaves every
// partial sum unchanged, so the guarded and the vector path give the same bits.
TB_EXPORT int tb_gemm_f32_nt(const float* A, int64_t lda, const float* W, int64_t ldw, float* C, int64_t ldc,
                             int M, int N, int K, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (K <= 0) return TB_ERR_BAD_SIZE;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return TB_ERR_BAD_SIZE;
    const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((uintptr_t)A % 16 == 0) &&
                     ((uintptr_t)W % 16 == 0);
    if (vec)
        gemm_f32_nt_kernel<true><<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
    else
        gemm_f32_nt_kernel<false><<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
    return tb_launch_status();
}
