// Skinny matrix products for decode steps (at most 16 rows), bfloat16 weights streamed once from HBM.
//
//   y[M, N] = X[M, K] . W[N, K]^T          with M <= 16, 32-bit accumulation
//
// with, fused in front, the residual addition and RMSNorm that produce X
//   c = res + upd (32-bit, unrounded); res_out = round(c); X = round(c * rsqrt(mean(c^2) + eps) * w)
//   (src/cuda/kernels.rs:59-103), or the plain RMSNorm of res (src/cuda/kernels.rs:26-57),
// and, fused behind, either a plain store (bfloat16 or 32-bit) or the SwiGLU activation
//   out[m, j] = round(silu(gate_j) * up_j)   (src/cuda/kernels.rs:191-208), for a weight whose rows
// interleave gate and up in blocks of eight: rows 16b..16b+7 = gate 8b..8b+7, rows 16b+8..16b+15 = up 8b..8b+7.
//
// Why not the library: at these sizes a decode layer is a chain of launches of a few microseconds
// each, and the norm and activation kernels between the products cost as much as the products.
// One CTA owns 16 output features; its 8 warps split K, each streaming its slice of the 16 weight
// rows straight from global memory into mma.sync.m16n8k16 A fragments (weights are the 16-row
// operand, the batch rows the 8-column operand), and are summed in a fixed order in shared memory.
// Each lane loads 16 contiguous bytes per weight row and 32-wide K block; the products pair weight
// and activation elements in the same permuted K order, so no shuffle or shared-memory transpose is
// needed.  The reduction order depends on K alone.
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

enum Prologue : int { PRO_NONE = 0, PRO_NORM = 1, PRO_ADD_NORM = 2 };
enum Epilogue : int { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_F32 = 2 };

struct LinearParams {
    const __nv_bfloat16* x;        // PRO_NONE: [M, K] activations (row stride x_stride)
    const __nv_bfloat16* res;      // PRO_*: residual rows [M, K]
    const __nv_bfloat16* upd;      // PRO_ADD_NORM: pending update [M, K]
    const float* norm_w;           // PRO_*: [K]
    __nv_bfloat16* res_out;        // PRO_ADD_NORM: round(res + upd), written by CTA 0; must not alias res
    const __nv_bfloat16* w;        // [N, K]
    void* out;                     // [M, N] (EPI_SWIGLU: [M, N/2])
    int64_t x_stride, out_stride;
    int M, N, K;
    float eps;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;  // weights are read once: do not keep them in L1
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// MT: number of 8-row batch tiles (1 or 2).
template <int MT, int PRO, int EPI>
__global__ void __launch_bounds__(kThreads) decode_linear_kernel(const LinearParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int K = p.K;
    constexpr int ROWS = 8 * MT;

    // shared memory: [ROWS][K + 32] bf16 normalised activations (PRO only), then the warps' partial sums
    const int x_pitch = K + 32;  // 64 bytes of padding: the eight rows a quarter-warp reads hit distinct banks
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);
    float* partial = reinterpret_cast<float*>(smem + (PRO != PRO_NONE ? (size_t)ROWS * x_pitch * 2 : 0));

    if (PRO != PRO_NONE) {
        // every CTA normalises the (few) rows itself; CTA 0 also stores the new residual
        for (int row = warp; row < ROWS; row += kWarps) {
            __nv_bfloat16* dst = xs + (size_t)row * x_pitch;
            if (row >= p.M) {
                for (int j = lane * 8; j < K; j += 256) *reinterpret_cast<uint4*>(dst + j) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const __nv_bfloat16* r = p.res + (int64_t)row * K;
            const __nv_bfloat16* u = PRO == PRO_ADD_NORM ? p.upd + (int64_t)row * K : nullptr;
            float ss = 0.0f;
            for (int j = lane * 8; j < K; j += 256) {
                float v[8];
                Packet<__nv_bfloat16>::load(r + j, v);
                if (PRO == PRO_ADD_NORM) {
                    float a[8];
                    Packet<__nv_bfloat16>::load(u + j, a);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] += a[e];
                    if (blockIdx.x == 0) Packet<__nv_bfloat16>::store(p.res_out + (int64_t)row * K + j, v);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
            }
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)K + p.eps);
            for (int j = lane * 8; j < K; j += 256) {
                float v[8];
                Packet<__nv_bfloat16>::load(r + j, v);
                if (PRO == PRO_ADD_NORM) {
                    float a[8];
                    Packet<__nv_bfloat16>::load(u + j, a);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] += a[e];
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = v[e] * inv * p.norm_w[j + e];
                Packet<__nv_bfloat16>::store(dst + j, v);
            }
        }
        __syncthreads();
    }

    // K is cut into 32-wide blocks; warp w takes blocks w, w + 8, ...  (fixed by K alone)
    const int blocks = K / 32;
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.0f;
    const __nv_bfloat16* w_lo = p.w + (int64_t)(n0 + g) * K + 8 * t;
    const __nv_bfloat16* w_hi = w_lo + (int64_t)8 * K;

    constexpr int UNROLL = 4;
    for (int b0 = warp; b0 < blocks; b0 += kWarps * UNROLL) {
        uint4 wa[UNROLL], wb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int b = b0 + u * kWarps;
            if (b < blocks) {
                wa[u] = ldg_stream(w_lo + b * 32);
                wb[u] = ldg_stream(w_hi + b * 32);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int b = b0 + u * kWarps;
            if (b >= blocks) break;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint4 xb;
                const int row = mt * 8 + g;
                if (PRO != PRO_NONE) {
                    xb = *reinterpret_cast<const uint4*>(xs + (size_t)row * x_pitch + b * 32 + 8 * t);
                } else if (row < p.M) {
                    xb = *reinterpret_cast<const uint4*>(p.x + (int64_t)row * p.x_stride + b * 32 + 8 * t);
                } else {
                    xb = make_uint4(0, 0, 0, 0);
                }
                mma_bf16(acc[mt], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xb.x, xb.y);
                mma_bf16(acc[mt], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xb.z, xb.w);
            }
        }
    }

    // sum the warps in a fixed order: partial[warp][feature 0..15][batch row 0..ROWS-1]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        float* dst = partial + (size_t)warp * 16 * ROWS;
        dst[g * ROWS + mt * 8 + 2 * t] = acc[mt][0];
        dst[g * ROWS + mt * 8 + 2 * t + 1] = acc[mt][1];
        dst[(g + 8) * ROWS + mt * 8 + 2 * t] = acc[mt][2];
        dst[(g + 8) * ROWS + mt * 8 + 2 * t + 1] = acc[mt][3];
    }
    __syncthreads();
    if (EPI == EPI_SWIGLU) {
        // features 0..7 are gates, 8..15 the matching up projections
        for (int idx = threadIdx.x; idx < 8 * ROWS; idx += kThreads) {
            const int f = idx / ROWS, m = idx - f * ROWS;
            if (m >= p.M) continue;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                gate += partial[(size_t)w * 16 * ROWS + f * ROWS + m];
                up += partial[(size_t)w * 16 * ROWS + (f + 8) * ROWS + m];
            }
            const float act = gate * (1.0f / (1.0f + expf(-gate))) * up;
            reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)m * p.out_stride + blockIdx.x * 8 + f] =
                __float2bfloat16_rn(act);
        }
    } else {
        for (int idx = threadIdx.x; idx < 16 * ROWS; idx += kThreads) {
            const int m = idx / 16, f = idx - m * 16;  // consecutive threads write consecutive features
            if (m >= p.M) continue;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) sum += partial[(size_t)w * 16 * ROWS + f * ROWS + m];
            if (EPI == EPI_F32)
                reinterpret_cast<float*>(p.out)[(int64_t)m * p.out_stride + n0 + f] = sum;
            else
                reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)m * p.out_stride + n0 + f] = __float2bfloat16_rn(sum);
        }
    }
}

template <int MT, int PRO, int EPI>
int launch(const LinearParams& p, cudaStream_t stream) {
    constexpr int ROWS = 8 * MT;
    size_t smem = (size_t)kWarps * 16 * ROWS * sizeof(float);
    if (PRO != PRO_NONE) smem += (size_t)ROWS * (p.K + 32) * 2;
    auto kernel = decode_linear_kernel<MT, PRO, EPI>;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return TB_ERR_BAD_SIZE;
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    kernel<<<p.N / 16, kThreads, smem, stream>>>(p);
    return tb_launch_status();
}

template <int MT>
int dispatch(const LinearParams& p, int prologue, int epilogue, cudaStream_t stream) {
#define TB_CASE(PRO, EPI) \
    if (prologue == PRO && epilogue == EPI) return launch<MT, PRO, EPI>(p, stream);
    TB_CASE(PRO_NONE, EPI_BF16)
    TB_CASE(PRO_NONE, EPI_F32)
    TB_CASE(PRO_NONE, EPI_SWIGLU)
    TB_CASE(PRO_NORM, EPI_BF16)
    TB_CASE(PRO_NORM, EPI_F32)
    TB_CASE(PRO_NORM, EPI_SWIGLU)
    TB_CASE(PRO_ADD_NORM, EPI_BF16)
    TB_CASE(PRO_ADD_NORM, EPI_F32)
    TB_CASE(PRO_ADD_NORM, EPI_SWIGLU)
#undef TB_CASE
    return TB_ERR_BAD_SIZE;
}

}  // namespace

// 1 if the sizes are ones this kernel takes, else 0 (the caller then uses the general path).
TB_EXPORT int tb_decode_linear_supported(int M, int N, int K, int prologue) {
    if (M < 1 || M > 16 || N < 16 || N % 16 != 0 || K < 32 || K % 32 != 0) return 0;
    if (prologue != PRO_NONE && (size_t)(M <= 8 ? 8 : 16) * (K + 32) * 2 > 160 * 1024) return 0;
    return 1;
}

// x: PRO_NONE only.  res/upd/norm_w/res_out: see LinearParams.  out_stride in elements of the output type.
TB_EXPORT int tb_decode_linear(const void* x, int64_t x_stride, const void* res, const void* upd,
                               const float* norm_w, float eps, void* res_out, const void* w, void* out,
                               int64_t out_stride, int M, int N, int K, int prologue, int epilogue,
                               cudaStream_t stream) {
    if (!tb_decode_linear_supported(M, N, K, prologue)) return TB_ERR_BAD_SIZE;
    const uintptr_t bits = (uintptr_t)x | (uintptr_t)res | (uintptr_t)upd | (uintptr_t)res_out | (uintptr_t)w;
    if (bits % 16 != 0 || (prologue == PRO_NONE && x_stride % 8 != 0)) return TB_ERR_BAD_ALIGN;
    if (prologue == PRO_ADD_NORM && (res_out == nullptr || res_out == res)) return TB_ERR_BAD_ALIGN;
    LinearParams p;
    p.x = (const __nv_bfloat16*)x;
    p.res = (const __nv_bfloat16*)res;
    p.upd = (const __nv_bfloat16*)upd;
    p.norm_w = norm_w;
    p.res_out = (__nv_bfloat16*)res_out;
    p.w = (const __nv_bfloat16*)w;
    p.out = out;
    p.x_stride = x_stride;
    p.out_stride = out_stride;
    p.M = M;
    p.N = N;
    p.K = K;
    p.eps = eps;
    return M <= 8 ? dispatch<1>(p, prologue, epilogue, stream) : dispatch<2>(p, prologue, epilogue, stream);
}
