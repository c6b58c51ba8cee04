// Token selection from 32-bit logits.
//
//   tb_argmax   token = lowest index attaining the row maximum
//               (two-stage argmax with ties to the lowest id, src/cuda/kernels.rs:803-873)
//   tb_sample   per row: temperature <= 0 -> argmax, else inverse-CDF sampling:
//               w_i = exp(double(l_i / T - max_j l_j / T)); token = first i (in token-id order)
//               with w_0 + ... + w_i > u * sum(w), for a caller-supplied uniform u in [0, 1)
//               (the reference's host sampler with top_p = 1, src/engine/sampling.rs:38-75,
//               which orders candidates by weight; without a top-p cut the order only decides
//               which token a given u maps to, not the distribution).
//
// One block of 1024 threads per row.  Each warp owns a contiguous segment of the vocabulary
// and scans it 32 tokens at a time, so prefix sums are taken in token order with coalesced reads.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;

struct MaxIdx {
    float v;
    int i;
};

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ MaxIdx block_argmax(const float* __restrict__ row, int vocab, MaxIdx* scratch) {
    MaxIdx best{-INFINITY, 0x7fffffff};
    if (((uintptr_t)row & 15) == 0) {
        // 16-byte loads, four of them in flight per thread; ascending i per thread keeps the lowest index on ties
        const int packets = vocab >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        int i = threadIdx.x;
        for (; i + 3 * (int)blockDim.x < packets; i += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = row4[i + u * blockDim.x];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int base = (i + u * blockDim.x) * 4;
                if (v[u].x > best.v) best = MaxIdx{v[u].x, base};
                if (v[u].y > best.v) best = MaxIdx{v[u].y, base + 1};
                if (v[u].z > best.v) best = MaxIdx{v[u].z, base + 2};
                if (v[u].w > best.v) best = MaxIdx{v[u].w, base + 3};
            }
        }
        for (; i < packets; i += blockDim.x) {
            const float4 v = row4[i];
            if (v.x > best.v) best = MaxIdx{v.x, i * 4};
            if (v.y > best.v) best = MaxIdx{v.y, i * 4 + 1};
            if (v.z > best.v) best = MaxIdx{v.z, i * 4 + 2};
            if (v.w > best.v) best = MaxIdx{v.w, i * 4 + 3};
        }
        for (int j = packets * 4 + threadIdx.x; j < vocab; j += blockDim.x) {
            const float v = row[j];
            if (v > best.v) best = MaxIdx{v, j};
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            if (v > best.v) best = MaxIdx{v, i};
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    MaxIdx t = lane < kWarps ? scratch[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
        t = better(t, other);
    }
    if (t.i == 0x7fffffff) t.i = 0;  // a row without any finite maximum (all NaN): token 0
    return t;
}

__device__ __forceinline__ double warp_inclusive_scan(double v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

__global__ void __launch_bounds__(kThreads)
argmax_kernel(const float* __restrict__ logits, int64_t stride, int* __restrict__ out, int vocab) {
    __shared__ MaxIdx scratch[kWarps];
    const MaxIdx best = block_argmax(logits + (int64_t)blockIdx.x * stride, vocab, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = best.i;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int64_t stride, const float* __restrict__ temperature,
              const double* __restrict__ uniform, int* __restrict__ out, int vocab) {
    __shared__ MaxIdx scratch[kWarps];
    __shared__ double warp_total[kWarps];
    __shared__ double warp_base[kWarps];
    __shared__ int chosen_warp;
    __shared__ double target_s;
    const float* row = logits + (int64_t)blockIdx.x * stride;
    const float temp = temperature[blockIdx.x];
    const MaxIdx best = block_argmax(row, vocab, scratch);
    if (!(temp > 0.0f)) {
        if (threadIdx.x == 0) out[blockIdx.x] = best.i;
        return;
    }
    const float inv_t = 1.0f / temp;
    const float top = best.v * inv_t;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = ((vocab + kWarps - 1) / kWarps + 31) / 32 * 32;  // tokens per warp, multiple of 32
    const int begin = warp * seg;
    const int end = min(vocab, begin + seg);

    double carry = 0.0;
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        const double w = i < end ? exp((double)(row[i] * inv_t - top)) : 0.0;
        const double incl = warp_inclusive_scan(w, lane);
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) warp_total[warp] = carry;
    __syncthreads();
    if (threadIdx.x == 0) {
        double run = 0.0;
        for (int w = 0; w < kWarps; ++w) {
            warp_base[w] = run;
            run += warp_total[w];
        }
        const double target = uniform[blockIdx.x] * run;
        int pick = -1;
        for (int w = 0; w < kWarps; ++w)
            if (pick < 0 && warp_total[w] > 0.0 && warp_base[w] + warp_total[w] > target) pick = w;
        if (pick < 0) {  // rounding left no crossing: last warp that holds any mass
            for (int w = kWarps - 1; w >= 0; --w)
                if (pick < 0 && warp_total[w] > 0.0) pick = w;
            if (pick < 0) pick = 0;
        }
        chosen_warp = pick;
        target_s = target;
    }
    __syncthreads();
    if (warp != chosen_warp) return;
    const double target = target_s;
    const double base = warp_base[warp];
    carry = 0.0;
    int token = -1, last_positive = -1;
    for (int i0 = begin; i0 < end && token < 0; i0 += 32) {
        const int i = i0 + lane;
        const double w = i < end ? exp((double)(row[i] * inv_t - top)) : 0.0;
        const double incl = warp_inclusive_scan(w, lane);
        const unsigned crossed = __ballot_sync(0xffffffffu, w > 0.0 && base + (carry + incl) > target);
        const unsigned positive = __ballot_sync(0xffffffffu, w > 0.0);
        if (positive) last_positive = i0 + 31 - __clz(positive);
        if (crossed) token = i0 + __ffs(crossed) - 1;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (token < 0) token = last_positive >= 0 ? last_positive : best.i;
    if (lane == 0) out[blockIdx.x] = token;
}

}  // namespace

TB_EXPORT int tb_argmax(const float* logits, int64_t stride, int* out, int rows, int vocab, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (vocab <= 0) return TB_ERR_BAD_SIZE;
    argmax_kernel<<<rows, kThreads, 0, stream>>>(logits, stride, out, vocab);
    return tb_launch_status();
}

TB_EXPORT int tb_sample(const float* logits, int64_t stride, const float* temperature, const double* uniform,
                        int* out, int rows, int vocab, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (vocab <= 0) return TB_ERR_BAD_SIZE;
    sample_kernel<<<rows, kThreads, 0, stream>>>(logits, stride, temperature, uniform, out, vocab);
    return tb_launch_status();
}
