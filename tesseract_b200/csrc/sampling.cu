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
// A row is shared by a thread-block cluster of 1, 2, 4 or 8 blocks of 1024 threads (as many as keep the grid
// within one wave): block c owns a contiguous chunk of the vocabulary, each of its warps a contiguous segment
// of the chunk, scanned 32 tokens at a time, so prefix sums are taken in token order with coalesced reads.  The
// blocks exchange their maxima and their sums through distributed shared memory; every block applies the same
// rule to the same numbers, so they agree on the block that holds the sampled token without a leader.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kPartStride = 16;     // rows per CTA in the partial results that a product leaves (at most 16 rows)

struct MaxIdx {
    float v;
    int i;
};

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// The block's best of tokens [first, first + vocab) of a row that starts at `row - first`.
__device__ MaxIdx block_argmax(const float* __restrict__ row, int vocab, MaxIdx* scratch, int first = 0) {
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
                if (v[u].x > best.v) best = MaxIdx{v[u].x, first + base};
                if (v[u].y > best.v) best = MaxIdx{v[u].y, first + base + 1};
                if (v[u].z > best.v) best = MaxIdx{v[u].z, first + base + 2};
                if (v[u].w > best.v) best = MaxIdx{v[u].w, first + base + 3};
            }
        }
        for (; i < packets; i += blockDim.x) {
            const float4 v = row4[i];
            if (v.x > best.v) best = MaxIdx{v.x, first + i * 4};
            if (v.y > best.v) best = MaxIdx{v.y, first + i * 4 + 1};
            if (v.z > best.v) best = MaxIdx{v.z, first + i * 4 + 2};
            if (v.w > best.v) best = MaxIdx{v.w, first + i * 4 + 3};
        }
        for (int j = packets * 4 + threadIdx.x; j < vocab; j += blockDim.x) {
            const float v = row[j];
            if (v > best.v) best = MaxIdx{v, first + j};
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            if (v > best.v) best = MaxIdx{v, first + i};
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
    return t;  // index 0x7fffffff: no finite maximum in the range
}

__device__ __forceinline__ double warp_inclusive_scan(double v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
    }
    return v;
}

// ---- thread-block clusters: barrier and loads from a peer's shared memory
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_address(const void* local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n"
                 : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    return remote;
}
__device__ __forceinline__ float peer_f32(const float* local, uint32_t rank) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(peer_address(local, rank)) : "memory");
    return v;
}
__device__ __forceinline__ int peer_s32(const int* local, uint32_t rank) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];\n" : "=r"(v) : "r"(peer_address(local, rank)) : "memory");
    return v;
}
__device__ __forceinline__ double peer_f64(const double* local, uint32_t rank) {
    double v;
    asm volatile("ld.shared::cluster.f64 %0, [%1];\n" : "=d"(v) : "r"(peer_address(local, rank)) : "memory");
    return v;
}

// The row's best over all blocks of the cluster (every block computes the same answer); `mine` is this block's.
__device__ MaxIdx cluster_argmax(MaxIdx mine, int blocks, float* x_value, int* x_index) {
    if (blocks == 1) return mine;
    if (threadIdx.x == 0) {
        *x_value = mine.v;
        *x_index = mine.i;
    }
    cluster_sync();
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int c = 0; c < blocks; ++c) best = better(best, MaxIdx{peer_f32(x_value, c), peer_s32(x_index, c)});
    return best;
}

// grid (blocks per row, rows); the blocks of a row are one cluster.
__global__ void __launch_bounds__(kThreads)
argmax_kernel(const float* __restrict__ logits, int64_t stride, int* __restrict__ out, int vocab, int chunk) {
    __shared__ MaxIdx scratch[kWarps];
    __shared__ float x_value;
    __shared__ int x_index;
    pdl_trigger();
    pdl_wait();   // the logits come from the kernel in front
    const int blocks = gridDim.x, block = blockIdx.x, r = blockIdx.y;
    const int first = min(vocab, block * chunk), count = min(vocab, first + chunk) - first;
    const float* row = logits + (int64_t)r * stride;
    const MaxIdx best = cluster_argmax(block_argmax(row + first, count, scratch, first), blocks, &x_value, &x_index);
    if (block == 0 && threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;   // all NaN: token 0
    if (blocks > 1) cluster_sync();   // no block leaves while a peer may still read its shared memory
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, int64_t stride, const float* __restrict__ temperature,
              const double* __restrict__ uniform, int* __restrict__ out, const float* __restrict__ part_value,
              const int* __restrict__ part_index, int parts, int vocab, int chunk) {
    __shared__ MaxIdx scratch[kWarps];
    __shared__ double warp_total[kWarps];
    __shared__ double warp_base[kWarps];
    __shared__ int chosen_warp;
    __shared__ double target_s;
    __shared__ float x_value;
    __shared__ int x_index;
    __shared__ double x_total;        // this block's mass
    pdl_trigger();
    pdl_wait();   // the logits come from the kernel in front
    const int blocks = gridDim.x, block = blockIdx.x, r = blockIdx.y;
    const int first = min(vocab, block * chunk), last = min(vocab, first + chunk);
    const float* row = logits + (int64_t)r * stride;
    const float temp = temperature[r];
    MaxIdx best;
    if (part_value != nullptr) {
        // The product that wrote the logits also left each of its CTAs' best token of the row (the reference's
        // two-stage argmax, src/cuda/kernels.rs:803-873): the row's best is the best of those, and the logits need
        // not be read for it.  Every block works it out for itself; nothing is exchanged.
        MaxIdx mine{-INFINITY, 0x7fffffff};
        if (threadIdx.x < 32) {
            for (int c = threadIdx.x; c < parts; c += 32)
                mine = better(mine, MaxIdx{part_value[c * kPartStride + r], part_index[c * kPartStride + r]});
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                mine = better(mine, MaxIdx{__shfl_xor_sync(0xffffffffu, mine.v, o), __shfl_xor_sync(0xffffffffu, mine.i, o)});
            if (threadIdx.x == 0) scratch[0] = mine;
        }
        __syncthreads();
        best = scratch[0];
        __syncthreads();
    } else {
        best = cluster_argmax(block_argmax(row + first, last - first, scratch, first), blocks, &x_value, &x_index);
    }
    if (best.i == 0x7fffffff) best.i = 0;
    if (!(temp > 0.0f)) {
        if (block == 0 && threadIdx.x == 0) out[r] = best.i;
        if (blocks > 1 && part_value == nullptr) cluster_sync();   // (with partial results no peer reads this block)
        return;
    }
    const float inv_t = 1.0f / temp;
    const float top = best.v * inv_t;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = ((last - first + kWarps - 1) / kWarps + 31) / 32 * 32;  // tokens per warp, multiple of 32
    const int begin = min(last, first + warp * seg);
    const int end = min(last, begin + seg);

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
        x_total = run;
    }
    if (blocks > 1) cluster_sync(); else __syncthreads();
    // every block: the masses in front of it, the whole mass, and the block in which the target falls
    double before = 0.0, all = 0.0;
    int chosen_block = -1, fallback_block = -1;
    {
        double run = 0.0;
        const double u = uniform[r];
        for (int c = 0; c < blocks; ++c) all += (blocks > 1 ? peer_f64(&x_total, c) : x_total);
        const double target = u * all;
        for (int c = 0; c < blocks; ++c) {
            const double mass = blocks > 1 ? peer_f64(&x_total, c) : x_total;
            if (c == block) before = run;
            if (chosen_block < 0 && mass > 0.0 && run + mass > target) chosen_block = c;
            if (mass > 0.0) fallback_block = c;
            run += mass;
        }
        if (chosen_block < 0) chosen_block = fallback_block;   // rounding left no crossing: the last block with mass
        if (threadIdx.x == 0) target_s = target;
    }
    if (chosen_block < 0) {                                    // no mass anywhere (all NaN): the best token
        if (block == 0 && threadIdx.x == 0) out[r] = best.i;
        if (blocks > 1) cluster_sync();
        return;
    }
    if (block == chosen_block && threadIdx.x == 0) {
        const double target = target_s;
        int pick = -1;
        for (int w = 0; w < kWarps; ++w)
            if (pick < 0 && warp_total[w] > 0.0 && before + warp_base[w] + warp_total[w] > target) pick = w;
        if (pick < 0) {  // rounding left no crossing: last warp that holds any mass
            for (int w = kWarps - 1; w >= 0; --w)
                if (pick < 0 && warp_total[w] > 0.0) pick = w;
            if (pick < 0) pick = 0;
        }
        chosen_warp = pick;
    }
    __syncthreads();
    if (block == chosen_block && warp == chosen_warp) {
        const double target = target_s;
        const double base = before + warp_base[warp];
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
        if (lane == 0) out[r] = token;
    }
    if (blocks > 1) cluster_sync();   // no block leaves while a peer may still read its shared memory
}

// Blocks per row: as many (a power of two up to the portable cluster size) as keep the grid within one wave.
int blocks_per_row(int rows, int vocab) {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 1;
    }
    int blocks = 8;
    while (blocks > 1 && (rows * blocks > sms || vocab < blocks * kThreads)) blocks >>= 1;
    return blocks;
}

template <typename Kernel, typename... Args>
int launch_rows(Kernel kernel, int rows, int vocab, cudaStream_t stream, Args... args) {
    const int blocks = blocks_per_row(rows, vocab);
    const int chunk = ((vocab + blocks - 1) / blocks + kThreads - 1) / kThreads * kThreads;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(blocks, rows, 1);
    config.blockDim = dim3(kThreads);
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = blocks;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start under the end of the head
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 2;
    cudaError_t err = cudaLaunchKernelEx(&config, kernel, args..., vocab, chunk);
    return err == cudaSuccess ? tb_launch_status() : (int)err;
}

}  // namespace

TB_EXPORT int tb_argmax(const float* logits, int64_t stride, int* out, int rows, int vocab, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (vocab <= 0 || rows > 65535) return TB_ERR_BAD_SIZE;
    return launch_rows(argmax_kernel, rows, vocab, stream, logits, stride, out);
}

// part_value / part_index (or null): [parts][16] per-CTA best value and token of each of at most 16 rows, left by
// the product that wrote the logits; with them a greedy row is decided without reading its logits and a sampled
// row skips the pass that finds its maximum.
TB_EXPORT int tb_sample(const float* logits, int64_t stride, const float* temperature, const double* uniform,
                        int* out, int rows, int vocab, const float* part_value, const int* part_index, int parts,
                        cudaStream_t stream) {
    if (rows == 0) return 0;
    if (vocab <= 0 || rows > 65535) return TB_ERR_BAD_SIZE;
    if (part_value != nullptr && (part_index == nullptr || parts < 1 || rows > kPartStride)) return TB_ERR_BAD_SIZE;
    return launch_rows(sample_kernel, rows, vocab, stream, logits, stride, temperature, uniform, out, part_value,
                       part_index, parts);
}
