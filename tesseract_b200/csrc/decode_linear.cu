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
// Two more forms move a norm's work out of the product behind it and into the product in front of it:
//   EPI_ADD_NORM (a product without a norm in front, bfloat16 out): with o = round(y), c = res + o (32-bit),
//     it stores res_out = round(c), xw = round(c * w) (w: the weights of the norm that FOLLOWS this product)
//     and, per 16- or 32-feature tile and batch row, the sum of c^2 over the tile's features;
//   PRO_SCALED: X = xw as it stands, and y = s * sum_k xw_k W_k with s = rsqrt(sum over the tiles' sums / K + eps).
//   Together: y = s * sum_k round(c_k w_k) W_k, where the reference has sum_k round(c_k s w_k) W_k
//   (src/cuda/kernels.rs:59-103): the same single rounding of the operand, the same 32-bit statistics of the
//   unrounded c, the scale applied to the 32-bit sums (a per-row scalar commutes with the sum).  The product
//   behind then starts like one without a norm (measured alone at 8 rows of the 1B sizes: QKV 3.6 against 5.7 us
//   with the norm folded in front, gate/up 11.0 against 12.6).
//
// Why not the library: at these sizes a decode layer is a chain of launches of a few microseconds
// each, and the norm and activation kernels between the products cost as much as the products.
// A CTA owns tiles of 32 (or, for narrow outputs, 16) output features; its 16 warps split K, each streaming its slice of the 32 weight
// rows through a private cp.async ring in shared memory into mma.sync.m16n8k16 A fragments (weights are
// the 16-row operand, the batch rows the 8-column operand); the warps are summed in a fixed order.
// Each lane loads 16 contiguous bytes per weight row and 32-wide K block; the products pair weight
// and activation elements in the same permuted K order, so no shuffle or shared-memory transpose is
// needed.  The reduction order depends on K alone.
#include "common.cuh"

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
// One CTA per SM (the prologue, which every CTA repeats, then costs each SM once) with rings deep enough for it
// to cover the memory latency alone: five stages of 32-feature tiles or six of 16-feature tiles per warp.

enum Prologue : int { PRO_NONE = 0, PRO_NORM = 1, PRO_ADD_NORM = 2, PRO_SCALED = 3, PRO_SCALED_RESIDENT = 4 };
enum Epilogue : int { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_F32 = 2, EPI_ADD_NORM = 3 };
constexpr int kSsStride = 16;      // floats per tile in the sums-of-squares array (rows beyond M hold zeros)

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
    // PRO_SCALED: sums of squares [ss_tiles][kSsStride] that an EPI_ADD_NORM product left; eps above
    const float* ss_in;
    int ss_tiles;
    // EPI_ADD_NORM: the residual rows [M, N] that this product's output is added to, the following norm's weights
    // [N], and what it leaves: the new residual [M, N], round(c * w) [M, N], sums of squares [N / TF][kSsStride]
    const __nv_bfloat16* epi_res;
    const float* epi_norm_w;
    __nv_bfloat16* epi_res_out;
    __nv_bfloat16* epi_xw;
    float* epi_ss;
    // EPI_F32 (or null): this CTA's best value and its lowest column per row, [gridDim.x][kSsStride] each: the first
    // stage of a two-stage argmax over the output columns (src/cuda/kernels.rs:803-873)
    float* best_value;
    int* best_index;
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Blackwell's packed pairs of 32-bit floats (one instruction for the two halves of a 64-bit register pair): the
// norm in front of a product is bound by the instructions each CTA issues for it.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// MT: number of 8-row batch tiles (1 or 2).
// NH: 16-feature halves per tile (2 where there are tiles enough for every SM, else 1).
template <int MT, int PRO, int EPI, int NH, int STAGES>
__global__ void __launch_bounds__(kThreads, 1) decode_linear_kernel(const LinearParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = p.K;
    constexpr int ROWS = 8 * MT;
    // The input rows either ride in the ring beside the weights, block by block (read from L2 once per tile: right
    // for a CTA with a tile or two), or lie in shared memory for all tiles (a norm in front puts them there anyway;
    // PRO_SCALED_RESIDENT copies them there: right for a CTA with many tiles, the head has 27).
    constexpr bool kRowsRide = PRO == PRO_NONE || PRO == PRO_SCALED;
    constexpr bool kNormInFront = PRO == PRO_NORM || PRO == PRO_ADD_NORM;
    constexpr bool kRowsResident = kNormInFront || PRO == PRO_SCALED_RESIDENT;
    constexpr bool kScaled = PRO == PRO_SCALED || PRO == PRO_SCALED_RESIDENT;
    __shared__ float scale_s[16];          // PRO_SCALED: the rows' reciprocal root mean squares
    __shared__ float tile_ss[kWarps][16];  // EPI_ADD_NORM: the warps' sums of squares of a tile

    // shared memory: [ROWS][K + 32] bf16 normalised activations (PRO only), the warps' partial sums, the rings
    const int x_pitch = K + 32;  // 64 bytes of padding: the eight rows a quarter-warp reads hit distinct banks
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);
    float* partial = reinterpret_cast<float*>(smem + (kRowsResident ? (size_t)ROWS * x_pitch * 2 : 0));

    // K is cut into 32-wide blocks; warp w takes blocks w, w + 16, ... of every tile (fixed by K alone).  A tile
    // is 32 output features (two 16-row operands that share the activation fragments).  A CTA walks over several
    // tiles, so that the prologue above is paid once.  Each warp keeps a private ring of STAGES blocks in shared
    // memory, filled by cp.async: a lane copies exactly the 16-byte pieces that it later reads back itself, so the
    // ring needs no barrier, only cp.async.wait_group, and runs on across tile boundaries.
    constexpr int X_BYTES = kRowsRide ? 512 * MT : 0;   // activations ride along when they come from memory
    constexpr int TF = 16 * NH;                                  // features per tile
    constexpr int STAGE_BYTES = 1024 * NH + X_BYTES;
    const int blocks = K / 32;
    const int bpw = (blocks + kWarps - 1) / kWarps;              // blocks per warp and tile
    const int num_tiles = p.N / TF;
    const int my_tiles = (num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    unsigned char* ring = smem + (kRowsResident ? (size_t)ROWS * x_pitch * 2 : 0) +
                          (size_t)kWarps * TF * ROWS * sizeof(float) + (size_t)warp * STAGES * STAGE_BYTES;
    const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
    const uint32_t lane_off = (uint32_t)(g * 64 + t * 16);
    const int64_t tile_stride = (int64_t)gridDim.x * TF * K;     // elements between this CTA's consecutive tiles

    // producer cursor: tile pi, block-of-warp pj, ring slot ps
    int pi = 0, pj = 0, ps = 0;
    const __nv_bfloat16* p_src = p.w + ((int64_t)blockIdx.x * TF + g) * K + 8 * t;   // row g of the current tile
    auto issue = [&](bool with_x) {
        int issued = -1;   // the K block whose weights went out (for the caller that adds the activations later)
        if (pi < my_tiles) {
            const int b = warp + pj * kWarps;
            if (b < blocks) {
                issued = b;
                const uint32_t dst = ring_addr + (uint32_t)ps * STAGE_BYTES + lane_off;
                const __nv_bfloat16* src = p_src + b * 32;
#pragma unroll
                for (int h = 0; h < 2 * NH; ++h) cp_async16(dst + 512 * h, src + (int64_t)(8 * h) * K);
                if (kRowsRide && with_x) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const int row = mt * 8 + g;
                        if (row < p.M)
                            cp_async16(dst + 1024 * NH + mt * 512, p.x + (int64_t)row * p.x_stride + b * 32 + 8 * t);
                    }
                }
            }
            if (++pj == bpw) {
                pj = 0;
                ++pi;
                p_src += tile_stride;
            }
            if (++ps == STAGES) ps = 0;
        }
        cp_async_commit();   // a group per slot, empty or not, keeps the wait count fixed
        return issued;
    };

    float acc[NH][MT][4];
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[h][mt][e] = 0.0f;
    pdl_trigger();
    float4 nw_first = make_float4(0.0f, 0.0f, 0.0f, 0.0f);   // the norm's weights are weights too: fetch them early
    if (kNormInFront && (int)threadIdx.x * 4 < K) nw_first = *reinterpret_cast<const float4*>(p.norm_w + threadIdx.x * 4);
    // Weights do not depend on the kernel before: their first stages go out ahead of the dependency wait.  With a
    // norm in front, the last POST of them are held back until the rows' own loads are out: those would otherwise
    // queue behind the whole ring (some microseconds of HBM time), and the memory would then idle while the norm
    // is computed; held back, they arrive under it (a decode step of eight rows: 0.783 -> 0.772 ms; with sixteen
    // rows and their shallower rings it cost 2 %, so those keep the whole prefetch in front).
    constexpr int POST = !kNormInFront || MT > 1 ? 0 : (NH == 2 ? 2 : 3) < STAGES - 1 ? (NH == 2 ? 2 : 3) : STAGES - 2;
    constexpr int PRE = STAGES - 1 - POST;
    int early[STAGES - 1];
#pragma unroll
    for (int q = 0; q < PRE; ++q) early[q] = issue(false);
    pdl_wait();                                      // from here on the previous kernel's results are visible
    if (kScaled) {
        // The rows' sums of squares that the product in front left, one value per tile of its features: every warp
        // sums the tiles w, w + 16, ... (two lanes a row, each every other one of them), in an order that depends
        // on the sizes alone; the first tile's epilogue, behind a block barrier, adds the sixteen warps' sums.
        const int m = lane & 15;
        float part = 0.0f;
        for (int tile = warp + kWarps * (lane >> 4); tile < p.ss_tiles; tile += 2 * kWarps)
            part += __ldcg(p.ss_in + tile * kSsStride + m);
        part += __shfl_xor_sync(0xffffffffu, part, 16);
        if (lane < 16) tile_ss[warp][lane] = part;
    }
    if (kRowsRide) {
        // the activations of the blocks above, a group each: the loop's wait count then covers them as well
#pragma unroll
        for (int q = 0; q < STAGES - 1; ++q) {
            if (early[q] >= 0) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int row = mt * 8 + g;
                    if (row < p.M)
                        cp_async16(ring_addr + (uint32_t)q * STAGE_BYTES + lane_off + 1024 * NH + mt * 512,
                                   p.x + (int64_t)row * p.x_stride + early[q] * 32 + 8 * t);
                }
            }
            cp_async_commit();
        }
    }

    if (PRO == PRO_SCALED_RESIDENT) {
        // the rows as they are, into shared memory once (rows beyond M as zeros)
        for (int idx = threadIdx.x; idx < ROWS * (K / 8); idx += kThreads) {
            const int row = idx / (K / 8), j = (idx - row * (K / 8)) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < p.M) v = *reinterpret_cast<const uint4*>(p.x + (int64_t)row * p.x_stride + j);
            *reinterpret_cast<uint4*>(xs + (size_t)row * x_pitch + j) = v;
        }
        __syncthreads();
    }
    if (kNormInFront) {
        // Every CTA normalises the (few) rows itself, all threads side by side along K; CTA 0 also stores the
        // new residual.  Two passes over the rows (the second one hits L1): sums of squares, then the scaling.
        // Eight rows at a time, all their loads issued before the first use (rows beyond M repeat row M - 1, so
        // that no load depends on a branch), four elements per thread and row.
        float* red = partial;  // [kWarps][ROWS] partial sums of squares (the partial-sum area is free until later)
        auto fetch_rows = [&](int r0, int j, uint2 (&a)[8], uint2 (&b)[8]) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int row = min(r0 + r, p.M - 1);
                a[r] = *reinterpret_cast<const uint2*>(p.res + (int64_t)row * K + j);
                if (PRO == PRO_ADD_NORM) b[r] = *reinterpret_cast<const uint2*>(p.upd + (int64_t)row * K + j);
            }
        };
        // c[r] = the four sums of a row as two pairs (elements 0,1 | 2,3), each sum exact in 32 bits
        auto sum_rows = [&](const uint2 (&a)[8], const uint2 (&b)[8], uint64_t (&c)[8][2]) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                c[r][0] = pack2(__uint_as_float(a[r].x << 16), __uint_as_float(a[r].x & 0xffff0000u));
                c[r][1] = pack2(__uint_as_float(a[r].y << 16), __uint_as_float(a[r].y & 0xffff0000u));
                if (PRO == PRO_ADD_NORM) {
                    c[r][0] = add2(c[r][0], pack2(__uint_as_float(b[r].x << 16), __uint_as_float(b[r].x & 0xffff0000u)));
                    c[r][1] = add2(c[r][1], pack2(__uint_as_float(b[r].y << 16), __uint_as_float(b[r].y & 0xffff0000u)));
                }
            }
        };
        auto load_rows = [&](int r0, int j, uint64_t (&c)[8][2]) {
            uint2 a[8], b[8];
            fetch_rows(r0, j, a, b);
            sum_rows(a, b, c);
        };
        // the first eight rows' first columns go out before the held-back weight stages
        uint2 first_a[8], first_b[8];
        const bool has_first = (int)threadIdx.x * 4 < K;
        if (POST > 0 && has_first) fetch_rows(0, threadIdx.x * 4, first_a, first_b);
#pragma unroll
        for (int q = PRE; q < STAGES - 1; ++q) early[q] = issue(false);
        auto pack4 = [](uint64_t v01, uint64_t v23) {
            float v0, v1, v2, v3;
            unpack2(v01, v0, v1);
            unpack2(v23, v2, v3);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v0, v1), hi = __floats2bfloat162_rn(v2, v3);
            return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        };
        uint64_t ss2[ROWS];   // per row a pair of partial sums of squares (even and odd elements)
#pragma unroll
        for (int r = 0; r < ROWS; ++r) ss2[r] = 0;   // the bit pattern of (0.0f, 0.0f)
        // With K up to four elements per thread the sums stay in registers between the two passes and the rows are
        // read once (every CTA reads all rows, so a second reading costs the L2 as much again); otherwise the
        // second pass reads them again.
        const bool keep = K <= kThreads * 4;
        uint64_t kept[ROWS][2];
        for (int j = threadIdx.x * 4; j < K; j += kThreads * 4) {
#pragma unroll
            for (int r0 = 0; r0 < ROWS; r0 += 8) {
                uint64_t c[8][2];
                if (POST > 0 && r0 == 0 && j == (int)threadIdx.x * 4) sum_rows(first_a, first_b, c);
                else load_rows(r0, j, c);
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    if (PRO == PRO_ADD_NORM && blockIdx.x == 0 && r0 + r < p.M)
                        *reinterpret_cast<uint2*>(p.res_out + (int64_t)(r0 + r) * K + j) = pack4(c[r][0], c[r][1]);
                    ss2[r0 + r] = fma2(c[r][0], c[r][0], ss2[r0 + r]);
                    ss2[r0 + r] = fma2(c[r][1], c[r][1], ss2[r0 + r]);
                    kept[r0 + r][0] = c[r][0];
                    kept[r0 + r][1] = c[r][1];
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float even, odd;
            unpack2(ss2[r], even, odd);
            const float ss = warp_sum(even + odd);
            if (lane == 0) red[warp * ROWS + r] = ss;
        }
        __syncthreads();
        float* inv_s = red + kWarps * ROWS;   // [ROWS] reciprocal root mean squares
        if (threadIdx.x < ROWS) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) total += red[w * ROWS + threadIdx.x];
            inv_s[threadIdx.x] = 1.0f / sqrtf(total / (float)K + p.eps);
        }
        __syncthreads();
        for (int j = threadIdx.x * 4; j < K; j += kThreads * 4) {
            const float4 nw = j == (int)threadIdx.x * 4 ? nw_first : *reinterpret_cast<const float4*>(p.norm_w + j);
            const uint64_t nw01 = pack2(nw.x, nw.y), nw23 = pack2(nw.z, nw.w);
#pragma unroll
            for (int r0 = 0; r0 < ROWS; r0 += 8) {
                uint64_t c[8][2];
                if (!keep) load_rows(r0, j, c);
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const float inv = inv_s[r0 + r];
                    const uint64_t inv2 = pack2(inv, inv);
                    // element * (inv * weight), as two pairs
                    uint64_t v01 = mul2(keep ? kept[r0 + r][0] : c[r][0], mul2(inv2, nw01));
                    uint64_t v23 = mul2(keep ? kept[r0 + r][1] : c[r][1], mul2(inv2, nw23));
                    if (r0 + r >= p.M) v01 = v23 = 0;
                    *reinterpret_cast<uint2*>(xs + (size_t)(r0 + r) * x_pitch + j) = pack4(v01, v23);
                }
            }
        }
        __syncthreads();
    }

    float best_v = -INFINITY;      // EPI_F32: the best value this thread has stored for its row, and its column
    int best_i = 0x7fffffff;
    int cs = 0;        // consumer ring slot
    for (int ti = 0; ti < my_tiles; ++ti) {
        // EPI_ADD_NORM: what this thread's item of the tile's epilogue adds to and multiplies with does not depend
        // on the products: asked for now, it is there when the products are done
        __nv_bfloat162 epi_r = __floats2bfloat162_rn(0.0f, 0.0f);
        float2 epi_w = make_float2(0.0f, 0.0f);
        if (EPI == EPI_ADD_NORM && (int)threadIdx.x < (TF / 2) * ROWS && (int)threadIdx.x % ROWS < p.M) {
            const int col = ((int)blockIdx.x + ti * (int)gridDim.x) * TF + 2 * ((int)threadIdx.x / ROWS);
            epi_r = *reinterpret_cast<const __nv_bfloat162*>(p.epi_res + (int64_t)((int)threadIdx.x % ROWS) * p.N + col);
            epi_w = *reinterpret_cast<const float2*>(p.epi_norm_w + col);
        }
        for (int j = 0; j < bpw; ++j) {
            issue(true);
            cp_async_wait<STAGES - 1>();
            const int b = warp + j * kWarps;
            if (b < blocks) {
                const unsigned char* st = ring + (size_t)cs * STAGE_BYTES + lane_off;
                uint4 w[2 * NH];
#pragma unroll
                for (int h = 0; h < 2 * NH; ++h) w[h] = *reinterpret_cast<const uint4*>(st + 512 * h);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint4 xa;
                    const int row = mt * 8 + g;
                    if (kRowsResident)
                        xa = *reinterpret_cast<const uint4*>(xs + (size_t)row * x_pitch + b * 32 + 8 * t);
                    else if (row >= p.M)
                        xa = make_uint4(0, 0, 0, 0);
                    else
                        xa = *reinterpret_cast<const uint4*>(st + 1024 * NH + mt * 512);
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        mma_bf16(acc[h][mt], w[2 * h].x, w[2 * h + 1].x, w[2 * h].y, w[2 * h + 1].y, xa.x, xa.y);
                        mma_bf16(acc[h][mt], w[2 * h].z, w[2 * h + 1].z, w[2 * h].w, w[2 * h + 1].w, xa.z, xa.w);
                    }
                }
            }
            if (++cs == STAGES) cs = 0;
        }
        // end of a tile: sum the warps in a fixed order: partial[warp][feature 0..31][batch row 0..ROWS-1]
        const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
        const int n0 = tile * TF;
        float* dst = partial + (size_t)warp * TF * ROWS;
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                dst[(h * 16 + g) * ROWS + mt * 8 + 2 * t] = acc[h][mt][0];
                dst[(h * 16 + g) * ROWS + mt * 8 + 2 * t + 1] = acc[h][mt][1];
                dst[(h * 16 + g + 8) * ROWS + mt * 8 + 2 * t] = acc[h][mt][2];
                dst[(h * 16 + g + 8) * ROWS + mt * 8 + 2 * t + 1] = acc[h][mt][3];
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[h][mt][e] = 0.0f;
            }
        __syncthreads();
        if (kScaled && ti == 0 && threadIdx.x < 16) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) total += tile_ss[w][threadIdx.x];
            scale_s[threadIdx.x] = 1.0f / sqrtf(total / (float)K + p.eps);
        }
        if (kScaled && ti == 0) __syncthreads();
        if (EPI == EPI_SWIGLU) {
            // of every 16 features the first eight are gates, the last eight the matching up projections
            for (int idx = threadIdx.x; idx < 8 * NH * ROWS; idx += kThreads) {
                const int f = idx / ROWS, m = idx - f * ROWS;   // f: activation column within the tile
                if (m >= p.M) continue;
                const int gate_row = (f >> 3) * 16 + (f & 7);
                float gate = 0.0f, up = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) {
                    gate += partial[(size_t)w * TF * ROWS + gate_row * ROWS + m];
                    up += partial[(size_t)w * TF * ROWS + (gate_row + 8) * ROWS + m];
                }
                if (kScaled) {
                    gate *= scale_s[m];
                    up *= scale_s[m];
                }
                const float act = gate * (1.0f / (1.0f + expf(-gate))) * up;
                reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)m * p.out_stride + tile * 8 * NH + f] =
                    __float2bfloat16_rn(act);
            }
        } else {
            // A thread sums two neighbouring features of one batch row: consecutive lanes then read consecutive
            // batch rows of the partial sums (at most two lanes per bank; one feature per lane along the features
            // would put 8 or 16 lanes on a bank) and store the pair at once.
            static_assert((TF / 2) * ROWS <= kThreads, "one item per thread");
            float ss = 0.0f;                     // EPI_ADD_NORM: this thread's share of its row's sum of squares
            for (int idx = threadIdx.x; idx < (TF / 2) * ROWS; idx += kThreads) {
                const int f = 2 * (idx / ROWS), m = idx % ROWS;
                if (m >= p.M) continue;
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) {
                    sum0 += partial[(size_t)w * TF * ROWS + f * ROWS + m];
                    sum1 += partial[(size_t)w * TF * ROWS + (f + 1) * ROWS + m];
                }
                if (kScaled) {
                    sum0 *= scale_s[m];
                    sum1 *= scale_s[m];
                }
                if (EPI == EPI_ADD_NORM) {
                    // o = round(y) as the product alone would store it; c = res + o; the new residual, the
                    // following norm's operand round(c * w), and c^2 towards the row's statistics
                    const int64_t at = (int64_t)m * p.N + n0 + f;
                    const __nv_bfloat162 o = __floats2bfloat162_rn(sum0, sum1);
                    const __nv_bfloat162 r = epi_r;
                    const float c0 = __bfloat162float(r.x) + __bfloat162float(o.x);
                    const float c1 = __bfloat162float(r.y) + __bfloat162float(o.y);
                    const float2 w2 = epi_w;
                    *reinterpret_cast<__nv_bfloat162*>(p.epi_res_out + at) = __floats2bfloat162_rn(c0, c1);
                    *reinterpret_cast<__nv_bfloat162*>(p.epi_xw + at) = __floats2bfloat162_rn(c0 * w2.x, c1 * w2.y);
                    ss = fmaf(c0, c0, c1 * c1);
                } else if (EPI == EPI_F32) {
                    // columns rise from tile to tile, so "greater" alone keeps the lowest column of equal values
                    if (sum0 > best_v) { best_v = sum0; best_i = n0 + f; }
                    if (sum1 > best_v) { best_v = sum1; best_i = n0 + f + 1; }
                    float* o = reinterpret_cast<float*>(p.out) + (int64_t)m * p.out_stride + n0 + f;
                    if ((uintptr_t)o % 8 == 0) {
                        *reinterpret_cast<float2*>(o) = make_float2(sum0, sum1);
                    } else {
                        o[0] = sum0;
                        o[1] = sum1;
                    }
                } else {
                    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)m * p.out_stride + n0 + f;
                    if ((uintptr_t)o % 4 == 0) {
                        *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(sum0, sum1);
                    } else {
                        o[0] = __float2bfloat16_rn(sum0);
                        o[1] = __float2bfloat16_rn(sum1);
                    }
                }
            }
            if (EPI == EPI_ADD_NORM) {
                // a row's items sit in lanes m, m + ROWS, ...: sum them in a fixed order, one value per warp and row
                if (ROWS == 8) ss += __shfl_xor_sync(0xffffffffu, ss, 8);
                ss += __shfl_xor_sync(0xffffffffu, ss, 16);
                if (lane < ROWS) tile_ss[warp][lane] = ss;
            }
        }
        __syncthreads();  // the partial sums are reused by the next tile
        if (EPI == EPI_ADD_NORM && threadIdx.x < kSsStride) {
            float total = 0.0f;
            if ((int)threadIdx.x < ROWS) {
#pragma unroll
                for (int w = 0; w < kWarps; ++w) total += tile_ss[w][threadIdx.x];
            }
            p.epi_ss[(int64_t)tile * kSsStride + threadIdx.x] = total;    // rows beyond M (and beyond ROWS) hold zeros
        }
    }
    if (EPI == EPI_F32 && p.best_value != nullptr) {
        // this CTA's best per row: a row's items sit in lanes m, m + ROWS, ... of the warps that had items
        auto take = [&](float v, int i) {
            if (v > best_v || (v == best_v && i < best_i)) { best_v = v; best_i = i; }
        };
        if (ROWS == 8) take(__shfl_xor_sync(0xffffffffu, best_v, 8), __shfl_xor_sync(0xffffffffu, best_i, 8));
        take(__shfl_xor_sync(0xffffffffu, best_v, 16), __shfl_xor_sync(0xffffffffu, best_i, 16));
        float* best_vs = &tile_ss[0][0];                                   // [kWarps][16], free by now
        int* best_is = reinterpret_cast<int*>(partial);                     // the partial sums are done with
        if (lane < ROWS) {
            best_vs[warp * 16 + lane] = best_v;
            best_is[warp * 16 + lane] = best_i;
        }
        __syncthreads();
        if (threadIdx.x < kSsStride) {
            float v = -INFINITY;
            int i = 0x7fffffff;
            if ((int)threadIdx.x < ROWS) {
                for (int w = 0; w < kWarps; ++w) {
                    const float wv = best_vs[w * 16 + threadIdx.x];
                    const int wi = best_is[w * 16 + threadIdx.x];
                    if (wv > v || (wv == v && wi < i)) { v = wv; i = wi; }
                }
            }
            p.best_value[(int64_t)blockIdx.x * kSsStride + threadIdx.x] = v;
            p.best_index[(int64_t)blockIdx.x * kSsStride + threadIdx.x] = i;
        }
    }
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 1;
    }
    return sms;
}

// 32-feature tiles where that still gives every SM a tile, else 16-feature tiles.
bool wide_tiles(int N) { return N % 32 == 0 && N / 32 >= sm_count(); }
// Ring depth: five stages of 32-feature tiles or six of 16-feature tiles per warp for up to eight rows; sixteen rows
// take four or six where the activations and the partial sums leave the room (their size depends on K), else three.
constexpr int deep_stages(int nh, int rows8) { return rows8 > 1 ? (nh == 2 ? 4 : 6) : (nh == 2 ? 5 : 6); }
constexpr int kShallowStages = 3;

size_t smem_bytes(int rows8, bool prologue, int nh, int K, int stages) {
    const int rows = 8 * rows8, tf = 16 * nh;
    const size_t stage = 1024 * nh + (prologue ? 0 : 512 * rows8);
    size_t smem = (size_t)kWarps * tf * rows * sizeof(float) + (size_t)kWarps * stages * stage;
    if (prologue) smem += (size_t)rows * (K + 32) * 2;
    return smem;
}

constexpr size_t kMaxSmem = 227 * 1024;

// the ring depth that these sizes get, or 0 if even the shallow ring does not fit
int stages_for(int rows8, bool prologue, int nh, int K) {
    if (smem_bytes(rows8, prologue, nh, K, deep_stages(nh, rows8)) <= kMaxSmem) return deep_stages(nh, rows8);
    if (rows8 > 1 && smem_bytes(rows8, prologue, nh, K, kShallowStages) <= kMaxSmem) return kShallowStages;
    return 0;
}

template <int MT, int PRO, int EPI, int NH, int STAGES>
int launch_ring(const LinearParams& p, cudaStream_t stream) {
    constexpr int TF = 16 * NH;
    const size_t smem = smem_bytes(MT, PRO == PRO_NORM || PRO == PRO_ADD_NORM || PRO == PRO_SCALED_RESIDENT, NH, p.K, STAGES);
    auto kernel = decode_linear_kernel<MT, PRO, EPI, NH, STAGES>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    const int tiles = p.N / TF;
    const int max_ctas = sm_count();                                 // one CTA per SM at most
    // every SM takes part even where some CTAs then stream a tile more than others: the others' rings are in
    // flight from the start, and the last tiles have the memory to themselves (QKV at 8 rows: 3.86 -> 3.55 us)
    const int grid = tiles < max_ctas ? tiles : max_ctas;
    cudaError_t err = tb_launch_pdl(kernel, dim3(grid), dim3(kThreads), smem, stream, p);
    return err == cudaSuccess ? tb_launch_status() : (int)err;
}

template <int MT, int PRO, int EPI, int NH>
int launch_tiles(const LinearParams& p, cudaStream_t stream) {
    const int stages = stages_for(MT, PRO == PRO_NORM || PRO == PRO_ADD_NORM || PRO == PRO_SCALED_RESIDENT, NH, p.K);
    if (stages == deep_stages(NH, MT)) return launch_ring<MT, PRO, EPI, NH, deep_stages(NH, MT)>(p, stream);
    if constexpr (MT > 1) {
        if (stages == kShallowStages) return launch_ring<MT, PRO, EPI, NH, kShallowStages>(p, stream);
    }
    return TB_ERR_BAD_SIZE;
}

template <int MT, int PRO, int EPI>
int launch(const LinearParams& p, cudaStream_t stream) {
    if (wide_tiles(p.N)) return launch_tiles<MT, PRO, EPI, 2>(p, stream);
    return launch_tiles<MT, PRO, EPI, 1>(p, stream);
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
    TB_CASE(PRO_NONE, EPI_ADD_NORM)
    TB_CASE(PRO_SCALED, EPI_BF16)
    TB_CASE(PRO_SCALED, EPI_F32)
    TB_CASE(PRO_SCALED, EPI_SWIGLU)
    TB_CASE(PRO_SCALED_RESIDENT, EPI_BF16)
    TB_CASE(PRO_SCALED_RESIDENT, EPI_F32)
    TB_CASE(PRO_SCALED_RESIDENT, EPI_SWIGLU)
#undef TB_CASE
    return TB_ERR_BAD_SIZE;
}

}  // namespace

// 1 if the sizes are ones this kernel takes, else 0 (the caller then uses the general path).
TB_EXPORT int tb_decode_linear_supported(int M, int N, int K, int prologue) {
    if (M < 1 || M > 16 || N < 16 || N % 16 != 0 || K < 32 || K % 32 != 0) return 0;
    const bool norm_in_front = prologue == PRO_NORM || prologue == PRO_ADD_NORM;
    return stages_for(M <= 8 ? 1 : 2, norm_in_front, wide_tiles(N) ? 2 : 1, K) != 0;
}

// Features per tile for an output width (what EPI_ADD_NORM's sums of squares are counted in).
TB_EXPORT int tb_decode_linear_tile_features(int N) { return wide_tiles(N) ? 32 : 16; }

// CTAs that a product of this output width is launched with (what EPI_F32's per-CTA best values are counted in).
TB_EXPORT int tb_decode_linear_ctas(int N) {
    const int tiles = N / tb_decode_linear_tile_features(N);
    return tiles < sm_count() ? tiles : sm_count();
}

// x: PRO_NONE and PRO_SCALED (the rows as they are).  res/upd/norm_w/res_out: see LinearParams.  out_stride in
// elements of the output type.
// PRO_SCALED: ss_in [ss_tiles][16] sums of squares that an EPI_ADD_NORM call left; the scale uses eps.
// EPI_ADD_NORM (with PRO_NONE): epi_res [M, N] residual, epi_norm_w [N], and the outputs epi_res_out [M, N],
//   epi_xw [M, N], epi_ss [N / tb_decode_linear_tile_features(N)][16]; `out` is not written.
// EPI_F32 with best_value / best_index [tb_decode_linear_ctas(N)][16] (or null): each CTA's best output value per
//   row and its lowest column.
TB_EXPORT int tb_decode_linear_ex(const void* x, int64_t x_stride, const void* res, const void* upd,
                                  const float* norm_w, float eps, void* res_out, const void* w, void* out,
                                  int64_t out_stride, int M, int N, int K, int prologue, int epilogue,
                                  const float* ss_in, int ss_tiles, const void* epi_res, const float* epi_norm_w,
                                  void* epi_res_out, void* epi_xw, float* epi_ss, float* best_value, int* best_index,
                                  cudaStream_t stream) {
    if (!tb_decode_linear_supported(M, N, K, prologue)) return TB_ERR_BAD_SIZE;
    const uintptr_t bits = (uintptr_t)x | (uintptr_t)res | (uintptr_t)upd | (uintptr_t)res_out | (uintptr_t)w |
                           (uintptr_t)epi_res | (uintptr_t)epi_res_out | (uintptr_t)epi_xw;
    const bool rows_ride = prologue == PRO_NONE || prologue == PRO_SCALED;
    if (bits % 16 != 0 || (rows_ride && (x == nullptr || x_stride % 8 != 0))) return TB_ERR_BAD_ALIGN;
    if (prologue == PRO_ADD_NORM && (res_out == nullptr || res_out == res)) return TB_ERR_BAD_ALIGN;
    if (prologue == PRO_SCALED && (ss_in == nullptr || ss_tiles < 1)) return TB_ERR_BAD_ALIGN;
    if (epilogue == EPI_ADD_NORM &&
        (prologue != PRO_NONE || epi_res == nullptr || epi_norm_w == nullptr || epi_res_out == nullptr ||
         epi_xw == nullptr || epi_ss == nullptr || epi_res_out == epi_res || (uintptr_t)epi_norm_w % 8 != 0))
        return TB_ERR_BAD_ALIGN;
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
    p.ss_in = ss_in;
    p.ss_tiles = ss_tiles;
    p.epi_res = (const __nv_bfloat16*)epi_res;
    p.epi_norm_w = epi_norm_w;
    p.epi_res_out = (__nv_bfloat16*)epi_res_out;
    p.epi_xw = (__nv_bfloat16*)epi_xw;
    p.epi_ss = epi_ss;
    p.best_value = epilogue == EPI_F32 && best_index != nullptr ? best_value : nullptr;
    p.best_index = best_index;
    if (prologue == PRO_SCALED) {
        // a CTA with three tiles or more keeps the rows in shared memory instead of reading them again per tile
        const int tf = tb_decode_linear_tile_features(N);
        const int ctas = tb_decode_linear_ctas(N);
        if ((N / tf + ctas - 1) / ctas >= 3 && K % 8 == 0 && x_stride % 8 == 0 &&
            stages_for(M <= 8 ? 1 : 2, true, tf / 16, K) != 0)
            prologue = PRO_SCALED_RESIDENT;
    }
    return M <= 8 ? dispatch<1>(p, prologue, epilogue, stream) : dispatch<2>(p, prologue, epilogue, stream);
}

TB_EXPORT int tb_decode_linear(const void* x, int64_t x_stride, const void* res, const void* upd,
                               const float* norm_w, float eps, void* res_out, const void* w, void* out,
                               int64_t out_stride, int M, int N, int K, int prologue, int epilogue,
                               cudaStream_t stream) {
    if (prologue == PRO_SCALED || epilogue == EPI_ADD_NORM) return TB_ERR_BAD_SIZE;
    return tb_decode_linear_ex(x, x_stride, res, upd, norm_w, eps, res_out, w, out, out_stride, M, N, K, prologue,
                               epilogue, nullptr, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, stream);
}
