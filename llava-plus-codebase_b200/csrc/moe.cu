// Mixture-of-experts feed-forward of the layer-list decoders: sigmoid or softmax router with group-limited top-k choice, the plan that
// sorts (token, choice) pairs by expert into tiles of one expert each, the gated activation, and the weighted sum of the
// chosen experts' outputs. The expert products themselves are grouped Linears (linear_generic.cu). Router scores, the choice
// and the weights are fp32; the order of a pair inside its expert's tile does not change its result, and the sum over a
// token's choices runs in the order of the choice, so a token's output does not depend on what else is in the call.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

// (value, index) maximum over the warp; ties go to the lower index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi < i))) { v = ov; i = oi; }
    }
}

// One warp per row. Shared memory per warp: E scores, G group scores (later: group alive flags), E taken flags.
__global__ void moe_route_kernel(MoeRouteArgs a) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= a.rows) return;
    const int E = a.experts, G = a.groups, per = E / G;
    float* s = sm + (size_t)warp * (2 * E + G);
    float* gs = s + E;
    float* taken = gs + G;
    if (a.score_fn == MOE_SCORE_SOFTMAX) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, a.logits[(size_t)r * a.ld + e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float den = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(a.logits[(size_t)r * a.ld + e] - mx);
            s[e] = v;
            den += v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        for (int e = lane; e < E; e += 32) { s[e] /= den; taken[e] = 0.f; }
    } else {
        for (int e = lane; e < E; e += 32) {
            s[e] = 1.f / (1.f + expf(-a.logits[(size_t)r * a.ld + e]));
            taken[e] = 0.f;
        }
    }
    __syncwarp();
    // a group's score: the sum of its two largest scores (of its one score, when a group is a single expert), or its largest
    for (int g = lane; g < G; g += 32) {
        float b1 = -INFINITY, b2v = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) {
            const float v = s[e];
            if (v > b1) { b2v = b1; b1 = v; } else if (v > b2v) { b2v = v; }
        }
        gs[g] = (per > 1 && a.group_score != MOE_GROUP_MAX) ? b1 + b2v : b1;
    }
    __syncwarp();
    // keep the best groups: experts of the others are marked as taken. G - keep rounds remove the weakest group each
    // (ties: the higher index goes first, so that the lower index stays, as a stable descending sort would have it)
    if (lane == 0) {
        for (int k = 0; k < G - a.keep; ++k) {
            int worst = -1;
            for (int g = 0; g < G; ++g)
                if (gs[g] != INFINITY && (worst < 0 || gs[g] <= gs[worst])) worst = g;
            if (worst < 0) break;
            gs[worst] = INFINITY;   // marks a dropped group
            for (int e = worst * per; e < (worst + 1) * per; ++e) taken[e] = 1.f;
        }
    }
    __syncwarp();
    float sum = 0.f, mine = 0.f;   // lane k keeps the k-th choice's score (top <= 32)
    int mine_e = 0;
    for (int k = 0; k < a.top; ++k) {
        float bv = -INFINITY;
        int bi = -1;
        for (int e = lane; e < E; e += 32)
            if (taken[e] == 0.f && (bi < 0 || s[e] > bv)) { bv = s[e]; bi = e; }
        warp_argmax(bv, bi);
        if (bi < 0) { bi = 0; bv = 0.f; }   // fewer candidates than choices: a zero-weight pair on expert 0
        if (lane == 0) taken[bi] = 1.f;
        __syncwarp();
        if (lane == k) { mine = bv; mine_e = bi; }
        sum += bv;
    }
    if (lane < a.top) {
        a.idx[(size_t)r * a.top + lane] = mine_e;
        a.w[(size_t)r * a.top + lane] = a.raw_weights ? mine : mine / (sum + 1e-20f) * a.scale;
    }
}

// One block. pairs = rows * top (token, choice) pairs with their expert in idx. Every expert gets its pairs in consecutive
// positions, padded to a multiple of `tile` rows: pair_pos[pair] = position, src_row[position] = token row (-1: padding),
// tile_group[t] = expert of tile t (-1: unused), for max_tiles tiles.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int32_t* __restrict__ idx, int pairs, int top, int experts, int tile, int max_tiles,
                                                        int32_t* __restrict__ pair_pos, int32_t* __restrict__ src_row,
                                                        int32_t* __restrict__ tile_group) {
    extern __shared__ int cnt[];   // [experts] counts, then [experts] offsets
    int* off = cnt + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
    for (int p = threadIdx.x; p < max_tiles * tile; p += blockDim.x) src_row[p] = -1;
    for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_group[t] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) pair_pos[p] = atomicAdd(&cnt[idx[p]], 1);   // rank inside its expert
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0;
        for (int e = 0; e < experts; ++e) { off[e] = o; o += (cnt[e] + tile - 1) / tile * tile; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        for (int t = off[e] / tile; t < (off[e] + cnt[e] + tile - 1) / tile; ++t) tile_group[t] = e;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int pos = off[idx[p]] + pair_pos[p];
        pair_pos[p] = pos;
        src_row[pos] = p / top;
    }
}

// out[r, c] = act(in[r, c], in[r, ff + c]): the gated unit (SiLU(g) u, or its bounded and shifted form)
__global__ void glu_rows_kernel(const float* __restrict__ in, int64_t ld_in, float* __restrict__ out, int64_t ld_out, int ff,
                                __nv_bfloat16* __restrict__ out16, int64_t ld_out16, GluAct act) {
    const size_t r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < ff) {
        const float v = glu_act(in[r * ld_in + c], in[r * ld_in + ff + c], act);
        if (out != nullptr) out[r * ld_out + c] = v;
        if (out16 != nullptr) out16[r * ld_out16 + c] = __float2bfloat16_rn(v);
    }
}

__global__ void gather_rows_bf16_kernel(const float* __restrict__ A, int64_t lda, const int32_t* __restrict__ src_row, __nv_bfloat16* __restrict__ out,
                                        int64_t ld_out, int K) {
    const size_t p = blockIdx.y;
    const int src = src_row[p];
    const int k = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (k + 1 < K) {
        const float a = src >= 0 ? A[(size_t)src * lda + k] : 0.f, b = src >= 0 ? A[(size_t)src * lda + k + 1] : 0.f;
        *reinterpret_cast<__nv_bfloat162*>(out + p * ld_out + k) = __floats2bfloat162_rn(a, b);
    } else if (k < K) {
        out[p * ld_out + k] = __float2bfloat16_rn(src >= 0 ? A[(size_t)src * lda + k] : 0.f);
    }
}

// x[r] += alpha * sum_k w[r, k] * y[pair_pos[r * top + k]] (pair_pos null: position = pair)
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, int64_t ldy, const int32_t* __restrict__ pair_pos,
                                   const float* __restrict__ w, int top, int cols, float alpha) {
    const size_t r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
        const size_t p = r * top + k;
        const size_t pos = pair_pos != nullptr ? (size_t)pair_pos[p] : p;
        acc = fmaf(w[p], y[pos * ldy + c], acc);
    }
    x[r * cols + c] += alpha * acc;
}
}  // namespace

int moe_route_f32(const MoeRouteArgs& a, cudaStream_t st) {
    B2_CHECK_ARG(a.logits && a.idx && a.w && a.rows > 0, "moe_route: null argument");
    B2_CHECK_ARG(a.experts >= 1 && a.top >= 1 && a.top <= 32 && a.top <= a.experts, "moe_route: %d experts, top %d (at most 32 choices)", a.experts, a.top);
    B2_CHECK_ARG(a.groups >= 1 && a.experts % a.groups == 0 && a.keep >= 1 && a.keep <= a.groups, "moe_route: %d experts in %d groups, %d kept", a.experts,
                 a.groups, a.keep);
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * a.experts + a.groups) * sizeof(float);
    B2_CHECK_ARG(smem <= 48 * 1024, "moe_route: %d experts exceed the router kernel's shared memory", a.experts);
    moe_route_kernel<<<(a.rows + warps - 1) / warps, warps * 32, smem, st>>>(a);
    B2_LAUNCH_CHECK();
    return 0;
}

int moe_plan(const int32_t* idx, int rows, int top, int experts, int tile, int max_tiles, int32_t* pair_pos, int32_t* src_row, int32_t* tile_group,
             cudaStream_t st) {
    B2_CHECK_ARG(idx && pair_pos && src_row && tile_group && rows > 0 && top > 0 && experts > 0 && tile > 0, "moe_plan: bad argument");
    B2_CHECK_ARG((size_t)max_tiles * tile >= (size_t)rows * top + (size_t)experts * (tile - 1), "moe_plan: %d tiles cannot hold the padded pairs", max_tiles);
    moe_plan_kernel<<<1, 1024, 2 * experts * sizeof(int), st>>>(idx, rows * top, top, experts, tile, max_tiles, pair_pos, src_row, tile_group);
    B2_LAUNCH_CHECK();
    return 0;
}

int glu_rows_f32(const float* in, int64_t ld_in, float* out, int64_t ld_out, int rows, int ff, const GluAct& act, cudaStream_t st, void* out16,
                 int64_t ld_out16) {
    B2_CHECK_ARG(in && (out || out16) && rows > 0 && ff > 0, "glu_rows: bad argument");
    glu_rows_kernel<<<dim3((ff + 255) / 256, rows), 256, 0, st>>>(in, ld_in, out, ld_out, ff, reinterpret_cast<__nv_bfloat16*>(out16), ld_out16, act);
    B2_LAUNCH_CHECK();
    return 0;
}

int swiglu_rows_f32(const float* in, int64_t ld_in, float* out, int64_t ld_out, int rows, int ff, cudaStream_t st, void* out16, int64_t ld_out16) {
    return glu_rows_f32(in, ld_in, out, ld_out, rows, ff, GluAct{}, st, out16, ld_out16);
}

int gather_rows_bf16(const float* A, int64_t lda, const int32_t* src_row, void* out, int64_t ld_out, int rows, int K, cudaStream_t st) {
    B2_CHECK_ARG(A && src_row && out && rows > 0 && K > 0 && ld_out % 2 == 0, "gather_rows_bf16: bad argument");
    gather_rows_bf16_kernel<<<dim3((K / 2 + 256) / 256, rows), 256, 0, st>>>(A, lda, src_row, reinterpret_cast<__nv_bfloat16*>(out), ld_out, K);
    B2_LAUNCH_CHECK();
    return 0;
}

int moe_combine_f32(float* x, const float* y, int64_t ldy, const int32_t* pair_pos, const float* w, int rows, int top, int cols, float alpha,
                    cudaStream_t st) {
    B2_CHECK_ARG(x && y && w && rows > 0 && top > 0 && cols > 0, "moe_combine: bad argument");
    moe_combine_kernel<<<dim3((cols + 255) / 256, rows), 256, 0, st>>>(x, y, ldy, pair_pos, w, top, cols, alpha);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b2
