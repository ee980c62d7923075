// Linear layers on fp32 activations for shapes the tcgen05 GEMMs do not take (any M, N, K; fp32 or bf16 weights) and for
// true-fp32 compute: a weight-streaming row kernel for a handful of rows (decode) and a shared-memory tiled kernel for
// portions of a prompt. Accumulation is fp32 FMA in both; with round_a the activations are rounded to bf16 first, so the
// product is the bf16 x bf16 -> fp32 product the tensor-core path computes.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

__device__ __forceinline__ float ld_w(const float* p) { return *p; }
__device__ __forceinline__ float ld_w(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float lin_act(float v, int act) {
    switch (act) {
        case LIN_SILU: return v / (1.f + expf(-v));
        case LIN_SIGMOID: return 1.f / (1.f + expf(-v));
        case LIN_TANH: return tanhf(v);
        case LIN_RELU_SQ: { const float r = v > 0.f ? v : 0.f; return r * r; }
        default: return v;
    }
}
__device__ __forceinline__ void lin_store(float* o, float acc, const float* bias, int n, int act, float alpha, int accumulate) {
    float v = acc + (bias ? bias[n] : 0.f);
    v = alpha * lin_act(v, act);
    *o = accumulate ? (*o + v) : v;
}

// ---- up to MR rows: one warp per output column, the weight row is read exactly once --------------------------------------
// VEC: a lane takes 8 consecutive k per step (16 B of bf16 weights, 2 x 16 B of fp32), two steps in flight.
constexpr int MR = 8;
__device__ __forceinline__ void ld_w8(const float* p, float (&w)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}
__device__ __forceinline__ void ld_w8(const __nv_bfloat16* p, float (&w)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    w[0] = __uint_as_float(t.x << 16); w[1] = __uint_as_float(t.x & 0xffff0000u);
    w[2] = __uint_as_float(t.y << 16); w[3] = __uint_as_float(t.y & 0xffff0000u);
    w[4] = __uint_as_float(t.z << 16); w[5] = __uint_as_float(t.z & 0xffff0000u);
    w[6] = __uint_as_float(t.w << 16); w[7] = __uint_as_float(t.w & 0xffff0000u);
}
// VEC kernel: a CTA of 8 warps works on groups of 16 output columns (2 per warp and two k-steps at a time, so a lane keeps
// 4 weight loads of 16 B in flight). The activation rows are staged in shared memory, already rounded to bf16 when the product
// is bf16: whole (K <= kc_max) and then shared by every column group the CTA walks, or kc_max columns at a time for one group.
constexpr int RW_COLS = 2, RW_SMEM_FLOATS = 16384;
template <typename TW>
__global__ void __launch_bounds__(256) linear_rows_vec_kernel(const float* __restrict__ A, int64_t lda, const TW* __restrict__ W, int64_t ldw,
                                                              const float* __restrict__ bias, float* __restrict__ out, int64_t ld_out, int M, int N,
                                                              int K, int kc_max, int act, float alpha, int accumulate, int round_a) {
    extern __shared__ float sA[];  // [M][kc]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ngroups = (N + 8 * RW_COLS - 1) / (8 * RW_COLS);
    const bool whole = K <= kc_max;      // otherwise gridDim.x == ngroups: one group per CTA, K in chunks
    for (int kc0 = 0; kc0 < K; kc0 += kc_max) {
        const int kc = min(kc_max, K - kc0);
        __syncthreads();
        for (int e = threadIdx.x * 4; e < M * kc; e += 1024) {
            const int m = e / kc, k = e % kc;
            float4 v = *reinterpret_cast<const float4*>(A + (size_t)m * lda + kc0 + k);
            if (round_a) { v.x = round_bf16(v.x); v.y = round_bf16(v.y); v.z = round_bf16(v.z); v.w = round_bf16(v.w); }
            *reinterpret_cast<float4*>(sA + e) = v;
        }
        __syncthreads();
        for (int grp = blockIdx.x; grp < ngroups; grp += gridDim.x) {
            const int n0 = (grp * 8 + warp) * RW_COLS;
            float acc[RW_COLS][MR];
#pragma unroll
            for (int c = 0; c < RW_COLS; ++c)
#pragma unroll
                for (int m = 0; m < MR; ++m) acc[c][m] = 0.f;
            for (int k0 = lane * 8; k0 < kc; k0 += 512) {
                // two k-steps x RW_COLS columns: 2 * RW_COLS weight loads of 16 B per lane are issued before the first is used
                float wv[2][RW_COLS][8];
                const bool second = k0 + 256 < kc;
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int c = 0; c < RW_COLS; ++c) {
                        const int n = min(n0 + c, N - 1);  // columns past N read the last row again: their sums are never stored
                        if (u == 0 || second) ld_w8(W + (size_t)n * ldw + kc0 + k0 + u * 256, wv[u][c]);
                    }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (u == 0 || second) {
#pragma unroll
                        for (int m = 0; m < MR; ++m) {
                            if (m < M) {
                                float av[8];
                                ld_w8(sA + m * kc + k0 + u * 256, av);
#pragma unroll
                                for (int c = 0; c < RW_COLS; ++c)
#pragma unroll
                                    for (int e = 0; e < 8; ++e) acc[c][m] = fmaf(av[e], wv[u][c][e], acc[c][m]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < RW_COLS; ++c)
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    float v = acc[c][m];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    // K in chunks: the first chunk stores (or adds to what the caller asked to keep), later chunks add;
                    // the activation is only legal on a whole K (checked on the host)
                    if (lane == 0 && m < M && n0 + c < N) {
                        if (whole) lin_store(out + (size_t)m * ld_out + n0 + c, v, bias, n0 + c, act, alpha, accumulate);
                        else lin_store(out + (size_t)m * ld_out + n0 + c, v, kc0 == 0 ? bias : nullptr, n0 + c, LIN_NONE, alpha, accumulate || kc0 > 0);
                    }
                }
        }
    }
}

// any K and alignment: one warp per output column, scalar loads
template <typename TW>
__global__ void __launch_bounds__(256) linear_rows_kernel(const float* __restrict__ A, int64_t lda, const TW* __restrict__ W, int64_t ldw,
                                                          const float* __restrict__ bias, float* __restrict__ out, int64_t ld_out, int M, int N,
                                                          int K, int act, float alpha, int accumulate, int round_a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const TW* w = W + (size_t)n * ldw;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float wv = ld_w(w + k);
#pragma unroll
        for (int m = 0; m < MR; ++m) {
            if (m < M) {
                float a = A[(size_t)m * lda + k];
                if (round_a) a = round_bf16(a);
                acc[m] = fmaf(a, wv, acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m < M) lin_store(out + (size_t)m * ld_out + n, v, bias, n, act, alpha, accumulate);
    }
}

// ---- portions of a prompt: 64 x 64 output tile, K in steps of 16, 4 x 4 outputs per thread -------------------------------
constexpr int TB = 64, TK = 16;
template <typename TW>
__global__ void __launch_bounds__(256) linear_tiled_kernel(const float* __restrict__ A, int64_t lda, const TW* __restrict__ W, int64_t ldw,
                                                           const float* __restrict__ bias, float* __restrict__ out, int64_t ld_out, int M, int N,
                                                           int K, int act, float alpha, int accumulate, int round_a) {
    __shared__ float As[TK][TB + 4];
    __shared__ float Ws[TK][TB + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TB, n0 = blockIdx.x * TB;
    const int tm = (tid >> 4) * 4, tn = (tid & 15) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;         // 64 rows x 16 k
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            float a = 0.f, w = 0.f;
            if (k < K) {
                if (m0 + r < M) { a = A[(size_t)(m0 + r) * lda + k]; if (round_a) a = round_bf16(a); }
                if (n0 + r < N) w = ld_w(W + (size_t)(n0 + r) * ldw + k);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][tm]);
            const float4 w = *reinterpret_cast<const float4*>(&Ws[kk][tn]);
            const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) lin_store(out + (size_t)m * ld_out + n, acc[i][j], bias, n, act, alpha, accumulate);
        }
    }
}

template <typename TW>
int launch_linear(const LinearArgs& a, cudaStream_t st) {
    const TW* W = reinterpret_cast<const TW*>(a.W);
    if (a.M <= MR) {
        const bool vec = a.K % 8 == 0 && a.lda % 4 == 0 && a.ldw % 8 == 0 && (reinterpret_cast<uintptr_t>(a.A) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(a.W) & 15) == 0;
        if (vec) {
            static bool attr_set = false;
            if (!attr_set) {
                B2_CUDA_CHECK(cudaFuncSetAttribute(linear_rows_vec_kernel<TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, RW_SMEM_FLOATS * 4));
                attr_set = true;
            }
            int kc_max = RW_SMEM_FLOATS / a.M / 8 * 8;
            // K in chunks accumulates through the output, which an activation forbids: such calls shrink nothing and take
            // the whole K when it fits at all, else the scalar kernel
            const int ngroups = (a.N + 8 * RW_COLS - 1) / (8 * RW_COLS);
            if (a.K <= kc_max || a.act == LIN_NONE) {
                const int grid = a.K <= kc_max ? std::min(ngroups, 3 * num_sms()) : ngroups;
                const size_t smem = (size_t)a.M * std::min(kc_max, a.K) * sizeof(float);
                linear_rows_vec_kernel<TW><<<grid, 256, smem, st>>>(a.A, a.lda, W, a.ldw, a.bias, a.out, a.ld_out, a.M, a.N, a.K, kc_max, a.act,
                                                                  a.alpha, a.accumulate, a.round_a);
                B2_LAUNCH_CHECK();
                return 0;
            }
        }
        {
            linear_rows_kernel<TW><<<(a.N + 7) / 8, 256, 0, st>>>(a.A, a.lda, W, a.ldw, a.bias, a.out, a.ld_out, a.M, a.N, a.K, a.act, a.alpha,
                                                                 a.accumulate, a.round_a);
        }
    } else {
        dim3 grid((a.N + TB - 1) / TB, (a.M + TB - 1) / TB);
        linear_tiled_kernel<TW><<<grid, 256, 0, st>>>(a.A, a.lda, W, a.ldw, a.bias, a.out, a.ld_out, a.M, a.N, a.K, a.act, a.alpha,
                                                      a.accumulate, a.round_a);
    }
    B2_LAUNCH_CHECK();
    return 0;
}
// ---- grouped Linear: every tile of output rows multiplies with the weight matrix of ITS group (mixture-of-experts) ------------
// 64-row tiles: the tiled kernel above with a per-tile weight matrix and gathered input rows. Tiles without a group return.
template <typename TW>
__global__ void __launch_bounds__(256) linear_grouped_tiled_kernel(GroupedLinearArgs g) {
    __shared__ float As[TK][TB + 4];
    __shared__ float Ws[TK][TB + 4];
    const int grp = g.tile_group[blockIdx.y];
    if (grp < 0) return;
    const TW* W = reinterpret_cast<const TW*>(g.W) + (size_t)grp * g.w_group_stride;
    const int tid = threadIdx.x, M = g.M, N = g.N, K = g.K;
    const int m0 = blockIdx.y * TB, n0 = blockIdx.x * TB;
    const int tm = (tid >> 4) * 4, tn = (tid & 15) * 4;
    // the tile's source rows: this thread stages rows r = (tid + e * 256) >> 4, e = 0..3
    int src[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int m = m0 + ((tid + e * 256) >> 4);
        src[e] = m < M ? (g.a_rows != nullptr ? g.a_rows[m] : m / g.a_div) : -1;
    }
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            float a = 0.f, w = 0.f;
            if (k < K) {
                if (src[e] >= 0) { a = g.A[(size_t)src[e] * g.lda + k]; if (g.round_a) a = round_bf16(a); }
                if (n0 + r < N) w = ld_w(W + (size_t)(n0 + r) * g.ldw + k);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][tm]);
            const float4 w = *reinterpret_cast<const float4*>(&Ws[kk][tn]);
            const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) lin_store(g.out + (size_t)m * g.ld_out + n, acc[i][j], nullptr, n, g.act, 1.f, 0);
        }
    }
}

// tiles of ONE row (a decode step: a handful of (token, choice) pairs): one warp per output column streams the weight row of
// the pair's group; VEC reads 16 bytes of weights per lane and step
template <typename TW, bool VEC>
__global__ void __launch_bounds__(256) linear_grouped_rows_kernel(GroupedLinearArgs g) {
    const int m = blockIdx.y;
    const int grp = g.tile_group[m];
    if (grp < 0) return;
    const int src = g.a_rows != nullptr ? g.a_rows[m] : m / g.a_div;
    if (src < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= g.N) return;
    const TW* w = reinterpret_cast<const TW*>(g.W) + (size_t)grp * g.w_group_stride + (size_t)n * g.ldw;
    const TW* w2 = w + (size_t)g.N * g.ldw;   // swiglu: the group's matrix is [gate rows | up rows] of N rows each
    const float* a = g.A + (size_t)src * g.lda;
    float acc = 0.f, acc2 = 0.f;
    if (VEC) {
        for (int k0 = lane * 8; k0 < g.K; k0 += 256) {
            float wv[8], av[8], uv[8];
            ld_w8(w + k0, wv);
            if (g.swiglu) ld_w8(w2 + k0, uv);
            ld_w8(a + k0, av);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float x = g.round_a ? round_bf16(av[e]) : av[e];
                acc = fmaf(x, wv[e], acc);
                if (g.swiglu) acc2 = fmaf(x, uv[e], acc2);
            }
        }
    } else {
        for (int k = lane; k < g.K; k += 32) {
            const float av = a[k], x = g.round_a ? round_bf16(av) : av;
            acc = fmaf(x, ld_w(w + k), acc);
            if (g.swiglu) acc2 = fmaf(x, ld_w(w2 + k), acc2);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { acc += __shfl_xor_sync(0xffffffffu, acc, o); acc2 += __shfl_xor_sync(0xffffffffu, acc2, o); }
    if (lane == 0) {
        if (g.swiglu) g.out[(size_t)m * g.ld_out + n] = glu_act(acc, acc2, GluAct{g.glu_slope, g.glu_limit, g.glu_up_shift});   // silu(gate) * up, or its bounded form
        else lin_store(g.out + (size_t)m * g.ld_out + n, acc, nullptr, n, g.act, 1.f, 0);
    }
}

// batched small Linears of a decode step: block = 8 output columns of one batch entry (a head), one warp per column; the
// weight row is read once and multiplied with every row of the step
template <typename TW, bool VEC>
__global__ void __launch_bounds__(256) linear_batched_rows_kernel(const float* __restrict__ A, int64_t lda, int64_t a_bs, const TW* __restrict__ W,
                                                                  int64_t w_bs, float* __restrict__ out, int64_t ld_out, int64_t o_bs, int M, int N,
                                                                  int K, int round_a, const float* __restrict__ gate, int64_t ldg) {
    const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const TW* w = W + (size_t)b * w_bs + (size_t)n * K;
    const float* a = A + (size_t)b * a_bs;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
    if (VEC) {
        for (int k0 = lane * 8; k0 < K; k0 += 256) {
            float wv[8];
            ld_w8(w + k0, wv);
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                if (m < M) {
                    float av[8];
                    ld_w8(a + (size_t)m * lda + k0, av);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[m] = fmaf(round_a ? round_bf16(av[e]) : av[e], wv[e], acc[m]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = ld_w(w + k);
#pragma unroll
            for (int m = 0; m < MR; ++m)
                if (m < M) { const float av = a[(size_t)m * lda + k]; acc[m] = fmaf(round_a ? round_bf16(av) : av, wv, acc[m]); }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        // gate: one sigmoid gate per (row, batch entry), e.g. a head's output gate
        if (lane == 0 && m < M) out[(size_t)m * ld_out + (size_t)b * o_bs + n] = gate != nullptr ? v / (1.f + expf(-gate[(size_t)m * ldg + b])) : v;
    }
}

template <typename TW>
int launch_batched_rows(const float* A, int64_t lda, int64_t a_bs, const void* W, int64_t w_bs, float* out, int64_t ld_out, int64_t o_bs, int batch, int M,
                        int N, int K, int round_a, const float* gate, int64_t ldg, cudaStream_t st) {
    const bool vec = K % 8 == 0 && lda % 4 == 0 && a_bs % 4 == 0 && w_bs % 8 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(W) & 15) == 0;
    dim3 grid((N + 7) / 8, batch);
    const TW* w = reinterpret_cast<const TW*>(W);
    if (vec) linear_batched_rows_kernel<TW, true><<<grid, 256, 0, st>>>(A, lda, a_bs, w, w_bs, out, ld_out, o_bs, M, N, K, round_a, gate, ldg);
    else linear_batched_rows_kernel<TW, false><<<grid, 256, 0, st>>>(A, lda, a_bs, w, w_bs, out, ld_out, o_bs, M, N, K, round_a, gate, ldg);
    B2_LAUNCH_CHECK();
    return 0;
}

template <typename TW>
int launch_grouped(const GroupedLinearArgs& g, cudaStream_t st) {
    if (g.tile_rows == 1) {
        const bool vec = g.K % 8 == 0 && g.lda % 4 == 0 && g.ldw % 8 == 0 && g.w_group_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(g.A) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(g.W) & 15) == 0;
        dim3 grid((g.N + 7) / 8, g.M);
        if (vec) linear_grouped_rows_kernel<TW, true><<<grid, 256, 0, st>>>(g);
        else linear_grouped_rows_kernel<TW, false><<<grid, 256, 0, st>>>(g);
    } else {
        dim3 grid((g.N + TB - 1) / TB, (g.M + TB - 1) / TB);
        linear_grouped_tiled_kernel<TW><<<grid, 256, 0, st>>>(g);
    }
    B2_LAUNCH_CHECK();
    return 0;
}
}  // namespace

int linear_batched_rows_f32(const float* A, int64_t lda, int64_t a_bs, const void* W, int64_t w_bs, int w_dtype, float* out, int64_t ld_out,
                            int64_t o_bs, int batch, int M, int N, int K, int round_a, cudaStream_t st, const float* gate, int64_t ldg) {
    B2_CHECK_ARG(A && W && out && batch > 0 && M > 0 && M <= MR && N > 0 && K > 0, "linear_batched_rows: bad argument (batch=%d M=%d N=%d K=%d)", batch, M, N, K);
    B2_CHECK_ARG(w_dtype == DT_F32 || w_dtype == DT_BF16, "linear_batched_rows: weights must be fp32 or bf16");
    return w_dtype == DT_F32 ? launch_batched_rows<float>(A, lda, a_bs, W, w_bs, out, ld_out, o_bs, batch, M, N, K, round_a, gate, ldg, st)
                             : launch_batched_rows<__nv_bfloat16>(A, lda, a_bs, W, w_bs, out, ld_out, o_bs, batch, M, N, K, round_a, gate, ldg, st);
}

int linear_grouped_f32(const GroupedLinearArgs& g, cudaStream_t st) {
    B2_CHECK_ARG(g.A && g.W && g.out && g.tile_group && g.M > 0 && g.N > 0 && g.K > 0, "linear_grouped: bad argument (M=%d N=%d K=%d)", g.M, g.N, g.K);
    B2_CHECK_ARG(g.tile_rows == 1 || g.tile_rows == TB, "linear_grouped: tiles of 1 or %d rows", TB);
    B2_CHECK_ARG(!g.swiglu || g.tile_rows == 1, "linear_grouped: the gated form is for tiles of one row");
    B2_CHECK_ARG(g.a_rows != nullptr || g.a_div >= 1, "linear_grouped: no source rows");
    B2_CHECK_ARG(g.w_dtype == DT_F32 || g.w_dtype == DT_BF16, "linear_grouped: weights must be fp32 or bf16");
    return g.w_dtype == DT_F32 ? launch_grouped<float>(g, st) : launch_grouped<__nv_bfloat16>(g, st);
}

namespace {
__global__ void cast_rows_bf16_kernel(const float* __restrict__ A, int64_t lda, __nv_bfloat16* __restrict__ out, int64_t ld_out, int K) {
    const size_t r = blockIdx.y;
    const int k = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (k + 1 < K) {
        *reinterpret_cast<__nv_bfloat162*>(out + r * ld_out + k) = __floats2bfloat162_rn(A[r * lda + k], A[r * lda + k + 1]);
    } else if (k < K) {
        out[r * ld_out + k] = __float2bfloat16_rn(A[r * lda + k]);
    }
}
}  // namespace

int cast_rows_bf16(const float* A, int64_t lda, void* out, int64_t ld_out, int M, int K, cudaStream_t st) {
    B2_CHECK_ARG(A && out && M > 0 && K > 0 && ld_out % 2 == 0, "cast_rows_bf16: bad argument");
    cast_rows_bf16_kernel<<<dim3((K / 2 + 256) / 256, M), 256, 0, st>>>(A, lda, reinterpret_cast<__nv_bfloat16*>(out), ld_out, K);
    B2_LAUNCH_CHECK();
    return 0;
}

int linear_f32(const LinearArgs& a, cudaStream_t st) {
    B2_CHECK_ARG(a.A && a.W && a.out && a.M > 0 && a.N > 0 && a.K > 0, "linear: bad argument (M=%d N=%d K=%d)", a.M, a.N, a.K);
    B2_CHECK_ARG(a.w_dtype == DT_F32 || a.w_dtype == DT_BF16, "linear: weights must be fp32 or bf16");
    return a.w_dtype == DT_F32 ? launch_linear<float>(a, st) : launch_linear<__nv_bfloat16>(a, st);
}

}  // namespace b2
