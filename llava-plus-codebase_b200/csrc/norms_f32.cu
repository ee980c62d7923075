// fp32 normalisations and row helpers of the layer-list decoders: LayerNorm of a sublayer's output added to the residual
// stream, gathered LayerNorm in front of the output head, grouped unit-RMS norm with a SiLU gate (before or after the
// norm), embedding rows as fp32, the row map of a call; for pre-norm blocks: the one-number RMS norm (with the opening of a
// looped pass folded in), the weighted RMS norm (plain, gathered, or added onto the residual stream), PolyNorm, the logit soft-cap, per-head sigmoid gates, token + hashed-bigram embedding, and the
// normalised latent row of a low-rank key/value cache. Statistics, sums and outputs are fp32 throughout; any width.
#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// sum over the block; every thread gets the result. `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // red may still be read from the previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// mean, then the mean of squared deviations (two passes over the row, which sits in L1 after the first)
__device__ __forceinline__ void row_stats(const float* y, int cols, float eps, float* red, float& mean, float& rstd) {
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += y[c];
    mean = block_sum(s, red) / (float)cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) { const float d = y[c] - mean; q = fmaf(d, d, q); }
    const float var = block_sum(q, red) / (float)cols;
    rstd = 1.f / sqrtf(var + eps);
}

__global__ void layernorm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, int cols, float eps) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const float* yr = y + r * cols;
    float mean, rstd;
    row_stats(yr, cols, eps, red, mean, rstd);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) x[r * cols + c] += (yr[c] - mean) * rstd * gamma[c] + beta[c];
}

__global__ void layernorm_gather_kernel(const float* __restrict__ x, const int32_t* __restrict__ row_index, const float* __restrict__ gamma,
                                        const float* __restrict__ beta, float* __restrict__ out, int cols, float eps) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const float* xr = x + (size_t)(row_index != nullptr ? row_index[r] : (int)r) * cols;  // null index: row r itself
    float mean, rstd;
    row_stats(xr, cols, eps, red, mean, rstd);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) out[r * cols + c] = (xr[c] - mean) * rstd * gamma[c] + beta[c];
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// one warp per (row, group)
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, int64_t ldy, const float* __restrict__ z, int64_t ldz,
                                           const float* __restrict__ gamma, float* __restrict__ out, int64_t ldo, int rows, int groups, int group,
                                           int gate_first, int gamma_shared, float eps) {
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows * groups) return;
    const int r = w / groups, g = w % groups;
    const float* yr = y + (size_t)r * ldy + (size_t)g * group;
    const float* zr = z != nullptr ? z + (size_t)r * ldz + (size_t)g * group : nullptr;   // null: no gate
    const float* gm = gamma + (gamma_shared ? 0 : (size_t)g * group);                      // one weight vector for all groups, or one each
    float q = 0.f;
    for (int c = lane; c < group; c += 32) {
        const float v = (gate_first && zr != nullptr) ? yr[c] * silu_f(zr[c]) : yr[c];
        q = fmaf(v, v, q);
    }
    q = warp_sum(q);
    const float rinv = 1.f / sqrtf(q / (float)group + eps);
    float* o = out + (size_t)r * ldo + (size_t)g * group;
    for (int c = lane; c < group; c += 32) {
        const float gz = zr != nullptr ? silu_f(zr[c]) : 1.f;
        o[c] = gate_first ? (yr[c] * gz) * rinv * gm[c] : yr[c] * rinv * gm[c] * gz;
    }
}

// differential attention: one warp per (row, head) subtracts lambda times the second map's output from the first map's and brings
// the difference to unit RMS
__global__ void diff_combine_kernel(const float* __restrict__ y, int64_t ldy, float* __restrict__ out, int64_t ldo, int rows, int heads, int dv,
                                    float lambda, float out_scale, float eps) {
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows * heads) return;
    const int r = w / heads, h = w % heads;
    const float* a1 = y + (size_t)r * ldy + (size_t)h * dv;
    const float* a2 = a1 + (size_t)heads * dv;
    float q = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float d = fmaf(-lambda, a2[c], a1[c]);
        q = fmaf(d, d, q);
    }
    q = warp_sum(q);
    const float mul = out_scale / sqrtf(q / (float)dv + eps);
    float* o = out + (size_t)r * ldo + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) o[c] = fmaf(-lambda, a2[c], a1[c]) * mul;
}

template <typename TT>
__global__ void embed_rows_kernel(const int32_t* __restrict__ tokens, const TT* __restrict__ table, float* __restrict__ x, int cols, int vocab,
                                  int* err_flag, float scale) {
    const size_t r = blockIdx.x;
    const int t = tokens[r];
    const bool ok = t >= 0 && t < vocab;
    if (!ok && threadIdx.x == 0 && err_flag != nullptr) err_flag[0] = 1;  // slot 0 = B2_ERR_TOKEN_RANGE
    for (int c = threadIdx.x; c < cols; c += blockDim.x) x[r * cols + c] = ok ? (float)table[(size_t)t * cols + c] * scale : 0.f;
}

__global__ void sigmoid_gate_kernel(const float* __restrict__ a, int64_t lda, const float* __restrict__ g, int64_t ldg, float* __restrict__ out,
                                    int64_t ldo, int cols) {
    const size_t r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < cols) out[r * ldo + c] = a[r * lda + c] / (1.f + expf(-g[r * ldg + c]));
}

// ---- pre-norm blocks with a one-number RMS norm -----------------------------------------------------------------------------
// out[i] = x[row_index[i]] / sqrt(mean(x^2) + eps) * g[0]; with `add`/`vec` the row is first updated in place:
// x += add[row] + vec (the opening of a pass of a looped block of layers)
__global__ void rms_scalar_kernel(float* __restrict__ x, const int32_t* __restrict__ row_index, const float* __restrict__ g,
                                  const float* __restrict__ add, const float* __restrict__ vec, float* __restrict__ out, int cols, float eps) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const size_t src = row_index != nullptr ? (size_t)row_index[r] : r;
    float* xr = x + src * cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float v = xr[c];
        if (add != nullptr || vec != nullptr) {
            v += (add != nullptr ? add[src * cols + c] : 0.f) + (vec != nullptr ? vec[c] : 0.f);
            xr[c] = v;
        }
        q = fmaf(v, v, q);
    }
    if (out == nullptr) return;   // only the update of x was asked for
    const float mul = g[0] / sqrtf(block_sum(q, red) / (float)cols + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) out[r * cols + c] = xr[c] * mul;
}

// weighted RMS norm of a (gathered) row; accumulate: added onto out
__global__ void rms_weight_kernel(const float* __restrict__ in, int64_t ld_in, const int32_t* __restrict__ row_index, const float* __restrict__ w,
                                  float* __restrict__ out, int64_t ld_out, int accumulate, int cols, float eps) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const float* xr = in + (row_index != nullptr ? (size_t)row_index[r] : r) * ld_in;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) q = fmaf(xr[c], xr[c], q);
    const float mul = 1.f / sqrtf(block_sum(q, red) / (float)cols + eps);
    float* o = out + r * ld_out;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = xr[c] * mul * w[c];
        o[c] = accumulate ? o[c] + v : v;
    }
}

// post-norm add of one sublayer, pre-norm of the next, and (decode steps) the input convolution with its carried inputs
__global__ void sandwich_norm_kernel(SandwichNormArgs a) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const int cols = a.cols;
    float* xr = a.x + r * cols;
    float q = 0.f;
    if (a.y != nullptr) {
        const float* yr = a.y + r * cols;
        float qy = 0.f;
#pragma unroll 4
        for (int c = threadIdx.x; c < cols; c += blockDim.x) qy = fmaf(yr[c], yr[c], qy);
        const float mul = 1.f / sqrtf(block_sum(qy, red) / (float)cols + a.eps);
#pragma unroll 4
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            const float v = fmaf(yr[c] * mul, a.w_post[c], xr[c]);
            xr[c] = v;
            q = fmaf(v, v, q);
        }
    } else {
#pragma unroll 4
        for (int c = threadIdx.x; c < cols; c += blockDim.x) q = fmaf(xr[c], xr[c], q);
    }
    if (a.w_pre == nullptr) return;
    const float mul = 1.f / sqrtf(block_sum(q, red) / (float)cols + a.eps);
    float* o = a.out + r * cols;
    if (a.conv_w == nullptr) {
#pragma unroll 4
        for (int c = threadIdx.x; c < cols; c += blockDim.x) o[c] = xr[c] * mul * a.w_pre[c];
        return;
    }
    const SeqSeg sg = a.segs[r];
    const int taps = a.taps;
    float* tl = a.tail + (size_t)sg.slot * (taps - 1) * cols;
    float* co = a.conv_out + r * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = xr[c] * mul * a.w_pre[c];
        o[c] = v;
        if (sg.n <= 0) continue;
        const float* wc = a.conv_w + (size_t)c * taps;
        float acc = fmaf(wc[taps - 1], v, v);
        for (int j = 0; j < taps - 1; ++j) {
            const float old = sg.pos0 > 0 ? tl[(size_t)j * cols + c] : 0.f;
            acc = fmaf(wc[j], old, acc);
            if (j > 0) tl[(size_t)(j - 1) * cols + c] = old;
        }
        if (taps > 1) tl[(size_t)(taps - 2) * cols + c] = v;
        co[c] = acc;
    }
}

// the same for rows of at most blockDim.x * V entries: a thread keeps its V entries in registers and the row is read once. Everything
// the kernel will need (both weights, and with TP > 0 the up to TP carried inputs and TP + 1 taps of the fused convolution) is loaded
// in front of the first reduction, so the launch costs one memory round trip and not one per pass (a decode step has ONE block per
// row and is bound by round trips, not by bandwidth).
template <int V, int TP>
__global__ void __launch_bounds__(512) sandwich_norm_reg_kernel(SandwichNormArgs a) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const int cols = a.cols, tid = threadIdx.x, nt = blockDim.x;
    float* xr = a.x + r * cols;
    float xv[V], yv[V], wpost[V], wpre[V];
    float old[TP > 0 ? TP : 1][V], cw[TP + 1][V];
    const bool conv = TP > 0 && a.conv_w != nullptr;
    const int taps = a.taps;
    SeqSeg sg = {0, 0, 0, 0};
    if (conv) sg = a.segs[r];
    float* tl = conv ? a.tail + (size_t)sg.slot * (taps - 1) * cols : nullptr;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = tid + i * nt;
        const bool ok = c < cols;
        xv[i] = ok ? xr[c] : 0.f;
        yv[i] = (ok && a.y != nullptr) ? a.y[r * cols + c] : 0.f;
        wpost[i] = (ok && a.y != nullptr) ? a.w_post[c] : 0.f;
        wpre[i] = (ok && a.w_pre != nullptr) ? a.w_pre[c] : 0.f;
        if (TP > 0) {
#pragma unroll
            for (int j = 0; j < TP; ++j) {   // carried input j and tap j, right-aligned: entry TP - 1 is the newest carried input
                const int tj = j - (TP - (taps - 1));
                old[j][i] = (conv && ok && tj >= 0 && sg.pos0 > 0) ? tl[(size_t)tj * cols + c] : 0.f;
                cw[j][i] = (conv && ok && tj >= 0) ? a.conv_w[(size_t)c * taps + tj] : 0.f;
            }
            cw[TP][i] = (conv && ok) ? a.conv_w[(size_t)c * taps + taps - 1] : 0.f;
        }
    }
    if (a.y != nullptr) {
        float qy = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) qy = fmaf(yv[i], yv[i], qy);
        const float mul = 1.f / sqrtf(block_sum(qy, red) / (float)cols + a.eps);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int c = tid + i * nt;
            xv[i] = fmaf(yv[i] * mul, wpost[i], xv[i]);
            if (c < cols) xr[c] = xv[i];
        }
    }
    if (a.w_pre == nullptr) return;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) q = fmaf(xv[i], xv[i], q);
    const float mul = 1.f / sqrtf(block_sum(q, red) / (float)cols + a.eps);
    float* o = a.out + r * cols;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = tid + i * nt;
        xv[i] = xv[i] * mul * wpre[i];
        if (c < cols) o[c] = xv[i];
    }
    if (!conv || sg.n <= 0) return;
    float* co = a.conv_out + r * cols;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = tid + i * nt;
        if (c >= cols) continue;
        float acc = fmaf(cw[TP][i], xv[i], xv[i]);
#pragma unroll
        for (int j = 0; j < TP; ++j) {
            acc = fmaf(cw[j][i], old[j][i], acc);
            const int tj = j - (TP - (taps - 1));
            if (tj >= 1) tl[(size_t)(tj - 1) * cols + c] = old[j][i];
        }
        if (taps > 1) tl[(size_t)(taps - 2) * cols + c] = xv[i];
        co[c] = acc;
    }
}

// dst[b][c][r] = src[b][r][c] for elements of 2 or 4 bytes
template <typename T>
__global__ void transpose_blocks_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows, int cols) {
    const size_t b = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows * cols) dst[b * rows * cols + (size_t)(i % cols) * rows + i / cols] = src[b * rows * cols + i];
}

// PolyNorm: out = a N(z) + b N(z^2) + c N(z^3) + e with z = in + bias, powers element-wise, N = division by the row's root mean square
__global__ void polynorm_kernel(const float* __restrict__ in, int64_t ld_in, const float* __restrict__ bias, const float* __restrict__ coef,
                                float* __restrict__ out, int64_t ld_out, int cols, float eps, int vec) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const float* zr = in + r * ld_in;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    if (vec) {   // 16 bytes at a time, four loads in flight: a decode step has ONE block per row and is bound by memory round trips
        const float4* z4 = reinterpret_cast<const float4*>(zr);
        const float4* b4 = reinterpret_cast<const float4*>(bias);
#pragma unroll 4
        for (int c = threadIdx.x; c < cols / 4; c += blockDim.x) {
            float4 z = z4[c];
            if (bias != nullptr) { const float4 b = b4[c]; z.x += b.x; z.y += b.y; z.z += b.z; z.w += b.w; }
            const float q0 = z.x * z.x, q1 = z.y * z.y, q2 = z.z * z.z, q3 = z.w * z.w;
            s2 += (q0 + q1) + (q2 + q3);
            s4 += fmaf(q0, q0, q1 * q1) + fmaf(q2, q2, q3 * q3);
            s6 += fmaf(q0 * q0, q0, q1 * q1 * q1) + fmaf(q2 * q2, q2, q3 * q3 * q3);
        }
    } else {
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            const float z = zr[c] + (bias != nullptr ? bias[c] : 0.f), z2 = z * z;
            s2 += z2; s4 = fmaf(z2, z2, s4); s6 = fmaf(z2 * z2, z2, s6);
        }
    }
    const float n = (float)cols;
    const float r1 = coef[0] / sqrtf(block_sum(s2, red) / n + eps);
    const float r2 = coef[1] / sqrtf(block_sum(s4, red) / n + eps);
    const float r3 = coef[2] / sqrtf(block_sum(s6, red) / n + eps);
    const float e = coef[3];
    if (vec) {
        const float4* z4 = reinterpret_cast<const float4*>(zr);
        const float4* b4 = reinterpret_cast<const float4*>(bias);
        float4* o4 = reinterpret_cast<float4*>(out + r * ld_out);
#pragma unroll 4
        for (int c = threadIdx.x; c < cols / 4; c += blockDim.x) {
            float4 z = z4[c];
            if (bias != nullptr) { const float4 b = b4[c]; z.x += b.x; z.y += b.y; z.z += b.z; z.w += b.w; }
            o4[c] = make_float4(fmaf(z.x, fmaf(z.x, fmaf(z.x, r3, r2), r1), e), fmaf(z.y, fmaf(z.y, fmaf(z.y, r3, r2), r1), e),
                                fmaf(z.z, fmaf(z.z, fmaf(z.z, r3, r2), r1), e), fmaf(z.w, fmaf(z.w, fmaf(z.w, r3, r2), r1), e));
        }
    } else {
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            const float z = zr[c] + (bias != nullptr ? bias[c] : 0.f);
            out[r * ld_out + c] = fmaf(z, fmaf(z, fmaf(z, r3, r2), r1), e);
        }
    }
}

// x[i] = cap * tanh(x[i] / cap)
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// out[r, h * dv + d] = a[r, h * dv + d] * sigmoid(g[r, h]): one gate per head
__global__ void head_gate_kernel(const float* __restrict__ a, int64_t lda, const float* __restrict__ g, int64_t ldg, float* __restrict__ out,
                                 int64_t ldo, int heads, int dv) {
    const size_t r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < heads * dv) out[r * ldo + c] = a[r * lda + c] / (1.f + expf(-g[r * ldg + c / dv]));
}

// Token embedding plus a hashed bigram row: x[row] = table[tok] + bigram[(prev * mul_prev + tok * mul_cur) mod buckets]; the first
// token of a sequence takes row `buckets`. The previous token of a call's first row is the slot's carried token, which the same
// block then replaces by the segment's last token. x0 (nullable) receives a copy of the rows.
template <typename TT>
__global__ void embed_bigram_kernel(const int32_t* __restrict__ tokens, const SeqSeg* __restrict__ segs, const TT* __restrict__ table,
                                    const TT* __restrict__ bigram, int32_t* __restrict__ last_tok, float* __restrict__ x, float* __restrict__ x0,
                                    int cols, int vocab, int buckets, int mul_prev, int mul_cur, int* err_flag) {
    const SeqSeg sg = segs[blockIdx.y];
    const int t = blockIdx.x;
    if (t >= sg.n) return;
    const size_t r = (size_t)sg.row0 + t;
    const int tok = tokens[r];
    int prev = -1;
    if (t > 0) prev = tokens[r - 1];
    else if (sg.pos0 > 0) prev = last_tok[sg.slot];
    __syncthreads();   // every thread has read the carried token before thread 0 replaces it
    if (t == 0 && threadIdx.x == 0) last_tok[sg.slot] = tokens[(size_t)sg.row0 + sg.n - 1];
    const bool ok = tok >= 0 && tok < vocab && prev < vocab;
    if (!ok && threadIdx.x == 0 && err_flag != nullptr) err_flag[0] = 1;  // slot 0 = B2_ERR_TOKEN_RANGE
    long long brow = buckets;
    if (prev >= 0) brow = (long long)(((unsigned long long)prev * (unsigned long long)mul_prev + (unsigned long long)tok * (unsigned long long)mul_cur) %
                                      (unsigned long long)buckets);
#pragma unroll 4
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float v = 0.f;
        if (ok) {
            v = (float)table[(size_t)tok * cols + c];
            if (bigram != nullptr) v += (float)bigram[(size_t)brow * cols + c];
        }
        x[r * cols + c] = v;
        if (x0 != nullptr) x0[r * cols + c] = v;
    }
}

// latent[slot][pos] = unit_rms(in[r]) * gamma: the normalised low-rank row that a token leaves in the cache
__global__ void latent_append_kernel(const float* __restrict__ in, int64_t ld_in, const float* __restrict__ gamma, float* __restrict__ cache,
                                     const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos, int rank, int Smax, float eps) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const int pos = row_pos[r];
    if (pos < 0) return;
    const float* src = in + r * ld_in;
    float q = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) q = fmaf(src[c], src[c], q);
    const float mul = 1.f / sqrtf(block_sum(q, red) / (float)rank + eps);
    float* dst = cache + ((size_t)row_slot[r] * Smax + pos) * rank;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = src[c] * mul * gamma[c];
}

__global__ void rowmap_portion_kernel(SeqSeg* segs, int32_t* row_slot, int32_t* row_pos, int32_t* len, int slot, int n, int restart) {
    const int pos0 = restart ? 0 : len[slot];
    __syncthreads();
    for (int r = threadIdx.x; r < n; r += blockDim.x) { row_slot[r] = slot; row_pos[r] = pos0 + r; }
    if (threadIdx.x == 0) {
        segs[0].slot = slot; segs[0].row0 = 0; segs[0].n = n; segs[0].pos0 = pos0;
        len[slot] = pos0 + n;
    }
}

__global__ void rowmap_decode_kernel(SeqSeg* segs, int32_t* row_slot, int32_t* row_pos, const int32_t* len, const SampleState* sstate,
                                     const RowState* rows_state, int slot0, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int slot = slot0 + b;
    // per-slot mode (continuous batching): a slot that is not armed keeps its state, cache rows and length
    const bool live = sstate == nullptr || rows_state == nullptr || sstate->per_row == 0 || rows_state[slot].active != 0;
    const int pos = len[slot];
    segs[b].slot = slot; segs[b].row0 = b; segs[b].n = live ? 1 : 0; segs[b].pos0 = pos;
    row_slot[b] = slot;
    row_pos[b] = live ? pos : -1;
}
}  // namespace

int layernorm_add_f32(float* x, const float* y, const float* gamma, const float* beta, int rows, int cols, float eps, cudaStream_t st) {
    B2_CHECK_ARG(x && y && gamma && beta && rows > 0 && cols > 0, "layernorm_add: bad argument");
    layernorm_add_kernel<<<rows, cols >= 1024 ? 256 : 128, 0, st>>>(x, y, gamma, beta, cols, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int layernorm_gather_f32(const float* x, const int32_t* row_index, const float* gamma, const float* beta, float* out, int rows, int cols,
                         float eps, cudaStream_t st) {
    B2_CHECK_ARG(x && gamma && beta && out && rows > 0 && cols > 0, "layernorm_gather: bad argument");
    layernorm_gather_kernel<<<rows, cols >= 1024 ? 256 : 128, 0, st>>>(x, row_index, gamma, beta, out, cols, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int gated_group_rmsnorm_f32(const float* y, int64_t ldy, const float* z, int64_t ldz, const float* gamma, float* out, int64_t ldo, int rows,
                            int cols, int group, int gate_first, float eps, cudaStream_t st, int gamma_shared) {
    B2_CHECK_ARG(y && z && gamma && out && rows > 0 && group > 0 && cols % group == 0, "gated_group_rmsnorm: cols %d is not a multiple of the group %d",
                 cols, group);
    const int groups = cols / group, warps = rows * groups;
    gated_group_rmsnorm_kernel<<<(warps + 7) / 8, 256, 0, st>>>(y, ldy, z, ldz, gamma, out, ldo, rows, groups, group, gate_first, gamma_shared, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int group_rmsnorm_f32(const float* y, int64_t ldy, const float* gamma, int gamma_shared, float* out, int64_t ldo, int rows, int cols, int group,
                      float eps, cudaStream_t st) {
    B2_CHECK_ARG(y && gamma && out && rows > 0 && group > 0 && cols % group == 0, "group_rmsnorm: cols %d is not a multiple of the group %d", cols, group);
    const int groups = cols / group, warps = rows * groups;
    gated_group_rmsnorm_kernel<<<(warps + 7) / 8, 256, 0, st>>>(y, ldy, nullptr, 0, gamma, out, ldo, rows, groups, group, 0, gamma_shared, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int diff_combine_f32(const float* y, int64_t ldy, float* out, int64_t ldo, int rows, int heads, int dv, float lambda, float out_scale, float eps,
                     cudaStream_t st) {
    B2_CHECK_ARG(y && out && y != out && rows > 0 && heads > 0 && dv > 0, "diff_combine: bad argument");
    const int warps = rows * heads;
    diff_combine_kernel<<<(warps + 7) / 8, 256, 0, st>>>(y, ldy, out, ldo, rows, heads, dv, lambda, out_scale, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int embed_rows_f32(const int32_t* tokens, const void* table, int table_dtype, float* x, int rows, int cols, int vocab, int* err_flag,
                   cudaStream_t st, float scale) {
    B2_CHECK_ARG(tokens && table && x && rows > 0, "embed_rows: bad argument");
    if (table_dtype == DT_F32)
        embed_rows_kernel<float><<<rows, 128, 0, st>>>(tokens, reinterpret_cast<const float*>(table), x, cols, vocab, err_flag, scale);
    else
        embed_rows_kernel<__nv_bfloat16><<<rows, 128, 0, st>>>(tokens, reinterpret_cast<const __nv_bfloat16*>(table), x, cols, vocab, err_flag, scale);
    B2_LAUNCH_CHECK();
    return 0;
}

int sigmoid_gate_f32(const float* a, int64_t lda, const float* g, int64_t ldg, float* out, int64_t ldo, int rows, int cols, cudaStream_t st) {
    B2_CHECK_ARG(a && g && out && rows > 0 && cols > 0, "sigmoid_gate: bad argument");
    sigmoid_gate_kernel<<<dim3((cols + 255) / 256, rows), 256, 0, st>>>(a, lda, g, ldg, out, ldo, cols);
    B2_LAUNCH_CHECK();
    return 0;
}

int rms_scalar_f32(float* x, const int32_t* row_index, const float* g, const float* add, const float* vec, float* out, int rows, int cols,
                   float eps, cudaStream_t st) {
    B2_CHECK_ARG(x && rows > 0 && cols > 0 && ((g && out) || (!out && (add || vec))), "rms_scalar: bad argument");
    rms_scalar_kernel<<<rows, cols >= 1024 ? 256 : 128, 0, st>>>(x, row_index, g, add, vec, out, cols, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int rms_weight_f32(const float* in, int64_t ld_in, const int32_t* row_index, const float* w, float* out, int64_t ld_out, int accumulate, int rows,
                   int cols, float eps, cudaStream_t st) {
    B2_CHECK_ARG(in && w && out && rows > 0 && cols > 0, "rms_weight: bad argument");
    rms_weight_kernel<<<rows, cols >= 1024 ? 256 : 128, 0, st>>>(in, ld_in, row_index, w, out, ld_out, accumulate, cols, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int sandwich_norm_f32(const SandwichNormArgs& a, cudaStream_t st) {
    B2_CHECK_ARG(a.x && a.rows > 0 && a.cols > 0 && (a.y == nullptr) == (a.w_post == nullptr) && (a.w_pre == nullptr || a.out != nullptr), "sandwich_norm: bad argument");
    B2_CHECK_ARG(a.conv_w == nullptr || (a.w_pre && (a.tail || a.taps == 1) && a.segs && a.conv_out && a.taps >= 1 && a.taps <= 16), "sandwich_norm: the fused convolution needs taps, tail and segments");
    // rows of up to 4096 entries live in registers (4 entries per thread for narrow rows, 8 otherwise); the fused convolution rides in
    // that kernel with up to 4 taps, and in the plain one otherwise
    const bool conv = a.conv_w != nullptr;
    if (a.cols <= 4096 && (!conv || a.taps <= 4)) {
        const int t4 = (a.cols + 127) / 128 * 32, t8 = (a.cols + 255) / 256 * 32;
        if (a.cols <= 512) { if (conv) sandwich_norm_reg_kernel<4, 3><<<a.rows, t4, 0, st>>>(a); else sandwich_norm_reg_kernel<4, 0><<<a.rows, t4, 0, st>>>(a); }
        else { if (conv) sandwich_norm_reg_kernel<8, 3><<<a.rows, t8, 0, st>>>(a); else sandwich_norm_reg_kernel<8, 0><<<a.rows, t8, 0, st>>>(a); }
    } else {
        sandwich_norm_kernel<<<a.rows, 256, 0, st>>>(a);
    }
    B2_LAUNCH_CHECK();
    return 0;
}

int transpose_blocks(const void* src, void* dst, int blocks, int rows, int cols, int elem_size, cudaStream_t st) {
    B2_CHECK_ARG(src && dst && blocks > 0 && rows > 0 && cols > 0 && (elem_size == 2 || elem_size == 4), "transpose_blocks: bad argument");
    dim3 grid((rows * cols + 255) / 256, blocks);
    if (elem_size == 2) transpose_blocks_kernel<uint16_t><<<grid, 256, 0, st>>>(reinterpret_cast<const uint16_t*>(src), reinterpret_cast<uint16_t*>(dst), rows, cols);
    else transpose_blocks_kernel<uint32_t><<<grid, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(src), reinterpret_cast<uint32_t*>(dst), rows, cols);
    B2_LAUNCH_CHECK();
    return 0;
}

int polynorm_f32(const float* in, int64_t ld_in, const float* bias, const float* coef, float* out, int64_t ld_out, int rows, int cols, float eps,
                 cudaStream_t st) {
    B2_CHECK_ARG(in && coef && out && rows > 0 && cols > 0, "polynorm: bad argument");
    const int vec = cols % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                                                                            reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
    polynorm_kernel<<<rows, cols >= 4096 ? 512 : (cols >= 1024 ? 256 : 128), 0, st>>>(in, ld_in, bias, coef, out, ld_out, cols, eps, vec);
    B2_LAUNCH_CHECK();
    return 0;
}

int softcap_f32(float* x, size_t n, float cap, cudaStream_t st) {
    B2_CHECK_ARG(x && n > 0 && cap > 0.f, "softcap: bad argument");
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, n, cap);
    B2_LAUNCH_CHECK();
    return 0;
}

int head_gate_f32(const float* a, int64_t lda, const float* g, int64_t ldg, float* out, int64_t ldo, int rows, int heads, int dv, cudaStream_t st) {
    B2_CHECK_ARG(a && g && out && rows > 0 && heads > 0 && dv > 0, "head_gate: bad argument");
    head_gate_kernel<<<dim3((heads * dv + 255) / 256, rows), 256, 0, st>>>(a, lda, g, ldg, out, ldo, heads, dv);
    B2_LAUNCH_CHECK();
    return 0;
}

int embed_bigram_rows_f32(const int32_t* tokens, const SeqSeg* segs, int nseg, int max_n, const void* table, const void* bigram, int table_dtype,
                          int32_t* last_tok, float* x, float* x0, int cols, int vocab, int buckets, int mul_prev, int mul_cur, int* err_flag,
                          cudaStream_t st) {
    B2_CHECK_ARG(tokens && segs && table && last_tok && x && nseg > 0 && max_n > 0, "embed_bigram_rows: bad argument");
    B2_CHECK_ARG(bigram == nullptr || buckets > 0, "embed_bigram_rows: a bigram table needs buckets");
    if (bigram == nullptr) buckets = 1;
    if (table_dtype == DT_F32)
        embed_bigram_kernel<float><<<dim3(max_n, nseg), 256, 0, st>>>(tokens, segs, reinterpret_cast<const float*>(table),
                                                                     reinterpret_cast<const float*>(bigram), last_tok, x, x0, cols, vocab, buckets,
                                                                     mul_prev, mul_cur, err_flag);
    else
        embed_bigram_kernel<__nv_bfloat16><<<dim3(max_n, nseg), 256, 0, st>>>(tokens, segs, reinterpret_cast<const __nv_bfloat16*>(table),
                                                                             reinterpret_cast<const __nv_bfloat16*>(bigram), last_tok, x, x0, cols,
                                                                             vocab, buckets, mul_prev, mul_cur, err_flag);
    B2_LAUNCH_CHECK();
    return 0;
}

int latent_append_f32(const float* in, int64_t ld_in, const float* gamma, float* cache, const int32_t* row_slot, const int32_t* row_pos, int rows,
                      int rank, int Smax, float eps, cudaStream_t st) {
    B2_CHECK_ARG(in && gamma && cache && row_slot && row_pos && rows > 0 && rank > 0, "latent_append: bad argument");
    latent_append_kernel<<<rows, rank >= 512 ? 256 : 128, 0, st>>>(in, ld_in, gamma, cache, row_slot, row_pos, rank, Smax, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int rowmap_portion(const RowMap& rm, int32_t* len, int slot, int n, int restart, cudaStream_t st) {
    B2_CHECK_ARG(rm.segs && rm.row_slot && rm.row_pos && len && n > 0, "rowmap_portion: bad argument");
    rowmap_portion_kernel<<<1, 256, 0, st>>>(rm.segs, rm.row_slot, rm.row_pos, len, slot, n, restart);
    B2_LAUNCH_CHECK();
    return 0;
}

int rowmap_decode(const RowMap& rm, const int32_t* len, const SampleState* sstate, const RowState* rows_state, int slot0, int B, cudaStream_t st) {
    B2_CHECK_ARG(rm.segs && rm.row_slot && rm.row_pos && len && B > 0, "rowmap_decode: bad argument");
    rowmap_decode_kernel<<<(B + 127) / 128, 128, 0, st>>>(rm.segs, rm.row_slot, rm.row_pos, len, sstate, rows_state, slot0, B);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b2
