// Recurrent mixers of the layer-list decoders: causal depthwise convolution with a carried tail, RWKV token shift, and the
// linear recurrence with a diagonal decay over a per-head [key, value] state (state-space, RWKV and HGRN2 forms). One code path
// serves a portion of a prompt (n rows of one slot) and a decode step (one row of each of B slots): the rows come as
// segments (kernels.h, SeqSeg). State, decays, step sizes and sums are fp32; a segment whose pos0 is 0 starts from zero
// state whatever its slot held before, so a slot that is handed to a new request needs no clearing.
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ---- causal depthwise convolution + SiLU -----------------------------------------------------------------------------------
// One thread per (channel, tile of CONV_TILE tokens): it primes its window from the inputs in front of the tile (rows of this
// call, or the carried tail for positions before the call) and walks the tile. The compute kernel only READS the tail; a
// second small kernel replaces it afterwards, so tiles never race with the update.
constexpr int CONV_MAX_TAPS = 16, CONV_TILE = 32;
template <int FLAGS>   // CONV_SILU | CONV_ADD_INPUT; own_tail: every segment is ONE tile, whose thread replaces the carried inputs itself
__global__ void __launch_bounds__(128) causal_conv_kernel(const float* __restrict__ in, int64_t ld_in, const float* __restrict__ w,
                                                          const float* __restrict__ bias, float* __restrict__ tail,
                                                          float* __restrict__ out, int64_t ld_out, int C, int taps,
                                                          const SeqSeg* __restrict__ segs, int own_tail) {
    const SeqSeg sg = segs[blockIdx.z];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int tt0 = blockIdx.y * CONV_TILE;
    if (c >= C || tt0 >= sg.n) return;
    // Window and taps are kept right-aligned in arrays of CONV_MAX_TAPS (all indices static): entry CONV_MAX_TAPS-1 is the
    // current token, the unused leading entries carry zero weights.
    float wt[CONV_MAX_TAPS], win[CONV_MAX_TAPS];
    const float* tl = tail + (size_t)sg.slot * (taps - 1) * C + c;
    const float* ip = in + (size_t)sg.row0 * ld_in + c;
#pragma unroll
    for (int jp = 0; jp < CONV_MAX_TAPS; ++jp) {
        const int tj = jp - (CONV_MAX_TAPS - taps);
        wt[jp] = tj >= 0 ? w[(size_t)c * taps + tj] : 0.f;
        // primed one step early (the loop shifts before it appends): entry jp holds the input of token tt0 - (CONV_MAX_TAPS - jp)
        const int t = tt0 - (CONV_MAX_TAPS - jp);
        float v = 0.f;
        if (jp >= CONV_MAX_TAPS - (taps - 1)) {  // the taps-1 tokens in front of the tile
            if (t >= 0) v = ip[(size_t)t * ld_in];
            else if (sg.pos0 > 0) v = tl[(size_t)(t + (taps - 1)) * C];
        }
        win[jp] = v;
    }
    const float b = bias != nullptr ? bias[c] : 0.f;
    float* op = out + (size_t)sg.row0 * ld_out + c;
    const int t_end = min(sg.n, tt0 + CONV_TILE);
    for (int t0 = tt0; t0 < t_end; t0 += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = t0 + u < t_end ? ip[(size_t)(t0 + u) * ld_in] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (t0 + u < t_end) {
#pragma unroll
                for (int jp = 0; jp < CONV_MAX_TAPS - 1; ++jp) win[jp] = win[jp + 1];
                win[CONV_MAX_TAPS - 1] = v[u];
                float acc = b;
#pragma unroll
                for (int jp = 0; jp < CONV_MAX_TAPS; ++jp) acc = fmaf(wt[jp], win[jp], acc);
                if (FLAGS & CONV_ADD_INPUT) acc += v[u];
                op[(size_t)(t0 + u) * ld_out] = (FLAGS & CONV_SILU) ? silu_f(acc) : acc;
            }
        }
    }
    if (own_tail && taps > 1) {   // the window now ends with the segment's last input: its last taps - 1 entries are the new carried inputs
        float* tw = tail + (size_t)sg.slot * (taps - 1) * C + c;
#pragma unroll
        for (int jp = 0; jp < CONV_MAX_TAPS; ++jp) {
            const int j = jp - (CONV_MAX_TAPS - (taps - 1));
            if (j >= 0) tw[(size_t)j * C] = win[jp];
        }
    }
}
// tail[j] := input of token n - (taps-1) + j of the segment; tokens before the call come from the old tail (or zero)
__global__ void __launch_bounds__(128) causal_conv_tail_kernel(const float* __restrict__ in, int64_t ld_in, float* __restrict__ tail, int C,
                                                               int taps, const SeqSeg* __restrict__ segs) {
    const SeqSeg sg = segs[blockIdx.y];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C || sg.n <= 0) return;
    float* tl = tail + (size_t)sg.slot * (taps - 1) * C + c;
    float nv[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        nv[j] = 0.f;
        if (j < taps - 1) {
            const int t = sg.n - (taps - 1) + j;
            if (t >= 0) nv[j] = in[(size_t)(sg.row0 + t) * ld_in + c];
            else if (sg.pos0 > 0) nv[j] = tl[(size_t)(t + (taps - 1)) * C];
        }
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
        if (j < taps - 1) tl[(size_t)j * C] = nv[j];
}

// ---- token shift: out[s][t] = x[t] + (x[t-1] - x[t]) * mu[s]; x[-1] of a call is the carried row (zero at a sequence start) ---
constexpr int SHIFT_MAX_MIX = 8, SHIFT_TILE = 8;
__global__ void __launch_bounds__(128) token_shift_mix_kernel(const float* __restrict__ x, const float* __restrict__ mu,
                                                              const float* __restrict__ prev, float* __restrict__ out, int64_t out_stride,
                                                              int cols, int n_mix, const SeqSeg* __restrict__ segs) {
    const SeqSeg sg = segs[blockIdx.z];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = blockIdx.y * SHIFT_TILE;
    if (c >= cols || t0 >= sg.n) return;
    float m[SHIFT_MAX_MIX];
#pragma unroll
    for (int s = 0; s < SHIFT_MAX_MIX; ++s) m[s] = s < n_mix ? mu[(size_t)s * cols + c] : 0.f;
    float v[SHIFT_TILE + 1];
    v[0] = t0 > 0 ? x[(size_t)(sg.row0 + t0 - 1) * cols + c] : (sg.pos0 > 0 ? prev[(size_t)sg.slot * cols + c] : 0.f);
#pragma unroll
    for (int u = 0; u < SHIFT_TILE; ++u) v[u + 1] = t0 + u < sg.n ? x[(size_t)(sg.row0 + t0 + u) * cols + c] : 0.f;
#pragma unroll
    for (int u = 0; u < SHIFT_TILE; ++u) {
        if (t0 + u < sg.n) {
            const float d = v[u] - v[u + 1];
#pragma unroll
            for (int s = 0; s < SHIFT_MAX_MIX; ++s)
                if (s < n_mix) out[(size_t)s * out_stride + (size_t)(sg.row0 + t0 + u) * cols + c] = fmaf(d, m[s], v[u + 1]);
        }
    }
}
__global__ void __launch_bounds__(128) token_shift_carry_kernel(const float* __restrict__ x, float* __restrict__ prev, int cols,
                                                                const SeqSeg* __restrict__ segs) {
    const SeqSeg sg = segs[blockIdx.y];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < cols && sg.n > 0) prev[(size_t)sg.slot * cols + c] = x[(size_t)(sg.row0 + sg.n - 1) * cols + c];
}

// ---- linear recurrence ------------------------------------------------------------------------------------------------
// Block = 32 value columns (threadIdx.x) x KS key slices (threadIdx.y) of one head of one segment. A thread keeps KPT keys
// of its column's state in registers. Tokens are staged TT at a time into shared memory with the per-token preparation done
// while staging (step size, decay, dt-scaled key), then walked in order with no barrier in between: the recurrence lives in
// registers, and the KS partial dot products of the tile's tokens meet in shared memory once per tile.
constexpr int TT = 16;   // KPT (template): keys of the state a thread keeps, 16, or 8 for key sizes <= 128 (twice the warps per CTA)

template <int MODE, int KPT>
__global__ void __launch_bounds__(512) linear_scan_kernel(ScanArgs a) {
    extern __shared__ float sm[];
    const SeqSeg sg = a.segs[blockIdx.z];
    if (sg.n <= 0) return;
    const int h = blockIdx.y, j = blockIdx.x * 32 + threadIdx.x, ks = threadIdx.y, KS = blockDim.y;
    const int dk = a.dk, dv = a.dv, dkp = KS * KPT;
    const int tid = threadIdx.y * 32 + threadIdx.x, nthr = KS * 32;
    float* sQ = sm;                    // [TT][dkp]
    float* sK = sQ + TT * dkp;         // [TT][dkp]
    float* sD = sK + TT * dkp;         // [TT][dkp] decay per key channel
    float* sV = sD + TT * dkp;         // [TT][32]
    float* sR = sV + TT * 32;          // [TT][KS][32] partial outputs of a tile
    const int g = MODE == SCAN_SSD ? h / (a.heads / a.groups) : h;  // SCAN_HGRN2 has no key input: a.k is not read
    const bool col_ok = j < dv;
    float S[KPT], bon[KPT];
    float* st = a.state + (((size_t)sg.slot * a.heads + h) * dk) * dv;
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int key = ks * KPT + i;
        S[i] = (sg.pos0 > 0 && col_ok && key < dk) ? st[(size_t)key * dv + j] : 0.f;
        bon[i] = (MODE == SCAN_RWKV && key < dk) ? a.bonus[(size_t)h * dk + key] : 0.f;
    }
    float neg_a = 0.f, dtb = 0.f, skip = 0.f;
    if (MODE == SCAN_SSD) { neg_a = -expf(a.a_log[h]); dtb = a.dt_bias[h]; skip = a.skip[h]; }

    // Staging is split in two so that global latency hides behind the walk of the previous tile: the raw inputs of tile
    // i+1 are requested into registers before tile i is walked, and turned into (q, dt*k, decay, v) in shared memory after.
    // A thread stages TT*KPT/32 key elements (dkp = KS*KPT over 32*KS threads) and up to TT value elements.
    constexpr int EPT = TT * KPT / 32;
    float rq[EPT], rk[EPT], rd[EPT], rv[TT];
    float rtok = 0.f;  // SSD: the raw step size of token `tid` of the tile (one scalar per token and head)
    auto fetch = [&](int t0) {
        const int nt = min(TT, sg.n - t0);
        if (MODE == SCAN_SSD && tid < nt) rtok = a.decay_in[(size_t)(sg.row0 + t0 + tid) * a.ldd + h];
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * nthr, t = e / dkp, key = e % dkp;
            rq[u] = 0.f; rk[u] = 0.f; rd[u] = 0.f;
            if (t < nt && key < dk) {
                const size_t row = (size_t)(sg.row0 + t0 + t);
                rq[u] = a.q[row * a.ldq + (size_t)g * dk + key];
                if (MODE != SCAN_HGRN2) rk[u] = a.k[row * a.ldk + (size_t)g * dk + key];
                if (MODE != SCAN_SSD) rd[u] = a.decay_in[row * a.ldd + (size_t)h * dk + key];
            }
        }
#pragma unroll
        for (int u = 0; u < TT; ++u) {
            const int e = tid + u * nthr, t = e >> 5, jj = blockIdx.x * 32 + (e & 31);
            rv[u] = (e < nt * 32 && jj < dv) ? a.v[(size_t)(sg.row0 + t0 + t) * a.ldv + (size_t)h * dv + jj] : 0.f;
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < sg.n; t0 += TT) {
        const int nt = min(TT, sg.n - t0);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < EPT; ++u) {
            const int e = tid + u * nthr, key = e % dkp;
            if (MODE == SCAN_HGRN2) {
                // forget gate bounded below: f = l + (1 - l) sigmoid(z + b); what is forgotten, 1 - f, is what is written
                float f = 1.f;
                if (key < dk) {
                    const float low = a.gate_lower[(size_t)h * dk + key];
                    f = fmaf(1.f - low, 1.f / (1.f + expf(-(rd[u] + a.gate_bias[(size_t)h * dk + key]))), low);
                }
                sQ[e] = silu_f(rq[u]); sK[e] = 1.f - f; sD[e] = f;
            } else if (MODE == SCAN_GLA) {
                // decay per key channel: sigmoid(z + b)^(1 / tau) = exp(log_sigmoid(z + b) / tau), log_sigmoid(u) = min(u, 0) - log1p(exp(-|u|))
                float al = 1.f;
                if (key < dk) {
                    const float z = rd[u] + a.gate_bias[(size_t)h * dk + key];
                    al = expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) / a.tau);
                }
                sQ[e] = rq[u] * a.q_scale; sK[e] = rk[u]; sD[e] = al;
            } else {
                sQ[e] = rq[u]; sK[e] = rk[u];
                if (MODE == SCAN_RWKV) sD[e] = key < dk ? expf(-expf(rd[u])) : 1.f;
            }
        }
        // SSD: the decay and the step size are scalars per token; the step size multiplies the value (dt B x^T = B (dt x)^T),
        // so the keys are staged as they are and sD holds [TT] step sizes followed by [TT] decays
        if (MODE == SCAN_SSD && tid < TT) {
            const float dt = softplus_f(rtok + dtb);
            sD[tid] = dt;
            sD[TT + tid] = expf(neg_a * dt);
        }
#pragma unroll
        for (int u = 0; u < TT; ++u) {
            const int e = tid + u * nthr;
            if (e < TT * 32) sV[e] = rv[u];
        }
        __syncthreads();
        if (t0 + TT < sg.n) fetch(t0 + TT);
        float part[TT];   // this thread's share of y[t][j] for the tokens of the tile
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            part[t] = 0.f;
            if (t < nt) {
                const float v = sV[t * 32 + threadIdx.x];
                float q[KPT], k[KPT], d[KPT];   // this slice's 16 keys of the token: four 16-byte broadcast reads per array
#pragma unroll
                for (int i4 = 0; i4 < KPT / 4; ++i4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(sQ + t * dkp + ks * KPT + i4 * 4);
                    const float4 k4 = *reinterpret_cast<const float4*>(sK + t * dkp + ks * KPT + i4 * 4);
                    q[i4 * 4] = q4.x; q[i4 * 4 + 1] = q4.y; q[i4 * 4 + 2] = q4.z; q[i4 * 4 + 3] = q4.w;
                    k[i4 * 4] = k4.x; k[i4 * 4 + 1] = k4.y; k[i4 * 4 + 2] = k4.z; k[i4 * 4 + 3] = k4.w;
                    if (MODE != SCAN_SSD) {
                        const float4 d4 = *reinterpret_cast<const float4*>(sD + t * dkp + ks * KPT + i4 * 4);
                        d[i4 * 4] = d4.x; d[i4 * 4 + 1] = d4.y; d[i4 * 4 + 2] = d4.z; d[i4 * 4 + 3] = d4.w;
                    }
                }
                float acc = 0.f;
                const float vdt = MODE == SCAN_SSD ? v * sD[t] : v, dec = MODE == SCAN_SSD ? sD[TT + t] : 0.f;
#pragma unroll
                for (int i = 0; i < KPT; ++i) {
                    const float kv = k[i] * vdt;
                    if (MODE == SCAN_RWKV) {
                        acc = fmaf(q[i], fmaf(bon[i], kv, S[i]), acc);
                        S[i] = fmaf(d[i], S[i], kv);
                    } else if (MODE == SCAN_HGRN2 || MODE == SCAN_GLA) {
                        S[i] = fmaf(d[i], S[i], kv);
                        acc = fmaf(q[i], S[i], acc);
                    } else {
                        S[i] = fmaf(dec, S[i], kv);
                        acc = fmaf(q[i], S[i], acc);
                    }
                }
                part[t] = acc;
            }
        }
        // the key slices meet once per tile: partial sums through shared memory, every thread finishes some (token, column) pairs
        if (KS > 1) {
#pragma unroll
            for (int t = 0; t < TT; ++t) sR[(t * KS + ks) * 32 + threadIdx.x] = part[t];
            __syncthreads();
            for (int t = ks; t < nt; t += KS) {
                float acc = 0.f;
                for (int s2 = 0; s2 < KS; ++s2) acc += sR[(t * KS + s2) * 32 + threadIdx.x];
                if (col_ok) {
                    if (MODE == SCAN_SSD) acc = fmaf(skip, sV[t * 32 + threadIdx.x], acc);
                    a.y[(size_t)(sg.row0 + t0 + t) * a.ldy + (size_t)h * dv + j] = acc;
                }
            }
        } else if (col_ok) {
#pragma unroll
            for (int t = 0; t < TT; ++t)
                if (t < nt) {
                    float acc = part[t];
                    if (MODE == SCAN_SSD) acc = fmaf(skip, sV[t * 32 + threadIdx.x], acc);
                    a.y[(size_t)(sg.row0 + t0 + t) * a.ldy + (size_t)h * dv + j] = acc;
                }
        }
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int key = ks * KPT + i;
        if (col_ok && key < dk) st[(size_t)key * dv + j] = S[i];
    }
}
}  // namespace

int causal_conv_silu_f32(const float* in, int64_t ld_in, const float* w, const float* bias, float* tail, float* out, int64_t ld_out, int C,
                         int taps, const SeqSeg* segs, int nseg, int max_n, cudaStream_t st) {
    B2_CHECK_ARG(bias != nullptr, "causal_conv_silu: null bias");
    return causal_conv_f32(in, ld_in, w, bias, tail, out, ld_out, C, taps, CONV_SILU, segs, nseg, max_n, st);
}

int causal_conv_f32(const float* in, int64_t ld_in, const float* w, const float* bias, float* tail, float* out, int64_t ld_out, int C, int taps,
                    int flags, const SeqSeg* segs, int nseg, int max_n, cudaStream_t st) {
    B2_CHECK_ARG(in && w && (tail || taps == 1) && out && in != out && segs && C > 0 && nseg > 0, "causal_conv: bad argument");
    B2_CHECK_ARG(taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: 1..%d taps are supported (got %d)", CONV_MAX_TAPS, taps);
    // the grid covers the longest segment the call may hold; tiles past a segment's end return at once
    const dim3 grid((C + 127) / 128, (max_n + CONV_TILE - 1) / CONV_TILE, nseg);
    const int own = max_n <= CONV_TILE;   // one tile per segment (decode steps, short portions): no second kernel for the carried inputs
    switch (flags & (CONV_SILU | CONV_ADD_INPUT)) {
        case 0: causal_conv_kernel<0><<<grid, 128, 0, st>>>(in, ld_in, w, bias, tail, out, ld_out, C, taps, segs, own); break;
        case CONV_SILU: causal_conv_kernel<CONV_SILU><<<grid, 128, 0, st>>>(in, ld_in, w, bias, tail, out, ld_out, C, taps, segs, own); break;
        case CONV_ADD_INPUT: causal_conv_kernel<CONV_ADD_INPUT><<<grid, 128, 0, st>>>(in, ld_in, w, bias, tail, out, ld_out, C, taps, segs, own); break;
        default: causal_conv_kernel<CONV_SILU | CONV_ADD_INPUT><<<grid, 128, 0, st>>>(in, ld_in, w, bias, tail, out, ld_out, C, taps, segs, own); break;
    }
    B2_LAUNCH_CHECK();
    if (taps > 1 && !own) {
        causal_conv_tail_kernel<<<dim3((C + 127) / 128, nseg), 128, 0, st>>>(in, ld_in, tail, C, taps, segs);
        B2_LAUNCH_CHECK();
    }
    return 0;
}

int token_shift_mix_f32(const float* x, const float* mu, float* prev, float* out, int64_t out_stride, int cols, int n_mix, const SeqSeg* segs,
                        int nseg, int max_n, cudaStream_t st) {
    B2_CHECK_ARG(x && mu && prev && out && segs && cols > 0 && nseg > 0, "token_shift: bad argument");
    B2_CHECK_ARG(n_mix >= 1 && n_mix <= SHIFT_MAX_MIX, "token_shift: 1..%d mixes are supported (got %d)", SHIFT_MAX_MIX, n_mix);
    token_shift_mix_kernel<<<dim3((cols + 127) / 128, (max_n + SHIFT_TILE - 1) / SHIFT_TILE, nseg), 128, 0, st>>>(x, mu, prev, out, out_stride, cols,
                                                                                                                 n_mix, segs);
    B2_LAUNCH_CHECK();
    token_shift_carry_kernel<<<dim3((cols + 127) / 128, nseg), 128, 0, st>>>(x, prev, cols, segs);
    B2_LAUNCH_CHECK();
    return 0;
}

template <int MODE, int KPT>
int launch_scan(const ScanArgs& a, cudaStream_t st) {
    const int KS = (a.dk + KPT - 1) / KPT;
    const size_t smem = ((size_t)3 * TT * KS * KPT + TT * 32 + (size_t)TT * KS * 32) * sizeof(float);
    dim3 grid((a.dv + 31) / 32, a.heads, a.nseg), block(32, KS);
    if (smem > 48 * 1024) B2_CUDA_CHECK(cudaFuncSetAttribute(linear_scan_kernel<MODE, KPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    linear_scan_kernel<MODE, KPT><<<grid, block, smem, st>>>(a);
    B2_LAUNCH_CHECK();
    return 0;
}

int linear_scan_f32(const ScanArgs& a, cudaStream_t st) {
    B2_CHECK_ARG(a.q && (a.k || a.mode == SCAN_HGRN2) && a.v && a.decay_in && a.state && a.y && a.segs && a.nseg > 0, "linear_scan: null argument");
    B2_CHECK_ARG(a.heads > 0 && a.dk > 0 && a.dv > 0, "linear_scan: bad sizes");
    B2_CHECK_ARG(a.dk <= 256, "linear_scan: key size %d exceeds 256", a.dk);
    // 8 keys per thread where 16 key slices cover the key size: twice the warps hide the shared-memory latency of the token walk
    static const bool narrow_ok = [] { const char* e = getenv("B2_SCAN_KPT8"); return !(e != nullptr && e[0] == '0'); }();
    const bool narrow = narrow_ok && a.dk <= 128 && a.dk > 16;
    if (a.mode == SCAN_SSD) {
        B2_CHECK_ARG(a.groups > 0 && a.heads % a.groups == 0 && a.dt_bias && a.a_log && a.skip, "linear_scan(ssd): heads %d / groups %d", a.heads, a.groups);
        return narrow ? launch_scan<SCAN_SSD, 8>(a, st) : launch_scan<SCAN_SSD, 16>(a, st);
    }
    if (a.mode == SCAN_HGRN2) {
        B2_CHECK_ARG(a.gate_bias && a.gate_lower, "linear_scan(hgrn2): null gate bias / lower bound");
        return narrow ? launch_scan<SCAN_HGRN2, 8>(a, st) : launch_scan<SCAN_HGRN2, 16>(a, st);
    }
    if (a.mode == SCAN_GLA) {
        B2_CHECK_ARG(a.gate_bias && a.tau > 0.f, "linear_scan(gla): null decay bias or a non-positive tau");
        return narrow ? launch_scan<SCAN_GLA, 8>(a, st) : launch_scan<SCAN_GLA, 16>(a, st);
    }
    B2_CHECK_ARG(a.mode == SCAN_RWKV, "linear_scan: unknown mode %d", a.mode);
    B2_CHECK_ARG(a.bonus != nullptr, "linear_scan(rwkv): null bonus");
    return narrow ? launch_scan<SCAN_RWKV, 8>(a, st) : launch_scan<SCAN_RWKV, 16>(a, st);
}

}  // namespace b2
