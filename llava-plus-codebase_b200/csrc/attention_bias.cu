// Causal softmax attention for layer-list decoders whose positions enter only through the scores: q and k are brought to
// unit RMS per head (no weight), q carries a temperature that grows with the logarithm of its position, the scaled score is
// soft-capped with tanh, and a learned bias indexed by a bucket of the distance is added (exact rows for near keys,
// logarithmic rows up to a far limit, one row beyond; the bucket of every distance is tabulated on the host). Query heads
// share key/value heads in groups; key and value sizes are free (dk, dv <= 256). Everything is fp32: scores, softmax,
// the cache. One warp per (row, head [, key split]); a row is a token of a prompt portion or a decode step, and it attends
// to its slot's cache, which attn_prepare has already extended by the rows of this call.
// The same kernels serve attention over a shared latent (one cached row per token that is key AND value of every head:
// kcache == vcache, dk == dv <= 512, G = 1), without bias table or soft-cap (rel == null), and with a per-head sink: one
// extra term exp(sink[h]) in the softmax denominator that has no key and no value (or exp(sink_value) for every head). A cached
// row may be longer than the value it holds (dv < dk: a latent followed by a rotated key part). The visible keys of a row may be
// limited to a sliding window or to the row's chunk of positions: keys in front of the first visible one are never loaded. A
// window may keep the sequence's first positions visible (mask_keep): the visible keys are then two ranges, [0, keep) and the
// window, and the tiles of the gap between them are never staged. Value heads may be fewer than key heads (Gv < G: key head g
// reads value head g mod Gv), which is how the two maps of differential attention share one set of values.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// first position a row at position pos sees
__device__ __forceinline__ int mask_first(int pos, int kind, int size) {
    if (kind == MASK_WINDOW) return max(0, pos - size + 1);
    if (kind == MASK_CHUNK) return pos / size * size;
    return 0;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// unit = q head (normalise, temperature, in place) | k head (normalise, append) | v head (append)
__global__ void attn_prepare_kernel(BiasAttnArgs a) {
    const int units = a.H + 2 * a.G;
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= a.rows * units) return;
    const int r = w / units, u = w % units;
    const int pos = a.row_pos[r], slot = a.row_slot[r];
    if (pos < 0) return;
    if (u < a.H + a.G) {
        const bool is_q = u < a.H;
        float* src = is_q ? a.q + (size_t)r * a.ldq + (size_t)u * a.dk
                          : const_cast<float*>(a.k) + (size_t)r * a.ldk + (size_t)(u - a.H) * a.dk;
        float ss = 0.f;
        for (int d = lane; d < a.dk; d += 32) ss = fmaf(src[d], src[d], ss);
        ss = warp_sum(ss);
        float mul = 1.f / sqrtf(ss / (float)a.dk + a.eps);
        float* dst = src;
        if (is_q) {
            mul *= 1.f + a.temp_coef * logf(floorf((float)(pos + 1) / a.temp_every) + 1.f);
        } else {
            dst = a.kcache + (((size_t)slot * a.G + (u - a.H)) * a.Smax + pos) * a.dk;
        }
        for (int d = lane; d < a.dk; d += 32) dst[d] = src[d] * mul;
    } else {
        const int g = u - a.H - a.G;
        const float* src = a.v + (size_t)r * a.ldv + (size_t)g * a.dv;
        float* dst = a.vcache + (((size_t)slot * a.G + g) * a.Smax + pos) * a.dv;
        for (int d = lane; d < a.dv; d += 32) dst[d] = src[d];
    }
}

constexpr int AT_WARPS = 4, AT_MAXC = 8;  // dv <= 32 * AT_MAXC

template <bool VEC>
__global__ void __launch_bounds__(AT_WARPS * 32) attn_bias_kernel(BiasAttnArgs a) {
    extern __shared__ float sq[];  // [AT_WARPS][dk]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int w = blockIdx.x * AT_WARPS + warp;
    const int sp = blockIdx.y;
    if (w >= a.rows * a.H) return;
    const int r = w / a.H, h = w % a.H;
    const int pos = a.row_pos[r];
    if (pos < 0) return;
    const int slot = a.row_slot[r], g = h / (a.H / a.G);
    float* q = sq + warp * a.dk;
    for (int d = lane; d < a.dk; d += 32) q[d] = a.q[(size_t)r * a.ldq + (size_t)h * a.dk + d];
    __syncwarp();
    const float* K = a.kcache + ((size_t)slot * a.G + g) * a.Smax * a.dk;
    const size_t vrs = a.vcache == a.kcache ? (size_t)a.dk : (size_t)a.dv;   // keys that hold the value: the key row's pitch
    const int Gv = a.Gv > 0 ? a.Gv : a.G;
    const float* V = a.vcache + ((size_t)slot * Gv + g % Gv) * a.Smax * vrs;
    // visible keys: [0, nA) (the kept first positions in front of the window; empty without them) and [first, pos], walked as
    // tiles of 32 that the key splits share out
    const int first = mask_first(pos, a.mask_kind, a.mask_size);
    const int nA = a.mask_kind == MASK_WINDOW ? min(a.mask_keep, first) : 0, tilesA = (nA + 31) / 32;
    const int T = tilesA + (pos + 1 - first + 31) / 32;
    int t_lo = 0, t_hi = T;
    if (a.nsplit > 1) {
        const int per = (T + a.nsplit - 1) / a.nsplit;
        t_lo = sp * per;
        t_hi = min(T, t_lo + per);
    }
    float m = -INFINITY, l = 0.f, o[AT_MAXC];
#pragma unroll
    for (int c = 0; c < AT_MAXC; ++c) o[c] = 0.f;
    for (int t = t_lo; t < t_hi; ++t) {
        const int j0 = t < tilesA ? t * 32 : first + (t - tilesA) * 32, hi = t < tilesA ? nA : pos + 1;
        const int j = j0 + lane;
        const bool valid = j < hi;
        float s = -INFINITY;
        if (valid) {
            const float* kr = K + (size_t)j * a.dk;
            float acc = 0.f;
            if (VEC) {
                for (int d = 0; d < a.dk; d += 4) {
                    const float4 kv = *reinterpret_cast<const float4*>(kr + d);
                    const float4 qv = *reinterpret_cast<const float4*>(q + d);
                    acc = fmaf(qv.x, kv.x, acc); acc = fmaf(qv.y, kv.y, acc); acc = fmaf(qv.z, kv.z, acc); acc = fmaf(qv.w, kv.w, acc);
                }
            } else {
                for (int d = 0; d < a.dk; ++d) acc = fmaf(q[d], kr[d], acc);
            }
            s = acc * a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            if (a.rel != nullptr) s += a.rel[(size_t)a.bucket_of[pos - j] * a.H + h];
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = fmaf(l, corr, warp_sum(p));
        m = m_new;
        const int nk = min(32, hi - j0);
#pragma unroll
        for (int c = 0; c < AT_MAXC; ++c) o[c] *= corr;
        for (int jj = 0; jj < nk; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* vr = V + (size_t)(j0 + jj) * vrs;
#pragma unroll
            for (int c = 0; c < AT_MAXC; ++c) {
                const int d = lane + 32 * c;
                if (d < a.dv) o[c] = fmaf(pj, vr[d], o[c]);
            }
        }
    }
    if (a.nsplit > 1) {
        float* part = a.partial + ((size_t)w * a.nsplit + sp) * (a.dv + 2);
        if (lane == 0) { part[0] = m; part[1] = l; }
#pragma unroll
        for (int c = 0; c < AT_MAXC; ++c) {
            const int d = lane + 32 * c;
            if (d < a.dv) part[2 + d] = o[c];
        }
    } else {
        float inv = 1.f / l;
        if (a.sink != nullptr || a.sink_fixed) {   // the sink joins the denominator once, under the common maximum
            const float sk = a.sink != nullptr ? a.sink[h] : a.sink_value, mf = fmaxf(m, sk), c0 = expf(m - mf);
            inv = c0 / fmaf(l, c0, expf(sk - mf));
        }
        if (a.head_gate != nullptr) inv /= 1.f + expf(-a.head_gate[(size_t)r * a.ldg + h]);
#pragma unroll
        for (int c = 0; c < AT_MAXC; ++c) {
            const int d = lane + 32 * c;
            if (d < a.dv) a.out[(size_t)r * a.ldo + (size_t)h * a.dv + d] = o[c] * inv;
        }
    }
}

// ---- tiled kernel: a CTA takes a tile of query rows of ONE slot x one key/value head x one key split. Keys and values are
// staged 32 at a time in shared memory with coalesced loads and shared by every (query row, query head of the group) pair of
// the CTA, so a key/value row crosses the memory system once per CTA instead of once per pair. 8 warps, <= 4 pairs per warp.
// A group of more than 32 query heads is cut into chunks of HC heads (blockIdx.y = group * chunks + chunk). When keys and
// values are the same cached rows (kcache == vcache), the staged key tile is the value tile too. MAXC * 32 >= dv.
constexpr int TL_KT = 32, TL_WARPS = 8, TL_PPW = 4;

// dst[r * dpitch + c] = src[r * spitch + c] for r < nrows, c < 4 * n4, 16 bytes at a time; a thread issues N loads before its
// first store, so the copy is bound by bandwidth and not by one memory round trip per element
template <int N>
__device__ __forceinline__ void copy_rows_f4(float* __restrict__ dst, int dpitch, const float* __restrict__ src, size_t spitch, int nrows, int n4,
                                             int tid) {
    const int total = nrows * n4;
    for (int base = 0; base < total; base += TL_WARPS * 32 * N) {
        float4 v[N];
        int off[N];
#pragma unroll
        for (int u = 0; u < N; ++u) {
            const int e = base + tid + u * TL_WARPS * 32;
            off[u] = -1;
            if (e < total) {
                const int r = e / n4, c = e - r * n4;
                v[u] = *reinterpret_cast<const float4*>(src + (size_t)r * spitch + c * 4);
                off[u] = r * dpitch + c * 4;
            }
        }
#pragma unroll
        for (int u = 0; u < N; ++u)
            if (off[u] >= 0) *reinterpret_cast<float4*>(dst + off[u]) = v[u];
    }
}

template <bool VEC, int MAXC>
__global__ void __launch_bounds__(TL_WARPS * 32, MAXC == 16 ? 1 : 2) attn_tile_kernel(BiasAttnArgs a, int QT, int HC) {
    extern __shared__ float sm[];
    const int HGall = a.H / a.G, chunks = (HGall + HC - 1) / HC;
    const int g = blockIdx.y / chunks, h0 = g * HGall + (blockIdx.y % chunks) * HC, HG = min(HC, g * HGall + HGall - h0);
    const int sp = blockIdx.z;
    const int r0 = blockIdx.x * QT, nrows = min(QT, a.rows - r0), P = nrows * HG;
    const int dk = a.dk, dv = a.dv, dkp = VEC ? dk + 4 : (dk | 1);
    const bool shared_kv = a.vcache == a.kcache;
    float* sQ = sm;                              // [QT * HC][dk]
    float* sK = sQ + (size_t)QT * HC * dk;       // [TL_KT][dkp]
    float* sV = sK + TL_KT * dkp;                // [TL_KT][dv] (unused when the key tile serves as the value tile)
    const int vp = shared_kv ? dkp : dv;         // pitch of a staged value row
    const float* sVal = shared_kv ? sK : sV;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int slot = a.row_slot[r0];
    int maxpos = -1, first = 0x7fffffff;   // last and first key position any row of the tile sees (kept first positions aside)
    for (int i = 0; i < nrows; ++i) {
        const int p = a.row_pos[r0 + i];
        maxpos = max(maxpos, p);
        if (p >= 0) first = min(first, mask_first(p, a.mask_kind, a.mask_size));
    }
    if (maxpos < 0) return;
    const int keep = a.mask_kind == MASK_WINDOW ? a.mask_keep : 0;
    if (VEC && a.ldq % 4 == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0) {
        // a row's heads of this chunk are consecutive in q: HG * dk floats per row, copied 16 bytes at a time
        for (int i = 0; i < nrows; ++i)
            copy_rows_f4<4>(sQ + (size_t)i * HG * dk, 0, a.q + (size_t)(r0 + i) * a.ldq + (size_t)h0 * dk, 0, 1, (HG * dk) >> 2, tid);
    } else {
        for (int e = tid; e < P * dk; e += TL_WARPS * 32) {
            const int p = e / dk, d = e % dk;
            sQ[e] = a.q[(size_t)(r0 + p / HG) * a.ldq + (size_t)(h0 + p % HG) * dk + d];
        }
    }
    // The keys the tile's rows see are two ranges: [0, nA), the kept first positions in front of the earliest window (empty without
    // them), and [first, maxpos]. They are walked as tiles of TL_KT keys, none of which straddles the gap, and the key splits of a
    // decode step share out the tiles.
    const int nA = min(keep, first), tilesA = (nA + TL_KT - 1) / TL_KT;
    const int T = tilesA + (maxpos + 1 - first + TL_KT - 1) / TL_KT;
    int t_lo = 0, t_hi = T;
    if (a.nsplit > 1) {
        const int per = (T + a.nsplit - 1) / a.nsplit;
        t_lo = sp * per;
        t_hi = min(T, t_lo + per);
    }
    // cache slabs [slot][head][position][size], or (kv_row_stride > 0) one matrix [position][head * size] made for this call
    const bool mat = a.kv_row_stride > 0;
    const int Gv = a.Gv > 0 ? a.Gv : a.G, gv = g % Gv;   // fewer value heads than key heads: key head g reads value head g mod Gv
    const size_t krs = mat ? (size_t)a.kv_row_stride : (size_t)dk, vrs = mat ? (size_t)a.kv_row_stride_v : (size_t)dv;
    const float* K = mat ? a.kcache + (size_t)g * dk : a.kcache + ((size_t)slot * a.G + g) * a.Smax * dk;
    const float* V = mat ? a.vcache + (size_t)gv * dv : a.vcache + ((size_t)slot * Gv + gv) * a.Smax * dv;
    const bool vecv = VEC && dv % 4 == 0 && vrs % 4 == 0 && (reinterpret_cast<uintptr_t>(V) & 15) == 0;   // 16-byte value rows
    float m[TL_PPW], l[TL_PPW], o[TL_PPW][MAXC];
    int ppos[TL_PPW], pfirst[TL_PPW];
#pragma unroll
    for (int i = 0; i < TL_PPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
        const int p = warp + TL_WARPS * i;
        ppos[i] = p < P ? a.row_pos[r0 + p / HG] : -1;
        pfirst[i] = mask_first(max(ppos[i], 0), a.mask_kind, a.mask_size);
#pragma unroll
        for (int c = 0; c < MAXC; ++c) o[i][c] = 0.f;
    }
    for (int t = t_lo; t < t_hi; ++t) {
        const int j0 = t < tilesA ? t * TL_KT : first + (t - tilesA) * TL_KT;
        const int nk = min(TL_KT, (t < tilesA ? nA : maxpos + 1) - j0);
        const bool kept = j0 < keep;   // the tile holds kept first positions: visible to every row behind them, whatever its window
        __syncthreads();
        if (VEC) {
            copy_rows_f4<4>(sK, dkp, K + (size_t)j0 * krs, krs, nk, dk >> 2, tid);
        } else {
            for (int e = tid; e < nk * dk; e += TL_WARPS * 32) sK[(e / dk) * dkp + e % dk] = K[(size_t)(j0 + e / dk) * krs + e % dk];
        }
        if (!shared_kv) {
            if (vecv) copy_rows_f4<4>(sV, dv, V + (size_t)j0 * vrs, vrs, nk, dv >> 2, tid);
            else for (int e = tid; e < nk * dv; e += TL_WARPS * 32) sV[e] = V[(size_t)(j0 + e / dv) * vrs + e % dv];
        }
        __syncthreads();
        // The warp's pairs go through the tile TOGETHER: a lane reads its key row once for all of them, and a value element
        // once per key for all of them (shared-memory bandwidth, not the FMA pipe, limits this loop).
        float sc[TL_PPW];
#pragma unroll
        for (int i = 0; i < TL_PPW; ++i) sc[i] = 0.f;
        if (lane < nk) {
            const float* kr = sK + lane * dkp;
            if (VEC) {
                for (int d = 0; d < dk; d += 4) {
                    const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
                    for (int i = 0; i < TL_PPW; ++i) {
                        if (ppos[i] >= j0 && (kept || pfirst[i] < j0 + nk)) {   // idle pairs and pairs whose keys all lie ahead or behind skip (warp-uniform)
                            const float4 qv = *reinterpret_cast<const float4*>(sQ + (warp + TL_WARPS * i) * dk + d);
                            sc[i] = fmaf(qv.x, kv.x, sc[i]); sc[i] = fmaf(qv.y, kv.y, sc[i]);
                            sc[i] = fmaf(qv.z, kv.z, sc[i]); sc[i] = fmaf(qv.w, kv.w, sc[i]);
                        }
                    }
                }
            } else {
                for (int d = 0; d < dk; ++d) {
                    const float kv = kr[d];
#pragma unroll
                    for (int i = 0; i < TL_PPW; ++i)
                        if (ppos[i] >= j0 && (kept || pfirst[i] < j0 + nk)) sc[i] = fmaf(sQ[(warp + TL_WARPS * i) * dk + d], kv, sc[i]);
                }
            }
        }
        float pr[TL_PPW];
        bool any = false;
#pragma unroll
        for (int i = 0; i < TL_PPW; ++i) {
            pr[i] = 0.f;
            const int pos = ppos[i];
            if (pos < j0 || (!kept && pfirst[i] >= j0 + nk)) continue;   // no key of this tile is visible: the running maximum stays as it is
            any = true;
            const int head = h0 + (warp + TL_WARPS * i) % HG;
            const int j = j0 + lane;
            const bool valid = lane < nk && j <= pos && (j >= pfirst[i] || j < keep);
            float sv = -INFINITY;
            if (valid) {
                sv = sc[i] * a.scale;
                if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
                if (a.rel != nullptr) sv += a.rel[(size_t)a.bucket_of[pos - j] * a.H + head];
            }
            const float m_new = fmaxf(m[i], warp_max(sv));
            pr[i] = valid ? expf(sv - m_new) : 0.f;
            const float corr = expf(m[i] - m_new);
            l[i] = fmaf(l[i], corr, warp_sum(pr[i]));
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < MAXC; ++c) o[i][c] *= corr;
        }
        if (any) {
            for (int jj = 0; jj < nk; ++jj) {
                float pj[TL_PPW];
#pragma unroll
                for (int i = 0; i < TL_PPW; ++i) pj[i] = __shfl_sync(0xffffffffu, pr[i], jj);
                const float* vr = sVal + jj * vp;
#pragma unroll
                for (int c = 0; c < MAXC; ++c) {
                    const int d = lane + 32 * c;
                    if (d < dv) {
                        const float vv = vr[d];
#pragma unroll
                        for (int i = 0; i < TL_PPW; ++i) o[i][c] = fmaf(pj[i], vv, o[i][c]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < TL_PPW; ++i) {
        const int p = warp + TL_WARPS * i;
        if (p >= P || ppos[i] < 0) continue;
        const int row = r0 + p / HG, head = h0 + p % HG;
        if (a.nsplit > 1) {
            float* part = a.partial + ((size_t)(row * a.H + head) * a.nsplit + sp) * (dv + 2);
            if (lane == 0) { part[0] = m[i]; part[1] = l[i]; }
#pragma unroll
            for (int c = 0; c < MAXC; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) part[2 + d] = o[i][c];
            }
        } else {
            float inv = 1.f / l[i];
            if (a.sink != nullptr || a.sink_fixed) {
                const float sk = a.sink != nullptr ? a.sink[head] : a.sink_value, mf = fmaxf(m[i], sk), c0 = expf(m[i] - mf);
                inv = c0 / fmaf(l[i], c0, expf(sk - mf));
            }
            if (a.head_gate != nullptr) inv /= 1.f + expf(-a.head_gate[(size_t)row * a.ldg + head]);   // the head's sigmoid gate
#pragma unroll
            for (int c = 0; c < MAXC; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) a.out[(size_t)row * a.ldo + (size_t)head * dv + d] = o[i][c] * inv;
            }
        }
    }
}

// one block per (row, head): every thread turns the splits' (max, sum) into weights (nsplit <= 64 values from L1) and combines
// its value columns in split order
__global__ void __launch_bounds__(512) attn_merge_kernel(BiasAttnArgs a) {
    const int w = blockIdx.x;
    const int r = w / a.H, h = w % a.H;
    if (a.row_pos[r] < 0) return;
    const int stride = a.dv + 2;
    const float* part = a.partial + (size_t)w * a.nsplit * stride;
    __shared__ float wgt[64];
    __shared__ float inv_s;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float mx = -INFINITY;
        for (int s = lane; s < a.nsplit; s += 32)
            if (part[(size_t)s * stride + 1] > 0.f) mx = fmaxf(mx, part[(size_t)s * stride]);
        mx = warp_max(mx);
        const bool has_sink = a.sink != nullptr || a.sink_fixed;
        const float sk = a.sink != nullptr ? a.sink[h] : (a.sink_fixed ? a.sink_value : -INFINITY);
        mx = fmaxf(mx, sk);
        float lsum = (has_sink && lane == 0) ? expf(sk - mx) : 0.f;
        for (int s = lane; s < a.nsplit; s += 32) {
            const float* ps = part + (size_t)s * stride;
            const float ws = ps[1] > 0.f ? expf(ps[0] - mx) : 0.f;
            wgt[s] = ws;
            lsum = fmaf(ps[1], ws, lsum);
        }
        lsum = warp_sum(lsum);
        if (lane == 0) inv_s = a.head_gate != nullptr ? 1.f / (lsum * (1.f + expf(-a.head_gate[(size_t)r * a.ldg + h]))) : 1.f / lsum;
    }
    __syncthreads();
    const float inv = inv_s;
    for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
        // every split wrote its partial sums (zeros when it had no keys): the loads need no guard and run four at a time
        float acc = 0.f;
        int s = 0;
        for (; s + 4 <= a.nsplit; s += 4) {
            const float p0 = part[(size_t)s * stride + 2 + d], p1 = part[(size_t)(s + 1) * stride + 2 + d];
            const float p2 = part[(size_t)(s + 2) * stride + 2 + d], p3 = part[(size_t)(s + 3) * stride + 2 + d];
            acc = fmaf(p0, wgt[s], acc); acc = fmaf(p1, wgt[s + 1], acc); acc = fmaf(p2, wgt[s + 2], acc); acc = fmaf(p3, wgt[s + 3], acc);
        }
        for (; s < a.nsplit; ++s) acc = fmaf(part[(size_t)s * stride + 2 + d], wgt[s], acc);
        a.out[(size_t)r * a.ldo + (size_t)h * a.dv + d] = acc * inv;
    }
}

int check_args(const BiasAttnArgs& a, const char* who) {
    B2_CHECK_ARG(a.q && a.kcache && a.vcache && a.row_slot && a.row_pos && a.rows > 0, "%s: null argument", who);
    B2_CHECK_ARG(a.H > 0 && a.G > 0 && a.H % a.G == 0, "%s: %d query heads cannot share %d key/value heads", who, a.H, a.G);
    B2_CHECK_ARG(a.dk > 0 && a.dk <= 768 && a.dv > 0 && a.dv <= 512, "%s: head sizes %d / %d exceed 768 / 512", who, a.dk, a.dv);
    B2_CHECK_ARG(a.vcache != a.kcache || a.dv <= a.dk, "%s: keys that also hold the values need dv <= dk", who);
    B2_CHECK_ARG(a.mask_kind == MASK_CAUSAL || ((a.mask_kind == MASK_WINDOW || a.mask_kind == MASK_CHUNK) && a.mask_size >= 1), "%s: mask %d of size %d", who, a.mask_kind, a.mask_size);
    B2_CHECK_ARG(a.mask_keep >= 0 && (a.mask_keep == 0 || a.mask_kind == MASK_WINDOW), "%s: kept first positions belong to a window", who);
    B2_CHECK_ARG(a.Gv >= 0 && (a.Gv == 0 || (a.G % a.Gv == 0 && a.vcache != a.kcache && a.kv_row_stride == 0)), "%s: %d key heads cannot share %d value heads", who, a.G, a.Gv);
    B2_CHECK_ARG(a.kv_row_stride == 0 || (a.kv_row_stride_v > 0 && a.tile_rows >= 1 && a.vcache != a.kcache), "%s: key/value matrices need both pitches and the tiled kernel", who);
    return 0;
}
}  // namespace

int attn_prepare_f32(const BiasAttnArgs& a, cudaStream_t st) {
    B2_TRY(check_args(a, "attn_prepare"));
    B2_CHECK_ARG(a.k && a.v && a.temp_every > 0.f, "attn_prepare: null k / v or a non-positive temperature period");
    const int warps = a.rows * (a.H + 2 * a.G);
    attn_prepare_kernel<<<(warps + 7) / 8, 256, 0, st>>>(a);
    B2_LAUNCH_CHECK();
    return 0;
}

template <bool VEC, int MAXC>
int launch_tile(const BiasAttnArgs& a, int QT, int HC, dim3 grid, size_t smem, cudaStream_t st) {
    if (smem > 48 * 1024) B2_CUDA_CHECK(cudaFuncSetAttribute(attn_tile_kernel<VEC, MAXC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_tile_kernel<VEC, MAXC><<<grid, TL_WARPS * 32, smem, st>>>(a, QT, HC);
    B2_LAUNCH_CHECK();
    if (a.nsplit > 1) {
        attn_merge_kernel<<<a.rows * a.H, a.dv > 256 ? 512 : (a.dv > 128 ? 256 : 128), 0, st>>>(a);
        B2_LAUNCH_CHECK();
    }
    return 0;
}

int attn_bias_f32(const BiasAttnArgs& a, cudaStream_t st) {
    B2_TRY(check_args(a, "attn_bias"));
    B2_CHECK_ARG(a.out && (a.rel == nullptr || a.bucket_of != nullptr), "attn_bias: null argument");
    B2_CHECK_ARG(a.nsplit >= 1 && a.nsplit <= 64 && (a.nsplit == 1 || a.partial != nullptr), "attn_bias: 1..64 key splits, with scratch");
    const int warps = a.rows * a.H;
    const bool vec = a.dk % 4 == 0 && (reinterpret_cast<uintptr_t>(a.kcache) & 15) == 0;
    const int HG = a.H / a.G;
    if (a.tile_rows >= 1) {
        // (row, head) pairs per CTA: 32. Query rows per CTA: as many as the heads of a chunk allow; rows of a tile share their
        // slot (tile_rows is 1 for a decode step, where every row has its own)
        const int HC = HG < TL_WARPS * TL_PPW ? HG : TL_WARPS * TL_PPW, chunks = (HG + HC - 1) / HC;
        int QT = (TL_WARPS * TL_PPW) / HC;
        if (QT > a.tile_rows) QT = a.tile_rows;
        const int dkp = vec ? a.dk + 4 : (a.dk | 1);
        const bool shared_kv = a.vcache == a.kcache;
        const size_t smem = ((size_t)QT * HC * a.dk + (size_t)TL_KT * dkp + (shared_kv ? 0 : (size_t)TL_KT * a.dv)) * sizeof(float);
        dim3 grid((a.rows + QT - 1) / QT, a.G * chunks, a.nsplit);
        if (a.dv <= 128) return vec ? launch_tile<true, 4>(a, QT, HC, grid, smem, st) : launch_tile<false, 4>(a, QT, HC, grid, smem, st);
        if (a.dv <= 32 * AT_MAXC) return vec ? launch_tile<true, AT_MAXC>(a, QT, HC, grid, smem, st) : launch_tile<false, AT_MAXC>(a, QT, HC, grid, smem, st);
        return vec ? launch_tile<true, 2 * AT_MAXC>(a, QT, HC, grid, smem, st) : launch_tile<false, 2 * AT_MAXC>(a, QT, HC, grid, smem, st);
    }
    B2_CHECK_ARG(a.dk <= 256 && a.dv <= 32 * AT_MAXC, "attn_bias: the untiled kernel takes head sizes up to 256");
    dim3 grid((warps + AT_WARPS - 1) / AT_WARPS, a.nsplit);
    const size_t smem = (size_t)AT_WARPS * a.dk * sizeof(float);
    if (vec) attn_bias_kernel<true><<<grid, AT_WARPS * 32, smem, st>>>(a);
    else attn_bias_kernel<false><<<grid, AT_WARPS * 32, smem, st>>>(a);
    B2_LAUNCH_CHECK();
    if (a.nsplit > 1) {
        attn_merge_kernel<<<warps, a.dv > 256 ? 512 : (a.dv > 128 ? 256 : 128), 0, st>>>(a);
        B2_LAUNCH_CHECK();
    }
    return 0;
}

}  // namespace b2
