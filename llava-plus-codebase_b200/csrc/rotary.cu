// Rotary positions for the layer-list decoders: pairs (2m, 2m+1) of a head's leading dimensions (or, in the half layout, pairs
// (m, m + pairs)) turn by position * f_m.
// cos and sin come from a table [position][pair] that the cache builds on the host in double precision (the plain
// frequencies base^(-2m/dims), optionally blended towards f_m / factor over a ramp of pairs with cos / sin scaled, the long-context
// form known as YaRN), so an angle never carries the rounding of a 32-bit product of a large position. One kernel serves
// queries (in place), keys and values on their way into the cache slabs, a rotated part copied to another layout, and the
// turn back of an attention output by its query's position with the sigmoid output gate applied in the same pass. When a head is
// normed before it turns (weighted RMS norm over the head, one weight vector for all heads), one warp takes a (row, head): it sums
// the squares, then every lane norms and turns the pairs it owns. A further kernel writes the row of a low-rank key/value cache that
// holds a normed latent AND one rotated key part.
#include <math.h>

#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

// Units of a head: single elements outside the rotated range, pairs inside it, so that a thread owns everything it reads and
// the call may run in place.
struct RotateParts { RotateArgs p[3]; };
__device__ __forceinline__ void rotate_rows_body(const RotateArgs& a);
__global__ void __launch_bounds__(256) rotate_rows_kernel(RotateArgs a) { rotate_rows_body(a); }
__global__ void __launch_bounds__(256) rotate_rows_multi_kernel(RotateParts ps) { rotate_rows_body(ps.p[blockIdx.z]); }
__device__ __forceinline__ void rotate_rows_body(const RotateArgs& a) {
    const int units = a.size - a.pairs;
    const int r = blockIdx.y;
    const int pos = a.row_pos[r];
    if (pos < 0) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.heads * units) return;
    const int h = i / units, u = i - h * units;
    const float* src = a.in + (size_t)r * a.ld_in + (size_t)h * a.hs_in;
    float* dst = a.cache != nullptr ? a.cache + (((size_t)a.row_slot[r] * a.heads + h) * a.Smax + pos) * a.size
                                    : a.out + (size_t)r * a.ld_out + (size_t)h * a.hs_out;
    const float* gate = a.gate != nullptr ? a.gate + (size_t)r * a.ldg + (size_t)h * a.size : nullptr;
    if (u >= a.offset && u < a.offset + a.pairs) {
        const int mp = u - a.offset, d = a.half ? a.offset + mp : a.offset + 2 * mp, d2 = a.half ? d + a.pairs : d + 1;
        const float2 cs = a.table[(size_t)pos * a.pairs + mp];
        const float sn = a.inverse ? -cs.y : cs.y;
        const float x = src[d], y = src[d2];
        float o0 = x * cs.x - y * sn, o1 = y * cs.x + x * sn;
        if (gate != nullptr) { o0 *= 1.f / (1.f + expf(-gate[d])); o1 *= 1.f / (1.f + expf(-gate[d2])); }
        dst[d] = o0; dst[d2] = o1;
    } else {
        const int d = u < a.offset ? u : u + a.pairs;
        float o = src[d];
        if (gate != nullptr) o *= 1.f / (1.f + expf(-gate[d]));
        dst[d] = o;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One warp per (row, head) of up to three parts: optional weighted RMS norm over the head, then the turn of its pairs. A lane reads
// everything it writes before it writes (its own pairs and single entries), and the sum of squares is complete before any lane writes,
// so the call may run in place.
__global__ void __launch_bounds__(256) rotate_rows_warp_kernel(RotateParts ps, int n_parts) {
    const int r = blockIdx.y, lane = threadIdx.x & 31;
    int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int pi = 0;
    while (pi < n_parts && w >= ps.p[pi].heads) { w -= ps.p[pi].heads; ++pi; }
    if (pi >= n_parts) return;
    const RotateArgs& a = ps.p[pi];
    const int pos = a.row_pos[r];
    if (pos < 0) return;
    const int h = w;
    const float* src = a.in + (size_t)r * a.ld_in + (size_t)h * a.hs_in;
    float* dst = a.cache != nullptr ? a.cache + (((size_t)a.row_slot[r] * a.heads + h) * a.Smax + pos) * a.size
                                    : a.out + (size_t)r * a.ld_out + (size_t)h * a.hs_out;
    const float* gate = a.gate != nullptr ? a.gate + (size_t)r * a.ldg + (size_t)h * a.size : nullptr;
    float mul = 1.f;
    if (a.norm_w != nullptr) {
        float q = 0.f;
        for (int d = lane; d < a.size; d += 32) q = fmaf(src[d], src[d], q);
        q = warp_sum(q);
        mul = 1.f / sqrtf(q / (float)a.size + a.eps);
    }
    __syncwarp();
    const int units = a.size - a.pairs;
    for (int u = lane; u < units; u += 32) {
        if (u >= a.offset && u < a.offset + a.pairs) {
            const int mp = u - a.offset, d = a.half ? a.offset + mp : a.offset + 2 * mp, d2 = a.half ? d + a.pairs : d + 1;
            const float2 cs = a.table[(size_t)pos * a.pairs + mp];
            const float sn = a.inverse ? -cs.y : cs.y;
            float x = src[d] * mul, y = src[d2] * mul;
            if (a.norm_w != nullptr) { x *= a.norm_w[d]; y *= a.norm_w[d2]; }
            float o0 = x * cs.x - y * sn, o1 = y * cs.x + x * sn;
            if (gate != nullptr) { o0 *= 1.f / (1.f + expf(-gate[d])); o1 *= 1.f / (1.f + expf(-gate[d2])); }
            dst[d] = o0; dst[d2] = o1;
        } else {
            const int d = u < a.offset ? u : u + a.pairs;
            float o = src[d] * mul;
            if (a.norm_w != nullptr) o *= a.norm_w[d];
            if (gate != nullptr) o *= 1.f / (1.f + expf(-gate[d]));
            dst[d] = o;
        }
    }
}

// cache[slot][pos] = [ unit_rms(in[r, :rank]) * gamma | the rot entries behind them, their first `pairs` pairs turned by pos ]
__global__ void __launch_bounds__(128) latent_rot_append_kernel(const float* __restrict__ in, int64_t ld_in, const float* __restrict__ gamma,
                                                                float* __restrict__ cache, const int32_t* __restrict__ row_slot,
                                                                const int32_t* __restrict__ row_pos, int rank, int rot, int pairs,
                                                                const float2* __restrict__ table, int Smax, float eps) {
    __shared__ float red[4];
    const size_t r = blockIdx.x;
    const int pos = row_pos[r];
    if (pos < 0) return;
    const float* src = in + r * ld_in;
    float q = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) q = fmaf(src[c], src[c], q);
    q = warp_sum(q);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
    __syncthreads();
    const float mul = 1.f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)rank + eps);
    float* dst = cache + ((size_t)row_slot[r] * Smax + pos) * (rank + rot);
    for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = src[c] * mul * gamma[c];
    for (int mp = threadIdx.x; mp < pairs; mp += blockDim.x) {
        const float2 cs = table[(size_t)pos * pairs + mp];
        const float x = src[rank + 2 * mp], y = src[rank + 2 * mp + 1];
        dst[rank + 2 * mp] = x * cs.x - y * cs.y;
        dst[rank + 2 * mp + 1] = y * cs.x + x * cs.y;
    }
    for (int c = rank + 2 * pairs + threadIdx.x; c < rank + rot; c += blockDim.x) dst[c] = src[c];
}
}  // namespace

int rotate_rows_f32(const RotateArgs& a, cudaStream_t st) {
    B2_CHECK_ARG(a.in && (a.out || a.cache) && (a.table || a.pairs == 0) && a.row_pos && a.rows > 0 && a.heads > 0 && a.size > 0, "rotate_rows: bad argument");
    B2_CHECK_ARG(a.pairs >= 0 && a.offset >= 0 && a.offset + 2 * a.pairs <= a.size, "rotate_rows: %d pairs from %d do not fit a head of %d", a.pairs, a.offset, a.size);
    B2_CHECK_ARG(a.cache == nullptr || (a.row_slot != nullptr && a.Smax > 0), "rotate_rows: a cache destination needs slots");
    if (a.norm_w != nullptr) return rotate_rows_multi_f32(&a, 1, st);
    const int units = a.heads * (a.size - a.pairs);
    rotate_rows_kernel<<<dim3((units + 255) / 256, a.rows), 256, 0, st>>>(a);
    B2_LAUNCH_CHECK();
    return 0;
}

int rotate_rows_multi_f32(const RotateArgs* parts, int n, cudaStream_t st) {
    B2_CHECK_ARG(parts && n >= 1 && n <= 3, "rotate_rows_multi: 1..3 parts");
    RotateParts ps;
    int units = 0, heads = 0;
    bool normed = false;
    for (int i = 0; i < n; ++i) {
        const RotateArgs& a = parts[i];
        B2_CHECK_ARG(a.in && (a.out || a.cache) && (a.table || a.pairs == 0) && a.row_pos && a.rows == parts[0].rows && a.heads > 0 && a.size > 0, "rotate_rows_multi: bad argument");
        B2_CHECK_ARG(a.pairs >= 0 && a.offset >= 0 && a.offset + 2 * a.pairs <= a.size, "rotate_rows_multi: %d pairs from %d do not fit a head of %d", a.pairs, a.offset, a.size);
        B2_CHECK_ARG(a.cache == nullptr || (a.row_slot != nullptr && a.Smax > 0), "rotate_rows_multi: a cache destination needs slots");
        ps.p[i] = a;
        units = std::max(units, a.heads * (a.size - a.pairs));
        normed = normed || a.norm_w != nullptr;
        heads += a.heads;
    }
    if (normed) {   // a normed head needs its sum of squares: one warp per (row, head) of every part
        rotate_rows_warp_kernel<<<dim3((heads + 7) / 8, parts[0].rows), 256, 0, st>>>(ps, n);
        B2_LAUNCH_CHECK();
        return 0;
    }
    rotate_rows_multi_kernel<<<dim3((units + 255) / 256, parts[0].rows, n), 256, 0, st>>>(ps);
    B2_LAUNCH_CHECK();
    return 0;
}

int latent_rot_append_f32(const float* in, int64_t ld_in, const float* gamma, float* cache, const int32_t* row_slot, const int32_t* row_pos, int rows,
                          int rank, int rot, int pairs, const float2* table, int Smax, float eps, cudaStream_t st) {
    B2_CHECK_ARG(in && gamma && cache && row_slot && row_pos && rows > 0 && rank > 0 && pairs >= 0 && 2 * pairs <= rot && (pairs == 0 || table), "latent_rot_append: bad argument");
    latent_rot_append_kernel<<<rows, 128, 0, st>>>(in, ld_in, gamma, cache, row_slot, row_pos, rank, rot, pairs, table, Smax, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

void rotary_frequencies(const RotaryDesc& d, std::vector<double>& freq, double& mag) {
    const int pairs = d.dims / 2;
    freq.resize(pairs);
    mag = 1.0;
    for (int i = 0; i < pairs; ++i) freq[i] = pow((double)d.base, -2.0 * i / d.dims);
    if (!(d.factor > 0.f)) return;
    const double two_pi = 6.283185307179586476925286766559;
    auto turn_dim = [&](double turns) { return d.dims * log((double)d.original / (two_pi * turns)) / (2.0 * log((double)d.base)); };
    const double lo = std::max(floor(turn_dim(d.fast)), 0.0), hi = std::min(ceil(turn_dim(d.slow)), (double)d.dims - 1.0);
    for (int i = 0; i < pairs; ++i) {
        const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
        freq[i] = freq[i] / d.factor * ramp + freq[i] * (1.0 - ramp);
    }
    mag = 0.1 * log((double)d.factor) + 1.0;
}

int rotary_table_build(const RotaryDesc& d, int positions, float2* table_dev) {
    B2_CHECK_ARG(d.dims >= 2 && d.base > 0.f && positions > 0 && table_dev, "rotary_table: bad argument");
    std::vector<double> freq;
    double mag;
    rotary_frequencies(d, freq, mag);
    const int pairs = d.dims / 2;
    std::vector<float2> tab((size_t)positions * pairs);
    for (int p = 0; p < positions; ++p)
        for (int i = 0; i < pairs; ++i) {
            const double ang = (double)p * freq[i];
            tab[(size_t)p * pairs + i] = make_float2((float)(cos(ang) * mag), (float)(sin(ang) * mag));
        }
    B2_CUDA_CHECK(cudaMemcpy(table_dev, tab.data(), tab.size() * sizeof(float2), cudaMemcpyHostToDevice));
    return 0;
}

}  // namespace b2
