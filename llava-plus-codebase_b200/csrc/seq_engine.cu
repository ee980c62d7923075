// Layer-list decoders behind the b2_model / b2_kv handles (include/b2llava.h, "layer-list decoders"): weights by tensor
// name, per-slot recurrent state and key/value slabs, and ONE forward over a set of rows that serves prompt portions
// (b2_append_tokens: n rows of one slot) and decode steps (one row per slot, replayed from the cache's CUDA graph by
// model.cu's decode_step_run with the same token selection and publication as the LLaMA path).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>

#include "engine.h"

namespace b2 {

struct SeqWeights {   // tensors of one layer that owns its weights
    // Linear weights in the compute dtype ([out, in]); vectors and small tables fp32
    DevBuf norm1, norm1_b, norm2, norm2_b;
    DevBuf in_w, conv_w, conv_b, dt_bias, a_log, skip, mnorm, o_w;                       // mamba2
    DevBuf lproj_w, rel, lo_w;                                                           // attention: [q | k | v | g] fused
    DevBuf mu, r_w, k_w, v_w, g_w, w1, w2, w0, bonus, rnorm, ro_w;                       // RWKV
    DevBuf up_w, down_w;                                                                 // feed-forward
    // pre-norm designs
    DevBuf qdg_w, dkv_norm, uk_w, ukT, uv_w, sink;      // latent attention: [q | dkv | g] fused; W_uk as stored and per head transposed to [rank][dim]
    DevBuf qfv_w, f_b, lower, hnorm;                    // HGRN2: [q | f | v] fused
    DevBuf up_b, down_b, down_b16, act_coef;            // PolyNorm feed-forward (bias of the second product also as bf16: GEMM epilogue)
    DevBuf router_w, egu_w, ed_w, sgu_w, sd_w;          // experts: [E][gate | up][width] (ungated: [E][up][width]), [E][width][ff]; shared expert likewise
    DevBuf canon1, canon2;                              // sandwich block: taps of the input convolutions [width][taps]
    DevBuf dq_norm, uq_w, ukx_w;                        // latent attention, further forms: norm of the queries' latent, W_uq, and W_uk widened per
                                                        // head by an identity block that carries the rotated key part ([H (dim + rot)][rank + rot])
    DevBuf qn_w, kn_w, lam4;                            // grouped attention, further forms: weights of the q / k norm; [lq1 | lk1 | lq2 | lk2] of
    float lambda = 0.f;                                 // differential attention and the layer's lambda (made from them when the model is finalized)
    DevBuf gla_w, a2_w, a2_b, gnorm;                    // gated linear attention: [q | k | v | g | a1] fused, W_a2 and its bias, the heads' norm weight
    std::map<std::string, int> got;
};

struct SeqLayerInfo {
    b2_seq_layer_desc d;
    int src = 0;                       // layer whose SeqWeights it uses
    // derived
    int inner = 0, conv_ch = 0, dproj = 0;            // mamba2: heads*vdim, inner + 2*groups*state, 2*inner + 2*groups*state + heads
    int nq = 0, nk = 0, nv = 0, ng = 0, lproj = 0;    // attention projection widths
    int rn = 0;                                       // RWKV heads*dim
    int dproj_ld = 0, lproj_ld = 0;                   // row pitch of the projection outputs (multiples of 8: tensor-core epilogue)
    int pq = 0, pproj = 0, pproj_ld = 0;              // latent attention / HGRN2: width of q, of the fused projection, its pitch
    int pv = 0;                                       // heads * vdim of those mixers
    int lqw = 0, lqw_ld = 0, lrow = 0;                // latent attention: heads * (dim + rot_dim) and its pitch, a cache row (rank + rot_dim)
    int maps = 1, gw = 0;                             // grouped attention: score maps per head (2: differential), width of the gate projection
};
struct SeqRun { int layer; int pass; int kv_run; };   // one layer run; pass >= 0: the run opens pass `pass` of the looped block; kv_run: the run
                                                      // whose cache rows a borrowing latent-attention layer reads (-1: its own)

struct SeqModel {
    b2_seq_model_desc d;
    std::vector<SeqLayerInfo> layers;
    std::vector<SeqRun> runs;          // what one forward pass executes, in order (a looped layer appears once per pass)
    std::vector<SeqWeights> w;
    DevBuf embed, head, final_w, final_b;
    DevBuf bigram, loop_step;          // [buckets + 1, width] in the weight dtype; [times, width] fp32
    DevBuf x0;                         // the embedding output, kept for the passes of a looped block
    DevBuf hin;                        // sandwich block: a sublayer's input after its convolution
    DevBuf qabs, olat;                 // latent attention: queries carried into the latent space, latent-space outputs [rows, heads*rank]
    DevBuf ffa;                        // activated feed-forward rows
    DevBuf rlogit, moe_idx, moe_w, moe_pos, moe_src, moe_tile, moe_h, moe_a, moe_y, moe_a16, zero_idx;   // router and grouped expert products
    int lat_w = 0, moe_rows = 0, moe_tiles = 0, moe_hw = 0, moe_aw = 0, moe_top = 0, moe_e = 0;
    std::map<std::string, int> got;
    int w_dtype = DT_BF16;             // dtype of the Linear weights and the embedding table on the device
    int rows = 0;                      // workspace rows
    // workspaces (fp32 unless noted)
    DevBuf x, proj, act, y, gated, mixout, mixes, rp, wl1, wlog, ff, xn, tok, want;
    DevBuf a16;                        // bf16 copy of a GEMM's A operand (tensor-core path of the bf16 compute mode)
    int a16_w = 0;
    DevBuf segs, row_slot, row_pos;
    int proj_w = 0, act_w = 0, y_w = 0, rp_w = 0, rank_w = 0, ff_w = 0;
};

struct SeqLayerState {
    DevBuf ssm, conv_tail;             // mamba2: [slots][heads][state][vdim], [slots][taps-1][channels]
    DevBuf kc, vc, bucket_of;          // attention: [slots][G][Smax][dk], [slots][G][Smax][dv], int32 [Smax]
    DevBuf wkv, prev;                  // RWKV: [slots][heads][dim][dim], [slots][width]
    DevBuf lat;                        // latent attention: [slots][Smax][rank]
    DevBuf gla;                        // HGRN2, gated linear attention: [slots][heads][dim][vdim]
    DevBuf canon1, canon2;             // sandwich block: the last taps-1 inputs of both sublayers [slots][taps-1][width]
    DevBuf rot_tab, vrot_tab;          // rotation tables (cos, sin) [Smax][pairs] of the queries / keys and of the values
};
struct SeqState {
    std::vector<SeqLayerState> layer;  // one per layer RUN
    DevBuf last_tok;                   // int32 [slots]: the token in front of the next one (hashed bigram embedding)
    DevBuf kmat, vmat;                 // latent attention, long prompt portions: per-head keys / values of one slot's positions [Smax][heads*size]
    int kmat_ld = 0, vmat_ld = 0;
    DevBuf attn_partial;
    int nsplit_max = 1;
};

namespace {

const size_t F4 = sizeof(float);
size_t esz(int dt) { return dt == DT_F32 ? 4 : 2; }

int64_t numel(const int64_t* shape, int ndim) {
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    return n;
}

// host-or-device tensor of `dtype` -> device buffer of `to` (DT_F32 or DT_BF16), at element offset `off` of a buffer of
// `total` elements (allocated on first use)
int put_tensor(DevBuf& buf, int to, size_t total, size_t off, const void* src, int dtype, int64_t n) {
    if (buf.p == nullptr) {
        B2_TRY(buf.alloc(total * esz(to)));
        B2_CUDA_CHECK(cudaMemset(buf.p, 0, total * esz(to)));
    }
    cudaPointerAttributes attr;
    bool on_device = false;
    if (cudaPointerGetAttributes(&attr, src) == cudaSuccess) on_device = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    else cudaGetLastError();
    const size_t sz = dtype == DT_F32 ? 4 : 2;
    DevBuf tmp;
    const void* dsrc = src;
    if (!on_device) {
        B2_TRY(tmp.alloc((size_t)n * sz));
        B2_CUDA_CHECK(cudaMemcpy(tmp.p, src, (size_t)n * sz, cudaMemcpyDefault));
        dsrc = tmp.p;
    }
    int r = to == DT_F32 ? convert_to_f32(dsrc, dtype, buf.as<float>() + off, n, 0)
                         : convert_to_bf16(dsrc, dtype, buf.as<__nv_bfloat16>() + off, n, 0);
    cudaError_t e = cudaStreamSynchronize(0);
    tmp.free();
    if (r != 0) return r;
    B2_CUDA_CHECK(e);
    return 0;
}

int want_shape(const char* key, const int64_t* shape, int ndim, int64_t a, int64_t b = -1) {
    const bool ok = b < 0 ? (numel(shape, ndim) == a) : (ndim == 2 && shape[0] == a && shape[1] == b);
    if (!ok) {
        char got[96] = {0};
        int o = 0;
        for (int i = 0; i < ndim && o < 80; ++i) o += snprintf(got + o, sizeof(got) - o, "%s%lld", i ? "x" : "", (long long)shape[i]);
        if (b < 0) set_error("set_weight(%s): shape %s, expected %lld elements", key, got, (long long)a);
        else set_error("set_weight(%s): shape %s, expected %lldx%lld", key, got, (long long)a, (long long)b);
        return -1;
    }
    return 0;
}

bool tc_enabled() {  // B2_SEQ_TC=0: every Linear on the FMA kernels (A/B runs, tests of the two paths against each other)
    const char* e = getenv("B2_SEQ_TC");
    return !(e != nullptr && e[0] == '0');
}

int tc_min_rows() {  // fewest rows that take the tensor-core GEMM (below: the weight-streaming FMA kernels)
    const char* e = getenv("B2_SEQ_TC_MIN_ROWS");
    const int v = e != nullptr ? atoi(e) : 0;
    // measured at widths 2048 / 4096 (decode step, ms): 4 rows 0.76 / 1.38 on the tile GEMM vs 0.78 / 1.48 on the FMA kernel,
    // 8 rows 0.87 / 1.59 vs 1.14 / 3.45; 2 rows 0.71 / 1.28 vs 0.62 / 1.10
    return v >= 1 ? v : 4;
}

struct Lin {  // one Linear call on the model's compute dtype
    const b2_model* m;
    cudaStream_t st;
    // whether a product of these sizes takes the tensor-core GEMM (bf16 compute, a portion of a prompt)
    bool tensor_cores(int N, int K, float* out, int64_t ldo, int M, const float* bias = nullptr, size_t w_row0 = 0, const void* bias16 = nullptr) const {
        const SeqModel& s = *m->seq;
        const int Np = (N + 7) / 8 * 8;
        return s.d.compute == B2_COMPUTE_BF16 && M >= tc_min_rows() && N >= 32 && K % 8 == 0 && K >= 32 && K <= s.a16_w && ldo % 8 == 0 && Np <= ldo &&
               (bias == nullptr || bias16 != nullptr) && (w_row0 == 0 || (N % 8 == 0 && (w_row0 * (size_t)K) % 8 == 0)) &&
               (reinterpret_cast<uintptr_t>(out) & 15) == 0 && tc_enabled();
    }
    // a16_ready: A is already there as bf16 rows of pitch K in the model's a16 buffer (the producing kernel wrote them): no cast
    int operator()(const float* A, int64_t lda, const DevBuf& W, int N, int K, float* out, int64_t ldo, int M, int act = LIN_NONE,
                   float alpha = 1.f, int accumulate = 0, const float* bias = nullptr, size_t w_row0 = 0, const void* bias16 = nullptr,
                   bool a16_ready = false) const {
        LinearArgs a;
        const SeqModel& s = *m->seq;
        a.A = A; a.lda = lda; a.ldw = K; a.w_dtype = s.w_dtype;
        a.W = reinterpret_cast<const char*>(W.p) + w_row0 * (size_t)K * esz(s.w_dtype);
        a.bias = bias; a.out = out; a.ld_out = ldo; a.M = M; a.N = N; a.K = K; a.act = act; a.alpha = alpha; a.accumulate = accumulate;
        a.round_a = s.d.compute == B2_COMPUTE_BF16;
        // bf16 compute, a portion of a prompt: the tcgen05 GEMM on a bf16 copy of A (weights are stored with their rows
        // padded to a multiple of 8, zero-filled, so N rounds up; the pitch of every projection buffer is a multiple of 8)
        const int Np = (N + 7) / 8 * 8;
        // a block of rows inside a matrix (w_row0 > 0) has no zero rows behind it: then N itself must be a multiple of 8; a bias
        // rides the epilogue as bf16
        if (tensor_cores(N, K, out, ldo, M, bias, w_row0, bias16)) {
            if (!a16_ready) B2_TRY(cast_rows_bf16(A, lda, s.a16.p, K, M, K, st));
            GemmArgs g;
            g.A = s.a16.p; g.lda = K; g.W = a.W; g.ldw = K; g.out = out; g.ld_out = (int)ldo; g.out_fp32 = 1; g.bias = bias16;
            g.M = M; g.N = Np; g.K = K; g.act = ACT_NONE; g.post = act; g.alpha = alpha; g.accumulate = accumulate;
            return gemm_bf16(g, st);
        }
        return linear_f32(a, st);
    }
};

int router_rows(int experts) { return std::max(32, (experts + 7) / 8 * 8); }   // rows of the (zero-padded) router matrix

int latent_materialise_rows() {  // prompt portions of at least this many rows make per-head keys / values instead of absorbing W_uk / W_uv
    const char* e = getenv("B2_LATENT_MATERIALISE_ROWS");
    const int v = e != nullptr ? atoi(e) : 0;
    return v >= 1 ? v : 64;
}

int attn_nsplit(int rows, int G, int max_seq) {
    // a decode step has few (row, key/value head) CTAs: cut the keys so that the step fills the SMs twice over, but keep
    // at least 32 keys (one staged tile) per cut at the cache's capacity
    if (rows > 8) return 1;
    int n = (2 * num_sms()) / (rows * G);
    const int cap = max_seq / 32;   // a cut is at least one tile of 32 keys
    if (n > cap) n = cap;
    if (n > 64) n = 64;
    return n < 1 ? 1 : n;
}

}  // namespace

// ------------------------------------------------------------------------------------------------------------------
// mixers and feed-forwards of the pre-norm and sandwich blocks: they read h [R, width] and write alpha * (their output) to
// `target` [R, width] (accumulate: onto what it holds)
// ------------------------------------------------------------------------------------------------------------------
static void mask_of(const b2_seq_layer_desc& d, BiasAttnArgs& aa) {
    aa.mask_kind = d.mask_kind;
    aa.mask_size = d.mask_size;
    aa.mask_keep = d.mask_keep;
}

// Attention over a low-rank latent. S: the run's own state (rotation table); KS: the state whose cache rows it reads (its own,
// or an earlier layer's). slot / ctx_end as for seq_forward.
static int latent_mixer(b2_model* m, b2_kv* kv, const SeqLayerInfo& L, SeqWeights& W, SeqLayerState& S, SeqLayerState& KS, const float* h, float* target,
                        float alpha, int accumulate, int R, int nseg, int slot, int ctx_end, cudaStream_t st) {
    SeqModel& s = *m->seq;
    SeqState& state = *kv->seq;
    const b2_seq_layer_desc& d = L.d;
    const Lin lin{m, st};
    const int width = s.d.width;
    const float eps = s.d.norm_eps;
    const int H = d.la_heads, dk = d.la_dim, dv = d.la_vdim, rank = d.la_rank, rd = d.la_rot_dim, qh = dk + rd, lrow = L.lrow;
    const int pairs = rd > 0 ? d.rot_dims / 2 : 0;
    const bool own = d.la_kv_from == 0, gate = d.la_no_gate == 0;
    const int max_n = nseg == 1 ? R : 1;
    const int32_t* row_slot = s.row_slot.as<int32_t>();
    const int32_t* row_pos = s.row_pos.as<int32_t>();
    const float2* tab = S.rot_tab.as<float2>();
    float* proj = s.proj.as<float>();  // [R, q (or the queries' latent) | dkv | g]
    B2_TRY(lin(h, width, W.qdg_w, L.pproj, width, proj, L.pproj_ld, R));
    float* q = proj;
    int64_t ldq = L.pproj_ld;
    if (d.la_q_rank > 0) {   // queries through their latent: norm in place, then up
        B2_TRY(rms_weight_f32(proj, L.pproj_ld, nullptr, W.dq_norm.as<float>(), proj, L.pproj_ld, 0, R, d.la_q_rank, eps, st));
        q = s.act.as<float>();
        ldq = L.lqw_ld;
        B2_TRY(lin(proj, L.pproj_ld, W.uq_w, L.lqw, d.la_q_rank, q, ldq, R));
    }
    if (own) B2_TRY(latent_rot_append_f32(proj + L.pq, L.pproj_ld, W.dkv_norm.as<float>(), S.lat.as<float>(), row_slot, row_pos, R, rank, rd, pairs, tab,
                                          kv->max_seq, eps, st));
    const float* gates = gate ? proj + L.pq + (own ? lrow : 0) : nullptr;
    float* lat_cache = KS.lat.as<float>();
    BiasAttnArgs aa;
    aa.sink = d.la_no_sink ? nullptr : W.sink.as<float>();
    aa.H = H; aa.Smax = kv->max_seq; aa.rows = R;
    aa.eps = eps; aa.scale = d.la_scale; aa.softcap = 0.f;
    aa.row_slot = row_slot; aa.row_pos = row_pos;
    aa.tile_rows = max_n;
    aa.partial = state.attn_partial.as<float>();
    mask_of(d, aa);
    float* y = s.y.as<float>();
    if (nseg == 1 && R >= latent_materialise_rows() && ctx_end > 0) {
        // a long portion: per-head keys and values of every visible position of the slot so far are made from the cached rows
        // with two products (the key product carries the rotated part through an identity block), and the attention runs over
        // them with the heads' own sizes
        if (pairs > 0) {
            RotateArgs ra;
            ra.in = q; ra.ld_in = ldq; ra.hs_in = qh; ra.out = q; ra.ld_out = ldq; ra.hs_out = qh;
            ra.table = tab; ra.heads = H; ra.size = qh; ra.offset = dk; ra.pairs = pairs; ra.rows = R; ra.row_pos = row_pos;
            B2_TRY(rotate_rows_f32(ra, st));
        }
        const float* lat = lat_cache + (size_t)slot * kv->max_seq * lrow;
        const int first = d.mask_kind == B2_MASK_WINDOW ? (d.mask_keep > 0 ? 0 : std::max(0, ctx_end - R - d.mask_size + 1))
                        : d.mask_kind == B2_MASK_CHUNK ? (ctx_end - R) / d.mask_size * d.mask_size : 0;
        const DevBuf& wk = rd > 0 ? W.ukx_w : W.uk_w;
        for (int m0 = first; m0 < ctx_end; m0 += s.rows) {
            const int mc = std::min(s.rows, ctx_end - m0);
            B2_TRY(lin(lat + (size_t)m0 * lrow, lrow, wk, L.lqw, lrow, state.kmat.as<float>() + (size_t)m0 * state.kmat_ld, state.kmat_ld, mc));
            B2_TRY(lin(lat + (size_t)m0 * lrow, lrow, W.uv_w, L.pv, rank, state.vmat.as<float>() + (size_t)m0 * state.vmat_ld, state.vmat_ld, mc));
        }
        aa.q = q; aa.ldq = ldq;
        aa.kcache = state.kmat.as<float>(); aa.vcache = state.vmat.as<float>();
        aa.kv_row_stride = state.kmat_ld; aa.kv_row_stride_v = state.vmat_ld;
        aa.out = y; aa.ldo = L.pv;
        aa.G = H; aa.dk = qh; aa.dv = dv; aa.nsplit = 1;
        B2_TRY(attn_bias_f32(aa, st));
    } else {
        // absorbed form: q_h -> W_uk_h^T q_h lives in the latent space (the rotated part rides behind it), so scores and values
        // read the cached rows directly, and W_uv_h carries the latent-space output to the head's values
        float* qabs = s.qabs.as<float>();
        const int64_t lq = (int64_t)H * lrow, lo = (int64_t)H * rank;
        const int round_a = s.d.compute == B2_COMPUTE_BF16;
        if (R <= 8) {
            B2_TRY(linear_batched_rows_f32(q, ldq, qh, W.ukT.p, (int64_t)rank * dk, s.w_dtype, qabs, lq, lrow, H, R, rank, dk, round_a, st));
        } else {
            for (int hh = 0; hh < H; ++hh)
                B2_TRY(lin(q + (size_t)hh * qh, ldq, W.ukT, rank, dk, qabs + (size_t)hh * lrow, lq, R, LIN_NONE, 1.f, 0, nullptr, (size_t)hh * rank));
        }
        if (rd > 0) {
            RotateArgs ra;
            ra.in = q + dk; ra.ld_in = ldq; ra.hs_in = qh; ra.out = qabs + rank; ra.ld_out = lq; ra.hs_out = lrow;
            ra.table = tab; ra.heads = H; ra.size = rd; ra.offset = 0; ra.pairs = pairs; ra.rows = R; ra.row_pos = row_pos;
            B2_TRY(rotate_rows_f32(ra, st));
        }
        aa.q = qabs; aa.ldq = lq;
        aa.kcache = lat_cache; aa.vcache = lat_cache;
        aa.out = s.olat.as<float>(); aa.ldo = lo;
        aa.G = 1; aa.dk = lrow; aa.dv = rank;
        aa.nsplit = attn_nsplit(R, (H + 31) / 32, kv->max_seq);
        if (aa.nsplit > state.nsplit_max) aa.nsplit = state.nsplit_max;
        B2_TRY(attn_bias_f32(aa, st));
        if (R <= 8) {   // with the heads' sigmoid gates in the same launch
            y = s.gated.as<float>();
            B2_TRY(linear_batched_rows_f32(s.olat.as<float>(), lo, rank, W.uv_w.p, (int64_t)dv * rank, s.w_dtype, y, L.pv, dv, H, R, dv, rank, round_a, st,
                                           gates, L.pproj_ld));
        } else {
            for (int hh = 0; hh < H; ++hh)
                B2_TRY(lin(s.olat.as<float>() + (size_t)hh * rank, lo, W.uv_w, dv, rank, y + (size_t)hh * dv, L.pv, R, LIN_NONE, 1.f, 0, nullptr, (size_t)hh * dv));
        }
    }
    if (gate && y != s.gated.as<float>()) {
        B2_TRY(head_gate_f32(y, L.pv, gates, L.pproj_ld, s.gated.as<float>(), L.pv, R, H, dv, st));
        y = s.gated.as<float>();
    }
    return lin(y, L.pv, W.o_w, width, L.pv, target, width, R, LIN_NONE, alpha, accumulate);
}

// Attention with grouped key/value heads, a short convolution on q / k / v, an optional weighted norm of the q / k heads, rotary q / k in
// either pair layout, optionally rotated values, a masked softmax with an optional fixed sink, and a sigmoid output gate per channel or
// per head. With two maps (differential attention) the projection rows were ordered [map][head][dim] when the tensors were set, so the
// maps are simply twice the query and key heads over the same value heads, and a head's two outputs are joined after the softmax.
static int gqa_mixer(b2_model* m, b2_kv* kv, const SeqLayerInfo& L, SeqWeights& W, SeqLayerState& S, const float* h, float* target, float alpha,
                     int accumulate, int R, int nseg, cudaStream_t st) {
    SeqModel& s = *m->seq;
    SeqState& state = *kv->seq;
    const b2_seq_layer_desc& d = L.d;
    const Lin lin{m, st};
    const int width = s.d.width;
    const int H = d.ga_heads, G = d.ga_kv_heads, dk = d.ga_dim, dv = d.ga_vdim, maps = L.maps;
    const int max_n = nseg == 1 ? R : 1;
    const SeqSeg* segs = s.segs.as<SeqSeg>();
    const int32_t* row_slot = s.row_slot.as<int32_t>();
    const int32_t* row_pos = s.row_pos.as<int32_t>();
    float* proj = s.proj.as<float>();  // [R, nq | nk | nv | gate]
    B2_TRY(lin(h, width, W.lproj_w, L.lproj, width, proj, L.lproj_ld, R));
    float* qkv = proj;
    int64_t ldc = L.lproj_ld;
    if (d.ga_conv >= 1) {
        qkv = s.act.as<float>();
        ldc = L.conv_ch;
        B2_TRY(causal_conv_f32(proj, L.lproj_ld, W.conv_w.as<float>(), nullptr, S.conv_tail.as<float>(), qkv, ldc, L.conv_ch, d.ga_conv, 0, segs, nseg, max_n, st));
    }
    // queries in place, keys into the cache, values into the cache (turned by their own position over all of vdim when the design
    // says so): one launch
    RotateArgs rq[3];
    for (RotateArgs& ra : rq) { ra.rows = R; ra.row_slot = row_slot; ra.row_pos = row_pos; ra.Smax = kv->max_seq; ra.ld_in = ldc; ra.offset = 0; }
    rq[0].in = qkv; rq[0].hs_in = dk; rq[0].out = qkv; rq[0].ld_out = ldc; rq[0].hs_out = dk; rq[0].heads = maps * H; rq[0].size = dk;
    rq[1].in = qkv + L.nq; rq[1].hs_in = dk; rq[1].cache = S.kc.as<float>(); rq[1].heads = maps * G; rq[1].size = dk;
    rq[0].table = rq[1].table = S.rot_tab.as<float2>(); rq[0].pairs = rq[1].pairs = d.rot_dims / 2;
    rq[0].half = rq[1].half = d.ga_rot_half;
    if (d.ga_qk_norm) { rq[0].norm_w = W.qn_w.as<float>(); rq[1].norm_w = W.kn_w.as<float>(); rq[0].eps = rq[1].eps = s.d.norm_eps; }
    rq[2].in = qkv + L.nq + L.nk; rq[2].hs_in = dv; rq[2].cache = S.vc.as<float>(); rq[2].heads = G; rq[2].size = dv;
    rq[2].table = S.vrot_tab.as<float2>(); rq[2].pairs = d.ga_rot_values ? dv / 2 : 0;
    B2_TRY(rotate_rows_multi_f32(rq, 3, st));
    BiasAttnArgs aa;
    aa.q = qkv; aa.ldq = ldc;
    aa.kcache = S.kc.as<float>(); aa.vcache = S.vc.as<float>();
    aa.out = s.y.as<float>(); aa.ldo = (int64_t)maps * L.ng;
    aa.H = maps * H; aa.G = maps * G; aa.Gv = maps > 1 ? G : 0; aa.dk = dk; aa.dv = dv; aa.Smax = kv->max_seq; aa.rows = R;
    aa.scale = d.ga_scale;
    aa.sink_fixed = d.ga_sink != 0; aa.sink_value = d.ga_sink_value;
    aa.row_slot = row_slot; aa.row_pos = row_pos;
    aa.nsplit = attn_nsplit(R, maps * G, kv->max_seq);
    aa.tile_rows = max_n;
    if (aa.nsplit > state.nsplit_max) aa.nsplit = state.nsplit_max;
    aa.partial = state.attn_partial.as<float>();
    mask_of(d, aa);
    const float* gates = proj + L.nq + L.nk + L.nv;
    // one sigmoid per head rides in the attention's last write (unless the head's output is still to be joined or turned back)
    const bool gate_in_attn = d.ga_gate == B2_GATE_HEAD && maps == 1 && !d.ga_rot_values;
    if (gate_in_attn) { aa.head_gate = gates; aa.ldg = L.lproj_ld; }
    B2_TRY(attn_bias_f32(aa, st));
    const float* yo = s.y.as<float>();
    float* gated = s.gated.as<float>();
    if (maps > 1) {   // a head's two maps: unit_rms(a1 - lambda a2) * (1 - diff)
        B2_TRY(diff_combine_f32(yo, (int64_t)maps * L.ng, gated, L.ng, R, H, dv, W.lambda, 1.f - d.ga_diff, s.d.norm_eps, st));
        yo = gated;
    }
    if (d.ga_rot_values || d.ga_gate == B2_GATE_CHANNEL) {
        // every head's output is turned back by the query's position, and the per-channel sigmoid gate is applied in the same pass
        RotateArgs rb;
        rb.in = yo; rb.ld_in = L.ng; rb.hs_in = dv; rb.out = gated; rb.ld_out = L.ng; rb.hs_out = dv;
        if (d.ga_gate == B2_GATE_CHANNEL) { rb.gate = gates; rb.ldg = L.lproj_ld; }
        rb.table = S.vrot_tab.as<float2>(); rb.heads = H; rb.size = dv; rb.offset = 0; rb.pairs = d.ga_rot_values ? dv / 2 : 0; rb.inverse = 1;
        rb.rows = R; rb.row_pos = row_pos;
        B2_TRY(rotate_rows_f32(rb, st));
        yo = gated;
    }
    if (d.ga_gate == B2_GATE_HEAD && !gate_in_attn) {   // one sigmoid per head
        B2_TRY(head_gate_f32(yo, L.ng, gates, L.lproj_ld, gated, L.ng, R, H, dv, st));
        yo = gated;
    }
    return lin(yo, L.ng, W.o_w, width, L.ng, target, width, R, LIN_NONE, alpha, accumulate);
}

// Gated linear attention: one fused projection [q | k | v | g | a1], the decay logits through the second low-rank matrix, the
// recurrence (decay, scaled query and state in fp32), per-head RMS norm with the gate, out-projection.
static int gla_mixer(b2_model* m, const SeqLayerInfo& L, SeqWeights& W, SeqLayerState& S, const float* h, float* target, float alpha, int accumulate,
                     int R, int nseg, cudaStream_t st) {
    SeqModel& s = *m->seq;
    const b2_seq_layer_desc& d = L.d;
    const Lin lin{m, st};
    const int width = s.d.width, H = d.gl_heads, dk = d.gl_dim, dv = d.gl_vdim;
    float* proj = s.proj.as<float>();
    B2_TRY(lin(h, width, W.gla_w, L.pproj, width, proj, L.pproj_ld, R));
    float* z = s.wlog.as<float>();   // [R, heads * dim] decay logits without their bias (the recurrence adds it in fp32)
    B2_TRY(lin(proj + 2 * L.pq + 2 * L.pv, L.pproj_ld, W.a2_w, L.pq, d.gl_rank, z, L.pq, R));
    ScanArgs sa;
    sa.mode = SCAN_GLA;
    sa.q = proj; sa.ldq = L.pproj_ld;
    sa.k = proj + L.pq; sa.ldk = L.pproj_ld;
    sa.v = proj + 2 * L.pq; sa.ldv = L.pproj_ld;
    sa.decay_in = z; sa.ldd = L.pq;
    sa.gate_bias = W.a2_b.as<float>();
    sa.q_scale = 1.f / sqrtf((float)dk); sa.tau = d.gl_tau;
    sa.state = S.gla.as<float>();
    sa.y = s.y.as<float>(); sa.ldy = L.pv;
    sa.heads = H; sa.groups = H; sa.dk = dk; sa.dv = dv;
    sa.segs = s.segs.as<SeqSeg>(); sa.nseg = nseg;
    B2_TRY(linear_scan_f32(sa, st));
    B2_TRY(gated_group_rmsnorm_f32(s.y.as<float>(), L.pv, proj + 2 * L.pq + L.pv, L.pproj_ld, W.gnorm.as<float>(), s.gated.as<float>(), L.pv, R, L.pv, dv,
                                   0, s.d.norm_eps, st, 1));
    return lin(s.gated.as<float>(), L.pv, W.o_w, width, L.pv, target, width, R, LIN_NONE, alpha, accumulate);
}

// What a sublayer of a sandwich block reads: the pending sublayer output (weight `post`, in mixout) joins x, x is normed with
// `norm` into xn, and the input convolution adds to it (a decode step: in the same launch). *h: where the result lies.
static int sandwich_input(SeqModel& s, const float* post, const DevBuf& norm, const DevBuf& taps_w, DevBuf& tail, int R, int nseg, int max_n,
                          cudaStream_t st, const float** h) {
    const int width = s.d.width, ctaps = s.d.input_conv_taps;
    SandwichNormArgs na;
    if (post != nullptr) { na.y = s.mixout.as<float>(); na.w_post = post; }
    na.x = s.x.as<float>(); na.w_pre = norm.as<float>(); na.out = s.xn.as<float>(); na.rows = R; na.cols = width; na.eps = s.d.norm_eps;
    *h = s.xn.as<float>();
    if (ctaps >= 1 && max_n == 1) {
        na.conv_w = taps_w.as<float>(); na.tail = tail.as<float>(); na.taps = ctaps; na.segs = s.segs.as<SeqSeg>(); na.conv_out = s.hin.as<float>();
        *h = s.hin.as<float>();
        return sandwich_norm_f32(na, st);
    }
    B2_TRY(sandwich_norm_f32(na, st));
    if (ctaps >= 1) {
        B2_TRY(causal_conv_f32(s.xn.as<float>(), width, taps_w.as<float>(), nullptr, tail.as<float>(), s.hin.as<float>(), width, width, ctaps, CONV_ADD_INPUT,
                               s.segs.as<SeqSeg>(), nseg, max_n, st));
        *h = s.hin.as<float>();
    }
    return 0;
}

// The feed-forward of a pre-norm or sandwich block in its three kinds.
static int seq_feed_forward(b2_model* m, const SeqLayerInfo& L, SeqWeights& W, const float* h, float* target, float alpha, int accumulate, int R,
                            cudaStream_t st) {
    SeqModel& s = *m->seq;
    const b2_seq_layer_desc& d = L.d;
    const Lin lin{m, st};
    const int width = s.d.width;
    const float eps = s.d.norm_eps;
    if (d.ff_kind == B2_FF_POLYNORM) {
        const int ffl = (d.ff + 7) / 8 * 8;
        B2_TRY(lin(h, width, W.up_w, d.ff, width, s.ff.as<float>(), ffl, R));
        B2_TRY(polynorm_f32(s.ff.as<float>(), ffl, W.up_b.as<float>(), W.act_coef.as<float>(), s.ffa.as<float>(), d.ff, R, d.ff, eps, st));
        return lin(s.ffa.as<float>(), d.ff, W.down_w, width, d.ff, target, width, R, LIN_NONE, alpha, accumulate, W.down_b.as<float>(), 0, W.down_b16.p);
    }
    if (d.ff_kind == B2_FF_CLAMP_GLU) {
        // [gate | up] in one matrix; the bounded gated unit a(g) (u + 1); a decode step of one row takes product and unit in one launch (more rows would
        // stream the matrix once per row there)
        const int ff = d.ff, ffl = (2 * ff + 7) / 8 * 8;
        const GluAct act{d.ff_act_slope, d.ff_limit, 1.f};
        if (R == 1) {
            GroupedLinearArgs gs;
            gs.A = h; gs.lda = width; gs.a_div = 1; gs.W = W.up_w.p; gs.ldw = width; gs.w_group_stride = 0; gs.w_dtype = s.w_dtype;
            gs.tile_group = s.zero_idx.as<int32_t>(); gs.tile_rows = 1; gs.out = s.ffa.as<float>(); gs.ld_out = ff;
            gs.M = R; gs.N = ff; gs.K = width; gs.round_a = s.d.compute == B2_COMPUTE_BF16; gs.swiglu = 1;
            gs.glu_slope = act.slope; gs.glu_limit = act.limit; gs.glu_up_shift = act.up_shift;
            B2_TRY(linear_grouped_f32(gs, st));
        } else {
            B2_TRY(lin(h, width, W.up_w, 2 * ff, width, s.ff.as<float>(), ffl, R));
            if (lin.tensor_cores(width, ff, target, width, R)) {   // the unit writes the bf16 rows that the second product reads
                B2_TRY(glu_rows_f32(s.ff.as<float>(), ffl, nullptr, 0, R, ff, act, st, s.a16.p, ff));
                return lin(nullptr, 0, W.down_w, width, ff, target, width, R, LIN_NONE, alpha, accumulate, nullptr, 0, nullptr, true);
            }
            B2_TRY(glu_rows_f32(s.ff.as<float>(), ffl, s.ffa.as<float>(), ff, R, ff, act, st));
        }
        return lin(s.ffa.as<float>(), ff, W.down_w, width, ff, target, width, R, LIN_NONE, alpha, accumulate);
    }
    if (d.ff_kind != B2_FF_MOE) {
        B2_TRY(lin(h, width, W.up_w, d.ff, width, s.ff.as<float>(), (d.ff + 7) / 8 * 8, R, LIN_RELU_SQ));
        return lin(s.ff.as<float>(), (d.ff + 7) / 8 * 8, W.down_w, width, d.ff, target, width, R, LIN_NONE, alpha, accumulate);
    }
    const int E = d.moe_experts, top = d.moe_top, ff = d.ff;
    const bool gated = d.moe_act == B2_MOE_ACT_SWIGLU;
    const int un = gated ? 2 * ff : ff;   // rows of an expert's first matrix: [gate | up], or up alone
    const int round_a = s.d.compute == B2_COMPUTE_BF16;
    B2_TRY(lin(h, width, W.router_w, router_rows(E), width, s.rlogit.as<float>(), router_rows(E), R));
    MoeRouteArgs ra;
    ra.logits = s.rlogit.as<float>(); ra.ld = router_rows(E); ra.rows = R; ra.experts = E; ra.top = top;
    ra.groups = d.moe_groups; ra.keep = d.moe_keep; ra.scale = d.moe_scale;
    ra.score_fn = d.moe_score; ra.group_score = d.moe_group_score; ra.raw_weights = d.moe_raw_weights;
    ra.idx = s.moe_idx.as<int32_t>(); ra.w = s.moe_w.as<float>();
    B2_TRY(moe_route_f32(ra, st));
    if (d.moe_shared_ff > 0) {
        const int sf = d.moe_shared_ff;
        if (!gated) {
            const int sfl = (sf + 7) / 8 * 8;
            B2_TRY(lin(h, width, W.sgu_w, sf, width, s.ff.as<float>(), sfl, R, LIN_RELU_SQ));
            B2_TRY(lin(s.ff.as<float>(), sfl, W.sd_w, width, sf, target, width, R, LIN_NONE, alpha, accumulate));
        } else {
            const int sfl = (2 * sf + 7) / 8 * 8;
            if (R <= 8) {   // decode step: both projections and the gate in one launch (the shared expert is "group 0" of its matrix)
                GroupedLinearArgs gs;
                gs.A = h; gs.lda = width; gs.a_div = 1; gs.W = W.sgu_w.p; gs.ldw = width; gs.w_group_stride = 0; gs.w_dtype = s.w_dtype;
                gs.tile_group = s.zero_idx.as<int32_t>(); gs.tile_rows = 1; gs.out = s.ffa.as<float>(); gs.ld_out = sf;
                gs.M = R; gs.N = sf; gs.K = width; gs.round_a = round_a; gs.swiglu = 1;
                B2_TRY(linear_grouped_f32(gs, st));
            } else {
                B2_TRY(lin(h, width, W.sgu_w, 2 * sf, width, s.ff.as<float>(), sfl, R));
                B2_TRY(swiglu_rows_f32(s.ff.as<float>(), sfl, s.ffa.as<float>(), sf, R, sf, st));
            }
            B2_TRY(lin(s.ffa.as<float>(), sf, W.sd_w, width, sf, target, width, R, LIN_NONE, alpha, accumulate));
        }
    } else if (!accumulate) {
        B2_CUDA_CHECK(cudaMemsetAsync(target, 0, (size_t)R * width * F4, st));
    }
    // routed experts: (token, choice) pairs as rows of grouped products. A decode step keeps the pairs where
    // they are (tiles of one row); a prompt portion sorts them by expert into tiles of 64 rows.
    GroupedLinearArgs ga;
    ga.A = h; ga.lda = width; ga.W = W.egu_w.p; ga.ldw = width; ga.w_group_stride = (int64_t)un * width; ga.w_dtype = s.w_dtype;
    ga.out = s.moe_h.as<float>(); ga.ld_out = un; ga.N = un; ga.K = width; ga.round_a = round_a;
    if (!gated) { ga.act = LIN_RELU_SQ; ga.out = s.moe_a.as<float>(); ga.ld_out = ff; }
    const int32_t* pos = nullptr;
    int P = R * top;
    const bool tc = ga.round_a && R >= 64 && tc_enabled() && width % 8 == 0 && ff % 8 == 0 && width >= 32 && ff >= 32;
    if (R <= 8) {   // decode step: gate, up and the gated activation of a pair in one launch
        ga.tile_rows = 1; ga.tile_group = s.moe_idx.as<int32_t>(); ga.a_div = top; ga.M = P;
        if (gated) { ga.swiglu = 1; ga.N = ff; ga.out = s.moe_a.as<float>(); ga.ld_out = ff; }
    } else {
        const int tile = tc ? 128 : GROUPED_TILE_ROWS;
        const int tiles = (R * top + E * (tile - 1) + tile - 1) / tile;
        B2_TRY(moe_plan(s.moe_idx.as<int32_t>(), R, top, E, tile, tiles, s.moe_pos.as<int32_t>(), s.moe_src.as<int32_t>(),
                        s.moe_tile.as<int32_t>(), st));
        pos = s.moe_pos.as<int32_t>();
        P = tiles * tile;
        ga.tile_rows = GROUPED_TILE_ROWS; ga.tile_group = s.moe_tile.as<int32_t>(); ga.a_rows = s.moe_src.as<int32_t>(); ga.M = P;
    }
    if (tc) {
        // tensor cores: the sorted pairs' input rows are gathered as bf16, every 128-row tile multiplies with its
        // expert's rows of the stacked weight matrices in ONE launch per product
        __nv_bfloat16* a16 = s.moe_a16.as<__nv_bfloat16>();
        __nv_bfloat16* h16 = a16 + (size_t)s.moe_rows * width;
        B2_TRY(gather_rows_bf16(h, width, s.moe_src.as<int32_t>(), a16, width, P, width, st));
        GemmArgs g1;
        g1.A = a16; g1.lda = width; g1.W = W.egu_w.p; g1.ldw = width; g1.out = s.moe_h.p; g1.ld_out = un; g1.out_fp32 = 1;
        g1.M = P; g1.N = un; g1.K = width; g1.tile_group = s.moe_tile.as<int32_t>(); g1.groups = E;
        if (!gated) g1.post = LIN_RELU_SQ;
        B2_TRY(gemm_bf16(g1, st));
        if (gated) B2_TRY(swiglu_rows_f32(s.moe_h.as<float>(), 2 * ff, nullptr, 0, P, ff, st, h16, ff));
        else B2_TRY(cast_rows_bf16(s.moe_h.as<float>(), ff, h16, ff, P, ff, st));
        GemmArgs g2;
        g2.A = h16; g2.lda = ff; g2.W = W.ed_w.p; g2.ldw = ff; g2.out = s.moe_y.p; g2.ld_out = width; g2.out_fp32 = 1;
        g2.M = P; g2.N = width; g2.K = ff; g2.tile_group = s.moe_tile.as<int32_t>(); g2.groups = E;
        B2_TRY(gemm_bf16(g2, st));
    } else {
        B2_TRY(linear_grouped_f32(ga, st));
        if (gated && !ga.swiglu) B2_TRY(swiglu_rows_f32(s.moe_h.as<float>(), 2 * ff, s.moe_a.as<float>(), ff, P, ff, st));
        GroupedLinearArgs gd = ga;
        gd.swiglu = 0; gd.act = LIN_NONE;
        gd.A = s.moe_a.as<float>(); gd.lda = ff; gd.a_rows = nullptr; gd.a_div = 1;
        gd.W = W.ed_w.p; gd.ldw = ff; gd.w_group_stride = (int64_t)width * ff;
        gd.out = s.moe_y.as<float>(); gd.ld_out = width; gd.N = width; gd.K = ff;
        B2_TRY(linear_grouped_f32(gd, st));
    }
    return moe_combine_f32(target, s.moe_y.as<float>(), width, pos, s.moe_w.as<float>(), R, top, width, alpha, st);
}

// ------------------------------------------------------------------------------------------------------------------
// forward over R rows described by the model's row map (nseg segments). x holds the embedded rows on entry.
// ------------------------------------------------------------------------------------------------------------------
// slot / ctx_end: for a prompt portion (nseg == 1) its slot and the slot's length after the call; 0 / 0 for a decode step
static int seq_forward(b2_model* m, b2_kv* kv, int R, int nseg, int slot, int ctx_end, float* resid_out, cudaStream_t st) {
    SeqModel& s = *m->seq;
    SeqState& state = *kv->seq;
    const int width = s.d.width;
    const float eps = s.d.norm_eps;
    const Lin lin{m, st};
    float* x = s.x.as<float>();
    float* mix = s.mixout.as<float>();
    const SeqSeg* segs = s.segs.as<SeqSeg>();
    const int max_n = nseg == 1 ? R : 1;  // a prompt portion is one segment of R rows; a decode step is R segments of one row
    const bool pre = s.d.block == B2_BLOCK_PRE_RMS1, sandwich = s.d.block == B2_BLOCK_SANDWICH_RMS, parallel = s.d.block == B2_BLOCK_PARALLEL_RMS;
    const bool direct = pre || parallel;   // a sublayer's last product adds residual_mult * its output onto x
    const float rm = s.d.residual_mult;
    float* xn = s.xn.as<float>();
    const float* post = nullptr;   // sandwich block: weight of the sublayer output in `mix` that has not joined x yet
    for (size_t ri = 0; ri < s.runs.size(); ++ri) {
        const size_t li = (size_t)s.runs[ri].layer;
        const SeqLayerInfo& L = s.layers[li];
        const b2_seq_layer_desc& d = L.d;
        SeqWeights& W = s.w[L.src];
        SeqLayerState& S = state.layer[ri];
        // a run that opens a pass of the looped block: x += (the embedding output, from the second pass on) + the pass's vector
        const int pass = s.runs[ri].pass;
        const float* pass_add = pass > 0 ? s.x0.as<float>() : nullptr;
        const float* pass_vec = pass >= 0 ? s.loop_step.as<float>() + (size_t)pass * width : nullptr;
        if (pre || sandwich || parallel) {
            // pre-norm block: a sublayer reads g * unit_rms(x) and adds residual_mult * its output onto x in its last product.
            // parallel block: ONE weighted RMS norm per layer; mixer and feed-forward both read it and both add onto x the same way.
            // sandwich block: a sublayer reads u + conv(u), u = rms_w(x); its output lands in `mix`, and its weighted RMS norm joins x in
            // the same pass that norms x for the next sublayer (`post`: the weight of a sublayer output that has not joined x yet).
            float* target = direct ? x : mix;
            const float alpha = direct ? rm : 1.f;
            const int acc = direct ? 1 : 0;
            const float* h = xn;
            if (pre) B2_TRY(rms_scalar_f32(x, nullptr, W.norm1.as<float>(), pass_add, pass_vec, xn, R, width, eps, st));
            else if (parallel) B2_TRY(rms_weight_f32(x, width, nullptr, W.norm1.as<float>(), xn, width, 0, R, width, eps, st));
            else B2_TRY(sandwich_input(s, post, W.norm1, W.canon1, S.canon1, R, nseg, max_n, st, &h));
            if (d.type == B2_MIXER_LATENT_ATTN) {
                SeqLayerState& KS = d.la_kv_from > 0 ? state.layer[s.runs[ri].kv_run] : S;
                B2_TRY(latent_mixer(m, kv, L, W, S, KS, h, target, alpha, acc, R, nseg, slot, ctx_end, st));
            } else if (d.type == B2_MIXER_GQA_ATTN) {
                B2_TRY(gqa_mixer(m, kv, L, W, S, h, target, alpha, acc, R, nseg, st));
            } else if (d.type == B2_MIXER_GLA) {
                B2_TRY(gla_mixer(m, L, W, S, h, target, alpha, acc, R, nseg, st));
            } else {
                float* proj = s.proj.as<float>();  // [R, q | f | v]
                const int H = d.g_heads, dk = d.g_dim, dv = d.g_vdim;
                B2_TRY(lin(h, width, W.qfv_w, L.pproj, width, proj, L.pproj_ld, R));
                ScanArgs sa;
                sa.mode = SCAN_HGRN2;
                sa.q = proj; sa.ldq = L.pproj_ld;
                sa.decay_in = proj + L.pq; sa.ldd = L.pproj_ld;
                sa.v = proj + 2 * L.pq; sa.ldv = L.pproj_ld;
                sa.gate_bias = W.f_b.as<float>(); sa.gate_lower = W.lower.as<float>();
                sa.state = S.gla.as<float>();
                sa.y = s.y.as<float>(); sa.ldy = L.pv;
                sa.heads = H; sa.groups = H; sa.dk = dk; sa.dv = dv;
                sa.segs = segs; sa.nseg = nseg;
                B2_TRY(linear_scan_f32(sa, st));
                B2_TRY(group_rmsnorm_f32(s.y.as<float>(), L.pv, W.hnorm.as<float>(), 1, s.gated.as<float>(), L.pv, R, L.pv, dv, eps, st));
                B2_TRY(lin(s.gated.as<float>(), L.pv, W.o_w, width, L.pv, target, width, R, LIN_NONE, alpha, acc));
            }
            post = sandwich ? W.norm1_b.as<float>() : nullptr;
            if (d.ff > 0) {
                h = xn;   // parallel block: the feed-forward reads what the mixer read
                if (pre) B2_TRY(rms_scalar_f32(x, nullptr, W.norm2.as<float>(), nullptr, nullptr, xn, R, width, eps, st));
                else if (sandwich) B2_TRY(sandwich_input(s, post, W.norm2, W.canon2, S.canon2, R, nseg, max_n, st, &h));
                B2_TRY(seq_feed_forward(m, L, W, h, target, alpha, acc, R, st));
                post = sandwich ? W.norm2_b.as<float>() : nullptr;
            }
            if (post != nullptr && (resid_out != nullptr || ri + 1 == s.runs.size())) {   // the last sublayer's output joins x now
                SandwichNormArgs na;
                na.y = mix; na.w_post = post; na.x = x; na.rows = R; na.cols = width; na.eps = eps;
                B2_TRY(sandwich_norm_f32(na, st));
                post = nullptr;
            }
            if (resid_out != nullptr)
                B2_CUDA_CHECK(cudaMemcpyAsync(resid_out + ri * (size_t)R * width, x, (size_t)R * width * F4, cudaMemcpyDeviceToDevice, st));
            continue;
        }
        if (pass >= 0) B2_TRY(rms_scalar_f32(x, nullptr, nullptr, pass_add, pass_vec, nullptr, R, width, eps, st));
        if (d.type == B2_MIXER_MAMBA2) {
            float* proj = s.proj.as<float>();
            const int gn = d.m_groups * d.m_state;
            B2_TRY(lin(x, width, W.in_w, L.dproj, width, proj, L.dproj_ld, R));
            float* act = s.act.as<float>();  // [R, conv_ch] = silu(conv(x | B | C))
            B2_TRY(causal_conv_silu_f32(proj + L.inner, L.dproj_ld, W.conv_w.as<float>(), W.conv_b.as<float>(), S.conv_tail.as<float>(), act,
                                        L.conv_ch, L.conv_ch, d.m_conv, segs, nseg, max_n, st));
            ScanArgs sa;
            sa.mode = SCAN_SSD;
            sa.v = act; sa.ldv = L.conv_ch;
            sa.k = act + L.inner; sa.ldk = L.conv_ch;
            sa.q = act + L.inner + gn; sa.ldq = L.conv_ch;
            sa.decay_in = proj + 2 * L.inner + 2 * gn; sa.ldd = L.dproj_ld;
            sa.dt_bias = W.dt_bias.as<float>(); sa.a_log = W.a_log.as<float>(); sa.skip = W.skip.as<float>();
            sa.state = S.ssm.as<float>();
            sa.y = s.y.as<float>(); sa.ldy = L.inner;
            sa.heads = d.m_heads; sa.groups = d.m_groups; sa.dk = d.m_state; sa.dv = d.m_vdim;
            sa.segs = segs; sa.nseg = nseg;
            B2_TRY(linear_scan_f32(sa, st));
            B2_TRY(gated_group_rmsnorm_f32(s.y.as<float>(), L.inner, proj, L.dproj_ld, W.mnorm.as<float>(), s.gated.as<float>(), L.inner, R, L.inner,
                                           L.inner / d.m_norm_groups, 1, eps, st));
            B2_TRY(lin(s.gated.as<float>(), L.inner, W.o_w, width, L.inner, mix, width, R));
        } else {
            // ---- left: attention -------------------------------------------------------------------------------------
            float* proj = s.proj.as<float>();  // [R, nq | nk | nv | ng]
            B2_TRY(lin(x, width, W.lproj_w, L.lproj, width, proj, L.lproj_ld, R));
            BiasAttnArgs aa;
            aa.q = proj; aa.ldq = L.lproj_ld;
            aa.k = proj + L.nq; aa.ldk = L.lproj_ld;
            aa.v = proj + L.nq + L.nk; aa.ldv = L.lproj_ld;
            aa.kcache = S.kc.as<float>(); aa.vcache = S.vc.as<float>();
            aa.out = s.y.as<float>(); aa.ldo = L.ng;
            aa.rel = W.rel.as<float>(); aa.bucket_of = S.bucket_of.as<int32_t>();
            aa.H = d.a_heads; aa.G = d.a_kv_heads; aa.dk = d.a_dim; aa.dv = d.a_vdim; aa.Smax = kv->max_seq; aa.rows = R;
            aa.eps = eps; aa.scale = d.a_scale; aa.softcap = d.a_softcap; aa.temp_coef = d.a_temp_coef; aa.temp_every = d.a_temp_every;
            aa.row_slot = s.row_slot.as<int32_t>(); aa.row_pos = s.row_pos.as<int32_t>();
            aa.nsplit = attn_nsplit(R, d.a_kv_heads, kv->max_seq);
            aa.tile_rows = max_n;
            if (aa.nsplit > state.nsplit_max) aa.nsplit = state.nsplit_max;
            aa.partial = state.attn_partial.as<float>();
            B2_TRY(attn_prepare_f32(aa, st));
            B2_TRY(attn_bias_f32(aa, st));
            B2_TRY(sigmoid_gate_f32(s.y.as<float>(), L.ng, proj + L.nq + L.nk + L.nv, L.lproj_ld, s.gated.as<float>(), L.ng, R, L.ng, st));
            B2_TRY(lin(s.gated.as<float>(), L.ng, W.lo_w, width, L.ng, mix, width, R, LIN_NONE, d.left_scale));
            // ---- right: RWKV time mixing -------------------------------------------------------------------------------
            const size_t ms = (size_t)s.rows * width;  // stride between the five mixes (r, k, v, g, w)
            float* mixes = s.mixes.as<float>();
            B2_TRY(token_shift_mix_f32(x, W.mu.as<float>(), S.prev.as<float>(), mixes, ms, width, 5, segs, nseg, max_n, st));
            float* rp = s.rp.as<float>();      // [4][rows][rn]: r, k, v, g
            const size_t rs = (size_t)s.rows * L.rn;
            B2_TRY(lin(mixes + 0 * ms, width, W.r_w, L.rn, width, rp + 0 * rs, L.rn, R));
            B2_TRY(lin(mixes + 1 * ms, width, W.k_w, L.rn, width, rp + 1 * rs, L.rn, R));
            B2_TRY(lin(mixes + 2 * ms, width, W.v_w, L.rn, width, rp + 2 * rs, L.rn, R));
            B2_TRY(lin(mixes + 3 * ms, width, W.g_w, L.rn, width, rp + 3 * rs, L.rn, R));
            B2_TRY(lin(mixes + 4 * ms, width, W.w1, d.r_decay_rank, width, s.wl1.as<float>(), d.r_decay_rank, R, LIN_TANH));
            B2_TRY(lin(s.wl1.as<float>(), d.r_decay_rank, W.w2, L.rn, d.r_decay_rank, s.wlog.as<float>(), L.rn, R, LIN_NONE, 1.f, 0, W.w0.as<float>()));
            ScanArgs sa;
            sa.mode = SCAN_RWKV;
            sa.q = rp; sa.ldq = L.rn;
            sa.k = rp + rs; sa.ldk = L.rn;
            sa.v = rp + 2 * rs; sa.ldv = L.rn;
            sa.decay_in = s.wlog.as<float>(); sa.ldd = L.rn;
            sa.bonus = W.bonus.as<float>();
            sa.state = S.wkv.as<float>();
            sa.y = s.y.as<float>(); sa.ldy = L.rn;
            sa.heads = d.r_heads; sa.groups = d.r_heads; sa.dk = d.r_dim; sa.dv = d.r_dim;
            sa.segs = segs; sa.nseg = nseg;
            B2_TRY(linear_scan_f32(sa, st));
            B2_TRY(gated_group_rmsnorm_f32(s.y.as<float>(), L.rn, rp + 3 * rs, L.rn, W.rnorm.as<float>(), s.gated.as<float>(), L.rn, R, L.rn, d.r_dim,
                                           0, eps, st));
            B2_TRY(lin(s.gated.as<float>(), L.rn, W.ro_w, width, L.rn, mix, width, R, LIN_NONE, d.right_scale, 1));
        }
        B2_TRY(layernorm_add_f32(x, mix, W.norm1.as<float>(), W.norm1_b.as<float>(), R, width, eps, st));
        if (d.ff > 0) {
            B2_TRY(lin(x, width, W.up_w, d.ff, width, s.ff.as<float>(), d.ff, R, LIN_RELU_SQ));
            B2_TRY(lin(s.ff.as<float>(), d.ff, W.down_w, width, d.ff, mix, width, R));
            B2_TRY(layernorm_add_f32(x, mix, W.norm2.as<float>(), W.norm2_b.as<float>(), R, width, eps, st));
        }
        if (resid_out != nullptr)
            B2_CUDA_CHECK(cudaMemcpyAsync(resid_out + ri * (size_t)R * width, x, (size_t)R * width * F4, cudaMemcpyDeviceToDevice, st));
    }
    return 0;
}

// token rows -> x (and the kept copy x0 of a looped model); tokens are indexed by row
static int seq_embed(b2_model* m, b2_kv* kv, const int32_t* tokens, int R, int nseg, cudaStream_t st) {
    SeqModel& s = *m->seq;
    if (s.d.bigram_buckets > 0 || s.x0.p != nullptr)
        return embed_bigram_rows_f32(tokens, s.segs.as<SeqSeg>(), nseg, nseg == 1 ? R : 1, s.embed.p, s.bigram.p, s.w_dtype, kv->seq->last_tok.as<int32_t>(),
                                     s.x.as<float>(), s.x0.as<float>(), s.d.width, s.d.vocab, s.d.bigram_buckets, s.d.bigram_mul_prev, s.d.bigram_mul_cur,
                                     m->err_dev, st);
    return embed_rows_f32(tokens, s.embed.p, s.w_dtype, s.x.as<float>(), R, s.d.width, s.d.vocab, m->err_dev, st, s.d.embed_scale != 0.f ? s.d.embed_scale : 1.f);
}

// rows `index` (null: all) of x -> final norm -> head -> soft-cap: fp32 logits [n, vocab]
static int seq_head(b2_model* m, const int32_t* index, int n, float* logits, int64_t ld, cudaStream_t st) {
    SeqModel& s = *m->seq;
    if (s.d.block == B2_BLOCK_PRE_RMS1)
        B2_TRY(rms_scalar_f32(s.x.as<float>(), index, s.final_w.as<float>(), nullptr, nullptr, s.xn.as<float>(), n, s.d.width, s.d.norm_eps, st));
    else if (s.d.block == B2_BLOCK_SANDWICH_RMS || s.d.block == B2_BLOCK_PARALLEL_RMS)
        B2_TRY(rms_weight_f32(s.x.as<float>(), s.d.width, index, s.final_w.as<float>(), s.xn.as<float>(), s.d.width, 0, n, s.d.width, s.d.norm_eps, st));
    else
        B2_TRY(layernorm_gather_f32(s.x.as<float>(), index, s.final_w.as<float>(), s.final_b.as<float>(), s.xn.as<float>(), n, s.d.width, s.d.norm_eps, st));
    const Lin lin{m, st};
    B2_TRY(lin(s.xn.as<float>(), s.d.width, s.head, s.d.vocab, s.d.width, logits, ld, n, LIN_NONE, s.d.logit_scale != 0.f ? s.d.logit_scale : 1.f));
    if (s.d.logit_softcap > 0.f) {
        B2_CHECK_ARG(ld == s.d.vocab, "seq_head: soft-capped logits are contiguous rows");
        B2_TRY(softcap_f32(logits, (size_t)n * s.d.vocab, s.d.logit_softcap, st));
    }
    return 0;
}

// one decode step over the slots [slot0, slot0 + B): kv->tok -> logits (m->logits) -> token selection, lengths += 1
int seq_decode_launch(b2_model* m, b2_kv* kv, int B, int slot0, cudaStream_t st) {
    SeqModel& s = *m->seq;
    RowMap rm{s.segs.as<SeqSeg>(), s.row_slot.as<int32_t>(), s.row_pos.as<int32_t>()};
    B2_TRY(rowmap_decode(rm, kv->len_dev.as<int32_t>(), kv->sstate.as<SampleState>(), kv->rows_dev.as<RowState>(), slot0, B, st));
    B2_TRY(seq_embed(m, kv, kv->tok.as<int32_t>() + slot0, B, B, st));
    B2_TRY(seq_forward(m, kv, B, B, 0, 0, nullptr, st));
    B2_TRY(seq_head(m, nullptr, B, m->logits.as<float>(), s.d.vocab, st));
    B2_TRY(sample_publish(m->logits.as<float>(), s.d.vocab, B, kv->sstate.as<SampleState>(), kv->rows_dev.as<RowState>() + slot0,
                          kv->tok.as<int32_t>() + slot0, kv->out_tokens.as<int32_t>(), kv->step_counter.as<int32_t>(),
                          kv->len_dev.as<int32_t>() + slot0, kv->ring_dev, kv->ring_cap, SP_SELECT | SP_WRITE_OUT | SP_BUMP, 0, st));
    return 0;
}

// ------------------------------------------------------------------------------------------------------------------
// weights
// ------------------------------------------------------------------------------------------------------------------
int seq_set_weight(b2_model* m, const char* key, const void* ptr, const int64_t* shape, int ndim, int dt) {
    SeqModel& s = *m->seq;
    const int width = s.d.width, V = s.d.vocab, WD = s.w_dtype;
    const std::string k(key);
    if (k == "embed") { B2_TRY(want_shape(key, shape, ndim, V, width)); s.got[k] = 1; return put_tensor(s.embed, WD, (size_t)V * width, 0, ptr, dt, (int64_t)V * width); }
    if (k == "head") { B2_TRY(want_shape(key, shape, ndim, V, width)); s.got[k] = 1; return put_tensor(s.head, WD, (size_t)((V + 7) / 8 * 8) * width, 0, ptr, dt, (int64_t)V * width); }
    const bool sandwich = s.d.block == B2_BLOCK_SANDWICH_RMS, parallel = s.d.block == B2_BLOCK_PARALLEL_RMS;
    const bool pre = s.d.block == B2_BLOCK_PRE_RMS1 || sandwich || parallel;   // blocks whose layers are made of the mixers / feed-forwards below
    if (k == "final.norm" && s.d.block == B2_BLOCK_PRE_RMS1) { B2_TRY(want_shape(key, shape, ndim, 1)); s.got[k] = 1; return put_tensor(s.final_w, DT_F32, 1, 0, ptr, dt, 1); }
    if (k == "bigram" && s.d.bigram_buckets > 0) {
        const int64_t rows = (int64_t)s.d.bigram_buckets + 1;
        B2_TRY(want_shape(key, shape, ndim, rows, width)); s.got[k] = 1;
        return put_tensor(s.bigram, WD, (size_t)rows * width, 0, ptr, dt, rows * width);
    }
    if (k == "loop.step" && s.d.loop_times >= 1 && !s.d.loop_plain) {
        B2_TRY(want_shape(key, shape, ndim, s.d.loop_times, width)); s.got[k] = 1;
        return put_tensor(s.loop_step, DT_F32, (size_t)s.d.loop_times * width, 0, ptr, dt, (int64_t)s.d.loop_times * width);
    }
    if (k == "final.norm") { B2_TRY(want_shape(key, shape, ndim, width)); s.got[k] = 1; return put_tensor(s.final_w, DT_F32, width, 0, ptr, dt, width); }
    if (k == "final.norm.b") { B2_TRY(want_shape(key, shape, ndim, width)); s.got[k] = 1; return put_tensor(s.final_b, DT_F32, width, 0, ptr, dt, width); }
    int li = -1, used = 0;
    if (sscanf(key, "l%d.%n", &li, &used) != 1 || used == 0 || li < 0 || li >= (int)s.layers.size()) {
        set_error("set_weight: unknown tensor '%s'", key);
        return -1;
    }
    const SeqLayerInfo& L = s.layers[li];
    B2_CHECK_ARG(L.src == li, "set_weight(%s): layer %d uses the tensors of layer %d and has none of its own", key, li, L.src);
    const b2_seq_layer_desc& d = L.d;
    SeqWeights& W = s.w[li];
    const std::string r = k.substr(used);
    auto vec = [&](DevBuf& b, int64_t n) -> int { B2_TRY(want_shape(key, shape, ndim, n)); W.got[r] = 1; return put_tensor(b, DT_F32, n, 0, ptr, dt, n); };
    // Linear weights are allocated with their rows padded to a multiple of 8 (zeros): the tensor-core GEMM wants N % 8 == 0
    auto mat = [&](DevBuf& b, int64_t o, int64_t i) -> int { B2_TRY(want_shape(key, shape, ndim, o, i)); W.got[r] = 1; return put_tensor(b, WD, (size_t)((o + 7) / 8 * 8) * i, 0, ptr, dt, o * i); };
    if (pre) {
        // a fused matrix of several projections that share their input: part j lands at its row offset
        auto part = [&](DevBuf& b, int total_rows, int row0, int rows, int cols) -> int {
            B2_TRY(want_shape(key, shape, ndim, rows, cols));
            W.got[r] = 1;
            return put_tensor(b, WD, (size_t)((total_rows + 7) / 8 * 8) * cols, (size_t)row0 * cols, ptr, dt, (int64_t)rows * cols);
        };
        auto taps_of = [&](DevBuf& b, int64_t ch, int64_t total_ch, int64_t ch0, int taps) -> int {   // [channels][taps] at its channel offset
            B2_TRY(want_shape(key, shape, ndim, ch, taps));
            W.got[r] = 1;
            return put_tensor(b, DT_F32, (size_t)total_ch * taps, (size_t)ch0 * taps, ptr, dt, ch * taps);
        };
        if (sandwich) {
            const int ct = s.d.input_conv_taps;
            if (r == "norm1") return vec(W.norm1, width);
            if (r == "norm1b") return vec(W.norm1_b, width);
            if (r == "canon1" && ct >= 1) return taps_of(W.canon1, width, width, 0, ct);
            if (d.ff > 0) {
                if (r == "norm2") return vec(W.norm2, width);
                if (r == "norm2b") return vec(W.norm2_b, width);
                if (r == "canon2" && ct >= 1) return taps_of(W.canon2, width, width, 0, ct);
            }
        } else if (parallel) {
            if (r == "norm1") return vec(W.norm1, width);
        } else {
            if (r == "norm1") return vec(W.norm1, 1);
            if (r == "norm2" && d.ff > 0) return vec(W.norm2, 1);
        }
        if (d.type == B2_MIXER_LATENT_ATTN) {
            const int H = d.la_heads, dk = d.la_dim, dv = d.la_vdim, rank = d.la_rank, rd = d.la_rot_dim;
            const bool own = d.la_kv_from == 0;
            if (r == "mix.q" && d.la_q_rank == 0) return part(W.qdg_w, L.pproj, 0, L.pq, width);
            if (r == "mix.dq" && d.la_q_rank > 0) return part(W.qdg_w, L.pproj, 0, L.pq, width);
            if (r == "mix.dq.norm" && d.la_q_rank > 0) return vec(W.dq_norm, d.la_q_rank);
            if (r == "mix.uq" && d.la_q_rank > 0) return mat(W.uq_w, L.lqw, d.la_q_rank);
            if (r == "mix.dkv" && own) return part(W.qdg_w, L.pproj, L.pq, L.lrow, width);
            if (r == "mix.g" && !d.la_no_gate) return part(W.qdg_w, L.pproj, L.pq + (own ? L.lrow : 0), H, width);
            if (r == "mix.dkv.norm" && own) return vec(W.dkv_norm, rank);
            if (r == "mix.sink" && !d.la_no_sink) return vec(W.sink, H);
            if (r == "mix.uv") return mat(W.uv_w, (int64_t)H * dv, rank);
            if (r == "mix.o") return mat(W.o_w, width, (int64_t)H * dv);
            if (r == "mix.uk") {
                // kept as stored (keys of long prompt portions) and per head as [rank][dim] (the query is carried into the latent
                // space by a Linear with this matrix)
                B2_TRY(mat(W.uk_w, (int64_t)H * dk, rank));
                int rc = W.ukT.alloc(((size_t)H * rank + 8) * dk * esz(WD));
                if (rc == 0) rc = cudaMemset(W.ukT.p, 0, W.ukT.bytes) == cudaSuccess ? 0 : -2;
                if (rc == 0) rc = transpose_blocks(W.uk_w.p, W.ukT.p, H, dk, rank, (int)esz(WD), 0);
                cudaStreamSynchronize(0);
                if (rc != 0 || rd == 0) return rc;
                // with a rotated key part: head h's rows [W_uk_h 0; 0 I], so that ONE product over the cached rows [c | rotated part]
                // gives every head's whole key
                const size_t e = esz(WD), lrow = (size_t)L.lrow, qh = (size_t)dk + rd;
                B2_TRY(W.ukx_w.alloc(((size_t)H * qh + 8) * lrow * e));
                B2_CUDA_CHECK(cudaMemset(W.ukx_w.p, 0, W.ukx_w.bytes));
                std::vector<unsigned char> eye((size_t)rd * rd * e, 0);
                for (int i = 0; i < rd; ++i) {
                    if (WD == DT_F32) reinterpret_cast<float*>(eye.data())[(size_t)i * rd + i] = 1.f;
                    else reinterpret_cast<uint16_t*>(eye.data())[(size_t)i * rd + i] = 0x3F80;   // 1.0 as bfloat16
                }
                for (int hh = 0; hh < H; ++hh) {
                    char* dst = W.ukx_w.as<char>() + (size_t)hh * qh * lrow * e;
                    B2_CUDA_CHECK(cudaMemcpy2D(dst, lrow * e, W.uk_w.as<char>() + (size_t)hh * dk * rank * e, (size_t)rank * e, (size_t)rank * e, dk,
                                               cudaMemcpyDeviceToDevice));
                    B2_CUDA_CHECK(cudaMemcpy2D(dst + ((size_t)dk * lrow + rank) * e, lrow * e, eye.data(), (size_t)rd * e, (size_t)rd * e, rd,
                                               cudaMemcpyHostToDevice));
                }
                return 0;
            }
        } else if (d.type == B2_MIXER_GQA_ATTN) {
            // the four projections share their input: one [nq + nk + nv + gate, width] matrix, one product; the taps of q, k, v side by side
            const char* parts[4] = {"mix.q", "mix.k", "mix.v", "mix.g"};
            const int sizes[4] = {L.nq, L.nk, L.nv, L.gw};
            const int heads_of[2] = {d.ga_heads, d.ga_kv_heads};
            int row0 = 0;
            for (int j = 0; j < 4; ++j) {
                const bool is_w = r == parts[j] && sizes[j] > 0, is_taps = j < 3 && d.ga_conv >= 1 && r == std::string(parts[j]) + ".conv";
                if ((is_w || is_taps) && j < 2 && L.maps > 1) {
                    // two maps: the checkpoint orders the rows [head][map][dim]; here they lie [map][head][dim], so that the maps are further
                    // heads (query head index = map * heads + head, the same for the keys) and share the value heads
                    const int cols = is_w ? width : d.ga_conv, nh = heads_of[j], dk = d.ga_dim;
                    B2_TRY(want_shape(key, shape, ndim, sizes[j], cols));
                    W.got[r] = 1;
                    const size_t sz = dt == DT_F32 ? 4 : 2;
                    for (int hh = 0; hh < nh; ++hh)
                        for (int mp = 0; mp < L.maps; ++mp) {
                            const char* src = reinterpret_cast<const char*>(ptr) + (size_t)(hh * L.maps + mp) * dk * cols * sz;
                            const size_t dst_row = (size_t)row0 + (size_t)(mp * nh + hh) * dk;
                            if (is_w) B2_TRY(put_tensor(W.lproj_w, WD, (size_t)((L.lproj + 7) / 8 * 8) * cols, dst_row * cols, src, dt, (int64_t)dk * cols));
                            else B2_TRY(put_tensor(W.conv_w, DT_F32, (size_t)L.conv_ch * cols, dst_row * cols, src, dt, (int64_t)dk * cols));
                        }
                    return 0;
                }
                if (is_w) return part(W.lproj_w, L.lproj, row0, sizes[j], width);
                if (is_taps) return taps_of(W.conv_w, sizes[j], L.conv_ch, row0, d.ga_conv);
                row0 += sizes[j];
            }
            if (r == "mix.o") return mat(W.o_w, width, L.ng);
            if (d.ga_qk_norm) {
                if (r == "mix.q.norm") return vec(W.qn_w, d.ga_dim);
                if (r == "mix.k.norm") return vec(W.kn_w, d.ga_dim);
            }
            if (L.maps > 1) {
                const char* lam[4] = {"mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"};
                for (int j = 0; j < 4; ++j)
                    if (r == lam[j]) {
                        B2_TRY(want_shape(key, shape, ndim, d.ga_dim));
                        W.got[r] = 1;
                        return put_tensor(W.lam4, DT_F32, (size_t)4 * d.ga_dim, (size_t)j * d.ga_dim, ptr, dt, d.ga_dim);
                    }
            }
        } else if (d.type == B2_MIXER_GLA) {
            // [q | k | v | g | a1]: one matrix, one product
            const int H = d.gl_heads, dk = d.gl_dim, dv = d.gl_vdim;
            if (r == "mix.q") return part(W.gla_w, L.pproj, 0, L.pq, width);
            if (r == "mix.k") return part(W.gla_w, L.pproj, L.pq, L.pq, width);
            if (r == "mix.v") return part(W.gla_w, L.pproj, 2 * L.pq, L.pv, width);
            if (r == "mix.g") return part(W.gla_w, L.pproj, 2 * L.pq + L.pv, L.pv, width);
            if (r == "mix.a1") return part(W.gla_w, L.pproj, 2 * L.pq + 2 * L.pv, d.gl_rank, width);
            if (r == "mix.a2") return mat(W.a2_w, (int64_t)H * dk, d.gl_rank);
            if (r == "mix.a2.b") return vec(W.a2_b, (int64_t)H * dk);
            if (r == "mix.norm") return vec(W.gnorm, dv);
            if (r == "mix.o") return mat(W.o_w, width, (int64_t)H * dv);
        } else if (d.type == B2_MIXER_HGRN2) {
            const int H = d.g_heads, dk = d.g_dim, dv = d.g_vdim;
            if (r == "mix.q") return part(W.qfv_w, L.pproj, 0, L.pq, width);
            if (r == "mix.f") return part(W.qfv_w, L.pproj, L.pq, L.pq, width);
            if (r == "mix.v") return part(W.qfv_w, L.pproj, 2 * L.pq, H * dv, width);
            if (r == "mix.f.b") return vec(W.f_b, (int64_t)H * dk);
            if (r == "mix.lower") return vec(W.lower, (int64_t)H * dk);
            if (r == "mix.norm") return vec(W.hnorm, dv);
            if (r == "mix.o") return mat(W.o_w, width, (int64_t)H * dv);
        }
        if (d.ff > 0 && d.ff_kind == B2_FF_POLYNORM) {
            if (r == "mlp.up") return mat(W.up_w, d.ff, width);
            if (r == "mlp.down") return mat(W.down_w, width, d.ff);
            if (r == "mlp.up.b") return vec(W.up_b, d.ff);
            if (r == "mlp.act") return vec(W.act_coef, 4);
            if (r == "mlp.down.b") {
                B2_TRY(vec(W.down_b, width));
                return put_tensor(W.down_b16, DT_BF16, (size_t)(width + 7) / 8 * 8, 0, ptr, dt, width);
            }
        } else if (d.ff > 0 && d.ff_kind == B2_FF_MOE) {
            const int E = d.moe_experts, ff = d.ff, sf = d.moe_shared_ff;
            const bool gated = d.moe_act == B2_MOE_ACT_SWIGLU;
            const int un = gated ? 2 : 1;   // matrices in front of an expert's activation
            if (r == "mlp.router") {   // at least 32 rows (zeros behind the experts): the tensor-core product of a prompt portion takes it
                B2_TRY(want_shape(key, shape, ndim, E, width));
                W.got[r] = 1;
                return put_tensor(W.router_w, WD, (size_t)router_rows(E) * width, 0, ptr, dt, (int64_t)E * width);
            }
            if (sf > 0) {
                if (r == "mlp.shared.gate" && gated) return part(W.sgu_w, 2 * sf, 0, sf, width);
                if (r == "mlp.shared.up") return part(W.sgu_w, un * sf, gated ? sf : 0, sf, width);
                if (r == "mlp.shared.down") return mat(W.sd_w, width, sf);
            }
            int e = -1, eu = 0;
            if (sscanf(r.c_str(), "mlp.e%d.%n", &e, &eu) == 1 && eu > 0 && e >= 0 && e < E) {
                const std::string which = r.substr(eu);
                // experts side by side: [E][gate | up][width] and [E][width][ff] (8 spare rows behind the last one)
                if ((which == "gate" && gated) || which == "up") {
                    B2_TRY(want_shape(key, shape, ndim, ff, width));
                    W.got[r] = 1;
                    return put_tensor(W.egu_w, WD, ((size_t)E * un * ff + 8) * width, ((size_t)e * un + (gated && which == "up")) * ff * width, ptr, dt,
                                      (int64_t)ff * width);
                }
                if (which == "down") {
                    B2_TRY(want_shape(key, shape, ndim, width, ff));
                    W.got[r] = 1;
                    return put_tensor(W.ed_w, WD, ((size_t)E * width + 8) * ff, (size_t)e * width * ff, ptr, dt, (int64_t)width * ff);
                }
            }
        } else if (d.ff > 0 && d.ff_kind == B2_FF_CLAMP_GLU) {
            if (r == "mlp.gate") return part(W.up_w, 2 * d.ff, 0, d.ff, width);
            if (r == "mlp.up") return part(W.up_w, 2 * d.ff, d.ff, d.ff, width);
            if (r == "mlp.down") return mat(W.down_w, width, d.ff);
        } else if (d.ff > 0) {
            if (r == "mlp.up") return mat(W.up_w, d.ff, width);
            if (r == "mlp.down") return mat(W.down_w, width, d.ff);
        }
        set_error("set_weight: tensor '%s' does not belong to a layer of this kind", key);
        return -1;
    }
    if (r == "norm1") return vec(W.norm1, width);
    if (r == "norm1.b") return vec(W.norm1_b, width);
    if (d.ff > 0) {
        if (r == "norm2") return vec(W.norm2, width);
        if (r == "norm2.b") return vec(W.norm2_b, width);
        if (r == "mlp.up") return mat(W.up_w, d.ff, width);
        if (r == "mlp.down") return mat(W.down_w, width, d.ff);
    }
    if (d.type == B2_MIXER_MAMBA2) {
        if (r == "mix.in") return mat(W.in_w, L.dproj, width);
        if (r == "mix.conv") { B2_TRY(want_shape(key, shape, ndim, L.conv_ch, d.m_conv)); W.got[r] = 1; return put_tensor(W.conv_w, DT_F32, (size_t)L.conv_ch * d.m_conv, 0, ptr, dt, (int64_t)L.conv_ch * d.m_conv); }
        if (r == "mix.conv.b") return vec(W.conv_b, L.conv_ch);
        if (r == "mix.dt_bias") return vec(W.dt_bias, d.m_heads);
        if (r == "mix.A_log") return vec(W.a_log, d.m_heads);
        if (r == "mix.D") return vec(W.skip, d.m_heads);
        if (r == "mix.norm") return vec(W.mnorm, L.inner);
        if (r == "mix.o") return mat(W.o_w, width, L.inner);
    } else {
        // the four attention projections share their input: one [nq + nk + nv + ng, width] matrix, one product
        const char* parts[4] = {"mix.left.q", "mix.left.k", "mix.left.v", "mix.left.g"};
        const int sizes[4] = {L.nq, L.nk, L.nv, L.ng};
        size_t row0 = 0;
        for (int j = 0; j < 4; ++j) {
            if (r == parts[j]) {
                B2_TRY(want_shape(key, shape, ndim, sizes[j], width));
                W.got[r] = 1;
                return put_tensor(W.lproj_w, WD, (size_t)L.lproj_ld * width, row0 * width, ptr, dt, (int64_t)sizes[j] * width);
            }
            row0 += sizes[j];
        }
        if (r == "mix.left.rel") { B2_TRY(want_shape(key, shape, ndim, d.a_rel_rows, d.a_heads)); W.got[r] = 1; return put_tensor(W.rel, DT_F32, (size_t)d.a_rel_rows * d.a_heads, 0, ptr, dt, (int64_t)d.a_rel_rows * d.a_heads); }
        if (r == "mix.left.o") return mat(W.lo_w, width, L.ng);
        const char* mus[5] = {"mix.right.mu.r", "mix.right.mu.k", "mix.right.mu.v", "mix.right.mu.g", "mix.right.mu.w"};
        for (int j = 0; j < 5; ++j)
            if (r == mus[j]) {
                B2_TRY(want_shape(key, shape, ndim, width));
                W.got[r] = 1;
                return put_tensor(W.mu, DT_F32, (size_t)5 * width, (size_t)j * width, ptr, dt, width);
            }
        if (r == "mix.right.r") return mat(W.r_w, L.rn, width);
        if (r == "mix.right.k") return mat(W.k_w, L.rn, width);
        if (r == "mix.right.v") return mat(W.v_w, L.rn, width);
        if (r == "mix.right.g") return mat(W.g_w, L.rn, width);
        if (r == "mix.right.w1") return mat(W.w1, d.r_decay_rank, width);
        if (r == "mix.right.w2") return mat(W.w2, L.rn, d.r_decay_rank);
        if (r == "mix.right.w0") return vec(W.w0, L.rn);
        if (r == "mix.right.u") return vec(W.bonus, L.rn);
        if (r == "mix.right.norm") return vec(W.rnorm, L.rn);
        if (r == "mix.right.o") return mat(W.ro_w, width, L.rn);
    }
    set_error("set_weight: tensor '%s' does not belong to a layer of this kind", key);
    return -1;
}

static std::vector<std::string> required_of(const SeqLayerInfo& L, int block, int ctaps) {
    const bool sandwich = block == B2_BLOCK_SANDWICH_RMS, parallel = block == B2_BLOCK_PARALLEL_RMS;
    if (block != B2_BLOCK_POST_LN) {
        std::vector<std::string> v = {"norm1", "mix.o"};
        const b2_seq_layer_desc& d = L.d;
        if (sandwich) { v.push_back("norm1b"); if (ctaps >= 1) v.push_back("canon1"); }
        if (d.type == B2_MIXER_LATENT_ATTN) {
            for (const char* n : {"mix.uk", "mix.uv"}) v.push_back(n);
            if (d.la_q_rank > 0) for (const char* n : {"mix.dq", "mix.dq.norm", "mix.uq"}) v.push_back(n);
            else v.push_back("mix.q");
            if (d.la_kv_from == 0) for (const char* n : {"mix.dkv", "mix.dkv.norm"}) v.push_back(n);
            if (!d.la_no_sink) v.push_back("mix.sink");
            if (!d.la_no_gate) v.push_back("mix.g");
        } else if (d.type == B2_MIXER_GQA_ATTN) {
            for (const char* n : {"mix.q", "mix.k", "mix.v"}) v.push_back(n);
            if (L.gw > 0) v.push_back("mix.g");
            if (d.ga_conv >= 1) for (const char* n : {"mix.q.conv", "mix.k.conv", "mix.v.conv"}) v.push_back(n);
            if (d.ga_qk_norm) for (const char* n : {"mix.q.norm", "mix.k.norm"}) v.push_back(n);
            if (L.maps > 1) for (const char* n : {"mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"}) v.push_back(n);
        } else if (d.type == B2_MIXER_GLA) {
            for (const char* n : {"mix.q", "mix.k", "mix.v", "mix.g", "mix.a1", "mix.a2", "mix.a2.b", "mix.norm"}) v.push_back(n);
        } else for (const char* n : {"mix.q", "mix.f", "mix.f.b", "mix.lower", "mix.v", "mix.norm"}) v.push_back(n);
        if (L.d.ff > 0) {
            if (!parallel) v.push_back("norm2");
            if (sandwich) { v.push_back("norm2b"); if (ctaps >= 1) v.push_back("canon2"); }
            if (L.d.ff_kind == B2_FF_POLYNORM) for (const char* n : {"mlp.up", "mlp.up.b", "mlp.down", "mlp.down.b", "mlp.act"}) v.push_back(n);
            else if (L.d.ff_kind == B2_FF_MOE) {
                v.push_back("mlp.router");
                const bool gated = L.d.moe_act == B2_MOE_ACT_SWIGLU;
                for (int e = 0; e < L.d.moe_experts; ++e)
                    for (const char* n : {"gate", "up", "down"})
                        if (gated || n[0] != 'g') v.push_back("mlp.e" + std::to_string(e) + "." + n);
                if (L.d.moe_shared_ff > 0)
                    for (const char* n : {"mlp.shared.gate", "mlp.shared.up", "mlp.shared.down"})
                        if (gated || n[11] != 'g') v.push_back(n);
            } else if (L.d.ff_kind == B2_FF_CLAMP_GLU) for (const char* n : {"mlp.gate", "mlp.up", "mlp.down"}) v.push_back(n);
            else for (const char* n : {"mlp.up", "mlp.down"}) v.push_back(n);
        }
        return v;
    }
    std::vector<std::string> v = {"norm1", "norm1.b"};
    if (L.d.ff > 0) for (const char* n : {"norm2", "norm2.b", "mlp.up", "mlp.down"}) v.push_back(n);
    if (L.d.type == B2_MIXER_MAMBA2) {
        for (const char* n : {"mix.in", "mix.conv", "mix.conv.b", "mix.dt_bias", "mix.A_log", "mix.D", "mix.norm", "mix.o"}) v.push_back(n);
    } else {
        for (const char* n : {"mix.left.q", "mix.left.k", "mix.left.v", "mix.left.g", "mix.left.rel", "mix.left.o", "mix.right.mu.r", "mix.right.mu.k",
                              "mix.right.mu.v", "mix.right.mu.g", "mix.right.mu.w", "mix.right.r", "mix.right.k", "mix.right.v", "mix.right.g",
                              "mix.right.w1", "mix.right.w2", "mix.right.w0", "mix.right.u", "mix.right.norm", "mix.right.o"})
            v.push_back(n);
    }
    return v;
}

int seq_finalize(b2_model* m) {
    SeqModel& s = *m->seq;
    std::string missing;
    const bool sandwich = s.d.block == B2_BLOCK_SANDWICH_RMS;
    const bool pre = s.d.block != B2_BLOCK_POST_LN;
    std::vector<std::string> top = {"embed", "head", "final.norm"};
    if (!pre) top.push_back("final.norm.b");
    if (s.d.bigram_buckets > 0) top.push_back("bigram");
    if (s.d.loop_times >= 1 && !s.d.loop_plain) top.push_back("loop.step");
    for (const std::string& n : top)
        if (!s.got.count(n) && missing.size() < 600) { missing += n; missing += ' '; }
    for (size_t i = 0; i < s.layers.size(); ++i) {
        if (s.layers[i].src != (int)i) continue;
        for (const std::string& n : required_of(s.layers[i], s.d.block, s.d.input_conv_taps))
            if (!s.w[i].got.count(n) && missing.size() < 600) missing += "l" + std::to_string(i) + "." + n + " ";
    }
    if (!missing.empty()) {
        set_error("b2_model_finalize: missing tensors: %s", missing.c_str());
        return -3;
    }
    // differential attention: the layer's lambda from its four vectors (double precision on the host, once)
    for (size_t i = 0; i < s.layers.size(); ++i) {
        const SeqLayerInfo& L = s.layers[i];
        if (L.src != (int)i || L.d.type != B2_MIXER_GQA_ATTN || L.maps < 2) continue;
        const int dk = L.d.ga_dim;
        std::vector<float> v((size_t)4 * dk);
        B2_CUDA_CHECK(cudaMemcpy(v.data(), s.w[i].lam4.p, v.size() * F4, cudaMemcpyDeviceToHost));
        double d1 = 0.0, d2 = 0.0;
        for (int c = 0; c < dk; ++c) { d1 += (double)v[c] * v[dk + c]; d2 += (double)v[2 * dk + c] * v[3 * dk + c]; }
        s.w[i].lambda = (float)(exp(d1) - exp(d2) + (double)L.d.ga_diff);
    }
    const int width = s.d.width;
    int pw = 1, aw = 1, yw = 1, rw = 1, kw = 1, fw = 1;
    int latw = 0, moe_top = 0, moe_e = 0, moe_ff = 0;
    bool glu = false;
    for (const SeqLayerInfo& L : s.layers) {
        if (L.d.type == B2_MIXER_MAMBA2) {
            pw = std::max(pw, L.dproj_ld); aw = std::max(aw, L.conv_ch); yw = std::max(yw, L.inner);
        } else if (L.d.type == B2_MIXER_PARALLEL) {
            pw = std::max(pw, L.lproj_ld); yw = std::max(yw, std::max(L.ng, L.rn)); rw = std::max(rw, L.rn); kw = std::max(kw, L.d.r_decay_rank);
        } else if (L.d.type == B2_MIXER_GQA_ATTN) {
            pw = std::max(pw, L.lproj_ld); yw = std::max(yw, L.maps * L.ng); aw = std::max(aw, L.conv_ch);
        } else if (L.d.type == B2_MIXER_GLA) {
            pw = std::max(pw, L.pproj_ld); yw = std::max(yw, L.pv); rw = std::max(rw, L.pq);
        } else {
            pw = std::max(pw, L.pproj_ld); yw = std::max(yw, L.pv);
            if (L.d.type == B2_MIXER_LATENT_ATTN) {
                latw = std::max(latw, L.d.la_heads * L.lrow);
                if (L.d.la_q_rank > 0) aw = std::max(aw, L.lqw_ld);
            }
        }
        fw = std::max(fw, (L.d.ff + 7) / 8 * 8);
        if (L.d.ff > 0 && L.d.ff_kind == B2_FF_CLAMP_GLU) { fw = std::max(fw, (2 * L.d.ff + 7) / 8 * 8); glu = true; }
        if (L.d.ff > 0 && L.d.ff_kind == B2_FF_MOE) {
            fw = std::max(fw, (2 * L.d.moe_shared_ff + 7) / 8 * 8);
            moe_top = std::max(moe_top, L.d.moe_top); moe_e = std::max(moe_e, L.d.moe_experts); moe_ff = std::max(moe_ff, L.d.ff);
        }
    }

    s.proj_w = pw; s.act_w = aw; s.y_w = yw; s.rp_w = rw; s.rank_w = kw; s.ff_w = fw;
    const size_t R = (size_t)s.rows;
    B2_TRY(s.x.alloc(R * width * F4));
    B2_TRY(s.proj.alloc(R * pw * F4));
    B2_TRY(s.act.alloc(R * aw * F4));
    B2_TRY(s.y.alloc(R * yw * F4));
    B2_TRY(s.gated.alloc(R * yw * F4));
    B2_TRY(s.mixout.alloc(R * width * F4));
    B2_TRY(s.mixes.alloc(5 * R * width * F4));
    B2_TRY(s.rp.alloc(4 * R * rw * F4));
    B2_TRY(s.wl1.alloc(R * kw * F4));
    B2_TRY(s.wlog.alloc(R * rw * F4));
    B2_TRY(s.ff.alloc(R * fw * F4));
    B2_TRY(s.xn.alloc(R * width * F4));
    if (pre) B2_TRY(s.ffa.alloc(R * fw * F4));
    if (sandwich && s.d.input_conv_taps >= 1) B2_TRY(s.hin.alloc(R * width * F4));
    if (s.d.loop_times > 1 && !s.d.loop_plain) B2_TRY(s.x0.alloc(R * width * F4));
    if (glu && moe_e == 0) {   // the one-row grouped product of a decode step reads its group (always 0) from here
        B2_TRY(s.zero_idx.alloc(64 * 4));
        B2_CUDA_CHECK(cudaMemset(s.zero_idx.p, 0, 64 * 4));
    }
    if (latw > 0) {
        s.lat_w = latw;
        B2_TRY(s.qabs.alloc(R * latw * F4));
        B2_TRY(s.olat.alloc(R * latw * F4));
    }
    if (moe_e > 0) {
        // (token, choice) pairs sorted by expert, every expert padded to whole tiles
        s.moe_top = moe_top; s.moe_e = moe_e;
        // (sized for tiles of 128 rows, the tensor-core product's; tiles of 64 pad less)
        s.moe_tiles = (int)((R * moe_top + (size_t)moe_e * 127 + 127) / 128) * 2;
        s.moe_rows = s.moe_tiles * GROUPED_TILE_ROWS;
        const size_t P = (size_t)s.moe_rows;
        B2_TRY(s.rlogit.alloc(R * router_rows(moe_e) * F4));
        B2_TRY(s.moe_idx.alloc(R * moe_top * 4));
        B2_TRY(s.moe_w.alloc(R * moe_top * F4));
        B2_TRY(s.moe_pos.alloc(R * moe_top * 4));
        B2_TRY(s.moe_src.alloc(P * 4));
        B2_TRY(s.moe_tile.alloc((size_t)s.moe_tiles * 4));
        B2_TRY(s.moe_h.alloc(P * 2 * moe_ff * F4));
        B2_TRY(s.moe_a.alloc(P * moe_ff * F4));
        B2_TRY(s.moe_y.alloc(P * width * F4));
        B2_TRY(s.zero_idx.alloc(64 * 4));
        B2_CUDA_CHECK(cudaMemset(s.zero_idx.p, 0, 64 * 4));
        if (s.d.compute == B2_COMPUTE_BF16) B2_TRY(s.moe_a16.alloc(P * (size_t)(width + moe_ff) * 2));
    }
    {
        int kmax = width;
        for (const SeqLayerInfo& L : s.layers)
            kmax = std::max(kmax, std::max(std::max(std::max(L.inner, L.ng), std::max(L.rn, L.d.ff)), std::max(std::max(L.pv, std::max(L.lrow, L.d.la_q_rank)), std::max(L.d.la_dim, L.d.moe_shared_ff))));
        s.a16_w = (kmax + 7) / 8 * 8;
        if (s.d.compute == B2_COMPUTE_BF16) B2_TRY(s.a16.alloc(R * s.a16_w * 2));
    }
    B2_TRY(s.tok.alloc(R * 4));
    B2_TRY(s.want.alloc(R * 4));
    B2_TRY(s.segs.alloc((size_t)std::max(1, s.d.max_batch) * sizeof(SeqSeg)));
    B2_TRY(s.row_slot.alloc(R * 4));
    B2_TRY(s.row_pos.alloc(R * 4));
    B2_TRY(m->logits.alloc((size_t)s.d.max_batch * s.d.vocab * 4));
    return 0;
}

void seq_model_free(b2_model* m) {
    if (m->seq == nullptr) return;
    SeqModel& s = *m->seq;
    for (SeqWeights& W : s.w) {
        DevBuf* bs[] = {&W.norm1, &W.norm1_b, &W.norm2, &W.norm2_b, &W.in_w, &W.conv_w, &W.conv_b, &W.dt_bias, &W.a_log, &W.skip, &W.mnorm, &W.o_w,
                        &W.lproj_w, &W.rel, &W.lo_w, &W.mu, &W.r_w, &W.k_w, &W.v_w, &W.g_w, &W.w1, &W.w2, &W.w0, &W.bonus, &W.rnorm, &W.ro_w,
                        &W.up_w, &W.down_w, &W.qdg_w, &W.dkv_norm, &W.uk_w, &W.ukT, &W.uv_w, &W.sink, &W.qfv_w, &W.f_b, &W.lower, &W.hnorm, &W.up_b, &W.down_b,
                        &W.down_b16, &W.act_coef, &W.router_w, &W.egu_w, &W.ed_w, &W.sgu_w, &W.sd_w, &W.canon1, &W.canon2, &W.dq_norm, &W.uq_w, &W.ukx_w,
                        &W.qn_w, &W.kn_w, &W.lam4, &W.gla_w, &W.a2_w, &W.a2_b, &W.gnorm};
        for (DevBuf* b : bs) b->free();
    }
    DevBuf* bs[] = {&s.embed, &s.head, &s.final_w, &s.final_b, &s.x, &s.proj, &s.act, &s.y, &s.gated, &s.mixout, &s.mixes, &s.rp, &s.wl1, &s.wlog,
                    &s.ff, &s.xn, &s.tok, &s.want, &s.segs, &s.row_slot, &s.row_pos, &s.a16, &s.bigram, &s.loop_step, &s.x0, &s.qabs, &s.olat, &s.ffa,
                    &s.rlogit, &s.moe_idx, &s.moe_w, &s.moe_pos, &s.moe_src, &s.moe_tile, &s.moe_h, &s.moe_a, &s.moe_y, &s.moe_a16, &s.zero_idx, &s.hin};
    for (DevBuf* b : bs) b->free();
    delete m->seq;
    m->seq = nullptr;
}

// ------------------------------------------------------------------------------------------------------------------
// per-cache state
// ------------------------------------------------------------------------------------------------------------------
static int distance_bucket(int n, int rows, double far_) {
    const int half = rows / 2;
    if (n < half || half == 0) return n < rows ? n : rows - 1;
    const double v = log((double)n / half) / log(far_ / half) * (rows - half);
    const long b = half + (long)floor(v);
    return (int)(b < rows - 1 ? b : rows - 1);
}

int64_t seq_kv_bytes(const b2_model* m, int B, int Smax) {
    int64_t n = 0;
    for (const SeqRun& run : m->seq->runs) {
        const SeqLayerInfo& L = m->seq->layers[run.layer];
        const b2_seq_layer_desc& d = L.d;
        if (d.type == B2_MIXER_MAMBA2) n += (int64_t)B * d.m_heads * d.m_state * d.m_vdim + (int64_t)B * (d.m_conv - 1) * L.conv_ch;
        else if (d.type == B2_MIXER_PARALLEL)
            n += (int64_t)B * d.a_kv_heads * Smax * (d.a_dim + d.a_vdim) + (int64_t)B * d.r_heads * d.r_dim * d.r_dim + (int64_t)B * m->seq->d.width;
        else if (d.type == B2_MIXER_LATENT_ATTN) n += d.la_kv_from == 0 ? (int64_t)B * Smax * L.lrow : 0;
        else if (d.type == B2_MIXER_GQA_ATTN) n += (int64_t)B * d.ga_kv_heads * Smax * (L.maps * d.ga_dim + d.ga_vdim) + (int64_t)B * std::max(0, d.ga_conv - 1) * L.conv_ch;
        else if (d.type == B2_MIXER_GLA) n += (int64_t)B * d.gl_heads * d.gl_dim * d.gl_vdim;
        else n += (int64_t)B * d.g_heads * d.g_dim * d.g_vdim;
        if (m->seq->d.block == B2_BLOCK_SANDWICH_RMS && m->seq->d.input_conv_taps > 1)
            n += (int64_t)B * (m->seq->d.input_conv_taps - 1) * m->seq->d.width * (d.ff > 0 ? 2 : 1);
    }
    return n * 4 + (m->seq->d.bigram_buckets > 0 ? (int64_t)B * 4 : 0);
}

int seq_kv_alloc(b2_kv* kv) {
    const b2_model* m = kv->m;
    const SeqModel& s = *m->seq;
    const size_t B = kv->max_batch, Smax = kv->max_seq;
    kv->seq = new SeqState();
    kv->seq->layer.resize(s.runs.size());
    B2_TRY(kv->seq->last_tok.alloc(B * 4));
    cudaMemset(kv->seq->last_tok.p, 0, B * 4);
    int maxH = 1, maxdv = 1;
    for (size_t li = 0; li < s.runs.size(); ++li) {
        const SeqLayerInfo& L = s.layers[s.runs[li].layer];
        const b2_seq_layer_desc& d = L.d;
        SeqLayerState& S = kv->seq->layer[li];
        if (s.d.block == B2_BLOCK_SANDWICH_RMS && s.d.input_conv_taps > 1) {
            const size_t n = B * (s.d.input_conv_taps - 1) * s.d.width * F4;
            B2_TRY(S.canon1.alloc(n));
            cudaMemset(S.canon1.p, 0, n);
            if (d.ff > 0) {
                B2_TRY(S.canon2.alloc(n));
                cudaMemset(S.canon2.p, 0, n);
            }
        }
        if (d.rot_dims >= 2 && (d.type == B2_MIXER_GQA_ATTN || (d.type == B2_MIXER_LATENT_ATTN && d.la_rot_dim > 0))) {
            RotaryDesc rdesc;
            rdesc.dims = d.rot_dims; rdesc.base = d.rot_base; rdesc.factor = d.rot_factor; rdesc.original = d.rot_original; rdesc.fast = d.rot_fast;
            rdesc.slow = d.rot_slow;
            B2_TRY(S.rot_tab.alloc(Smax * (d.rot_dims / 2) * sizeof(float2)));
            B2_TRY(rotary_table_build(rdesc, (int)Smax, S.rot_tab.as<float2>()));
        }
        if (d.type == B2_MIXER_GQA_ATTN) {
            B2_TRY(S.kc.alloc(B * L.maps * d.ga_kv_heads * Smax * d.ga_dim * F4));
            B2_TRY(S.vc.alloc(B * d.ga_kv_heads * Smax * d.ga_vdim * F4));
            cudaMemset(S.kc.p, 0, S.kc.bytes);
            cudaMemset(S.vc.p, 0, S.vc.bytes);
            if (d.ga_conv > 1) {
                B2_TRY(S.conv_tail.alloc(B * (d.ga_conv - 1) * L.conv_ch * F4));
                cudaMemset(S.conv_tail.p, 0, S.conv_tail.bytes);
            }
            if (d.ga_rot_values && d.ga_vdim >= 2) {   // values turn over all of vdim (an odd last entry passes) with the plain frequencies of the same base
                RotaryDesc vdesc;
                vdesc.dims = d.ga_vdim; vdesc.base = d.rot_base;
                B2_TRY(S.vrot_tab.alloc(Smax * (d.ga_vdim / 2) * sizeof(float2)));
                B2_TRY(rotary_table_build(vdesc, (int)Smax, S.vrot_tab.as<float2>()));
            }
            maxH = std::max(maxH, L.maps * d.ga_heads);
            maxdv = std::max(maxdv, d.ga_vdim);
        } else if (d.type == B2_MIXER_LATENT_ATTN) {
            if (d.la_kv_from == 0) {   // a borrowing layer reads the owner's rows
                B2_TRY(S.lat.alloc(B * Smax * L.lrow * F4));
                cudaMemset(S.lat.p, 0, S.lat.bytes);
            }
            maxH = std::max(maxH, d.la_heads);
            maxdv = std::max(maxdv, d.la_rank);
        } else if (d.type == B2_MIXER_HGRN2) {
            B2_TRY(S.gla.alloc(B * d.g_heads * d.g_dim * d.g_vdim * F4));
            cudaMemset(S.gla.p, 0, S.gla.bytes);
        } else if (d.type == B2_MIXER_GLA) {
            B2_TRY(S.gla.alloc(B * d.gl_heads * d.gl_dim * d.gl_vdim * F4));
            cudaMemset(S.gla.p, 0, S.gla.bytes);
        } else if (d.type == B2_MIXER_MAMBA2) {
            B2_TRY(S.ssm.alloc(B * d.m_heads * d.m_state * d.m_vdim * F4));
            B2_TRY(S.conv_tail.alloc(std::max<size_t>(1, B * (d.m_conv - 1) * L.conv_ch) * F4));
            cudaMemset(S.ssm.p, 0, S.ssm.bytes);
            cudaMemset(S.conv_tail.p, 0, S.conv_tail.bytes);
        } else {
            B2_TRY(S.kc.alloc(B * d.a_kv_heads * Smax * d.a_dim * F4));
            B2_TRY(S.vc.alloc(B * d.a_kv_heads * Smax * d.a_vdim * F4));
            B2_TRY(S.wkv.alloc(B * d.r_heads * d.r_dim * d.r_dim * F4));
            B2_TRY(S.prev.alloc(B * s.d.width * F4));
            B2_TRY(S.bucket_of.alloc(Smax * 4));
            cudaMemset(S.kc.p, 0, S.kc.bytes);
            cudaMemset(S.vc.p, 0, S.vc.bytes);
            cudaMemset(S.wkv.p, 0, S.wkv.bytes);
            cudaMemset(S.prev.p, 0, S.prev.bytes);
            std::vector<int32_t> tab(Smax);
            for (size_t n = 0; n < Smax; ++n) tab[n] = distance_bucket((int)n, d.a_rel_rows, (double)d.a_bias_max);
            B2_CUDA_CHECK(cudaMemcpy(S.bucket_of.p, tab.data(), Smax * 4, cudaMemcpyHostToDevice));
            maxH = std::max(maxH, d.a_heads);
            maxdv = std::max(maxdv, d.a_vdim);
        }
    }
    int kw = 0, vw = 0;
    for (const SeqLayerInfo& L : s.layers)
        if (L.d.type == B2_MIXER_LATENT_ATTN) { kw = std::max(kw, L.lqw_ld); vw = std::max(vw, (L.pv + 7) / 8 * 8); }
    if (kw > 0) {
        kv->seq->kmat_ld = kw; kv->seq->vmat_ld = vw;
        B2_TRY(kv->seq->kmat.alloc(Smax * kw * F4));
        B2_TRY(kv->seq->vmat.alloc(Smax * vw * F4));
    }
    kv->seq->nsplit_max = 64;
    B2_TRY(kv->seq->attn_partial.alloc((size_t)8 * maxH * kv->seq->nsplit_max * (maxdv + 2) * F4));
    return 0;
}

void seq_kv_free(b2_kv* kv) {
    if (kv->seq == nullptr) return;
    for (SeqLayerState& S : kv->seq->layer) {
        DevBuf* bs[] = {&S.ssm, &S.conv_tail, &S.kc, &S.vc, &S.bucket_of, &S.wkv, &S.prev, &S.lat, &S.gla, &S.canon1, &S.canon2, &S.rot_tab, &S.vrot_tab};
        for (DevBuf* b : bs) b->free();
    }
    kv->seq->last_tok.free();
    kv->seq->kmat.free();
    kv->seq->vmat.free();
    kv->seq->attn_partial.free();
    delete kv->seq;
    kv->seq = nullptr;
}

}  // namespace b2

using namespace b2;

// ==================================================================================================================
// C ABI
// ==================================================================================================================
extern "C" {

int b2_seq_model_create(const b2_seq_model_desc* desc, const b2_seq_layer_desc* layers, b2_model** out) {
    B2_CHECK_ARG(desc && layers && out, "b2_seq_model_create: null argument");
    const b2_seq_model_desc& d = *desc;
    B2_CHECK_ARG(d.width > 0 && d.vocab > 0 && d.n_layers > 0, "b2_seq_model_create: width %d, vocab %d, %d layers", d.width, d.vocab, d.n_layers);
    B2_CHECK_ARG(d.compute == B2_COMPUTE_BF16 || d.compute == B2_COMPUTE_F32, "b2_seq_model_create: unknown compute mode %d", d.compute);
    B2_CHECK_ARG(d.max_batch >= 1 && d.max_rows >= 1, "b2_seq_model_create: bad workspace sizing");
    B2_CHECK_ARG(d.norm_eps >= 0.f, "b2_seq_model_create: negative eps");
    B2_CHECK_ARG(d.block >= B2_BLOCK_POST_LN && d.block <= B2_BLOCK_PARALLEL_RMS, "b2_seq_model_create: unknown block form %d", d.block);
    B2_CHECK_ARG(d.embed_scale == 0.f || d.bigram_buckets == 0, "b2_seq_model_create: a scaled embedding does not go with the hashed bigram rows");
    B2_CHECK_ARG(d.input_conv_taps >= 0 && d.input_conv_taps <= 16, "b2_seq_model_create: 0..16 taps of the input convolution");
    B2_CHECK_ARG(d.input_conv_taps == 0 || d.block == B2_BLOCK_SANDWICH_RMS, "b2_seq_model_create: the input convolution belongs to the sandwich block");
    B2_CHECK_ARG(d.bigram_buckets >= 0 && d.logit_softcap >= 0.f, "b2_seq_model_create: negative bigram buckets or soft-cap");
    SeqModel* s = new SeqModel();
    s->d = d;
    s->w_dtype = d.compute == B2_COMPUTE_F32 ? DT_F32 : DT_BF16;
    s->rows = std::max(d.max_batch, d.max_rows);
    s->layers.resize(d.n_layers);
    s->w.resize(d.n_layers);
    // a layer may name ANY other layer as the owner of its tensors (an owner that itself borrows is followed to its owner)
    for (int i = 0; i < d.n_layers; ++i) s->layers[i].d = layers[i];
    for (int i = 0; i < d.n_layers; ++i) {
        int j = i, hops = 0;
        while (j >= 0 && j < d.n_layers && s->layers[j].d.weights_of >= 0 && s->layers[j].d.weights_of != j && hops <= d.n_layers) {
            j = s->layers[j].d.weights_of;
            ++hops;
        }
        if (j < 0 || j >= d.n_layers || hops > d.n_layers) {
            set_error("b2_seq_model_create: layer %d: weights_of does not lead to a layer that owns its tensors", i);
            delete s;
            return -1;
        }
        s->layers[i].src = j;
    }
    for (int i = 0; i < d.n_layers; ++i) {
        SeqLayerInfo& L = s->layers[i];
        const b2_seq_layer_desc& l = L.d;
        const char* why = nullptr;
        if (l.ff < 0) why = "negative feed-forward width";
        else if (l.type == B2_MIXER_MAMBA2) {
            if (l.m_heads < 1 || l.m_vdim < 1 || l.m_state < 1 || l.m_groups < 1 || l.m_heads % l.m_groups) why = "mamba2: heads must be a positive multiple of groups";
            else if (l.m_conv < 1 || l.m_conv > 16) why = "mamba2: 1..16 convolution taps";
            else if (l.m_norm_groups < 1 || (l.m_heads * l.m_vdim) % l.m_norm_groups) why = "mamba2: norm_groups must divide heads*vdim";
            else if (l.m_state > 256) why = "mamba2: state size above 256";
            L.inner = l.m_heads * l.m_vdim;
            L.conv_ch = L.inner + 2 * l.m_groups * l.m_state;
            L.dproj = 2 * L.inner + 2 * l.m_groups * l.m_state + l.m_heads;
            L.dproj_ld = (L.dproj + 7) / 8 * 8;
        } else if (l.type == B2_MIXER_PARALLEL) {
            if (l.a_heads < 1 || l.a_kv_heads < 1 || l.a_heads % l.a_kv_heads) why = "attention: heads must be a positive multiple of kv_heads";
            else if (l.a_dim < 1 || l.a_dim > 256 || l.a_vdim < 1 || l.a_vdim > 256) why = "attention: head sizes 1..256";
            else if (l.a_rel_rows < 1 || !(l.a_bias_max > 0.f)) why = "attention: the distance bias needs rows and a positive far limit";
            else if (!(l.a_temp_every > 0.f)) why = "attention: q_temp.every must be positive";
            else if (l.r_heads < 1 || l.r_dim < 1 || l.r_dim > 256 || l.r_decay_rank < 1) why = "rwkv: heads, dim 1..256, decay rank";
            L.nq = l.a_heads * l.a_dim; L.nk = l.a_kv_heads * l.a_dim; L.nv = l.a_kv_heads * l.a_vdim; L.ng = l.a_heads * l.a_vdim;
            L.lproj = L.nq + L.nk + L.nv + L.ng;
            L.lproj_ld = (L.lproj + 7) / 8 * 8;
            L.rn = l.r_heads * l.r_dim;
        } else if (l.type == B2_MIXER_LATENT_ATTN) {
            if (l.la_heads < 1 || l.la_dim < 1 || l.la_vdim < 1) why = "latent attention: heads and head sizes must be positive";
            else if (l.la_rot_dim < 0 || l.la_q_rank < 0 || l.la_kv_from < 0) why = "latent attention: negative size";
            else if (l.la_rank < 1 || l.la_rank > 512 || l.la_rank + l.la_rot_dim > 768) why = "latent attention: latent size 1..512, with the rotated part at most 768";
            else if (l.la_rot_dim > 0 && (l.rot_dims < 1 || l.rot_dims > l.la_rot_dim || !(l.rot_base > 0.f))) why = "latent attention: rotated dimensions within the rotated part, positive base";
            else if (l.rot_factor > 0.f && !(l.rot_original > 0.f && l.rot_fast > 0.f && l.rot_slow > 0.f && l.rot_base > 1.f)) why = "rotation: scaled frequencies need original, fast and slow";
            else if (l.la_kv_from > 0) {
                const int j = l.la_kv_from - 1;
                if (j >= i) why = "latent attention: cache rows can only be read from an earlier layer";
                else {
                    const b2_seq_layer_desc& o = s->layers[j].d;
                    if (o.type != B2_MIXER_LATENT_ATTN || o.la_kv_from != 0) why = "latent attention: the layer named by kv_from has no cache rows of its own";
                    else if (o.la_rank != l.la_rank || o.la_rot_dim != l.la_rot_dim || o.rot_dims != l.rot_dims || o.rot_base != l.rot_base || o.rot_factor != l.rot_factor ||
                             o.rot_original != l.rot_original || o.rot_fast != l.rot_fast || o.rot_slow != l.rot_slow)
                        why = "latent attention: a layer that reads another's cache rows must have its latent size and rotation";
                }
            }
            if (why == nullptr && (l.mask_kind < B2_MASK_CAUSAL || l.mask_kind > B2_MASK_CHUNK || (l.mask_kind != B2_MASK_CAUSAL && l.mask_size < 1))) why = "mask: unknown kind or empty size";
            L.lrow = l.la_rank + l.la_rot_dim;
            L.lqw = l.la_heads * (l.la_dim + l.la_rot_dim); L.lqw_ld = (L.lqw + 7) / 8 * 8;
            L.pq = l.la_q_rank > 0 ? l.la_q_rank : L.lqw;   // rows of the query part of the fused projection
            L.pv = l.la_heads * l.la_vdim;
            L.pproj = L.pq + (l.la_kv_from == 0 ? L.lrow : 0) + (l.la_no_gate ? 0 : l.la_heads);
            L.pproj_ld = (L.pproj + 7) / 8 * 8;
        } else if (l.type == B2_MIXER_GQA_ATTN) {
            if (l.ga_heads < 1 || l.ga_kv_heads < 1 || l.ga_heads % l.ga_kv_heads) why = "attention: heads must be a positive multiple of kv_heads";
            else if (l.ga_dim < 1 || l.ga_dim > 512 || l.ga_vdim < 1 || l.ga_vdim > 512) why = "attention: head sizes 1..512";
            else if (l.ga_conv < 0 || l.ga_conv > 16) why = "attention: 0..16 convolution taps";
            else if (l.rot_dims < 0 || l.rot_dims > l.ga_dim || (l.rot_dims > 0 && !(l.rot_base > 0.f))) why = "attention: rotated dimensions within a head, positive base";
            else if (l.rot_factor > 0.f && !(l.rot_original > 0.f && l.rot_fast > 0.f && l.rot_slow > 0.f && l.rot_base > 1.f)) why = "rotation: scaled frequencies need original, fast and slow";
            else if (l.ga_rot_values && !(l.rot_base > 0.f)) why = "attention: rotated values need a base";
            else if (l.mask_kind < B2_MASK_CAUSAL || l.mask_kind > B2_MASK_CHUNK || (l.mask_kind != B2_MASK_CAUSAL && l.mask_size < 1)) why = "mask: unknown kind or empty size";
            else if (l.mask_keep < 0 || (l.mask_keep > 0 && l.mask_kind != B2_MASK_WINDOW)) why = "mask: kept first positions belong to a window";
            else if (l.ga_maps < 0 || l.ga_maps > 2) why = "attention: one or two maps";
            else if (l.ga_maps == 2 && l.ga_rot_values) why = "attention: two maps do not go with rotated values";
            else if (l.ga_gate < B2_GATE_CHANNEL || l.ga_gate > B2_GATE_NONE) why = "attention: unknown output gate";
            else if (l.ga_rot_half && l.rot_dims % 2) why = "attention: the half layout rotates an even number of dimensions";
            L.maps = l.ga_maps == 2 ? 2 : 1;
            L.nq = L.maps * l.ga_heads * l.ga_dim; L.nk = L.maps * l.ga_kv_heads * l.ga_dim; L.nv = l.ga_kv_heads * l.ga_vdim; L.ng = l.ga_heads * l.ga_vdim;
            L.gw = l.ga_gate == B2_GATE_CHANNEL ? L.ng : l.ga_gate == B2_GATE_HEAD ? l.ga_heads : 0;
            L.lproj = L.nq + L.nk + L.nv + L.gw;
            L.lproj_ld = (L.lproj + 7) / 8 * 8;
            L.conv_ch = L.nq + L.nk + L.nv;
        } else if (l.type == B2_MIXER_HGRN2) {
            if (l.g_heads < 1 || l.g_dim < 1 || l.g_dim > 256 || l.g_vdim < 1) why = "hgrn2: heads, dim 1..256, vdim";
            L.pq = l.g_heads * l.g_dim; L.pv = l.g_heads * l.g_vdim;
            L.pproj = 2 * L.pq + L.pv;
            L.pproj_ld = (L.pproj + 7) / 8 * 8;
        } else if (l.type == B2_MIXER_GLA) {
            if (l.gl_heads < 1 || l.gl_dim < 1 || l.gl_dim > 256 || l.gl_vdim < 1 || l.gl_rank < 1) why = "gla: heads, dim 1..256, vdim, decay rank";
            else if (!(l.gl_tau > 0.f)) why = "gla: tau must be positive";
            L.pq = l.gl_heads * l.gl_dim; L.pv = l.gl_heads * l.gl_vdim;
            L.pproj = 2 * L.pq + 2 * L.pv + l.gl_rank;
            L.pproj_ld = (L.pproj + 7) / 8 * 8;
        } else {
            why = "unknown mixer type";
        }
        const bool pre_mixer = l.type == B2_MIXER_LATENT_ATTN || l.type == B2_MIXER_HGRN2 || l.type == B2_MIXER_GQA_ATTN || l.type == B2_MIXER_GLA;
        if (why == nullptr && pre_mixer != (d.block != B2_BLOCK_POST_LN)) why = "this mixer does not go with the model's block form";
        if (why == nullptr && l.ff > 0) {
            if (l.ff_kind != B2_FF_RELU_SQ && d.block == B2_BLOCK_POST_LN) why = "this feed-forward needs a pre-norm or sandwich block";
            else if (l.ff_kind == B2_FF_MOE) {
                if (l.moe_experts < 1 || l.moe_top < 1 || l.moe_top > 32 || l.moe_top > l.moe_experts) why = "moe: experts >= top >= 1, at most 32 choices";
                else if (l.moe_groups < 1 || l.moe_experts % l.moe_groups || l.moe_keep < 1 || l.moe_keep > l.moe_groups) why = "moe: groups must divide experts, 1 <= keep <= groups";
                else if (l.moe_shared_ff < 0) why = "moe: negative shared width";
                else if (l.moe_score < 0 || l.moe_score > 1 || l.moe_group_score < 0 || l.moe_group_score > 1 || l.moe_act < 0 || l.moe_act > 1) why = "moe: unknown score, group score or activation";
            } else if (l.ff_kind == B2_FF_CLAMP_GLU) {
                if (l.ff_limit < 0.f) why = "gated feed-forward: negative limit";
            } else if (l.ff_kind != B2_FF_RELU_SQ && l.ff_kind != B2_FF_POLYNORM) why = "unknown feed-forward kind";
        }
        if (why == nullptr && L.src != i) {
            b2_seq_layer_desc a = l, b = s->layers[L.src].d;
            a.weights_of = b.weights_of = -1;
            if (memcmp(&a, &b, sizeof(a)) != 0) why = "a layer that borrows weights must have the sizes of their owner";
        }
        if (why != nullptr) {
            set_error("b2_seq_model_create: layer %d: %s", i, why);
            delete s;
            return -1;
        }
    }
    // layer runs: the layers in order, the looped block `times` times in a row
    {
        const bool looped = d.loop_times >= 1;   // one pass is still a pass: its vector is added in front of it
        if (looped && !(d.loop_start >= 0 && d.loop_start < d.loop_stop && d.loop_stop <= d.n_layers)) {
            set_error("b2_seq_model_create: loop [%d, %d) x %d does not fit %d layers", d.loop_start, d.loop_stop, d.loop_times, d.n_layers);
            delete s;
            return -1;
        }
        for (int i = 0; i < d.n_layers; ++i) {
            if (looped && i == d.loop_start) {
                for (int t = 0; t < d.loop_times; ++t)
                    for (int j = d.loop_start; j < d.loop_stop; ++j) s->runs.push_back(SeqRun{j, (j == d.loop_start && !d.loop_plain) ? t : -1, -1});
                i = d.loop_stop - 1;
            } else {
                s->runs.push_back(SeqRun{i, -1, -1});
            }
        }
        // a layer that reads another layer's cache rows reads those of that layer's latest run in front of it
        for (size_t r = 0; r < s->runs.size(); ++r) {
            const b2_seq_layer_desc& l = s->layers[s->runs[r].layer].d;
            if (l.type != B2_MIXER_LATENT_ATTN || l.la_kv_from == 0) continue;
            for (size_t q = r; q-- > 0;)
                if (s->runs[q].layer == l.la_kv_from - 1) { s->runs[r].kv_run = (int)q; break; }
            if (s->runs[r].kv_run < 0) {
                set_error("b2_seq_model_create: layer %d runs before the layer whose cache rows it reads", s->runs[r].layer);
                delete s;
                return -1;
            }
        }
    }
    b2_model* m = new b2_model();
    memset(&m->d, 0, sizeof(m->d));
    m->d.vocab = d.vocab; m->d.max_batch = d.max_batch; m->d.max_seq = d.max_rows; m->d.layers = d.n_layers; m->d.hidden = d.width;
    m->arch = B2_ARCH_LAYER_LIST;
    m->seq = s;
    cudaGetDevice(&m->device);
    *out = m;
    return 0;
}

int b2_seq_model_runs(const b2_model* m) {
    return (m != nullptr && m->arch == B2_ARCH_LAYER_LIST) ? (int)m->seq->runs.size() : -1;
}

int b2_append_tokens(b2_model* m, b2_kv* kv, int slot, const int32_t* tokens_host, int n, int restart, const int32_t* want_host, int n_want,
                     float* logits_out, float* resid_out, void* stream) {
    B2_CHECK_ARG(m && kv && kv->m == m && tokens_host, "b2_append_tokens: bad handle");
    B2_CHECK_ARG(m->arch == B2_ARCH_LAYER_LIST && m->finalized, "b2_append_tokens: needs a finalized layer-list model");
    SeqModel& s = *m->seq;
    B2_CHECK_ARG(slot >= 0 && slot < kv->max_batch, "b2_append_tokens: slot %d outside the cache (%d slots)", slot, kv->max_batch);
    B2_CHECK_ARG(n >= 1 && n <= s.d.max_rows, "b2_append_tokens: %d tokens in one call (at most %d)", n, s.d.max_rows);
    B2_CHECK_ARG(n_want >= 0 && n_want <= n && (n_want == 0 || (want_host && logits_out)), "b2_append_tokens: bad logits request");
    std::lock_guard<std::mutex> lk(m->mu);
    DeviceGuard dg(m->device);
    const int start = restart ? 0 : kv->len_host[slot];
    B2_CHECK_ARG(start + n <= kv->max_seq, "b2_append_tokens: %d + %d tokens exceed the cache's %d per slot", start, n, kv->max_seq);
    for (int i = 0; i < n_want; ++i) B2_CHECK_ARG(want_host[i] >= 0 && want_host[i] < n, "b2_append_tokens: wanted index %d outside the %d tokens", want_host[i], n);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    B2_TRY(ws_enter(m, st));
    B2_CUDA_CHECK(cudaMemcpyAsync(s.tok.p, tokens_host, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    RowMap rm{s.segs.as<SeqSeg>(), s.row_slot.as<int32_t>(), s.row_pos.as<int32_t>()};
    // a slot that starts over begins from position 0 whatever its device-side length says
    B2_TRY(rowmap_portion(rm, kv->len_dev.as<int32_t>(), slot, n, start == 0 ? 1 : 0, st));
    B2_TRY(seq_embed(m, kv, s.tok.as<int32_t>(), n, 1, st));
    B2_TRY(seq_forward(m, kv, n, 1, slot, start + n, resid_out, st));
    if (n_want > 0) {
        B2_CUDA_CHECK(cudaMemcpyAsync(s.want.p, want_host, (size_t)n_want * 4, cudaMemcpyHostToDevice, st));
        cudaPointerAttributes attr;
        bool dev_out = cudaPointerGetAttributes(&attr, logits_out) == cudaSuccess && (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged);
        cudaGetLastError();
        if (dev_out) {
            B2_TRY(seq_head(m, s.want.as<int32_t>(), n_want, logits_out, s.d.vocab, st));
        } else {
            // host destination: through the projection workspace, in pieces of what it holds
            const int per = (int)std::max<size_t>(1, ((size_t)s.rows * s.proj_w) / s.d.vocab);
            for (int i0 = 0; i0 < n_want; i0 += per) {
                const int c = std::min(per, n_want - i0);
                B2_TRY(seq_head(m, s.want.as<int32_t>() + i0, c, s.proj.as<float>(), s.d.vocab, st));
                B2_CUDA_CHECK(cudaMemcpyAsync(logits_out + (size_t)i0 * s.d.vocab, s.proj.p, (size_t)c * s.d.vocab * 4, cudaMemcpyDeviceToHost, st));
                B2_CUDA_CHECK(cudaStreamSynchronize(st));
            }
        }
    }
    kv->len_host[slot] = start + n;
    return ws_leave(m, st);
}

int b2_kv_free_slot(b2_kv* kv, int slot, void* stream) {
    B2_CHECK_ARG(kv && slot >= 0 && slot < kv->max_batch, "b2_kv_free_slot: bad slot");
    std::lock_guard<std::mutex> lk(kv->m->mu);
    DeviceGuard dg(kv->m->device);
    B2_CUDA_CHECK(cudaMemsetAsync(kv->len_dev.as<int32_t>() + slot, 0, 4, reinterpret_cast<cudaStream_t>(stream)));
    kv->len_host[slot] = 0;
    return 0;
}

int64_t b2_kv_bytes(b2_model* m, int max_batch, int max_seq) {
    if (m == nullptr || max_batch < 1 || max_seq < 1) return -1;
    if (m->arch == B2_ARCH_LAYER_LIST) return seq_kv_bytes(m, max_batch, max_seq);
    return (int64_t)2 * m->d.layers * max_batch * m->d.heads * max_seq * m->hd * 2;
}

}  // extern "C"
