// Internal launcher declarations for the b2llava kernels (C++ side, not part of the C ABI).
// All tensors are device pointers; activations/weights are bf16 unless stated otherwise.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

enum { ACT_NONE = 0, ACT_QUICK_GELU = 1, ACT_GELU_ERF = 2, ACT_SWIGLU = 3, ACT_ROPE_QKV = 4 };

// ACT_ROPE_QKV (CTA-pair kernel only): the GEMM is LLaMA's fused QKV projection of a prefill, rows = b*S + t. The epilogue
// rounds the projection to bf16, applies RoPE (HF rounding points, cos/sin from `table`) to the q and k heads, writes q to
// `out` and k / v straight into the KV cache [b][head][Smax][128] — the standalone rope_kv_write pass over qkv disappears.
struct RopeQkv {
    const void* table = nullptr;   // uint32 [Smax][64]: bf16 cos | bf16 sin << 16 of position t, frequency i (rope_table_build)
    void* kcache = nullptr;        // this layer's K slab of the first batch row written
    void* vcache = nullptr;
    int S = 0, H = 0, Smax = 0;
};
enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

int num_sms();

// ---- tcgen05 GEMM (gemm_tcgen05.cu) -------------------------------------------------------------
// out[M, N] = act(A[M,K] · W[N,K]^T + bias) + residual      (ACT_NONE / QUICK_GELU / GELU_ERF)
// out[M, N/2] = silu(gate) * up                               (ACT_SWIGLU; W rows block-64 interleaved)
struct GemmArgs {
    const void* A = nullptr; int lda = 0;        // bf16 [M, K]
    const void* W = nullptr; int ldw = 0;        // bf16 [N, K]
    const void* bias = nullptr;                  // bf16 [N] or null
    const void* residual = nullptr; int ld_res = 0;  // bf16 [M, N] or null (may alias out)
    void* out = nullptr; int ld_out = 0; int out_fp32 = 0;
    int M = 0, N = 0, K = 0;
    int act = ACT_NONE;
    int bn_override = 0;  // 0 = cost-model heuristic, else 64/128/192/256 (2 = CTA-pair kernel)
    RopeQkv rope;         // ACT_ROPE_QKV only
    // fp32 output only (layer-list decoders): out = alpha * post(acc + bias + residual) (+ out when accumulate); post = LIN_*
    int post = 0; float alpha = 1.f; int accumulate = 0;
    // grouped product (mixture of experts; single-CTA kernels only): M is a multiple of 128, tile t of 128 rows multiplies with
    // W rows [g * N, (g + 1) * N), g = tile_group[t] (device; negative: the tile is skipped); W holds `groups` matrices of N rows
    const int* tile_group = nullptr; int groups = 1;
};
int gemm_bf16(const GemmArgs& g, cudaStream_t stream);
// mm_projector mlp2x_gelu as ONE kernel (gemm_tcgen05.cu, projector_fused_kernel): out = gelu_erf(X W1^T + b1) W2^T + b2.
// H [M,N1] bf16 and row_done int[ceil(M/128)] are caller scratch.
int projector_fused_bf16(const void* X, int ldx, const void* W1, const void* b1, const void* W2, const void* b2, void* H,
                         void* out, int ld_out, int M, int K1, int N1, int N2, int* row_done, cudaStream_t stream);
// CTA-pair (cta_group::2, 256x256 pair tiles) variant, gemm_2cta.cu (chosen by gemm_bf16's cost model, or bn_override == 2)
int gemm_bf16_2cta(const GemmArgs& g, cudaStream_t stream);

// ---- swap-AB stream-K GEMM for decode at batch 9..128 (gemm_skinny.cu) ------------------------------------
// out[B, N] = x[B,K] · W[N,K]^T (+ residual); ACT_SWIGLU: out[B, N/2] (W rows block-64 interleaved).
struct SkinnyArgs {
    const void* x = nullptr; int ldx = 0;        // bf16 [B, K]
    const void* W = nullptr; int ldw = 0;        // bf16 [N, K]
    const void* residual = nullptr; int ld_res = 0;  // bf16 [B, N] or null (may alias out)
    void* out = nullptr; int ld_out = 0; int out_fp32 = 0;
    int B = 0, N = 0, K = 0;
    int act = ACT_NONE;                          // ACT_NONE | ACT_SWIGLU
    float* partial = nullptr; size_t partial_bytes = 0;  // >= gemm_skinny_workspace_bytes(B, N, K)
    int* counters = nullptr;                     // >= gemm_skinny_counter_bytes(N), zero-initialised once
    const float* w_scale = nullptr;              // fp8 variant: [N] per weight row; x / W then hold e4m3 bytes
    const float* x_scale = nullptr;              // fp8 variant: [B] per token
};
int gemm_skinny_bf16(const SkinnyArgs& g, cudaStream_t stream);
int gemm_skinny_fp8(const SkinnyArgs& g, cudaStream_t stream);
size_t gemm_skinny_workspace_bytes(int B, int N, int K);
size_t gemm_skinny_counter_bytes(int N);

// ---- e4m3 row quantisation for the fp8 decode path (quant_fp8.cu) ----------------------
// scale[r] = amax_r / 448 (1 for a zero row); q[r,k] = e4m3_rn_satfinite(x[r,k] * (448 / amax_r)); ld* in elements
int quantize_rows_e4m3(const void* x, int64_t ldx, int rows, int K, void* q, int64_t ldq, float* scale, cudaStream_t stream);
// RMSNorm (HF rounding points) fused with the per-token quantisation of its output
int rmsnorm_quant_e4m3(const void* x, int64_t x_row_stride, const void* gamma, void* q, int64_t ldq, float* scale, int rows,
                       int cols, float eps, cudaStream_t stream);

// ---- weight-streaming GEMV for decode (gemv.cu) ---------------------------------------------------
// out[B, N] = (rmsnorm(x) or x)[B,K] · W[N,K]^T (+ residual); B <= 8. ACT_SWIGLU: out[B, N/2].
struct GemvArgs {
    const void* x = nullptr; int64_t ldx = 0;   // bf16 [B, K], row stride ldx (elements)
    const void* W = nullptr; int ldw = 0;        // bf16 [N, K]
    const void* norm_gamma = nullptr; float eps = 0.f;  // fused RMSNorm on x when non-null
    const void* residual = nullptr; int ld_res = 0;     // bf16 [B, N] or null (may alias out)
    void* out = nullptr; int ld_out = 0; int out_fp32 = 0;
    int B = 0, N = 0, K = 0;
    int act = ACT_NONE;
};
int gemv_bf16(const GemvArgs& g, cudaStream_t stream);
bool gemv_fits(int B, int N, int K, int act);  // activation tile + partial table fit in shared memory

// ---- norms (norms.cu) ------------------------------------------------------------------------------
int layernorm_bf16(const void* x, const void* gamma, const void* beta, void* y, int rows, int cols, float eps,
                   cudaStream_t stream);
// HF LlamaRMSNorm semantics: y = gamma * bf16(x * rsqrt(mean(x^2) + eps)); x rows may be strided.
int rmsnorm_bf16(const void* x, int64_t x_row_stride, const void* gamma, void* y, int rows, int cols, float eps,
                 cudaStream_t stream);
// gather variant: row r of y is the RMSNorm of x[row_index[r]] (row_index on device)
int rmsnorm_gather_bf16(const void* x, const int32_t* row_index, const void* gamma, void* y, int rows, int cols,
                        float eps, cudaStream_t stream);

// ---- ViT helpers (vit_ops.cu) ----------------------------------------------------------------------
// pixels [B,3,img,img] bf16 -> patches [B*P, kpad] (k = c*patch*patch + i*patch + j, zero padded to kpad)
int vit_im2col(const void* pixels, void* out, int B, int img, int patch, int kpad, cudaStream_t stream);
// hidden[b, 0] = LN(cls + pos[0]); hidden[b, 1+p] = LN(patch_out[b*P+p] + pos[1+p])   (pre_layrnorm fused)
int vit_embed_ln(const void* patch_out, const void* cls, const void* pos, const void* gamma, const void* beta,
                 void* hidden, int B, int P, int D, float eps, cudaStream_t stream);
// out[b, p, :] = hidden[b, 1 + p, :]   (feature_select 'patch': drop CLS)
int vit_drop_cls(const void* hidden, void* out, int B, int P, int D, cudaStream_t stream);

// ---- attention (attention.cu) ----------------------------------------------------------------------
struct FlashArgs {
    const void* q = nullptr; int64_t q_bs = 0, q_ts = 0, q_hs = 0;  // element strides: batch, token, head
    const void* k = nullptr; int64_t k_bs = 0, k_ts = 0, k_hs = 0;
    const void* v = nullptr; int64_t v_bs = 0, v_ts = 0, v_hs = 0;
    void* o = nullptr;       int64_t o_bs = 0, o_ts = 0, o_hs = 0;
    const int32_t* seq_lens = nullptr;  // device [B] or null (=S)
    int B = 0, H = 0, S = 0, D = 0;     // S = padded/query length; D in {64, 128}
    int causal = 0;
    float scale = 1.f;
};
int flash_attn_bf16(const FlashArgs& a, cudaStream_t stream);      // dispatcher (tcgen05 unless B2_FLASH_TC=0)
int flash_attn_tc_bf16(const FlashArgs& a, cudaStream_t stream);   // attention_tc.cu: tcgen05 + TMEM + TMA
int flash_attn_mma_bf16(const FlashArgs& a, cudaStream_t stream);  // attention.cu: mma.sync variant

// prefill: RoPE on q (in place) and k inside qkv [B*S, 3*H*D]; roped k and v written to the cache
// kcache/vcache: [Bmax, H, Smax, D] for one layer. Positions are 0..S-1 (right-padded rows).
// (cos, sin) table of rope_kv_write's positions 0..Smax-1 (head_dim D): uint32 [Smax][D/2], bf16 cos | bf16 sin << 16
int rope_table_build(void* table, int Smax, int D, float theta, cudaStream_t stream);
int rope_kv_write(void* qkv, void* kcache, void* vcache, int B, int S, int H, int D, int Smax, float theta,
                  cudaStream_t stream);

// decode: q/k/v of the new token from qkv [B, 3*H*D]; RoPE at position cur_len[b]; append k,v to the cache;
// split-KV attention over cur_len[b]+1 keys; out [B, H*D] bf16.
struct DecodeAttnArgs {
    const void* qkv = nullptr;
    void* kcache = nullptr; void* vcache = nullptr;  // layer base, [Bmax, H, Smax, D]
    const int32_t* cur_len = nullptr;                // device [B]
    void* out = nullptr;
    float* partial = nullptr;                        // workspace [B*H*nsplit*(D+2)] fp32
    int32_t* counters = nullptr;                     // workspace [B*H], zero-initialised, self-resetting
    int B = 0, H = 0, D = 128, Smax = 0, nsplit = 1;
    float theta = 10000.f, scale = 1.f;
};
int decode_attn_ctas_per_sm();
int decode_attn_bf16(const DecodeAttnArgs& a, cudaStream_t stream);

// ---- persistent decode-step megakernel (decode_mega.cu), batch <= 8 ------------------------------------
struct MegaLayer {
    const __nv_bfloat16 *ln1, *wqkv, *wo, *ln2, *wgu, *wd;
    __nv_bfloat16 *kcache, *vcache;  // this layer's [Bmax, H, Smax, 128] slabs
};
struct MegaParams {
    const MegaLayer* layers = nullptr;  // device array [L]
    int L = 0, h = 0, I = 0, H = 0, V = 0, B = 0, Smax = 0, nsplit = 1;
    const __nv_bfloat16 *embed = nullptr, *final_norm = nullptr, *lm_head = nullptr;
    int32_t *tok = nullptr, *cur_len = nullptr, *out_tokens = nullptr, *step_counter = nullptr;
    __nv_bfloat16 *x = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr;
    float* logits = nullptr;
    float* attn_partial = nullptr;      // [B*H*nsplit*(128+2)]
    int32_t* attn_counters = nullptr;   // [B*H], zero-initialised, self-resetting
    unsigned int *bar_count = nullptr, *done_count = nullptr;  // zero-initialised
    unsigned int bar_base = 0;  // barrier-counter value before this launch = launches so far * (5L+2) * grid
    float eps = 1e-5f, theta = 10000.f, scale_log2 = 1.f;
    int l2_ahead = 0;       // weight tiles pulled into L2 in front of the shared-memory ring (0 = off), multiple of 4
    int l2_mode = 1;        // 1 = prefetch.global.L2 lines (LSU), 2 = cp.async.bulk.prefetch.L2 (TMA queue)
    int fast_prologue = 0;  // single-pass activation staging with pre-barrier RMSNorm-weight loads
    int gamma_smem = 0;     // next phase's RMSNorm weights staged in shared memory (cp.async) in front of the grid barrier
    long long* trace = nullptr;  // optional [n_phases+2][4] SM-clock timestamps of CTA 0 (B2_MEGA_TRACE=1)
    // token publication to the host ring (sampling.cu): non-null only for greedy streaming; with do_sample the separate
    // sample_publish kernel that follows the launch overrides the fused argmax and publishes instead
    struct SampleState* sstate = nullptr;
    int32_t* ring = nullptr;
    int ring_cap = 0;
    const struct RowState* rows = nullptr;  // continuous batching: only active slots advance their cache length
};
// one launch = embed -> all layers -> lm_head -> argmax -> token store; cur_len/step_counter advance on device
int decode_mega(const MegaParams& p, cudaStream_t stream);
bool decode_mega_fits(int B, int h, int I);

// ---- token selection + host-ring publication (sampling.cu) --------------------------------------------------
// Device-resident state of one generation (lives in the b2_kv): read by the kernels, so a captured CUDA graph of the decode
// step stays valid when the sampling parameters change.
struct SampleState {
    int do_sample;            // 0 = greedy argmax
    float temperature, top_p;
    int top_k;                // 0 = off
    unsigned long long seed;  // Philox key
    int tag;                  // generation epoch 1..2047 published with every token; 0 = do not publish to the host ring
    int pub_counter;          // index of the next token of this generation
    unsigned int done;        // rows finished in the current launch (self-resetting)
    int per_row;              // continuous batching: selection parameters and liveness come from RowState[b] instead
};
// One cache slot of a continuously batched decode (llava/_b2/batching.py): requests join and leave between steps, each with
// its own sampling parameters and its own Philox draw index; a slot that is not active keeps its cache length and token.
struct RowState {
    int active;
    int do_sample; float temperature, top_p; int top_k;
    unsigned long long seed;
    int index;                // draws made for this request so far
};
enum { SP_SELECT = 1,     // choose from `logits` (argmax or sample) and write tok[b]; otherwise tok[b] is already chosen
       SP_WRITE_OUT = 2,  // out_tokens[(*step_counter + step_offset) * B + b] = token
       SP_BUMP = 4 };     // last row: *step_counter += 1, cur_len[b] += 1
int sample_state_set(SampleState* st_dev, const SampleState& v, cudaStream_t stream);
int sample_publish(const float* logits, int V, int B, SampleState* st_dev, RowState* rows_dev, int32_t* tok, int32_t* out_tokens,
                   int32_t* step_counter, int32_t* cur_len, int32_t* ring_dev, int ring_cap, int flags, int step_offset,
                   cudaStream_t stream);
int row_state_set(RowState* row_dev, const RowState& v, int32_t* tok_dev, int token, cudaStream_t stream);

// ---- image preprocessing (preprocess.cu): uint8 HWC -> CLIP pixel_values, PIL-exact bicubic resize ------------------------
struct PreprocessArgs {
    const uint8_t* img = nullptr; int H = 0, W = 0;        // device, RGB HWC
    int pad_top = 0, pad_left = 0; uint8_t bg[3] = {0, 0, 0};  // virtual expand2square: reads outside the image return bg
    const int32_t *h_bounds = nullptr, *h_kk = nullptr; int h_ksize = 0, h_identity = 0;  // tables over the resized WIDTH
    const int32_t *v_bounds = nullptr, *v_kk = nullptr; int v_ksize = 0, v_identity = 0;  // tables over the resized HEIGHT
    int y0 = 0, rows = 0;        // source rows the vertical pass reads: [y0, y0 + rows)
    int x_lo = 0, y_lo = 0;      // centre-crop origin inside the resized image
    int cols = 0, out = 0;       // cols == out: crop width / output size
    uint8_t* tmp = nullptr;      // [rows, cols, 3] scratch
    float mean[3] = {0, 0, 0}, stdv[3] = {1, 1, 1}, rescale = 1.f / 255.f;
    void* pixels = nullptr;      // bf16 [3, out, out] or null
    uint8_t* u8_out = nullptr;   // uint8 [out, out, 3] (the resized + cropped image before normalisation) or null
};
int preprocess_clip_image(const PreprocessArgs& a, cudaStream_t stream);

// ---- misc (misc_ops.cu) ----------------------------------------------------------------------------
// out[r, :] = src_index[r] >= 0 ? table[src_index[r]] : (src_index[r] == INT32_MIN ? 0 : feats[-src_index[r]-1]).
// Rows whose index is outside [0, vocab) / [0, n_feat_rows) are written as zeros and reported through *err_flag
// (mapped host memory, B2_ERR_* codes, may be null): nothing is ever read out of bounds.
int splice_embed(const int32_t* src_index, const void* table, const void* feats, void* out, int rows, int h, int vocab,
                 int n_feat_rows, int* err_flag, cudaStream_t stream);
// device-built source index for equal-length unpadded rows with k_per_row image placeholders each (misc_ops.cu):
// ids int64 [B, Lt] on the device; feat_offsets_host[n_img + 1] = prefix sums of the feature rows of the image slots
int splice_index(const long long* ids, int B, int Lt, int k_per_row, const int32_t* feat_offsets_host, int n_img, int image_token,
                 int S, int32_t* src_index, int* err_flag, cudaStream_t stream);
int embed_tokens(const int32_t* tokens, const void* table, void* out, int rows, int h, int vocab, int* err_flag,
                 cudaStream_t stream);
enum { B2_ERR_TOKEN_RANGE = 1, B2_ERR_IMAGE_ROW_RANGE = 2, B2_ERR_SPLICE_SLOTS = 4 };
int argmax_f32(const float* logits, int B, int V, int32_t* out, cudaStream_t stream);
struct I32Pack { int32_t v[128]; };
// dst_a[i] = a_host[i] (and dst_b[i] = b_host[i] when dst_b != null), i < n: values travel as kernel parameters
int set_i32_pairs(int32_t* dst_a, const int32_t* a_host, int32_t* dst_b, const int32_t* b_host, int n, cudaStream_t stream);
int add_i32(int32_t* x, int n, int delta, cudaStream_t stream);
int convert_to_bf16(const void* src, int src_dtype, void* dst, int64_t n, cudaStream_t stream);
int convert_to_f32(const void* src, int src_dtype, float* dst, int64_t n, cudaStream_t stream);  // src on the device
// out[2I, h]: within each 128-row group g: rows [0,64) = gate[g*64 .. +64), rows [64,128) = up[g*64 .. +64)
int interleave_gate_up(const void* gate, const void* up, void* out, int I, int h, cudaStream_t stream);
int store_token(const int32_t* src, int32_t* dst_base, const int32_t* step_counter, int B, cudaStream_t stream);

// =====================================================================================================================
// Layer-list decoders (seq_engine.cu): fp32 residual stream, recurrent mixers, biased attention with generic head sizes.
// Rows of one call are described on the device so that a captured decode step follows the cache lengths by itself:
// a SEGMENT is a run of consecutive rows that belong to one cache slot (a prompt portion: n rows; a decode step: 1 row).
// =====================================================================================================================
struct SeqSeg {
    int slot;   // cache slot (state / key-value slab index)
    int row0;   // first row of the segment in the call's activation buffers
    int n;      // rows (0: the slot is idle in this step; nothing of its state is touched)
    int pos0;   // position of the first row inside its sequence (0: the state starts from zero, whatever the slot held)
};
struct RowMap {
    SeqSeg* segs = nullptr;     // device [nseg]
    int32_t* row_slot = nullptr;  // device [rows]
    int32_t* row_pos = nullptr;   // device [rows]; -1 = idle row
};
// one segment: rows [0, n) of slot `slot`; its start position is read on the device from len[slot] (and len[slot] += n)
int rowmap_portion(const RowMap& rm, int32_t* len, int slot, int n, int restart, cudaStream_t stream);
// B segments of one row each for slots slot0 .. slot0+B-1 at positions len[slot]; with sstate->per_row set, slots whose
// rows_state entry is not active become idle rows
int rowmap_decode(const RowMap& rm, const int32_t* len, const SampleState* sstate, const RowState* rows_state, int slot0, int B,
                  cudaStream_t stream);

// ---- generic Linear on fp32 activations (linear_generic.cu): any M, N, K -----------------------------------------------
enum { LIN_NONE = 0, LIN_SILU = 1, LIN_SIGMOID = 2, LIN_TANH = 3, LIN_RELU_SQ = 4 };
struct LinearArgs {
    const float* A = nullptr; int64_t lda = 0;   // fp32 [M, K]
    const void* W = nullptr; int64_t ldw = 0;    // [N, K], DT_BF16 or DT_F32
    int w_dtype = DT_F32;
    const float* bias = nullptr;                 // fp32 [N] or null
    float* out = nullptr; int64_t ld_out = 0;    // fp32 [M, N]
    int M = 0, N = 0, K = 0;
    int act = LIN_NONE;
    float alpha = 1.f;                           // out = alpha * act(A W^T + bias) (+ out when accumulate)
    int accumulate = 0;
    int round_a = 0;                             // round A to bf16 first (bf16 compute: the product is bf16 x bf16 -> fp32)
};
int linear_f32(const LinearArgs& a, cudaStream_t stream);
// out[r, :K] = bf16(A[r, :K]): the A operand of a tensor-core GEMM from fp32 activations (ld_out % 8 == 0)
int cast_rows_bf16(const float* A, int64_t lda, void* out, int64_t ld_out, int M, int K, cudaStream_t stream);

// Grouped Linear: output rows come in tiles of tile_rows (1 or 64) rows; tile t multiplies with the weight matrix of group
// tile_group[t] (W + group * w_group_stride elements; a negative group: the tile is unused). Output row m reads input row
// a_rows[m] (a_rows null: m / a_div; negative: a zero row). out[m, :N] = act(A[src] W_g^T); M bounds the rows (the launch grid).
struct GroupedLinearArgs {
    const float* A = nullptr; int64_t lda = 0;
    const int32_t* a_rows = nullptr; int a_div = 1;
    const void* W = nullptr; int64_t ldw = 0; int64_t w_group_stride = 0; int w_dtype = DT_F32;
    const int32_t* tile_group = nullptr; int tile_rows = 64;
    float* out = nullptr; int64_t ld_out = 0;
    int M = 0, N = 0, K = 0;
    int act = LIN_NONE;
    int round_a = 0;
    int swiglu = 0;   // one-row tiles only: a group's matrix is [gate | up] of N rows each and out[m, n] = silu(gate_n . a) * (up_n . a)
    float glu_slope = 1.f, glu_limit = 0.f, glu_up_shift = 0.f;   // with swiglu: the general gated unit (GluAct) instead of SiLU(g) u
};
int linear_grouped_f32(const GroupedLinearArgs& g, cudaStream_t stream);
// `batch` small Linears in one launch on a handful of rows (a decode step's per-head products): for b < batch,
// out[m, b * o_bs + n] = sum_k A[m, b * a_bs + k] * W[b * w_bs + n * K + k], m < M <= 8; weights in w_dtype, fp32 accumulation;
// gate (nullable, [M, ldg]): the result is multiplied by sigmoid(gate[m, b])
int linear_batched_rows_f32(const float* A, int64_t lda, int64_t a_bs, const void* W, int64_t w_bs, int w_dtype, float* out, int64_t ld_out,
                            int64_t o_bs, int batch, int M, int N, int K, int round_a, cudaStream_t stream, const float* gate = nullptr, int64_t ldg = 0);
enum { GROUPED_TILE_ROWS = 64 };

// ---- mixture of experts (moe.cu) ------------------------------------------------------------------------------------------
// Router: scores s = sigmoid(logits) (score_fn MOE_SCORE_SOFTMAX: softmax over the experts); experts form `groups` equal groups of
// neighbours, a group's score is the sum of its two largest scores (group_score MOE_GROUP_MAX: its largest), only experts of
// the best `keep` groups compete; the `top` largest are chosen (ties: the lower index); w = s / (sum of the chosen s + 1e-20) *
// scale (raw_weights: w = s). idx / w: [rows, top].
enum { MOE_SCORE_SIGMOID = 0, MOE_SCORE_SOFTMAX = 1, MOE_GROUP_TOP2_SUM = 0, MOE_GROUP_MAX = 1 };   // the values of B2_MOE_*
struct MoeRouteArgs {
    const float* logits = nullptr; int64_t ld = 0;
    int rows = 0, experts = 0, top = 0, groups = 1, keep = 1;
    int score_fn = 0, group_score = 0, raw_weights = 0;
    float scale = 1.f;
    int32_t* idx = nullptr; float* w = nullptr;
};
int moe_route_f32(const MoeRouteArgs& a, cudaStream_t stream);
// Sorts the rows * top pairs by expert into tiles of `tile` rows of one expert each: pair_pos[pair] = its position,
// src_row[position] = its token row (-1: padding), tile_group[t] = the expert of tile t (-1: unused).
// max_tiles * tile >= rows * top + experts * (tile - 1).
int moe_plan(const int32_t* idx, int rows, int top, int experts, int tile, int max_tiles, int32_t* pair_pos, int32_t* src_row, int32_t* tile_group,
             cudaStream_t stream);
// out[r, c] = silu(in[r, c]) * in[r, ff + c], c < ff; out16 (nullable, bf16 [rows, ld_out16]) receives the rounded copy that a
// tensor-core product reads next (out may then be null)
int swiglu_rows_f32(const float* in, int64_t ld_in, float* out, int64_t ld_out, int rows, int ff, cudaStream_t stream, void* out16 = nullptr,
                    int64_t ld_out16 = 0);
// The gated unit in its general form: with g = in[r, c] and u = in[r, ff + c], limit > 0 first bounds them, g = min(g, limit),
// u = clamp(u, -limit, limit); out = g sigmoid(slope g) (u + up_shift). (slope 1, no limit, shift 0: SiLU(g) u.)
struct GluAct { float slope = 1.f, limit = 0.f, up_shift = 0.f; };
__host__ __device__ inline float glu_act(float g, float u, const GluAct& a) {
    if (a.limit > 0.f) { g = fminf(g, a.limit); u = fminf(fmaxf(u, -a.limit), a.limit); }
    return g / (1.f + expf(-a.slope * g)) * (u + a.up_shift);
}
int glu_rows_f32(const float* in, int64_t ld_in, float* out, int64_t ld_out, int rows, int ff, const GluAct& act, cudaStream_t stream,
                 void* out16 = nullptr, int64_t ld_out16 = 0);
// out[p, :K] = bf16(A[src_row[p], :K]), zeros where src_row[p] < 0: the gathered A operand of a grouped tensor-core product
int gather_rows_bf16(const float* A, int64_t lda, const int32_t* src_row, void* out, int64_t ld_out, int rows, int K, cudaStream_t stream);
// x[r] += alpha * sum_k w[r, k] * y[pair_pos[r * top + k]] (pair_pos null: the pair's own index)
int moe_combine_f32(float* x, const float* y, int64_t ldy, const int32_t* pair_pos, const float* w, int rows, int top, int cols, float alpha,
                    cudaStream_t stream);

// ---- fp32 norms and row helpers (norms_f32.cu) ------------------------------------------------------------------------
// x[r] += LayerNorm(y[r]) * gamma + beta   (normalisation of a sublayer's OUTPUT, added to the residual stream)
int layernorm_add_f32(float* x, const float* y, const float* gamma, const float* beta, int rows, int cols, float eps, cudaStream_t stream);
// out[i] = LayerNorm(x[row_index[i]]) * gamma + beta
int layernorm_gather_f32(const float* x, const int32_t* row_index, const float* gamma, const float* beta, float* out, int rows, int cols,
                         float eps, cudaStream_t stream);
// Per row and per group of `group` consecutive channels (cols % group == 0):
//   gate_first: out = unit_rms(y * silu(z)) * gamma            (state-space mixer: the gate comes before the norm)
//   otherwise : out = unit_rms(y) * gamma * silu(z)            (RWKV mixer: per-head norm, then weight, then gate)
// gamma_shared: one weight vector [group] for every group instead of [cols]
int gated_group_rmsnorm_f32(const float* y, int64_t ldy, const float* z, int64_t ldz, const float* gamma, float* out, int64_t ldo, int rows,
                            int cols, int group, int gate_first, float eps, cudaStream_t stream, int gamma_shared = 0);
// ungated form; gamma_shared: one weight vector [group] for every group instead of [cols]
int group_rmsnorm_f32(const float* y, int64_t ldy, const float* gamma, int gamma_shared, float* out, int64_t ldo, int rows, int cols, int group,
                      float eps, cudaStream_t stream);
// One-number RMS norm of pre-norm blocks: out[i] = x[row_index[i]] / sqrt(mean(x^2) + eps) * g[0] (row_index null: row i). With add
// and/or vec the row is first updated in place, x += add[row] + vec: the opening of a pass of a looped block of layers.
int rms_scalar_f32(float* x, const int32_t* row_index, const float* g, const float* add, const float* vec, float* out, int rows, int cols,
                   float eps, cudaStream_t stream);
// dst[b][c][r] = src[b][r][c], elements of 2 or 4 bytes (a stack of matrices transposed one by one)
int transpose_blocks(const void* src, void* dst, int blocks, int rows, int cols, int elem_size, cudaStream_t stream);
// PolyNorm: out = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3, z = in + bias (bias nullable), N(u) = u / sqrt(mean(u^2) + eps) per row; coef on the device
int polynorm_f32(const float* in, int64_t ld_in, const float* bias, const float* coef, float* out, int64_t ld_out, int rows, int cols, float eps,
                 cudaStream_t stream);
// x[i] = cap * tanh(x[i] / cap)
int softcap_f32(float* x, size_t n, float cap, cudaStream_t stream);
// out[r, h*dv + d] = a[r, h*dv + d] * sigmoid(g[r, h])
int head_gate_f32(const float* a, int64_t lda, const float* g, int64_t ldg, float* out, int64_t ldo, int rows, int heads, int dv, cudaStream_t stream);
// x[row] = table[tok] + bigram[(prev * mul_prev + tok * mul_cur) mod buckets] (row `buckets` for a sequence's first token; bigram null:
// no such term). Rows come as segments; the token in front of a call's first row is last_tok[slot], which is replaced by the segment's
// last token. x0 (nullable) receives a copy of x. tokens is indexed by row.
int embed_bigram_rows_f32(const int32_t* tokens, const SeqSeg* segs, int nseg, int max_n, const void* table, const void* bigram, int table_dtype,
                          int32_t* last_tok, float* x, float* x0, int cols, int vocab, int buckets, int mul_prev, int mul_cur, int* err_flag,
                          cudaStream_t stream);
// cache[slot][pos][:rank] = unit_rms(in[r, :rank]) * gamma for every live row r
int latent_append_f32(const float* in, int64_t ld_in, const float* gamma, float* cache, const int32_t* row_slot, const int32_t* row_pos, int rows,
                      int rank, int Smax, float eps, cudaStream_t stream);
// x[r, :] = table[tokens[r], :] as fp32; ids outside [0, vocab) give a zero row and raise *err_flag (B2_ERR_TOKEN_RANGE)
int embed_rows_f32(const int32_t* tokens, const void* table, int table_dtype, float* x, int rows, int cols, int vocab, int* err_flag,
                   cudaStream_t stream, float scale = 1.f);   // scale: x = table[token] * scale, in fp32
// Differential attention, per (row, head): d = a1 - lambda a2 over the head's dv values, out = d / sqrt(mean(d^2) + eps) * out_scale.
// y holds map 1 of every head, then map 2 of every head: [rows, 2 * heads * dv]
int diff_combine_f32(const float* y, int64_t ldy, float* out, int64_t ldo, int rows, int heads, int dv, float lambda, float out_scale, float eps,
                     cudaStream_t stream);
// out[r, c] = a[r, c] * sigmoid(g[r, c])
int sigmoid_gate_f32(const float* a, int64_t lda, const float* g, int64_t ldg, float* out, int64_t ldo, int rows, int cols, cudaStream_t stream);

// out[i] = x[row_index[i]] / sqrt(mean(x^2) + eps) * w (row_index null: row i; rows of pitch ld_in / ld_out); accumulate: out[i] += ...
// (a normed sublayer output joining the residual stream)
int rms_weight_f32(const float* in, int64_t ld_in, const int32_t* row_index, const float* w, float* out, int64_t ld_out, int accumulate, int rows,
                   int cols, float eps, cudaStream_t stream);

// The norms around a sublayer of a sandwich block in one pass over a row: first (y, w_post non-null) x += rms_w_post(y), the normed
// output of the previous sublayer joining the residual stream; then (w_pre non-null) out = rms_w_pre(x), the next sublayer's input.
// With conv_w the input convolution of a decode step rides along: every row is a segment of ONE token (row r = segs[r]), conv_out =
// out + sum_j conv_w[c, j] * (the taps - 1 carried inputs of the slot, then out itself), and the carried inputs move on by one
// (a segment at position 0 starts from zeros; an idle segment, n == 0, is left alone).
struct SandwichNormArgs {
    const float* y = nullptr; const float* w_post = nullptr;
    float* x = nullptr;
    const float* w_pre = nullptr; float* out = nullptr;
    const float* conv_w = nullptr; float* tail = nullptr; int taps = 0; const SeqSeg* segs = nullptr; float* conv_out = nullptr;
    int rows = 0, cols = 0; float eps = 0.f;
};
int sandwich_norm_f32(const SandwichNormArgs& a, cudaStream_t stream);

// ---- rotary positions (rotary.cu) -------------------------------------------------------------------------------------------
// Pairs (2m, 2m+1) (or, in the half layout, (m, m + pairs)), m < floor(dims / 2), turn by position * f_m, f_m = base^(-2m / dims). factor > 0: f_m is blended towards f_m / factor
// over the pairs between lo = max(floor(dim(fast)), 0) and hi = min(ceil(dim(slow)), dims - 1), dim(t) = dims ln(original / (2 pi t)) /
// (2 ln base), and cos / sin are scaled by 0.1 ln(factor) + 1.
struct RotaryDesc { int dims = 0; float base = 10000.f, factor = 0.f, original = 0.f, fast = 0.f, slow = 0.f; };
// table_dev[p][m] = (cos, sin)(p * f_m) * scale for p < positions; computed on the host in double precision
int rotary_table_build(const RotaryDesc& d, int positions, float2* table_dev);
// For every live row r (position row_pos[r] >= 0) and head h < heads: the head's `size` entries at in[r * ld_in + h * hs_in] are copied
// to out[r * ld_out + h * hs_out] (or to cache[slot][h][position][size]); the `pairs` pairs from entry `offset` on are turned by the
// row's position (inverse: by minus the position); gate (nullable, [rows, ldg], entry h * size + d): the result times its sigmoid.
// in == out is allowed.
struct RotateArgs {
    const float* in = nullptr; int64_t ld_in = 0; int hs_in = 0;
    float* out = nullptr; int64_t ld_out = 0; int hs_out = 0;
    float* cache = nullptr; int Smax = 0;
    const float* gate = nullptr; int64_t ldg = 0;
    const float2* table = nullptr;               // [positions][pairs]
    int heads = 0, size = 0, offset = 0, pairs = 0, inverse = 0, rows = 0;
    const int32_t* row_slot = nullptr; const int32_t* row_pos = nullptr;
    int half = 0;                                // pair m is (offset + m, offset + m + pairs) instead of (offset + 2m, offset + 2m + 1)
    const float* norm_w = nullptr; float eps = 0.f;   // non-null: the head is first normed, x / sqrt(mean(x^2) + eps) * norm_w over its `size` entries
                                                      // (one weight vector for all heads); such calls run one warp per (row, head)
};
int rotate_rows_f32(const RotateArgs& a, cudaStream_t stream);
// up to three such calls over the same rows in one launch (queries, keys and values of an attention layer)
int rotate_rows_multi_f32(const RotateArgs* parts, int n, cudaStream_t stream);
// Row of a low-rank key/value cache with a rotated key part: cache[slot][pos] = [unit_rms(in[r, :rank]) * gamma | the rot entries
// behind them, of which the first `pairs` pairs are turned by the row's position]; rows of the cache have rank + rot entries
int latent_rot_append_f32(const float* in, int64_t ld_in, const float* gamma, float* cache, const int32_t* row_slot, const int32_t* row_pos, int rows,
                          int rank, int rot, int pairs, const float2* table, int Smax, float eps, cudaStream_t stream);

// ---- recurrent mixers (recurrent.cu) ----------------------------------------------------------------------------------
// Causal depthwise convolution + SiLU with a carried tail: out[t, c] = silu(bias[c] + sum_j w[c, j] * in[t - (taps-1-j), c]);
// inputs before the start of the call come from tail[slot][taps-1][C] (zeros when the segment starts a sequence); the tail is
// replaced by the last taps-1 inputs. taps <= 16.
// max_n: the longest segment of the call (the launch grid covers that many rows per segment).
int causal_conv_silu_f32(const float* in, int64_t ld_in, const float* w, const float* bias, float* tail, float* out, int64_t ld_out, int C,
                         int taps, const SeqSeg* segs, int nseg, int max_n, cudaStream_t stream);
// The same convolution in its other forms: bias nullable; flags CONV_SILU (the activation above), CONV_ADD_INPUT (out = in + conv(in):
// a sublayer input that passes a convolution beside itself). in and out are different buffers.
enum { CONV_SILU = 1, CONV_ADD_INPUT = 2 };
int causal_conv_f32(const float* in, int64_t ld_in, const float* w, const float* bias, float* tail, float* out, int64_t ld_out, int C, int taps,
                    int flags, const SeqSeg* segs, int nseg, int max_n, cudaStream_t stream);
// Token shift: out[s][t, c] = x[t, c] + (x[t-1, c] - x[t, c]) * mu[s][c] for s < n_mix, with x[-1] = prev[slot] (zeros at a sequence
// start); prev[slot] := the segment's last row. out is [n_mix][rows_total][cols].
int token_shift_mix_f32(const float* x, const float* mu, float* prev, float* out, int64_t out_stride, int cols, int n_mix, const SeqSeg* segs,
                        int nseg, int max_n, cudaStream_t stream);
// Linear recurrence with a diagonal decay over a [key, value] state per head, carried per slot in fp32:
//   SCAN_SSD : dt = softplus(dt_raw + dt_bias[h]); S = exp(-exp(a_log[h]) dt) S + (dt k) v^T ; y = S^T q + skip[h] v
//              (q, k: [rows, groups, dk] shared by heads/groups consecutive heads; v: [rows, heads, dv])
//   SCAN_RWKV: y = (S + diag(bonus[h]) k v^T)^T q ; S = diag(exp(-exp(w_log))) S + k v^T    (q, k, w_log: [rows, heads, dk])
//   SCAN_HGRN2: f = l + (1 - l) sigmoid(z + b) per key channel; S = diag(f) S + (1 - f) v^T ; y = S^T silu(q)   (q, z: [rows, heads, dk]
//              raw projections; l, b: [heads, dk]; there is no key input: what the gate forgets is what it writes)
//   SCAN_GLA : alpha = sigmoid(z + b)^(1 / tau) per key channel; S = diag(alpha) S + k v^T ; y = S^T (q_scale q)   (q, k, z: [rows, heads, dk];
//              b: [heads, dk] in gate_bias)
enum { SCAN_SSD = 0, SCAN_RWKV = 1, SCAN_HGRN2 = 2, SCAN_GLA = 3 };
struct ScanArgs {
    int mode = SCAN_SSD;
    const float *q = nullptr, *k = nullptr, *v = nullptr; int64_t ldq = 0, ldk = 0, ldv = 0;
    const float* decay_in = nullptr; int64_t ldd = 0;  // SSD: dt_raw [rows, heads]; RWKV: w_log [rows, heads*dk]; HGRN2, GLA: z [rows, heads*dk]
    const float *gate_bias = nullptr, *gate_lower = nullptr;              // HGRN2 (GLA: gate_bias alone), [heads, dk]
    const float *dt_bias = nullptr, *a_log = nullptr, *skip = nullptr;  // SSD, [heads]
    const float* bonus = nullptr;                                         // RWKV, [heads, dk]
    float q_scale = 1.f, tau = 1.f;                                       // GLA
    float* state = nullptr;                                               // [slots][heads][dk][dv]
    float* y = nullptr; int64_t ldy = 0;                                  // [rows, heads*dv]
    int heads = 0, groups = 0, dk = 0, dv = 0;
    const SeqSeg* segs = nullptr; int nseg = 0;
};
int linear_scan_f32(const ScanArgs& a, cudaStream_t stream);

// ---- attention with unit-RMS q/k, query temperature, tanh soft-cap and a bucketed distance bias (attention_bias.cu) -----
enum { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_CHUNK = 2 };
struct BiasAttnArgs {
    float* q = nullptr; int64_t ldq = 0;          // [rows, H*dk]: normalised and scaled in place by attn_prepare
    const float* k = nullptr; int64_t ldk = 0;    // [rows, G*dk] projections of this call's rows
    const float* v = nullptr; int64_t ldv = 0;    // [rows, G*dv]
    float* kcache = nullptr; float* vcache = nullptr;  // [slots][G][Smax][dk] / [..][dv] fp32; the same pointer (dv <= dk): a cached row
                                                       // is the key and, with its first dv entries, the value
    float* out = nullptr; int64_t ldo = 0;        // [rows, H*dv]
    const float* rel = nullptr;                   // [buckets, H] learned bias; null: no bias
    const int32_t* bucket_of = nullptr;           // [Smax]: bias row of a distance (built on the host)
    int H = 0, G = 0, dk = 0, dv = 0, Smax = 0, rows = 0;
    float eps = 0.f, scale = 1.f, softcap = 0.f;  // softcap <= 0: none
    float temp_coef = 0.f, temp_every = 1.f;      // q *= 1 + coef * ln(floor((p + 1) / every) + 1)
    const int32_t* row_slot = nullptr; const int32_t* row_pos = nullptr;
    int64_t kv_row_stride = 0, kv_row_stride_v = 0;  // > 0: kcache / vcache are matrices [position][G * dk] / [position][G * dv] of the call's
                                                  // one slot (keys and values made for this call) with these pitches, not cache slabs
    const float* sink = nullptr;                  // [H] or null: exp(sink[h]) joins the softmax denominator (no key, no value)
    int sink_fixed = 0; float sink_value = 0.f;   // sink_fixed (with sink null): exp(sink_value) does, for every head
    int mask_kind = 0, mask_size = 0;             // MASK_* (the values of B2_MASK_*): row at position i sees j <= i (causal), and only i - j < size (window) or
                                                  // floor(i / size) == floor(j / size) (chunk)
    int mask_keep = 0;                            // MASK_WINDOW: positions j < mask_keep stay visible whatever their distance
    int Gv = 0;                                   // > 0: vcache holds Gv <= G value heads per slot and key head g reads value head g mod Gv
                                                  // (the maps of differential attention: G = maps * Gv key heads over one set of values)
    const float* head_gate = nullptr; int64_t ldg = 0;   // non-null ([rows, ldg], entry h): a head's output is multiplied by sigmoid(head_gate[r, h])
    float* partial = nullptr; int nsplit = 1;     // split-KV scratch [rows*H*nsplit*(dv+2)] when nsplit > 1
    int tile_rows = 0;                            // consecutive rows that share a slot (a prompt portion: its rows; a decode step: 1);
                                                  // 0: one warp per (row, head) without shared key/value tiles
};
int attn_prepare_f32(const BiasAttnArgs& a, cudaStream_t stream);  // q/k norms, temperature, cache append
int attn_bias_f32(const BiasAttnArgs& a, cudaStream_t stream);     // causal softmax attention of every row against its slot's cache

}  // namespace b2
