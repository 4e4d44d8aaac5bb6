// Internal structures shared by the translation units of liblumi_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "../../include/lumi_b200.h"

namespace lumi {

// ---- errors -----------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int32_t fail(int32_t code, const char* fmt, ...);

#define LUMI_CUDA(expr)                                                                            \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return ::lumi::fail(_e == cudaErrorMemoryAllocation ? LUMI_E_NOMEM : LUMI_E_CUDA,      \
                                "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

#define LUMI_TRY(expr)                    \
    do {                                  \
        int32_t _s = (expr);              \
        if (_s != LUMI_OK) return _s;     \
    } while (0)

// ---- configuration (ModelConfig of the reference, inference/src/model.rs:20-86) -----------------
struct Config {
    int d_model = 0, n_layers = 0, d_state = 0, expand = 0, n_heads = 0, n_groups = 0, vocab = 0, max_seq_len = 0;
    int attention_interval = 0, attn_n_heads = 16, attn_kv_heads = 4, attn_mlp_expand = 4;
    std::vector<int> attn_window_sizes, attention_layers;
    bool byte_level = false;
    int attn_mlp_dim = 0;        // extension: 0 = attn_mlp_expand * d_model
    float attn_rope_base = 0.f;  // extension: 0 = no rotary embedding in attention
    float eps = 1e-5f;           // the reference hard-codes 1e-5 (model.rs:97) and has no norm_eps key

    int d_inner() const { return expand * d_model; }
    int head_dim() const { return d_inner() / n_heads; }
    int bc() const { return n_groups * d_state; }
    int in_proj_out() const { return 2 * d_inner() + 2 * bc() + 3 * n_heads + n_heads * d_state / 2; }
    int attn_head_dim() const { return d_model / attn_n_heads; }
    int kv_dim() const { return attn_kv_heads * attn_head_dim(); }
    int mlp_dim() const { return attn_mlp_dim > 0 ? attn_mlp_dim : attn_mlp_expand * d_model; }
    bool is_attention_layer(int i) const;
    int n_attn_layers() const;
    int attn_window_size(int attn_idx) const {
        return attn_idx < (int)attn_window_sizes.size() ? attn_window_sizes[attn_idx] : 0;
    }
};
int32_t parse_config(const char* json, Config& out);

// ---- device tensors -----------------------------------------------------------------------------
struct DevTensor {
    void* p = nullptr;
    int dtype = LUMI_DTYPE_F32;
    int64_t rows = 0, cols = 0;   // rank-1 tensors: rows = 1
    size_t bytes = 0;
};

struct MambaW {
    const float* norm_g = nullptr;
    DevTensor in_proj, out_proj;
    const float *b_gamma = nullptr, *c_gamma = nullptr, *b_bias = nullptr, *c_bias = nullptr;
    const float *d_skip = nullptr, *dt_bias = nullptr, *h_init = nullptr;   // h_init may stay null (zeros)
};
struct AttnW {
    const float *attn_norm_g = nullptr, *mlp_norm_g = nullptr;
    DevTensor qkv, o, gate_up, down;     // q|k|v and gate|up rows concatenated at finalize
};
struct Layer {
    bool is_attn = false;
    int kind_idx = 0;     // index among the Mamba layers, or among the attention layers
    int window = 0;
    MambaW m;
    AttnW a;
};

}  // namespace lumi

struct lumi_model {
    lumi::Config cfg;
    int device = 0;
    bool finalized = false;
    int wdtype = -1;                                  // dtype of rank-2 tensors (all must agree)
    std::map<std::string, lumi::DevTensor> tensors;   // by name without the "item." prefix
    std::vector<void*> owned;                         // extra device allocations made at finalize
    std::vector<lumi::Layer> layers;
    lumi::DevTensor embedding;
    const float* final_norm_g = nullptr;
    int n_mamba = 0, n_attn = 0;
    int64_t weight_bytes = 0;                         // bytes of weights one decode step reads
};

namespace lumi {

// Device-resident control block read by the kernels of a step, so that a captured CUDA graph stays
// valid from call to call: the host rewrites these fields, not kernel arguments.
struct StepCtl {
    int32_t step;            // index of the token being generated (Philox counter, output row)
    int32_t status;          // 0 ok; kernels OR in LUMI_STATUS_* bits
    int32_t record;          // 1: write sampled tokens to out_tokens[step][b] and track eos
    int32_t want_dump;       // 1: copy logits to dump[step][b][:]
    float temperature;
    int32_t top_k;
    uint32_t seed_lo, seed_hi;
    uint32_t eos_id;
    int32_t ignore_eos;
    uint32_t* out_tokens;    // [n_new][batch]
    float* dump;             // [n_new][batch][vocab]
    int32_t batch;
    int32_t prompt_len;      // prefill: tokens per sequence still to come from `prompt`
    int32_t prompt_pos;      // next prompt position; >= prompt_len means "consume tok_cur"
    int32_t pad;
    const uint32_t* prompt;  // [prompt_len][batch]
};
enum { STATUS_BAD_TOKEN = 1, STATUS_KV_FULL = 2, STATUS_TIMEOUT = 4 };

struct GraphEntry {
    cudaGraphExec_t exec = nullptr;
    int64_t launches = 0;
};

}  // namespace lumi

namespace lumi { struct B1Layer; }

struct lumi_session {
    lumi_model* m = nullptr;
    int max_batch = 0, max_tokens_kv = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev2 = nullptr;
    // two-lane execution of large tensor-core batches: GEMM kernels of each lane on a high-priority
    // stream, state steps on a low-priority one
    cudaStream_t lane_hi[2] = {nullptr, nullptr}, lane_lo[2] = {nullptr, nullptr};
    cudaEvent_t lane_ev[2][2] = {{nullptr, nullptr}, {nullptr, nullptr}}, ev_fork = nullptr, ev_stagger = nullptr, ev_join[2] = {nullptr, nullptr};
    int opt_overlap = 0;              // minimum batch for two-lane execution (0 = never)
    size_t act_ld = 0;                // elements per row of the activation-half buffers
    int opt_chunked_prefill = 128;    // minimum prompt length for the chunked SSD prefill (0 = never)
    int opt_prefill_rows = 131072;    // token rows processed per chunked-prefill pass (workspace size)
    // chunked-prefill workspace (grow-only): residual rows, in_proj output, bf16 halves, BCNorm scales
    float *pf_x = nullptr, *pf_proj = nullptr, *pf_rb = nullptr, *pf_rc = nullptr;
    __nv_bfloat16 *pf_hi = nullptr, *pf_lo = nullptr;
    size_t pf_rows = 0;
    // options
    int opt_gemm = 0, opt_split = 1, opt_graph = 1, opt_pdl = 1, opt_mega = 0;
    // greedy head with the argmax fused behind the lm_head GEMV (batch <= 8): set by the caller of a step that wants
    // neither sampling nor the logits; per (row, CTA) partials
    bool fused_head = false;
    float* amax_val = nullptr;
    int* amax_idx = nullptr;
    int amax_stride = 0;
    // batch-1 persistent kernel
    bool b1_ok = false;
    lumi::B1Layer* b1_layers = nullptr;
    void* b1_grid_ctl = nullptr;
    float* b1_amax_val = nullptr;
    int* b1_amax_idx = nullptr;
    unsigned long long* b1_timing = nullptr;
    unsigned long long* b1_tagged = nullptr;   // xt | pt | yt
    uint32_t b1_epoch = 1;
    // state, per Mamba layer l: base + l * max_batch * per-sequence size
    float *h = nullptr, *xprev = nullptr, *bprev = nullptr, *cum = nullptr;
    // attention cache: pool of pages of kPageTokens tokens, [n_attn][pages][2][kv_heads][kPageTokens][head_dim]
    void* kv_pool = nullptr;           // element type follows the weights (fp32 or bf16)
    size_t kv_layer_bytes = 0;
    int32_t* page_table = nullptr;     // [max_batch][pages_per_seq]
    int32_t* kv_pos = nullptr;         // [max_batch] tokens consumed so far (absolute position)
    float* attn_part = nullptr;        // partial (max, sum, context) of attention contexts split over CTAs
    int32_t* attn_part_count = nullptr;
    int32_t* slot_buf = nullptr;       // [max_batch] slot list of a partial reset
    int32_t* row_len = nullptr;        // [max_batch] prompt lengths of a ragged prefill
    float* xlast = nullptr;            // [max_batch][d_model] residual rows at each sequence's last prompt token
    int pages_per_seq = 0;
    // activations
    float *x = nullptr, *proj = nullptr, *y32 = nullptr, *logits = nullptr;
    __nv_bfloat16 *act_hi = nullptr, *act_lo = nullptr;
    __nv_bfloat16 *xn_hi = nullptr, *xn_lo = nullptr;   // residual rows x the next norm's weights, bf16 halves [rows][d_model]
    float* ssq = nullptr;              // [rows][ssq_stride] partial sums of squares of the residual rows
    int ssq_stride = 0;
    uint32_t *tok_cur = nullptr;       // [max_batch] tokens the next step consumes
    int32_t *finished = nullptr, *out_len = nullptr;   // [max_batch]
    int32_t* gemm_counters = nullptr;  // [2][kGemmCounters] zeroed ints for the split-K GEMM (second half: second lane)
    float* gemm_scratch = nullptr;     // [2][kGemmScratchFloats] partial tiles of the split-K GEMM
    lumi::StepCtl* ctl = nullptr;      // device
    lumi::StepCtl* ctl_host = nullptr; // pinned mirror
    uint32_t* pin_tokens = nullptr;    // pinned staging [max_batch]
    // grow-only buffers for lumi_generate outputs
    uint32_t* gen_out = nullptr; size_t gen_out_cap = 0;
    uint32_t* prompt_dev = nullptr; size_t prompt_cap = 0;
    float* gen_dump = nullptr; size_t gen_dump_cap = 0;
    float* score_logits = nullptr; size_t score_logits_cap = 0;    // logits of a block of prefill rows (scoring)
    std::map<int64_t, lumi::GraphEntry> graphs;
    int64_t launches = 0;              // kernels enqueued outside graphs since last reset of the counter
    int64_t launches_per_step = 0;
};

namespace lumi {

constexpr int kPageTokens = 64;
constexpr int kGemmCounters = 4096;
constexpr size_t kGemmScratchFloats = (size_t)4 << 20;      // 16 MiB per lane

// ---- kernel launchers (kernels.cu) --------------------------------------------------------------
// All take the stream to enqueue on and return a cudaError_t from the launch.
struct GemvArgs {
    const float* A; int lda;         // [M][K] fp32
    const void* W; int w_dtype;      // [N][K]
    float* D; int ldd;               // [M][N]
    const float* R;                  // residual, same layout as D, or null
    const float* gamma;              // RMSNorm weight applied to rows of A first, or null
    int M, N, K;
    float eps;
    int act;                         // 0 none; 1: D = sigmoid(W_gate a) * (W_up a), W = [gate rows | up rows], N = rows of each
    int32_t* status = nullptr;       // device word that receives STATUS_TIMEOUT if a bounded wait gives up; may be null
    bool allow_preload = true;       // false: never the single-wave preloading kernel (the only GEMV with a device-side wait)
    // greedy head: per (batch row, CTA) the best (value, row) of the CTA's rows goes to amax_val / amax_idx
    // [M][amax_stride]; *amax_parts (host) receives the number of partials per row; D may then be null (no logits written)
    float* amax_val = nullptr;
    int* amax_idx = nullptr;
    int amax_stride = 0;
    int* amax_parts = nullptr;
};
cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t st);
cudaError_t launch_logprob(const float* logits, int B, int V, const uint32_t* targets, float* out, int out_stride, int out_col,
                           cudaStream_t st);
cudaError_t launch_logprob_rows(const float* logits, int rows, int V, const uint32_t* prompt, int batch_total, int T, int ts, int t0,
                                int b0, int row0, float* out, cudaStream_t st);
// Kernels of kernels.cu launched by the calling thread from now on carry (or not) the
// programmatic-dependent-launch attribute.
void set_launch_pdl(bool on);
bool launch_pdl_on();
// The same for the tensor-core GEMM launches alone (their set-up may overlap the predecessor's tail at batch sizes where
// an early start of the CUDA-core kernels does not pay).
void set_launch_pdl_gemm(bool on);
bool launch_pdl_gemm_on();

cudaError_t launch_embed(const void* emb, int dtype, const uint32_t* tok_cur, float* x, int B, int D, int vocab,
                         StepCtl* ctl, cudaStream_t st, const int32_t* row_len = nullptr);
// x[B][D] fp32 -> RMSNorm(gamma) -> bf16 hi (+ lo if lo != null); gamma null = plain split.
// ssq != null: hi / lo = x * gamma without the per-row scale, ssq[b * ssq_stride] = sum of x^2 (for a GEMM with a folded norm)
cudaError_t launch_norm_split(const float* x, const float* gamma, __nv_bfloat16* hi, __nv_bfloat16* lo, int B, int D,
                              float eps, cudaStream_t st, float* ssq = nullptr, int ssq_stride = 0);

struct SsmArgs {
    const float* proj; int ldp;      // [B][in_proj_out]
    const float *bg, *cg, *bb, *cb, *dskip, *dtb;
    float *h, *xprev, *bprev, *cum;  // this layer's slices
    float* y32;                      // [B][d_inner] fp32, or null
    __nv_bfloat16 *yhi, *ylo;        // [B][d_inner] bf16 halves, or null
    int B, H, P, N, G;
    float eps;
    // prompts of different lengths (null otherwise): sequences whose prompt has ended (ctl->prompt_pos >= row_len[b]
    // while the prefill runs) are left untouched
    const int32_t* row_len = nullptr;
    const StepCtl* ctl = nullptr;
};
cudaError_t launch_ssm_step(const SsmArgs& a, cudaStream_t st);
bool ssm_shape_supported(int P, int N);

cudaError_t launch_state_reset(float* h, float* xprev, float* bprev, float* cum, const float* h_init, const int32_t* slots,
                               int n_slots, int H, int P, int N, cudaStream_t st);

cudaError_t launch_sample(const float* logits, int B, int V, StepCtl* ctl, uint32_t* tok_cur, int32_t* finished,
                          int32_t* out_len, cudaStream_t st);
cudaError_t launch_advance_step(StepCtl* ctl, int32_t* kv_pos, int B, int sampled, cudaStream_t st, const int32_t* row_len = nullptr);
cudaError_t launch_capture_last(const float* x, float* xlast, const int32_t* row_len, const StepCtl* ctl, int B, int D, cudaStream_t st);
// greedy head, second stage for batch <= 8: argmax over the GEMV's partials, token bookkeeping, end-of-step bookkeeping
cudaError_t launch_head_finish(const float* amax_val, const int* amax_idx, int nparts, int stride, int B, StepCtl* ctl, uint32_t* tok_cur,
                               int32_t* finished, int32_t* out_len, int32_t* kv_pos, cudaStream_t st);

// ---- attention (attention.cu) ---------------------------------------------------------------------
struct AttnArgs {
    const float* qkv; int ldq;       // [B][d_model + 2 kv_dim] fp32 (q | k | v) of the current token
    void* pool;                      // this layer's page pool (fp32 or bf16 elements)
    int kv_is_f32;
    const int32_t* page_table; int pages_per_seq;
    const int32_t* pos;              // [B] absolute position of the current token
    float* ctx32;                    // [B][d_model] fp32 or null
    __nv_bfloat16 *chi, *clo;        // bf16 halves or null
    int B, n_heads, kv_heads, head_dim, window, max_tokens;
    float rope_base;
    StepCtl* ctl;
    // Batched prefill: B counts token rows, row r = sequence (b0 + r / rows_per_seq), position pos[sequence] + r % rows_per_seq;
    // the rows of a slice are appended to the cache by one launch (phase 1) and attend to it in a second one (phase 2).
    // Decode: rows_per_seq = 1, phase 0 (append, then attend, in one launch).
    int rows_per_seq = 1, b0 = 0, phase = 0;
    // decode only: room for the partial results of a context split over several CTAs — part: [B * kv_heads][16 slices]
    // [hpk * (head_dim + 2)] floats, part_count: [B * kv_heads] zeroed ints (left zero) — and the longest context of the
    // batch as far as the host knows it (bounds the number of slices); null / 0: one CTA per (row, KV head)
    float* part = nullptr;
    int32_t* part_count = nullptr;
    int max_ctx_hint = 0;
    const int32_t* row_len = nullptr;    // prompts of different lengths: rows at or past their sequence's prompt length are skipped (decode form: by the
                                         // step's prompt position; prompt slices: by the row's own position, and their output rows are zero)
    size_t pool_bytes = 0;               // size of this layer's page pool (bounds the tensor map of the tensor-core kernel); 0: not given
};
constexpr int kAttnPartSlices = 16;
constexpr int kAttnPartUnits = 296;        // (row, KV head) pairs below which a context is split over CTAs: two CTAs per SM (sizes the partial-result buffer)
cudaError_t launch_attention_decode(const AttnArgs& a, cudaStream_t st);
cudaError_t launch_kv_advance(int32_t* kv_pos, int b0, int nb, int by, cudaStream_t st, const int32_t* lens = nullptr, int t_abs0 = 0);


// ---- tcgen05 GEMM (gemm_tcgen05.cu) ---------------------------------------------------------------
// D[M][N] (+)= A[M][K] W[N][K]^T ; A as bf16 hi (+ lo) halves, W bf16, fp32 accumulate and output.
// epi: 0 store, 1 add to existing D (residual), 2 sigmoid-gate: D[m][n] = sigmoid(acc[n]) * acc[n + N] is NOT
// done here (see gate kernel).  status_word: device int that receives STATUS_TIMEOUT if a bounded wait gives up.
// RMSNorm folded around a tensor-core product.  Consumer side (ssq_in): the A rows hold x * gamma without the
// per-row scale; the kernel sums `ssq_parts` partial sums of x^2 per row (stride ssq_stride) and multiplies its
// accumulator rows by 1 / sqrt(sum * inv_k + eps).  Producer side (out_hi): beside D the kernel writes
// D * gamma_next as bf16 hi (+ lo) rows of width N and, per row, the sum of D^2 over each strip of 32 columns into
// ssq_out[row * ssq_stride + column / 32] (independent of the tile width, so results do not depend on the row
// count) — the next product's consumer side.  All null: plain product.
struct NormFuse {
    const float* ssq_in = nullptr;
    int ssq_parts = 0;
    int ssq_stride = 0;
    float inv_k = 0.f, eps = 0.f;
    const float* gamma_next = nullptr;
    __nv_bfloat16 *out_hi = nullptr, *out_lo = nullptr;
    float* ssq_out = nullptr;
};

struct GemmArgs {
    const __nv_bfloat16 *a_hi, *a_lo;   // [M][K]
    const __nv_bfloat16* w;             // [N][K]
    float* d; int ldd;
    int M, N, K;
    int accumulate;
    int32_t* status_word;               // may be null
    int32_t* tile_counters = nullptr;   // zeroed device ints for split-K (the kernel leaves them zero); null: no split-K
    int n_counters = 0;
    float* scratch = nullptr;           // partial tiles of the splits
    size_t scratch_floats = 0;
    uint64_t wait_limit_ns = 0;         // limit of every device-side wait (0 = the default, 0.5 s)
    int debug_skip_unit = -1;           // test hook: the producer stops before this work unit, so the consumers' waits run out
    NormFuse nf;                        // RMSNorm folded around the product (persistent kernel only)
};
int32_t launch_gemm_tcgen05(const GemmArgs& a, cudaStream_t st);   // returns LUMI_* status
void gemm_tcgen05_plan(const GemmArgs& a, int* width, int* splits);     // the tile width and K split that launch would take
int32_t gemm_tcgen05_init();                                        // resolves the driver entry point

// ---- batch-1 persistent decode kernel (decode_b1.cu) ---------------------------------------------
struct B1Layer {
    const void *in_proj, *out_proj;
    const float *norm_g, *bg, *cg, *bb, *cb, *dskip, *dtb;
    float *h, *xprev, *bprev, *cum;          // slot 0 of this layer's state
};
struct B1Args {
    const B1Layer* layers; int n_layers;
    const void* emb; const float* final_g;
    int vocab, D, DI, R, H, G, BC;
    float eps;
    unsigned long long *xt, *pt, *yt;        // epoch-tagged activations: [D], [R], [DI]
    uint32_t epoch_base;                     // epochs used by this launch start at epoch_base (+1 per layer, token, ...)
    float* logits;
    uint32_t* tok_cur;
    int32_t *finished, *out_len;
    StepCtl* ctl;
    void* grid_ctl;                          // 32 bytes of barrier counters, zeroed per launch
    float* amax_val; int* amax_idx;          // [grid] argmax partials
    int n_tokens;
    int head_mode;                           // 0: never run the lm_head; 1: at the last prompt position and every decode position
    int do_argmax;                           // 1: pick the greedy token on the device and advance the step counter
    unsigned long long* timing;              // optional: [2][n_layers][10] globaltimer stamps of the last token (CTA 0 and CTA 100)
};
bool decode_b1_supported(const Config& c, int n_attn, int device);
cudaError_t launch_decode_b1(const B1Args& a, int w_dtype, int device, cudaStream_t st);

// ---- chunked SSD prefill (prefill_ssd.cu) ----------------------------------------------------------
struct PrefillArgs {
    const float* proj; int ldp;              // [nb * ts][in_proj_out], row = sequence * ts + token
    const float *bg, *cg, *bb, *cb, *dskip, *dtb;
    float *h, *xprev, *bprev, *cum;          // this layer's state, slot 0
    float *rb, *rc;                          // [nb * ts] BCNorm scales (scratch)
    __nv_bfloat16 *yhi, *ylo;                // [nb * ts][d_inner] gated output halves
    int H, G, ts, nb, b0;                    // heads, groups, tokens per sequence in this launch, sequences, first slot
    float eps;
    int32_t* status = nullptr;               // device word that receives STATUS_TIMEOUT if the bounded wait gives up
    // prompts of different lengths: lens[slot] = prompt length of the sequence, t_abs0 = prompt position of this launch's first
    // token; a sequence takes min(ts, lens - t_abs0) tokens of the launch (none: its state is left alone).  null: all take ts
    const int32_t* lens = nullptr;
    int t_abs0 = 0;
};
bool prefill_ssd_supported(const Config& c);
cudaError_t launch_prefill_embed(const void* emb, int dtype, const uint32_t* prompt, float* x, int D, int vocab, int rows, int ts,
                                 int t_abs0, int b_abs0, int batch_total, StepCtl* ctl, cudaStream_t st, const int32_t* lens = nullptr);
cudaError_t launch_prefill_scan(const PrefillArgs& a, cudaStream_t st);
cudaError_t launch_gather_last(const float* xr, float* x, int D, int ts, int nb, int b0, cudaStream_t st, const int32_t* lens = nullptr, int t_abs0 = 0);

cudaError_t launch_gate_mul(const float* gu, int ld, float* out32, __nv_bfloat16* hi, __nv_bfloat16* lo, int B, int mlp,
                            cudaStream_t st);

}  // namespace lumi
