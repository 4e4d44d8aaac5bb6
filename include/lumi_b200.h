/*
 * lumi_b200 — C ABI of the B200 (sm_100a) implementation of lumi's token loop:
 * prompt prefill plus the per-token Mamba-3 / attention decode step, with sampling on the device.
 *
 * This header is the whole drop-in boundary.  The reference's inference crate has no plugin
 * interface; the seam it offers is the Rust API `NmModel::{load, init_states, forward_step}`
 * called by `generate` (inference/src/main.rs:86,118,124,169), realised on its GPU path by the
 * `*_metal` bridge functions (inference/src/metal_ssm.rs:135,251,341,431,589,628).  The style is
 * that of the reference's own CUDA FFI (training/src/native_ops.rs:4-213): `extern "C"` free
 * functions over plain pointers and 32/64-bit integers — with two deliberate differences: every
 * call returns a status (the reference returns void and aborts, training/csrc/cublas_ops.cu:23-35)
 * and all state lives in opaque handles with their own CUDA stream (no process globals).
 *
 * Rules that hold for every function:
 *   - returns LUMI_OK (0) or a negative LUMI_E_* code; never aborts, never throws;
 *   - after a failure, lumi_last_error() (calling thread) holds a message;
 *   - host buffers passed in are borrowed for the duration of the call only;
 *   - the library owns all device memory; the decode step allocates nothing after lumi_session_create()
 *     (grow-only work areas exist for lumi_generate's outputs, the batched prefill and lumi_score: they are
 *     sized by the first call that needs them and reused afterwards);
 *   - one handle is driven by one host thread at a time; handles on different devices are
 *     independent (one host thread or process per GPU; the path needs no collective);
 *   - there is no CPU fallback: without a CUDA device every call that needs one fails.
 */
#ifndef LUMI_B200_H
#define LUMI_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LUMI_OK              0
#define LUMI_E_INVALID      -1   /* bad argument (null handle, batch out of range, ...)          */
#define LUMI_E_CONFIG       -2   /* config.json missing a key / inconsistent dimensions          */
#define LUMI_E_TENSOR       -3   /* unknown / missing / duplicate tensor, wrong shape or dtype   */
#define LUMI_E_IO           -4   /* file cannot be read, malformed safetensors                   */
#define LUMI_E_NOMEM        -5   /* device or host allocation failed                             */
#define LUMI_E_CUDA         -6   /* CUDA runtime error (message carries cudaGetErrorString)      */
#define LUMI_E_TIMEOUT      -7   /* a bounded device-side wait gave up (kernel returned cleanly) */
#define LUMI_E_TOKEN        -8   /* token id >= vocab_size                                       */
#define LUMI_E_KV_FULL      -9   /* attention cache capacity (max_tokens_kv) exceeded            */
#define LUMI_E_UNSUPPORTED  -10  /* shape outside what the kernels were built for                */

#define LUMI_DTYPE_F32  0
#define LUMI_DTYPE_BF16 1

typedef struct lumi_model   lumi_model;
typedef struct lumi_session lumi_session;

/* Sampling, replacing inference/src/main.rs:142-148,197-209.
 * temperature <= 0: greedy argmax (lowest index wins ties).  Otherwise softmax(logits / temperature)
 * and the reference's walk over the cumulative distribution in vocabulary order (first index whose
 * cumulative sum >= r).  top_k > 0 keeps the k largest logits (ties towards the lower index) and
 * renormalises before the walk (extension; 0 = reference behaviour).  r comes from Philox4x32-10:
 * key = seed, counter = (step, sequence, 0, 0), first word, top 24 bits * 2^-24. */
typedef struct lumi_sampling {
    float    temperature;
    int32_t  top_k;
    uint64_t seed;
    uint32_t eos_id;
    int32_t  ignore_eos;      /* benchmark only: keep generating past eos */
} lumi_sampling;

typedef struct lumi_stats {
    int64_t prompt_tokens;    /* batch * prompt length                          */
    int64_t decode_tokens;    /* tokens produced by decode steps                */
    float   ms_prefill;       /* CUDA-event time on the session stream          */
    float   ms_decode;
    int64_t bytes_per_step;   /* algorithmic bytes of one decode step at this batch:
                                 weights once + per sequence (state read+write, KV)   */
    int64_t kernel_launches;  /* kernels of this library launched in the timed phases  */
    float   achieved_gbps;    /* bytes_per_step * decode steps / ms_decode, in GB/s (0 without decode steps) */
    int32_t waves;            /* resident batches the call ran through: always 1 here — a host that holds more
                                 sequences than a session runs them as several calls (waves) and adds the times */
} lumi_stats;

/* Message for the last failure on the calling thread ("" if none). */
const char* lumi_last_error(void);

/* ---- model lifecycle: replaces load_model + NmModel::load (inference/src/main.rs:72-89,
 *      inference/src/model.rs:643-728, 185-231, 469-489) -------------------------------------- */

/* Parses config.json text (same keys and defaults as ModelConfig, inference/src/model.rs:20-48;
 * unknown keys ignored; byte_level forces vocab_size 259; optional extensions attn_mlp_dim,
 * attn_rope_base) and binds the model to a device. */
int32_t lumi_model_create(const char* config_json, int32_t device_id, lumi_model** out);

/* One call per safetensors entry, name including the `item.` prefix.  dtype F32 or BF16; rank-2
 * tensors keep their stored width on the device, rank-1 tensors become fp32.  `ssm.h_init` may be
 * rank 2 [n_heads, d_state] or rank 1 [n_heads * d_state]. */
int32_t lumi_model_load_tensor(lumi_model* m, const char* name, int32_t dtype, const int64_t* shape,
                               int32_t rank, const void* host_data, uint64_t nbytes);

/* Convenience: reads a .safetensors file and calls lumi_model_load_tensor for each entry. */
int32_t lumi_model_load_safetensors(lumi_model* m, const char* path);

/* Checks that every tensor the config requires is present (b_bias / c_bias default to ones and
 * h_init to zeros, as inference/src/model.rs:209-214) and prepares kernel-side tables. */
int32_t lumi_model_finalize(lumi_model* m);

void    lumi_model_free(lumi_model* m);

/* Fills: d_model, n_layers, d_state, n_heads, head_dim, n_groups, vocab_size, n_mamba, n_attention,
 * in_proj_out, weights dtype (LUMI_DTYPE_*), weight bytes read per step — 12 int64 values. */
int32_t lumi_model_info(const lumi_model* m, int64_t* out12);

/* ---- sessions: replaces NmModel::init_states + LayerState (inference/src/model.rs:112-159,
 *      731-763) for `max_batch` independent sequences ----------------------------------------- */

/* Allocates SSM state (fp32, rank-1 factors for prev_bx), the attention cache for max_tokens_kv
 * tokens per sequence (element type of the weights: bf16 or fp32; ignored for models without attention
 * layers) and the decode step's scratch, then resets every slot. */
int32_t lumi_session_create(lumi_model* m, int32_t max_batch, int32_t max_tokens_kv, lumi_session** out);

/* h <- h_init broadcast over head_dim, prev_bx <- 0, cum_angle <- 0, cache emptied.
 * slots == NULL resets all. */
int32_t lumi_session_reset(lumi_session* s, const int32_t* slots, int32_t n_slots);

void    lumi_session_free(lumi_session* s);

/* Options (name, value):  "gemm" = 0 auto | 1 SIMT only | 2 tcgen05 only;
 *                         "split_activations" = 1 (default) feeds tensor-core GEMMs with bf16 hi+lo
 *                         halves of each fp32 activation, 0 rounds activations to bf16 once;
 *                         "graph" = 1 (default) replays the decode step as a CUDA graph;
 *                         "pdl" = 1 (default) launches the kernels of small batches with programmatic dependent
 *                         launch so each one requests its weights / state while its predecessors still run;
 *                         "chunked_prefill" = minimum prompt length (default 128, 0 = never) from which bf16
 *                         models (attention layers included, unless one has a sliding window) prefill with the
 *                         chunked SSD scan (chunk 64), attention over all rows of a slice and tensor-core GEMMs
 *                         over all prompt tokens instead of token by token (same state to rounding); "prefill_rows" =
 *                         token rows per pass of that path (default 131072; sets its workspace size: 41 KB per row);
 *                         "overlap" = minimum batch (default 0 = never) from which the tensor-core path runs two
 *                         lanes of sequences side by side on prioritised streams (measured neutral: the state
 *                         step needs its L1 and cannot share an SM with the 198 KB GEMM);
 *                         "megakernel" = 1 runs batch-1 calls on Mamba-only models (head_dim 32, d_state 64) as
 *                         one persistent cooperative kernel per call (default 0: measured slower than the
 *                         graph-replayed chain of dependent-launched kernels). */
int32_t lumi_session_set_option(lumi_session* s, const char* name, int64_t value);

/* ---- token loop: replaces NmModel::forward_step (inference/src/model.rs:766-801) and the
 *      generate loop (inference/src/main.rs:118-170) ------------------------------------------ */

/* Feeds tokens[batch][T] (row-major) through the model: position by position, exactly as the
 * reference prefills (main.rs:121-125), or by the batched path the "chunked_prefill" option describes
 * (same resulting state to rounding).  last_logits (may be NULL): [batch][vocab] fp32 of the final
 * position.  Sequences occupy slots 0..batch-1. */
int32_t lumi_prefill(lumi_session* s, const uint32_t* tokens, int32_t batch, int32_t T, float* last_logits);

/* The same for prompts of different lengths: tokens[batch][T_max] row-major, of which sequence b uses the first
 * lengths[b] (1 <= lengths[b] <= T_max; what is stored behind them is not looked at).  Each sequence goes through its
 * own tokens (the reference's prefill, inference/src/main.rs:121-125, once per sequence) and ends in the state a
 * lumi_prefill of its own tokens alone would leave; last_logits [batch][vocab] (may be NULL) are those of each
 * sequence's own last position.  Token by token, or, where the longest prompt qualifies for it, by the batched path of
 * the "chunked_prefill" option over the rectangle of the longest prompt (same state to rounding).  At most 1024
 * sequences per call. */
int32_t lumi_prefill_ragged(lumi_session* s, const uint32_t* tokens, const int32_t* lengths, int32_t batch, int32_t T_max,
                            float* last_logits);

/* One forward_step for each of `batch` sequences: consumes in_tokens[batch], writes the sampled /
 * argmax next token to out_tokens[batch] (may be NULL) and, if logits_out != NULL, the logits
 * [batch][vocab].  `step` indexes the Philox counter. */
int32_t lumi_decode_step(lumi_session* s, const uint32_t* in_tokens, int32_t batch, const lumi_sampling* sp,
                         int32_t step, uint32_t* out_tokens, float* logits_out);

/* The whole generate loop on the device with one host synchronisation: prefill prompts[batch][T],
 * then n_new tokens per sequence.  out_tokens[batch][n_new]; out_lens[batch] = tokens before eos
 * (n_new when ignore_eos).  logits_dump (may be NULL): [n_new][batch][vocab], the logits each
 * generated token was chosen from.  stats may be NULL. */
int32_t lumi_generate(lumi_session* s, const uint32_t* prompts, int32_t batch, int32_t T, int32_t n_new,
                      const lumi_sampling* sp, uint32_t* out_tokens, int32_t* out_lens,
                      float* logits_dump, lumi_stats* stats);

/* Device-resident decode loop for measurement: runs n_steps decode steps, each consuming the
 * previous step's greedy tokens, no host traffic.  ms_out: CUDA-event time on the session stream. */
int32_t lumi_decode_loop_device(lumi_session* s, int32_t batch, int32_t n_steps, float* ms_out,
                                int64_t* launches_out);

/* One decode step launched kernel by kernel with a CUDA event in front of every launch, for live
 * per-kernel timing.  Fills 8 entries each: milliseconds and launch counts by family —
 * 0 embedding, 1 RMSNorm to bf16, 2 in_proj, 3 Mamba state step, 4 out_proj, 5 attention block,
 * 6 final norm + lm_head, 7 sampling + bookkeeping.  Advances the sequences by one (greedy) token. */
int32_t lumi_profile_step(lumi_session* s, int32_t batch, float* ms_by_family, int64_t* launches_by_family);

/* Copies one sequence's Mamba state of one layer to host (any pointer may be NULL):
 * h [H][P][N], x_prev [H][P], b_prev [H][N] (prev_bx = x_prev (x) b_prev), cum_angle [H][N/2]. */
int32_t lumi_session_read_state(lumi_session* s, int32_t slot, int32_t layer, float* h, float* x_prev,
                                float* b_prev, float* cum_angle);

/* Runs block `layer` alone on a caller-supplied residual stream x[batch][d_model] (host, in/out),
 * using and updating the session state — for per-layer parity tests. */
int32_t lumi_debug_run_block(lumi_session* s, int32_t layer, float* x, int32_t batch);

/* Teacher-forced scoring for the reference's `evaluate` command (inference/src/eval.rs:39-139: perplexity and
 * continuation scores from log-softmax over forward_window's logits, model.rs:806-826):
 * logprobs_out[b][t] = log p(tokens[b][t+1] | tokens[b][0..t]), t = 0 .. T-2 (row stride T-1), natural log.
 * tokens[batch][T] row-major as for lumi_prefill; afterwards the state is that of a prefill of all T tokens. */
int32_t lumi_score(lumi_session* s, const uint32_t* tokens, int32_t batch, int32_t T, float* logprobs_out);

/* ---- sequence snapshots: park a sequence on the host and resume it later, in any slot of any session of
 * the same model (slot reuse when a sequence ends, resuming a long generation).  The state is what
 * inference/src/model.rs:112-159 keeps per sequence (SsmState, KvCache); the reference has no call that
 * saves it.  A snapshot holds, for one slot: h, x_prev, B_prev and the cumulative angles of every Mamba
 * layer, the K/V pages and the position of every attention layer.  The token that the next step consumes
 * is NOT part of it (the caller feeds tokens to lumi_decode_step).
 * lumi_session_state_bytes: size of one snapshot for this session's model and max_tokens_kv.
 * save/load synchronise the session's stream; load checks the header written by save (LUMI_E_TENSOR on
 * a snapshot of another model or cache size). */
int32_t lumi_session_state_bytes(const lumi_session* s, int64_t* bytes);
int32_t lumi_session_save_state(lumi_session* s, int32_t slot, void* host_buf, int64_t nbytes);
int32_t lumi_session_load_state(lumi_session* s, int32_t slot, const void* host_buf, int64_t nbytes);

/* ---- single kernels over caller-owned DEVICE pointers (tests, profiling) -------------------- */

/* D[M][N] (fp32, row-major, leading dimension ldd) = A[M][K] * W[N][K]^T (+ D if accumulate != 0),
 * A given as bf16 hi (and optional lo, may be 0) halves, W bf16, K % 64 == 0.  tcgen05 + TMA.
 * stream: cudaStream_t as integer (0 = default stream). */
int32_t lumi_k_gemm_bf16_tcgen05(uint64_t a_hi, uint64_t a_lo, uint64_t w, uint64_t d, int32_t M, int32_t N,
                                 int32_t K, int32_t ldd, int32_t accumulate, uint64_t stream);

/* Failure-path test hook for the bounded device-side waits (no counterpart in the reference, whose kernels never wait
 * on one another): runs the same GEMM with activations a_hi only, every device-side wait limited to wait_limit_ns, and
 * the producer stopping before work unit `skip_unit` (units are 128-row x tile-width output tiles in launch order;
 * -1 = none), so that the waits of the consumers run out.  status_word: a zeroed device int32.  Returns LUMI_E_TIMEOUT
 * when a wait gave up — the kernel has then returned cleanly (copies drained, tensor memory freed) and further calls
 * work — or LUMI_OK when nothing was skipped.  Synchronises the default stream. */
int32_t lumi_debug_gemm_wait_timeout(uint64_t a_hi, uint64_t w, uint64_t d, int32_t M, int32_t N, int32_t K,
                                     uint64_t wait_limit_ns, int32_t skip_unit, uint64_t status_word);

/* Host-side only (no device is touched, nothing is launched; no counterpart in the reference): the output-tile width and
 * the number of CTAs K is split over that lumi_k_gemm_bf16_tcgen05 and the decode / prefill steps take for a product of
 * this shape.  two_planes: activations as bf16 hi + lo halves; producer: the epilogue also leaves the next RMSNorm's
 * input (tile widths are then multiples of 32).  For tests of the choice and for reading profiles. */
int32_t lumi_debug_gemm_plan(int32_t M, int32_t N, int32_t K, int32_t two_planes, int32_t producer, int32_t* width,
                             int32_t* splits);

/* Same contraction on CUDA cores with fp32 activations: D[M][N] = A[M][K] * W[N][K]^T (+ residual R).
 * w_dtype LUMI_DTYPE_*.  norm_gamma != 0 applies RMSNorm(gamma) to each row of A first. */
int32_t lumi_k_gemv(uint64_t a_f32, uint64_t w, int32_t w_dtype, uint64_t d, uint64_t residual,
                    uint64_t norm_gamma, int32_t M, int32_t N, int32_t K, uint64_t stream);

/* The fused Mamba-3 state step alone (inference/src/model.rs:301-370 after in_proj, before
 * out_proj): proj[B][ldp] holds in_proj's output rows; h[B][H][P][N], x_prev[B][H][P],
 * b_prev[B][H][N], cum_angle[B][H][N/2] are updated in place; y[B][H*P] receives the gated output. */
int32_t lumi_k_ssm_step(uint64_t proj, int32_t ldp, uint64_t b_gamma, uint64_t c_gamma, uint64_t b_bias, uint64_t c_bias,
                        uint64_t d_skip, uint64_t dt_bias, uint64_t h, uint64_t x_prev, uint64_t b_prev, uint64_t cum_angle,
                        uint64_t y, int32_t B, int32_t H, int32_t P, int32_t N, int32_t G, uint64_t stream);

/* The chunked prefill scan alone (chunk length 64; head_dim 32, d_state 64): the same recurrence as lumi_k_ssm_step
 * over `ts` consecutive tokens of each of `nb` sequences at once — what replaces `ts` sequential forward_step calls
 * (inference/src/main.rs:121-125) and what the reference's sequential CUDA scan computes for its trainer
 * (training/csrc/ssm_scan.cu:71-229, host entry :773).  proj[nb * ts][ldp]: in_proj output rows, row = sequence * ts +
 * token.  State arrays as for lumi_k_ssm_step (slot = sequence), updated in place to the state after the last token.
 * y_hi / y_lo [nb * ts][H * 32]: the gated output as bf16 hi + lo halves (y_lo may be 0).  scratch: 2 * nb * ts floats. */
int32_t lumi_k_ssd_prefill(uint64_t proj, int32_t ldp, uint64_t b_gamma, uint64_t c_gamma, uint64_t b_bias, uint64_t c_bias,
                           uint64_t d_skip, uint64_t dt_bias, uint64_t h, uint64_t x_prev, uint64_t b_prev, uint64_t cum_angle,
                           uint64_t y_hi, uint64_t y_lo, uint64_t scratch, int32_t nb, int32_t ts, int32_t H, int32_t G,
                           uint64_t stream);

/* One Mamba block (RMSNorm -> in_proj -> state step -> out_proj + residual, inference/src/model.rs:296-375
 * in arithmetic) WITHOUT any allocation.  This entry point has no counterpart in the reference.
 *
 * For hosts that cannot call cudaMalloc where they need the block: a process whose own memory pool
 * already holds the whole GPU, code inside a stream capture, or a loop that must not take the
 * device-wide synchronisation an allocation brings.  Such a host cannot create a lumi_session either,
 * since that allocates.  Here the caller passes every input and output as device pointers —
 * x[batch][d_model] fp32 (in/out, the residual stream) and this layer's state for `batch` sequences:
 * h[batch][H][P][N], x_prev[batch][H][P], b_prev[batch][H][N], cum_angle[batch][H][N/2] (all updated in
 * place; a fresh sequence has h = h_init broadcast over P and zeros elsewhere) — and the block's two
 * intermediates live in a fixed 512 KiB array inside the library's device image (held by every GPU
 * that loads the library, until the process exits).
 *
 * Limits: batch <= 8 and in_proj_out + d_inner <= 16384 floats; anything larger is refused with
 * LUMI_E_UNSUPPORTED.  The weights come from `m` (loaded and finalized earlier).  No cudaMalloc,
 * cudaFree or other allocating call is made.  The first call on a device looks up the array's
 * device address (cudaGetSymbolAddress, with that device current) and keeps it: make that first
 * call before any stream capture begins — with the same batch size and the same model as the calls
 * that follow, because the batch size (1, 2, 3-4 or 5-8) and the weight type select the kernels, and a
 * kernel's code is loaded at its first launch.  The call makes the model's device current
 * (cudaSetDevice) and leaves it so.  It enqueues three kernels on `stream` and returns without
 * synchronising; none of them waits on anything on the device, so there is no device-side failure it
 * would have to report later.  All calls on a device share the one array, which keeps
 * whatever the last call left in it; nothing in it needs clearing (every element is written
 * before it is read), but two calls whose kernels overlap on the GPU — different streams, or the same
 * stream from different threads — race on it: serialise them. */
int32_t lumi_mamba_block_static(lumi_model* m, int32_t layer, uint64_t x, uint64_t h, uint64_t x_prev, uint64_t b_prev,
                                uint64_t cum_angle, int32_t batch, uint64_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LUMI_B200_H */
