/* fm_attn.h -- C-ABI of the Blackwell (sm_100a) attention hot path of Flash-MoE.
 *
 * The reference engine has no plugin/FFI layer for this path: attention and
 * GatedDeltaNet are inline Metal encoder sequences inside
 * fused_layer_forward() and batched_prefill().  What a caller binds there is
 * (i) the argument lists of the Metal kernels, (ii) the KVCache /
 * LinearAttnState structs and the MetalCtx buffers that back them.  Each entry
 * point below replaces one such group and cites it.  All citations are paths
 * inside the reference project.
 *
 * Conventions
 *   - Every call returns fm_status; fm_last_error() gives the text (the
 *     reference prints "ERROR: ..." to stderr and returns early; this library
 *     prints nothing and changes no state on error).
 *   - Tensors are fp32 unless noted, row-major, with the reference's layouts:
 *       q_proj_out [n][H][2*D]   per head [q(D) | gate(D)]   (layer_forward.h:537-541)
 *       q, gate, out [n][H*D];  k, v [n][Hkv*D]
 *       qkv [n][2*Hk*dk + Hv*dv] = q | k | v                 (layer_forward.h:907-909)
 *       z, out [n][Hv*dv];  beta, alpha [n][Hv]
 *       norm / conv / dt_bias weights are bf16 bit patterns (uint16_t).
 *   - Data pointers are DEVICE pointers by default; fm_set_pointer_mode(ctx,
 *     FM_PTR_HOST) makes every data pointer a host pointer (the reference passes
 *     host floats because Apple memory is unified); the library then stages
 *     through its own pinned buffers.  seq[] / pos[] index arrays are always
 *     host arrays.
 *   - Work is queued on the context's stream (fm_set_stream; default: the
 *     legacy default stream).  In host-pointer mode calls return after the
 *     outputs have landed in the caller's buffers.
 *   - A context is not re-entrant (one inference thread), like the reference.
 */
#ifndef FM_ATTN_H
#define FM_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fm_status {
    FM_OK = 0,
    FM_ERR_INVALID = 1,     /* bad argument, nothing done */
    FM_ERR_CAPACITY = 2,    /* KV cache overflow: sequence full or page pool exhausted */
    FM_ERR_NOMEM = 3,       /* device / host allocation failed */
    FM_ERR_CUDA = 4,        /* a CUDA call failed; text in fm_last_error */
    FM_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up */
    FM_ERR_UNSUPPORTED = 6  /* shape outside what the kernels are built for */
} fm_status;

enum { FM_PTR_DEVICE = 0, FM_PTR_HOST = 1 };

/* Element type of the KV store (FmConfig.kv_dtype). */
enum { FM_KV_BF16 = 0, FM_KV_FP8_E4M3 = 1 };

/* Plain-data configuration; replaces the ModelConfig fields this path reads
 * (metal_infer/config.h:9-75) and the feature globals set before metal_setup()
 * (metal_infer/timing.h:82-111).  Head counts are those HELD BY THIS CONTEXT:
 * a head-sharded deployment creates one context per GPU with its share. */
typedef struct FmConfig {
    /* gated GQA full attention */
    int num_attn_heads;      /* query heads (32) */
    int num_kv_heads;        /* KV heads (2) */
    int head_dim;            /* 256 (the kernels are built for 256) */
    int rotary_dim;          /* leading dims that rotate (64); pairs (i, i+rotary_dim/2) */
    float rope_theta;        /* 1e7 */
    float rms_norm_eps;      /* eps of q/k norm and of the GatedDeltaNet output norm */
    int rope_scaling_mode;   /* 0 none, 1 linear, 2 NTK, 3 YaRN (layer_forward.h:22-70) */
    float rope_scale_factor; /* 1.0 */
    int rope_orig_max_pos;   /* original context length used by YaRN's wavelength bounds */
    int num_full_layers;     /* full-attention layers held (15) */
    /* GatedDeltaNet */
    int linear_num_v_heads;  /* 64 */
    int linear_num_k_heads;  /* 16; v head vh reads k head vh / (Hv/Hk) */
    int linear_key_dim;      /* 128 (kernels are built for 128) */
    int linear_value_dim;    /* 128 */
    int conv_kernel_size;    /* 4 */
    int num_linear_layers;   /* GatedDeltaNet layers held (45) */
    /* capacity */
    int max_seqs;            /* concurrent sequences (the reference has 1) */
    int max_seq_len;         /* positions per sequence (global, before sequence sharding) */
    int page_size;           /* positions per KV page; 64 */
    int64_t kv_pool_pages;   /* pages in the shared pool; 0 = enough for every sequence at max_seq_len */
    int max_batch_tokens;    /* largest n of a prefill call / batch of a decode call */
    /* sequence sharding of the KV store: page p of a sequence lives on the
     * context with seq_shard_rank == p % seq_shard_count */
    int seq_shard_rank;      /* 0 */
    int seq_shard_count;     /* 1 */
    int device;              /* CUDA device ordinal */
    /* long-context policy of the KV store (decode): 0 = keep every position; W > 0 = sliding window,
     * the store of a sequence is a circular buffer of W rows -- the token count keeps growing, row
     * count % W is overwritten, attention sees the last min(count, W) tokens
     * (g_sliding_window / KVCache.window_size: layer_forward.h:130-131,148-161,600-601,649-650,673-677) */
    int sliding_window;
    /* FM_KV_BF16 (default): rows are stored as bf16.  FM_KV_FP8_E4M3: rows are stored as E4M3 bytes with one
     * scale per position and tensor (K, V), scale = absmax over the row / 240, the reference's FP8 cache
     * (g_use_fp8_kv; metal_infer/fp8.h:19-118, KVCache fields metal_infer/layer_forward.h:124-127, append
     * :609-616, CPU attention :679-712, Metal kernels metal_infer/shaders.metal:1067-1143,1320-1430).  The
     * bytes and scales are the reference's, quirks of its encoder included, so a row decodes to what its CPU
     * attention would have read.  The absmax runs over the KV heads THIS CONTEXT holds (all of them on one
     * GPU, as in the reference).  Half the bytes per row of bf16. */
    int kv_dtype;
    /* Heavy-hitter eviction (H2O) of the KV store at decode: h2o_budget > 0 keeps at most that many rows per
     * (layer, sequence) -- the first h2o_num_sinks tokens, the last (budget - sinks) / 4 tokens and, of the rest,
     * those with the largest attention mass accumulated over the steps (softmax weight summed over the query heads).
     * A step appends its row, attends over budget + 1 rows at most, adds the step's mass and, past the budget, drops
     * the lightest unprotected row (g_h2o_budget / g_h2o_num_sinks; KVCache fields metal_infer/layer_forward.h:132-140,
     * kv_cache_h2o_accumulate_scores / kv_cache_evict_h2o :248-383, use in the step :591-727).  It replaces a sliding
     * window when both are set, as in the reference.  Decode only (the reference's batched prefill ignores it too:
     * metal_infer/batched_prefill.h:736); not with sequence sharding. */
    int h2o_budget;
    int h2o_num_sinks;       /* 4 in the reference */
} FmConfig;

typedef struct FmCtx FmCtx;

/* Fills *cfg with the Qwen3.5-397B shapes (32/2 heads x 256, rotary 64, theta 1e7; 64/16 heads x
 * 128, conv 4; 15 + 45 layers), one sequence, 8192 positions. */
void fm_default_config(FmConfig *cfg);

/* Allocates the KV page pool, page tables, recurrent state and staging buffers.
 * Replaces metal_setup()'s buf_kv_k/v, buf_attn_*, buf_delta_state, buf_conv_state
 * (metal_infer/metal_ctx.h:94-130,460-526) and kv_cache_new / linear_attn_state_new
 * (metal_infer/layer_forward.h:143-236,419-424).  State starts zeroed. */
fm_status fm_create(const FmConfig *cfg, FmCtx **out);
void fm_destroy(FmCtx *ctx);

/* Text of the last error on this context (ctx == NULL: last fm_create failure).
 * Mirrors flashmoe_last_error (FlashMoE-iOS/FlashMoEEngine/FlashMoEEngine.h:150-151). */
const char *fm_last_error(const FmCtx *ctx);

fm_status fm_set_stream(FmCtx *ctx, void *cuda_stream);
fm_status fm_set_pointer_mode(FmCtx *ctx, int mode);
fm_status fm_synchronize(FmCtx *ctx);

/* Forget a sequence (seq = -1: all): KV length 0, pages back to the pool, conv and recurrent
 * state zeroed.  Replaces reset_delta_net_state (metal_infer/metal_ctx.h:599-608) plus kv->len = 0
 * (FlashMoE-iOS/FlashMoEEngine/FlashMoEEngine.m:1239-1258). */
fm_status fm_reset(FmCtx *ctx, int seq);

/* Sequence `dst` becomes a copy of `src` (it is reset first): the reference's system-prompt cache
 * saves every layer's KV rows and recurrent state after the prompt and copies them back for each
 * request (metal_infer/generate.h:708-764, 887-947).  In the paged store the full pages of `src` are
 * shared by reference -- appends never touch a full page, so no copy is ever needed for them -- and
 * only the partly filled last page of each layer and the GatedDeltaNet state are copied.  Resetting
 * either sequence leaves the other intact.  Not available with a sliding window (pages are
 * rewritten in place).  With sequence sharding every rank calls it. */
fm_status fm_seq_fork(FmCtx *ctx, int src, int dst);

/* Pages of the KV pool not held by any sequence. */
int64_t fm_kv_free_pages(const FmCtx *ctx);

/* Rows held for (layer, sequence) -- KVCache.len (metal_infer/layer_forward.h:128). */
int fm_kv_len(const FmCtx *ctx, int fa_idx, int seq);

/* k RMS-norm (k_norm_w may be NULL) + partial RoPE at pos[i] + append of token i to sequence
 * seq[i]; cache row = the sequence's current length, which then grows by one.  K and V are stored
 * as bf16.  Replaces layer_forward.h:574-629 (CPU) and the Metal kernel prefill_kv_cache_bf16
 * (metal_infer/shaders.metal:2405-2482).  FM_ERR_CAPACITY on overflow, with nothing appended. */
fm_status fm_kv_append_rope(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int n,
                            const float *k, const float *v, const uint16_t *k_norm_w);

/* One decode step for `batch` sequences: q RMS-norm (q_norm_w may be NULL) + RoPE, append of the
 * new k, v (skipped if k == NULL: caller already appended), softmax(q K^T / sqrt(D)) V over the
 * whole sequence including the new row, times sigmoid(gate).
 * Give either q_proj_out (interleaved) or q and gate.
 * Replaces layer_forward.h:556-735 (CPU) and the Metal kernels attn_scores_batched /
 * attn_softmax_batched / attn_values_batched / fused_attention_online / sigmoid_gate
 * (metal_infer/shaders.metal:899-1040,1151-1313; dispatch layer_forward.h:3175-3367). */
fm_status fm_attn_decode(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                         const float *q_proj_out, const float *q, const float *gate,
                         const float *k, const float *v, const uint16_t *q_norm_w,
                         const uint16_t *k_norm_w, float *out);

/* The same step on a sequence-sharded store: attends over the rows this context holds and returns
 * the un-normalised partial result, o_part [batch][H][D] and ml_part [batch][H][2] = (running max
 * in log2 units, sum of weights).  The new k, v are appended only where this context owns the
 * row's page.  No reference counterpart (the reference is single-device). */
fm_status fm_attn_decode_partial(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                                 const float *q_proj_out, const float *q, const float *k,
                                 const float *v, const uint16_t *q_norm_w,
                                 const uint16_t *k_norm_w, float *o_part, float *ml_part);

/* Log-sum-exp merge of nparts partial results ([nparts][batch][H][D] and [nparts][batch][H][2])
 * followed by the sigmoid gate (gate [batch][H*D], or q_proj_out interleaved). */
fm_status fm_attn_merge_gate(FmCtx *ctx, int nparts, const float *o_parts, const float *ml_parts,
                             const float *q_proj_out, const float *gate, int batch, float *out);

/* The sequence-sharded decode step with the exchange done by this library over peer memory (plain
 * stores over NVLink into buffers that the ranks of a sequence group have mapped for each other --
 * e.g. CUDA IPC or symmetric memory -- no collective call on the path).  No reference counterpart.
 *   fm_exchange_bytes   size of the buffer every rank must provide (nranks <= 8)
 *   fm_exchange_attach  peer_bufs[r] = rank r's buffer as addressable from this GPU; peer_bufs[my_index]
 *                       is the local one and is zeroed here.  All ranks attach before the first step.
 *   ..._exchange_push   the partial step (as fm_attn_decode_partial), then each (token, head) partial is
 *                       stored into every rank's buffer and the step number published to every rank
 *   ..._exchange_merge  waits until every rank has published the step -- for about half a second at
 *                       most: FM_ERR_TIMEOUT, reported at the next synchronising call, with zeros in
 *                       `out`, and the context stays usable -- then merges by log-sum-exp and applies
 *                       the gate (gate, or q_proj_out interleaved)
 *   fm_attn_decode_exchange  push + merge.
 * All ranks of the group call these in lockstep (same number of steps); batch <= 64. */
size_t fm_exchange_bytes(const FmCtx *ctx, int nranks);
fm_status fm_exchange_attach(FmCtx *ctx, int nranks, int my_index, void *const *peer_bufs);
fm_status fm_attn_decode_exchange_push(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                                       const float *q_proj_out, const float *q, const float *k,
                                       const float *v, const uint16_t *q_norm_w,
                                       const uint16_t *k_norm_w);
fm_status fm_attn_decode_exchange_merge(FmCtx *ctx, int batch, const float *q_proj_out,
                                        const float *gate, float *out);
fm_status fm_attn_decode_exchange(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                                  const float *q_proj_out, const float *q, const float *gate,
                                  const float *k, const float *v, const uint16_t *q_norm_w,
                                  const uint16_t *k_norm_w, float *out);

/* One token of `batch` sequences through n_layers consecutive full-attention layers: the layer loop
 * of the reference's generation loop (metal_infer/generate.h:2187-2250, one fused_layer_forward per
 * layer) for hosts that have every layer's projections at hand.  Layer first_layer + l reads
 * q_proj_out + l * layer_stride_q (interleaved q | gate), k and v + l * layer_stride_kv, and writes
 * out + l * layer_stride_out (strides in floats).  exchange != 0 runs each layer through
 * fm_attn_decode_exchange (sequence-sharded store), else through fm_attn_decode. */
fm_status fm_attn_decode_layers(FmCtx *ctx, int first_layer, int n_layers, const int *seq, const int *pos,
                                int batch, const float *q_proj_out, size_t layer_stride_q, const float *k,
                                const float *v, size_t layer_stride_kv, const uint16_t *q_norm_w,
                                const uint16_t *k_norm_w, float *out, size_t layer_stride_out,
                                int exchange);

/* Causal prefill of n tokens of one sequence at positions start_pos..: q norm + RoPE, k norm +
 * RoPE + append, token t attends to rows [0, len_before + t], times sigmoid(gate).
 * Replaces batched_prefill.h:543-740 and the Metal kernels prefill_q_rope_norm_bf16 /
 * prefill_kv_cache_bf16 / prefill_causal_attn (metal_infer/shaders.metal:2228-2482). */
fm_status fm_attn_prefill(FmCtx *ctx, int fa_idx, int seq, int start_pos, int n,
                          const float *q_proj_out, const float *q, const float *gate,
                          const float *k, const float *v, const uint16_t *q_norm_w,
                          const uint16_t *k_norm_w, float *out);

/* One GatedDeltaNet step for `batch` sequences: depthwise causal conv + SiLU, conv-state shift,
 * q/k normalise, decay and beta, delta-rule update of the [Hv][dv][dk] fp32 state, gated RMS-norm.
 * A_log / dt_bias / norm_w may be NULL with the reference's meaning (A = 1, bias 0, no norm).
 * Replaces layer_forward.h:886-1025 (CPU) and the Metal kernels conv1d_step / rms_norm_qk /
 * compute_decay_beta / gated_delta_net_step(_fused) / gated_rms_norm
 * (metal_infer/shaders.metal:1591-1850; dispatch layer_forward.h:2114-2214). */
fm_status fm_gdn_decode(FmCtx *ctx, int li, const int *seq, int batch, const float *qkv,
                        const float *z, const float *beta, const float *alpha,
                        const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                        const uint16_t *norm_w, float *out);

/* n tokens of one sequence through the GatedDeltaNet layer in chunked form; output and final state
 * equal n sequential fm_gdn_decode steps.  chunk = 0 picks the default (64).
 * Replaces batched_prefill.h:798-1037 and the Metal kernels conv1d_step_batched /
 * rms_norm_qk_batched / compute_decay_beta_batched / gated_delta_net_step_batched /
 * gated_rms_norm_batched (metal_infer/shaders.metal:2639-2860). */
fm_status fm_gdn_prefill(FmCtx *ctx, int li, int seq, int n, int chunk, const float *qkv,
                         const float *z, const float *beta, const float *alpha,
                         const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                         const uint16_t *norm_w, float *out);

/* Snapshot / restore in the reference's fp32 layouts: k, v [len][Hkv*D] (KVCache.k_cache/v_cache,
 * layer_forward.h:121-123), conv [(ks-1)][conv_dim], ssm [Hv][dv][dk] (layer_forward.h:414-417).
 * Replaces the system-prompt snapshot/restore of metal_infer/generate.h:710-764,897-939.
 * On a sequence-sharded store export/import touch the rows this context owns (other rows of the
 * caller's arrays are left alone / ignored).  Pointers follow the pointer mode. */
fm_status fm_kv_export(FmCtx *ctx, int fa_idx, int seq, float *k, float *v, int max_rows, int *len_out);
fm_status fm_kv_import(FmCtx *ctx, int fa_idx, int seq, const float *k, const float *v, int len);
/* FP8 store only: the stored bytes and scales themselves, k8 / v8 [len][Hkv*D] E4M3 bytes and k_scales /
 * v_scales [len] -- KVCache.k_cache_fp8 / v_cache_fp8 / k_scales / v_scales (metal_infer/layer_forward.h:124-127),
 * what the reference's snapshot copies for an FP8 cache.  Unlike the fp32 pair above (which decodes on export
 * and quantises again on import) this round trip is exact. */
fm_status fm_kv_export_fp8(FmCtx *ctx, int fa_idx, int seq, uint8_t *k8, uint8_t *v8, float *k_scales, float *v_scales,
                           int max_rows, int *len_out);
fm_status fm_kv_import_fp8(FmCtx *ctx, int fa_idx, int seq, const uint8_t *k8, const uint8_t *v8, const float *k_scales,
                           const float *v_scales, int len);
/* H2O bookkeeping of (layer, sequence) in the cache's row order (the order fm_kv_export uses): accum [n] accumulated
 * attention mass (KVCache.attn_scores_accum), token_positions [n] original token index of each kept row
 * (KVCache.token_positions); *n_out = rows kept.  Pointers follow the pointer mode. */
fm_status fm_h2o_export(FmCtx *ctx, int fa_idx, int seq, float *accum, int *token_positions, int max_rows, int *n_out);
fm_status fm_state_export(FmCtx *ctx, int li, int seq, float *conv, float *ssm);
fm_status fm_state_import(FmCtx *ctx, int li, int seq, const float *conv, const float *ssm);

/* The step behind token mixing: output projection + residual + post-attention RMS-norm, i.e. what the reference
 * encodes after attention in fused_layer_forward (metal_infer/layer_forward.h:3369-3450): o_proj / out_proj as a
 * 4-bit dequantising matvec (cpu_dequant_matvec, metal_infer/cpu_kernels.h:199-232; Metal dequant_matvec_4bit*),
 * residual_add, rms_norm_sum_sq, rms_norm_apply_bf16 (metal_infer/shaders.metal:792-882):
 *     y = W x;   h_mid = residual + y;   h_post = h_mid * rsqrt(mean(h_mid^2) + rms_norm_eps) * norm_w
 * Weights in the reference's format: w uint32 [out_dim][in_dim / 8], eight 4-bit values per word, lowest nibble
 * first; scales, biases bf16 [out_dim][in_dim / group_size], weight = nibble * scale + bias; group_size 64.
 * Weight pointers are DEVICE pointers in either pointer mode (fm_proj_upload copies a host set to the device once);
 * x [n][in_dim], residual [n][out_dim] (may be NULL), norm_w bf16 [out_dim] (may be NULL: weight 1), h_mid and
 * h_post [n][out_dim] (h_post may be NULL) follow the pointer mode.  in_dim a multiple of 512, out_dim of 4. */
enum { FM_W_Q4_AFFINE = 0 };
typedef struct FmProjWeights {
    int format;              /* FM_W_Q4_AFFINE */
    int out_dim, in_dim;     /* 4096 x 8192 for both o_proj and out_proj of the 397B model */
    int group_size;          /* 64 */
    const uint32_t *w;
    const uint16_t *scales, *biases;
} FmProjWeights;
fm_status fm_proj_upload(FmCtx *ctx, const FmProjWeights *host, FmProjWeights *device);
void fm_proj_free(FmCtx *ctx, FmProjWeights *device);
fm_status fm_out_proj_norm(FmCtx *ctx, const FmProjWeights *w, int n, const float *x, const float *residual,
                           const uint16_t *norm_w, float *h_mid, float *h_post);

/* Off by default.  On: the caller vouches that the launch that precedes a fm_gdn_decode call in the stream does not
 * touch the state of the layer that call steps (in a model loop it never does: the previous launch belongs to another
 * layer or to a projection).  The step is then launched as a programmatic dependent of whatever precedes it: it
 * requests its recurrent state at once and waits for the previous launch to complete before it reads qkv, z, beta,
 * alpha or writes anything, so its start-up and the state's trip from HBM hide behind the previous kernel's tail.
 * Device-pointer mode, batches that take the one-launch form (fewer than 512 (head, sequence) pairs).  The library
 * itself keeps a step of the layer it stepped last, or one that follows its own prefill, import or reset, in plain
 * stream order; launches it does not know about are the caller's to vouch for. */
fm_status fm_set_layer_overlap(FmCtx *ctx, int on);

/* Number of kernels this context has launched since creation (bench bookkeeping). */
int64_t fm_launch_count(const FmCtx *ctx);

/* Device timing of the dominant kernel of each entry point (the split-KV decode kernel, the prefill
 * attention kernel, the GatedDeltaNet kernels): while enabled, every launch of those kernels is
 * bracketed by CUDA events on the context's stream.  fm_profile_read waits for the stream, returns
 * the number of bracketed launches and their summed duration in milliseconds, and clears the
 * record.  Replaces the reference's --timing accumulators (metal_infer/timing.h:9-39,257-296). */
fm_status fm_profile_enable(FmCtx *ctx, int on);
fm_status fm_profile_read(FmCtx *ctx, int *launches, double *total_ms);

/* Decode attention without any allocation -- no counterpart in the reference.
 *
 * For callers that are not allowed to allocate device memory and therefore cannot use fm_create:
 * a plugin living inside another engine's fixed memory plan, a serving loop that bans allocator
 * calls once it is running, code under a tool that intercepts allocation.  The caller owns
 * everything it passes in: the KV pages, the page table, q / gate and the output.  The scratch the
 * split-KV kernels need (the per-split partial results) is a fixed array inside the library image,
 * 8192 partial rows (8.45 MB), resident on every GPU that loads the library until process exit.
 *
 *   kv_pages    device, bf16; page p = [2 (K then V)][num_kv_heads][64 rows][256 dims]; K rows are
 *               already normalised and rotated (what fm_kv_append_rope stores)
 *   page_table  device, int [batch][max_pages_per_seq]; row r of sequence i lives in page
 *               page_table[i][r / 64] at row r % 64
 *   kv_len, pos HOST, int [batch]: rows to attend (>= 1) and the RoPE position of q
 *   q_proj_out  device, [batch][H][512] interleaved q | gate; or q and gate, [batch][H*256]
 *   out         device, [batch][H*256]
 *
 * Computes softmax(rope(norm(q)) K^T / 16) V * sigmoid(gate) like fm_attn_decode with k == NULL
 * (nothing is appended).  Limits: batch <= 64; batch * num_attn_heads <= 8192 (FM_ERR_CAPACITY
 * otherwise; the number of splits shrinks first so that batch * heads * splits fits).  Calls no
 * cudaMalloc / cudaFree or other allocating routine.  The first call on each device resolves the
 * scratch address (cudaGetSymbolAddress) with that device current: make that call before any
 * stream capture.  Every call on a device shares the one scratch array: each call overwrites the
 * rows it uses, nothing needs clearing, but two calls that overlap on the GPU (different streams)
 * race on it -- serialise them.  Error text, if any, is written to err (may be NULL). */
typedef struct FmStaticDecodeArgs {
    const void *kv_pages;
    const int *page_table;
    int max_pages_per_seq;
    const int *kv_len;
    const int *pos;
    int batch;
    int num_attn_heads, num_kv_heads, rotary_dim;
    float rope_theta, rms_norm_eps;
    const float *q_proj_out, *q, *gate;
    const uint16_t *q_norm_w;
    float *out;
    void *stream;
} FmStaticDecodeArgs;
fm_status fm_attn_decode_static(const FmStaticDecodeArgs *args, char *err, size_t err_cap);

#ifdef __cplusplus
}
#endif
#endif /* FM_ATTN_H */
