/* CPU checker interface -- TEST INFRASTRUCTURE ONLY.
 *
 * Two libraries export this interface: the plain-C restatement (prefix fmo_,
 * fm_oracle.c) and the harness around the reference project's own CPU code
 * (prefix fmr_, ref_harness.c).  Both run the reference semantics of one
 * decode step in fp32:
 *
 *   full attention (metal_infer/layer_forward.h:556-735):
 *     per-head q/k RMS-norm (optional) -> partial RoPE at `pos` -> append k,v
 *     at row `*len` -> *len += 1 -> softmax(q.K/sqrt(D)) V over rows [0,*len)
 *     -> multiply by sigmoid(gate).
 *   GatedDeltaNet (metal_infer/layer_forward.h:886-1025):
 *     depthwise causal conv (width 4) + SiLU -> shift conv state -> q,k
 *     RMS-normalise and scale -> decay / beta -> delta-rule recurrence on the
 *     per-head [dv][dk] state -> gated RMS-norm with SiLU(z).
 *
 * Only tests, the smoke check and the bench's CPU-baseline leg may load these
 * libraries.
 */
#ifndef FM_ORACLE_H
#define FM_ORACLE_H
#include <stdint.h>

typedef struct {
    int num_attn_heads;      /* 32 */
    int num_kv_heads;        /* 2  */
    int head_dim;            /* 256 */
    int rotary_dim;          /* 64 */
    float rope_theta;        /* 1e7 */
    float rms_norm_eps;      /* 1e-6 */
    int rope_scaling_mode;   /* 0 none, 1 linear, 2 NTK, 3 YaRN */
    float rope_scale_factor; /* 1.0 */
    int max_seq_len;         /* original context length (YaRN wavelength bounds) */
    int linear_num_v_heads;  /* 64 */
    int linear_num_k_heads;  /* 16 */
    int linear_key_dim;      /* 128 */
    int linear_value_dim;    /* 128 */
    int conv_kernel_size;    /* 4 */
    int store_bf16;          /* restatement only (the reference harness ignores it): round the
                                normalised, rotated k and the v to bf16 (nearest even) before the
                                append, i.e. reference arithmetic on top of a bf16 KV store */
    int sliding_window;      /* 0 unlimited; > 0: the cache is a circular buffer of that many rows
                                (capacity must equal it), metal_infer/layer_forward.h:130-161,600-601,
                                649-650,673-677; *len keeps counting every appended token */
} FmoDims;

/* A KV cache with the reference's optional policies (KVCache, metal_infer/layer_forward.h:121-141), caller-owned
 * arrays.  fp32 store: k_cache / v_cache [capacity][kv_dim].  FP8 store (use_fp8): k8 / v8 [capacity][kv_dim]
 * E4M3 bytes + k_scales / v_scales [capacity] (metal_infer/fp8.h:100-108).  window_size > 0: circular buffer
 * (capacity == window_size).  h2o_budget > 0: heavy-hitter eviction (metal_infer/layer_forward.h:248-383);
 * capacity >= budget + 1, attn_scores_accum / token_positions [capacity], num_recent = (budget - sinks) / 4 as
 * kv_cache_new() sets it (:203). */
typedef struct {
    float *k_cache, *v_cache;
    uint8_t *k8, *v8;
    float *k_scales, *v_scales;
    int len, capacity, use_fp8, window_size;
    int h2o_budget, h2o_num_sinks, h2o_num_recent, h2o_num_valid;
    float *attn_scores_accum;
    int *token_positions;
} FmoCache;

#define FMO_API(prefix)                                                                         \
    /* One decode step. k_cache/v_cache: [capacity][kv_heads*head_dim] fp32, *len rows valid.   \
       q, gate: [heads*head_dim] (already de-interleaved); k, v: [kv_heads*head_dim].           \
       q_norm_w/k_norm_w: bf16 [head_dim] or NULL. out: [heads*head_dim].                       \
       threads > 1 runs the per-head loop on that many OpenMP threads (same arithmetic).        \
       Returns 0, or -1 on cache overflow (nothing written). */                                 \
    int prefix##attn_step(const FmoDims *d, float *k_cache, float *v_cache, int *len,           \
                          int capacity, const float *q, const float *gate, const float *k,      \
                          const float *v, const uint16_t *q_norm_w, const uint16_t *k_norm_w,   \
                          int pos, float *out, int threads);                                    \
    /* n consecutive steps at positions start_pos.. (token-major inputs with leading [n]). */   \
    int prefix##attn_run(const FmoDims *d, float *k_cache, float *v_cache, int *len,            \
                         int capacity, const float *q, const float *gate, const float *k,       \
                         const float *v, const uint16_t *q_norm_w, const uint16_t *k_norm_w,    \
                         int start_pos, int n, float *out, int threads);                        \
    /* One GatedDeltaNet step. conv_state: [(ks-1)][conv_dim]; ssm_state: [Hv][dv][dk].          \
       qkv: [conv_dim] = q(Hk*dk) | k(Hk*dk) | v(Hv*dv); z: [Hv*dv]; beta, alpha: [Hv].          \
       conv_w: bf16 [conv_dim][ks]; A_log: fp32 [Hv] or NULL; dt_bias: bf16 [Hv] or NULL;        \
       norm_w: bf16 [dv] or NULL. out: [Hv*dv]. */                                              \
    int prefix##gdn_step(const FmoDims *d, float *conv_state, float *ssm_state,                 \
                         const float *qkv, const float *z, const float *beta,                   \
                         const float *alpha, const uint16_t *conv_w, const float *A_log,        \
                         const uint16_t *dt_bias, const uint16_t *norm_w, float *out,           \
                         int threads);                                                          \
    int prefix##gdn_run(const FmoDims *d, float *conv_state, float *ssm_state,                  \
                        const float *qkv, const float *z, const float *beta,                    \
                        const float *alpha, const uint16_t *conv_w, const float *A_log,         \
                        const uint16_t *dt_bias, const uint16_t *norm_w, int n, float *out,     \
                        int threads);                                                           \
    /* One decode step on a cache with the optional policies (FP8 store, sliding window, H2O     \
       eviction).  Same inputs and output as attn_step; the cache's len / h2o_num_valid move. */ \
    int prefix##attn_step_cache(const FmoDims *d, FmoCache *c, const float *q, const float *gate, \
                                const float *k, const float *v, const uint16_t *q_norm_w,       \
                                const uint16_t *k_norm_w, int pos, float *out, int threads);     \
    /* FP8 codec on n rows of kv_dim floats: bytes [n][kv_dim], scales [n]. */                   \
    void prefix##fp8_encode_rows(const float *src, int n, int kv_dim, uint8_t *dst, float *scales); \
    void prefix##fp8_decode_rows(const uint8_t *src, const float *scales, int n, int kv_dim, float *dst); \
    /* Output projection from 4-bit affine weights + residual + RMS-norm for one token                 \
       (metal_infer/cpu_kernels.h:199-246; order of use metal_infer/layer_forward.h:3369-3450):         \
       y = W x, h_mid = residual + y (residual may be NULL), h_post = rms_norm(h_mid) * norm_w. */      \
    void prefix##out_proj_norm(const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int out_dim, \
                               int in_dim, int group_size, const float *x, const float *residual,        \
                               const uint16_t *norm_w, float eps, float *h_mid, float *h_post);

FMO_API(fmo_)
FMO_API(fmr_)

#endif
