/* fm_compat.h -- the reference's own names for this path, for a host that wants a drop-in.
 *
 * The reference's callers (fused_layer_forward, batched_prefill, the generation loops) hold a
 * KVCache* per full-attention layer and a LinearAttnState* per GatedDeltaNet layer, create them with
 * kv_cache_new() / linear_attn_state_new(), read kv->len, and run the post-projection part of
 * full_attention_forward / linear_attention_forward on host float buffers.  This header keeps those
 * names and that calling style (plain C, host pointers, void functions that print
 * "ERROR: ..." to stderr and return) on top of include/fm_attn.h; the structs become handles into
 * the context's device-resident store.
 *
 *   reference                                              here
 *   metal_setup()                metal_ctx.h:157           fm_compat_init(cfg)
 *   kv_cache_new / _free         layer_forward.h:143-236   same names; k_cache/v_cache live on the GPU
 *   linear_attn_state_new/_free  layer_forward.h:419-432   same names
 *   reset_delta_net_state()      metal_ctx.h:599-608       same name
 *   full_attention_forward  :556-735 (after the projections)     full_attention_core()
 *   linear_attention_forward:886-1025 (after the projections)    linear_attention_core()
 *   batched_prefill(), full-attention layer, after the projection GEMMs, one chunk of <= MAX_PFB_GPU tokens
 *       (batched_prefill.h:543-740: deinterleave, prefill_q_rope_norm_bf16, prefill_kv_cache_bf16,
 *       prefill_causal_attn, kv->len = cache_start + n)          batched_prefill_full_attention()
 *   batched_prefill(), GatedDeltaNet layer, after the projection GEMMs (batched_prefill.h:798-1037:
 *       conv1d_step_batched ... gated_rms_norm_batched)           batched_prefill_linear_attention()
 */
#ifndef FM_COMPAT_H
#define FM_COMPAT_H
#include "fm_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct KVCache {
    int len;       /* rows written, kept in step with the device store (layer_forward.h:128) */
    int capacity;  /* max_seq_len of the context */
    int fa_idx;    /* which full-attention layer of the context this cache is */
} KVCache;

typedef struct LinearAttnState {
    int li;        /* which GatedDeltaNet layer of the context this state is */
} LinearAttnState;

/* One context for the process, host-pointer mode (the reference's globals g_metal / cfg). 0 or -1. */
int fm_compat_init(const FmConfig *cfg);
void fm_compat_shutdown(void);
FmCtx *fm_compat_ctx(void);

/* Handles are given out in layer order: the i-th call returns the cache of full-attention layer i. */
KVCache *kv_cache_new(void);
void kv_cache_free(KVCache *c);
LinearAttnState *linear_attn_state_new(void);
void linear_attn_state_free(LinearAttnState *s);
void reset_delta_net_state(void);

/* q_proj_out [H][2*D] interleaved q|gate, k, v [Hkv*D], norm weights bf16 [D] or NULL, attn_out [H*D]. */
void full_attention_core(const float *q_proj_out, const float *k, const float *v, const uint16_t *qnorm_w,
                         const uint16_t *knorm_w, KVCache *kv, int pos, float *attn_out);
/* qkv [conv_dim], z [Hv*dv], beta, alpha [Hv]; weights as the reference's tensors; gated_out [Hv*dv]. */
void linear_attention_core(const float *qkv, const float *z, const float *beta, const float *alpha,
                           const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                           const uint16_t *gated_norm_w, LinearAttnState *state, float *gated_out);

/* One chunk of n prompt tokens of a full-attention layer: q_proj_out [n][H][2*D] interleaved q|gate, k, v
 * [n][Hkv*D]; token t sits at position cache_start + t, its row is appended and it attends to rows
 * [0, cache_start + t]; attn_out [n][H*D] (already multiplied by the sigmoid gate).  kv->len becomes
 * cache_start + n.  n is bounded by the context's max_batch_tokens (the reference's MAX_PFB_GPU is 32). */
void batched_prefill_full_attention(const float *q_proj_out, const float *k, const float *v, const uint16_t *qnorm_w,
                                    const uint16_t *knorm_w, KVCache *kv, int cache_start, int n, float *attn_out);
/* One chunk of n prompt tokens of a GatedDeltaNet layer: qkv [n][conv_dim], z [n][Hv*dv], beta, alpha [n][Hv];
 * gated_out [n][Hv*dv]; the layer's conv history and recurrent state move on by n tokens. */
void batched_prefill_linear_attention(const float *qkv, const float *z, const float *beta, const float *alpha,
                                      const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                                      const uint16_t *gated_norm_w, LinearAttnState *state, int n, float *gated_out);

#ifdef __cplusplus
}
#endif
#endif
