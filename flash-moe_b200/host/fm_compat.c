/* Host-side mirror of the reference's attention / GatedDeltaNet calling style (see fm_compat.h).
 * Plain C on top of the C-ABI; no device code here. */
#include "fm_compat.h"

#include <stdio.h>
#include <stdlib.h>

static FmCtx *g_fm = NULL;
static FmConfig g_cfg;
static int g_next_fa = 0, g_next_li = 0;

int fm_compat_init(const FmConfig *cfg) {
    if (g_fm) fm_compat_shutdown();
    g_cfg = *cfg;
    if (fm_create(&g_cfg, &g_fm) != FM_OK) {
        fprintf(stderr, "ERROR: %s\n", fm_last_error(NULL));
        g_fm = NULL;
        return -1;
    }
    fm_set_pointer_mode(g_fm, FM_PTR_HOST); /* the reference passes host floats */
    g_next_fa = g_next_li = 0;
    return 0;
}

void fm_compat_shutdown(void) {
    if (g_fm) fm_destroy(g_fm);
    g_fm = NULL;
}

FmCtx *fm_compat_ctx(void) { return g_fm; }

KVCache *kv_cache_new(void) {
    if (!g_fm || g_next_fa >= g_cfg.num_full_layers) {
        fprintf(stderr, "ERROR: KV cache alloc failed (layer %d of %d)\n", g_next_fa, g_fm ? g_cfg.num_full_layers : 0);
        return NULL;
    }
    KVCache *c = calloc(1, sizeof(KVCache));
    if (!c) return NULL;
    c->fa_idx = g_next_fa++;
    c->capacity = g_cfg.max_seq_len;
    c->len = 0;
    return c;
}

void kv_cache_free(KVCache *c) { free(c); }

LinearAttnState *linear_attn_state_new(void) {
    if (!g_fm || g_next_li >= g_cfg.num_linear_layers) {
        fprintf(stderr, "ERROR: linear attention state alloc failed (layer %d)\n", g_next_li);
        return NULL;
    }
    LinearAttnState *s = calloc(1, sizeof(LinearAttnState));
    if (!s) return NULL;
    s->li = g_next_li++;
    return s;
}

void linear_attn_state_free(LinearAttnState *s) { free(s); }

void reset_delta_net_state(void) {
    if (g_fm && fm_reset(g_fm, -1) != FM_OK) fprintf(stderr, "ERROR: %s\n", fm_last_error(g_fm));
}

void full_attention_core(const float *q_proj_out, const float *k, const float *v, const uint16_t *qnorm_w,
                         const uint16_t *knorm_w, KVCache *kv, int pos, float *attn_out) {
    const int seq0 = 0;
    if (!g_fm || !kv) {
        fprintf(stderr, "ERROR: full_attention_core without a context or cache\n");
        return;
    }
    if (fm_attn_decode(g_fm, kv->fa_idx, &seq0, &pos, 1, q_proj_out, NULL, NULL, k, v, qnorm_w, knorm_w, attn_out) != FM_OK) {
        fprintf(stderr, "ERROR: %s\n", fm_last_error(g_fm)); /* e.g. "KV cache overflow (pos=.. >= cap=..)" */
        return;
    }
    kv->len = fm_kv_len(g_fm, kv->fa_idx, 0);
}

void linear_attention_core(const float *qkv, const float *z, const float *beta, const float *alpha,
                           const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                           const uint16_t *gated_norm_w, LinearAttnState *state, float *gated_out) {
    const int seq0 = 0;
    if (!g_fm || !state) {
        fprintf(stderr, "ERROR: linear_attention_core without a context or state\n");
        return;
    }
    if (fm_gdn_decode(g_fm, state->li, &seq0, 1, qkv, z, beta, alpha, conv_w, A_log, dt_bias, gated_norm_w, gated_out) != FM_OK)
        fprintf(stderr, "ERROR: %s\n", fm_last_error(g_fm));
}

void batched_prefill_full_attention(const float *q_proj_out, const float *k, const float *v, const uint16_t *qnorm_w,
                                    const uint16_t *knorm_w, KVCache *kv, int cache_start, int n, float *attn_out) {
    if (!g_fm || !kv) {
        fprintf(stderr, "ERROR: batched_prefill_full_attention without a context or cache\n");
        return;
    }
    if (fm_attn_prefill(g_fm, kv->fa_idx, 0, cache_start, n, q_proj_out, NULL, NULL, k, v, qnorm_w, knorm_w, attn_out) != FM_OK) {
        fprintf(stderr, "ERROR: %s\n", fm_last_error(g_fm));
        return;
    }
    kv->len = fm_kv_len(g_fm, kv->fa_idx, 0); /* = cache_start + n (batched_prefill.h:736) */
}

void batched_prefill_linear_attention(const float *qkv, const float *z, const float *beta, const float *alpha,
                                      const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                                      const uint16_t *gated_norm_w, LinearAttnState *state, int n, float *gated_out) {
    if (!g_fm || !state) {
        fprintf(stderr, "ERROR: batched_prefill_linear_attention without a context or state\n");
        return;
    }
    if (fm_gdn_prefill(g_fm, state->li, 0, n, 0, qkv, z, beta, alpha, conv_w, A_log, dt_bias, gated_norm_w, gated_out) != FM_OK)
        fprintf(stderr, "ERROR: %s\n", fm_last_error(g_fm));
}
