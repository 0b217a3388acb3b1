/* Harness around the reference project's own CPU attention / GatedDeltaNet code.
 * TEST INFRASTRUCTURE ONLY -- see fm_oracle.h.
 *
 * The *.inc files are line ranges of the reference checkout, cut into a
 * temporary directory by build_oracle.py at build time (they are never stored
 * in this repository).  This file supplies what the unity build around those
 * ranges would have supplied: the globals, a tensor lookup that answers by
 * name suffix from the pointers of the current call, and the local variables
 * the two function bodies expect.
 */
#include <math.h>
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "fm_oracle.h"

#include "ref_config_struct.inc"  /* ModelConfig + `static ModelConfig cfg` */

/* feature flags the sliced code reads (metal_infer/timing.h:82-111) */
static int g_sliding_window = 0;
static int g_h2o_budget = 0;
static int g_h2o_num_sinks = 4;
static int g_rope_scaling_mode = 0;
static float g_rope_scale_factor = 1.0f;
static int g_kv_seq_len = 0;

#include "ref_fp8.inc"
#include "ref_bf16.inc"
#include "ref_cpu_kernels.inc"

typedef struct WeightFile WeightFile;

/* tensors of the call in flight, answered by name suffix */
static struct {
    const void *q_norm, *k_norm, *conv1d, *A_log, *dt_bias, *gdn_norm;
} g_tensors;

static int ends_with(const char *s, const char *suffix) {
    size_t n = strlen(s), m = strlen(suffix);
    return n >= m && strcmp(s + n - m, suffix) == 0;
}

static void *get_tensor_ptr(WeightFile *wf, const char *name) {
    (void)wf;
    if (ends_with(name, "self_attn.q_norm.weight")) return (void *)g_tensors.q_norm;
    if (ends_with(name, "self_attn.k_norm.weight")) return (void *)g_tensors.k_norm;
    if (ends_with(name, "linear_attn.conv1d.weight")) return (void *)g_tensors.conv1d;
    if (ends_with(name, "linear_attn.A_log")) return (void *)g_tensors.A_log;
    if (ends_with(name, "linear_attn.dt_bias")) return (void *)g_tensors.dt_bias;
    if (ends_with(name, "linear_attn.norm.weight")) return (void *)g_tensors.gdn_norm;
    return NULL;
}

#include "ref_rope.inc"
#include "ref_kv.inc"
#include "ref_h2o.inc"
#include "ref_las.inc"
#include "ref_gdn_helpers.inc"

static void load_cfg(const FmoDims *d) {
    memset(&cfg, 0, sizeof(cfg));
    cfg.num_attn_heads = d->num_attn_heads;
    cfg.num_kv_heads = d->num_kv_heads;
    cfg.head_dim = d->head_dim;
    cfg.rotary_dim = d->rotary_dim;
    cfg.rope_theta = d->rope_theta;
    cfg.rms_norm_eps = d->rms_norm_eps;
    cfg.max_seq_len = d->max_seq_len;
    cfg.linear_num_v_heads = d->linear_num_v_heads;
    cfg.linear_num_k_heads = d->linear_num_k_heads;
    cfg.linear_key_dim = d->linear_key_dim;
    cfg.linear_value_dim = d->linear_value_dim;
    cfg.conv_kernel_size = d->conv_kernel_size;
    cfg.linear_total_key = d->linear_num_k_heads * d->linear_key_dim;
    cfg.linear_total_value = d->linear_num_v_heads * d->linear_value_dim;
    cfg.linear_conv_dim = 2 * cfg.linear_total_key + cfg.linear_total_value;
    g_rope_scaling_mode = d->rope_scaling_mode;
    g_rope_scale_factor = d->rope_scale_factor;
}

/* ---- full attention: the reference body as written (single thread) ---- */
static void fa_body_serial(WeightFile *wf, int layer_idx, float *q, float *q_gate, float *k,
                           float *v, KVCache *kv, int pos, int q_dim, int kv_dim, float *out,
                           int *ok) {
    char name[256];
    *ok = 0;
#include "ref_fa_core.inc"
    memcpy(out, attn_out, (size_t)q_dim * sizeof(float));
    free(attn_out);
    *ok = 1;
}

/* ---- same body, per-head loop threaded by the harness (loop body unchanged) ---- */
static void fa_body_threaded(WeightFile *wf, int layer_idx, float *q, float *q_gate, float *k,
                             float *v, KVCache *kv, int pos, int q_dim, int kv_dim, float *out,
                             int *ok, int threads) {
    char name[256];
    *ok = 0;
#include "ref_fa_pre.inc"
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int h = 0; h < cfg.num_attn_heads; h++) {
#include "ref_fa_head_body.inc"
    }
#include "ref_fa_post.inc"
    memcpy(out, attn_out, (size_t)q_dim * sizeof(float));
    free(attn_out);
    *ok = 1;
}

int fmr_attn_step(const FmoDims *d, float *k_cache, float *v_cache, int *len, int capacity,
                  const float *q_in, const float *gate_in, const float *k_in, const float *v_in,
                  const uint16_t *q_norm_w, const uint16_t *k_norm_w, int pos, float *out,
                  int threads) {
    load_cfg(d);
    int q_dim = d->num_attn_heads * d->head_dim;
    int kv_dim = d->num_kv_heads * d->head_dim;
    KVCache kv;
    memset(&kv, 0, sizeof(kv));
    kv.k_cache = k_cache;
    kv.v_cache = v_cache;
    kv.len = *len;
    kv.capacity = capacity;
    kv.window_size = d->sliding_window; /* as kv_cache_new() sets it from g_sliding_window */
    if (kv.window_size > 0 && capacity != kv.window_size) return -1;
    g_tensors.q_norm = q_norm_w;
    g_tensors.k_norm = k_norm_w;
    /* the body normalises / rotates q and k in place: work on copies */
    float *q = malloc((size_t)q_dim * sizeof(float));
    float *g = malloc((size_t)q_dim * sizeof(float));
    float *k = malloc((size_t)kv_dim * sizeof(float));
    float *v = malloc((size_t)kv_dim * sizeof(float));
    memcpy(q, q_in, (size_t)q_dim * sizeof(float));
    memcpy(g, gate_in, (size_t)q_dim * sizeof(float));
    memcpy(k, k_in, (size_t)kv_dim * sizeof(float));
    memcpy(v, v_in, (size_t)kv_dim * sizeof(float));
    int ok = 0;
    if (threads > 1)
        fa_body_threaded(NULL, 0, q, g, k, v, &kv, pos, q_dim, kv_dim, out, &ok, threads);
    else
        fa_body_serial(NULL, 0, q, g, k, v, &kv, pos, q_dim, kv_dim, out, &ok);
    *len = kv.len;
    free(q); free(g); free(k); free(v);
    return ok ? 0 : -1;
}

int fmr_attn_run(const FmoDims *d, float *k_cache, float *v_cache, int *len, int capacity,
                 const float *q, const float *gate, const float *k, const float *v,
                 const uint16_t *q_norm_w, const uint16_t *k_norm_w, int start_pos, int n,
                 float *out, int threads) {
    size_t q_dim = (size_t)d->num_attn_heads * d->head_dim;
    size_t kv_dim = (size_t)d->num_kv_heads * d->head_dim;
    for (int t = 0; t < n; t++) {
        int rc = fmr_attn_step(d, k_cache, v_cache, len, capacity, q + t * q_dim, gate + t * q_dim,
                               k + t * kv_dim, v + t * kv_dim, q_norm_w, k_norm_w, start_pos + t,
                               out + t * q_dim, threads);
        if (rc) return rc;
    }
    return 0;
}

/* ---- the same step on a cache with the reference's optional policies (FP8 store, sliding window, H2O) ---- */
int fmr_attn_step_cache(const FmoDims *d, FmoCache *c, const float *q_in, const float *gate_in, const float *k_in,
                        const float *v_in, const uint16_t *q_norm_w, const uint16_t *k_norm_w, int pos, float *out,
                        int threads) {
    load_cfg(d);
    int q_dim = d->num_attn_heads * d->head_dim;
    int kv_dim = d->num_kv_heads * d->head_dim;
    KVCache kv;
    memset(&kv, 0, sizeof(kv));
    kv.k_cache = c->k_cache; kv.v_cache = c->v_cache;
    kv.k_cache_fp8 = c->k8; kv.v_cache_fp8 = c->v8;
    kv.k_scales = c->k_scales; kv.v_scales = c->v_scales;
    kv.len = c->len; kv.capacity = c->capacity; kv.use_fp8 = c->use_fp8;
    kv.window_size = c->h2o_budget > 0 ? 0 : c->window_size;     /* kv_cache_new(): H2O replaces the window */
    if (kv.window_size > 0 && c->capacity != kv.window_size) return -1;
    kv.h2o_active = c->h2o_budget > 0;
    kv.h2o_budget = c->h2o_budget;
    kv.h2o_num_sinks = c->h2o_num_sinks;
    kv.h2o_num_recent = c->h2o_num_recent;
    kv.h2o_num_valid = c->h2o_num_valid;
    kv.attn_scores_accum = c->attn_scores_accum;
    kv.token_positions = c->token_positions;
    g_tensors.q_norm = q_norm_w;
    g_tensors.k_norm = k_norm_w;
    float *q = malloc((size_t)q_dim * sizeof(float));
    float *g = malloc((size_t)q_dim * sizeof(float));
    float *k = malloc((size_t)kv_dim * sizeof(float));
    float *v = malloc((size_t)kv_dim * sizeof(float));
    memcpy(q, q_in, (size_t)q_dim * sizeof(float));
    memcpy(g, gate_in, (size_t)q_dim * sizeof(float));
    memcpy(k, k_in, (size_t)kv_dim * sizeof(float));
    memcpy(v, v_in, (size_t)kv_dim * sizeof(float));
    int ok = 0;
    /* The reference's per-head loop shares one dequantisation buffer (FP8) and one score accumulator (H2O)
       between heads, so those two modes run it as written, on one thread. */
    if (threads > 1 && !kv.use_fp8 && !kv.h2o_active)
        fa_body_threaded(NULL, 0, q, g, k, v, &kv, pos, q_dim, kv_dim, out, &ok, threads);
    else
        fa_body_serial(NULL, 0, q, g, k, v, &kv, pos, q_dim, kv_dim, out, &ok);
    c->len = kv.len;
    c->h2o_num_valid = kv.h2o_num_valid;
    free(q); free(g); free(k); free(v);
    return ok ? 0 : -1;
}

void fmr_fp8_encode_rows(const float *src, int n, int kv_dim, uint8_t *dst, float *scales) {
    for (int i = 0; i < n; i++) scales[i] = fp8_encode_vec(src + (size_t)i * kv_dim, dst + (size_t)i * kv_dim, kv_dim);
}
void fmr_fp8_decode_rows(const uint8_t *src, const float *scales, int n, int kv_dim, float *dst) {
    for (int i = 0; i < n; i++) fp8_decode_vec(src + (size_t)i * kv_dim, dst + (size_t)i * kv_dim, kv_dim, scales[i]);
}

/* ---- the step behind attention: o_proj (4-bit dequant matvec) + residual + post-attention RMS-norm ---- */
void fmr_out_proj_norm(const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int out_dim, int in_dim,
                       int group_size, const float *x, const float *residual, const uint16_t *norm_w, float eps,
                       float *h_mid, float *h_post) {
    cpu_dequant_matvec(w, scales, biases, x, h_mid, out_dim, in_dim, group_size);
    if (residual)
        for (int i = 0; i < out_dim; i++) h_mid[i] = residual[i] + h_mid[i];   /* residual_add: a + b */
    if (h_post) cpu_rms_norm(h_mid, norm_w, h_post, out_dim, eps);
}

/* ---- GatedDeltaNet ---- */
static void gdn_body_serial(WeightFile *wf, int layer_idx, LinearAttnState *state, float *qkv,
                            int qkv_dim, float *z, float *beta, float *alpha, float *out) {
    char name[256];
#include "ref_gdn_core.inc"
    memcpy(out, gated_out, (size_t)cfg.linear_total_value * sizeof(float));
    free(gated_out);
    free(out_values);
    free(conv_out);
}

static void gdn_body_threaded(WeightFile *wf, int layer_idx, LinearAttnState *state, float *qkv,
                              int qkv_dim, float *z, float *beta, float *alpha, float *out,
                              int threads) {
    char name[256];
#include "ref_gdn_pre.inc"
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int vh = 0; vh < cfg.linear_num_v_heads; vh++) {
#include "ref_gdn_head_body.inc"
    }
#include "ref_gdn_post.inc"
    memcpy(out, gated_out, (size_t)cfg.linear_total_value * sizeof(float));
    free(gated_out);
    free(out_values);
    free(conv_out);
}

int fmr_gdn_step(const FmoDims *d, float *conv_state, float *ssm_state, const float *qkv,
                 const float *z, const float *beta, const float *alpha, const uint16_t *conv_w,
                 const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, float *out,
                 int threads) {
    load_cfg(d);
    LinearAttnState st = {conv_state, ssm_state};
    g_tensors.conv1d = conv_w;
    g_tensors.A_log = A_log;
    g_tensors.dt_bias = dt_bias;
    g_tensors.gdn_norm = norm_w;
    if (threads > 1)
        gdn_body_threaded(NULL, 0, &st, (float *)qkv, cfg.linear_conv_dim, (float *)z,
                          (float *)beta, (float *)alpha, out, threads);
    else
        gdn_body_serial(NULL, 0, &st, (float *)qkv, cfg.linear_conv_dim, (float *)z, (float *)beta,
                        (float *)alpha, out);
    return 0;
}

int fmr_gdn_run(const FmoDims *d, float *conv_state, float *ssm_state, const float *qkv,
                const float *z, const float *beta, const float *alpha, const uint16_t *conv_w,
                const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, int n,
                float *out, int threads) {
    size_t conv_dim = (size_t)(2 * d->linear_num_k_heads * d->linear_key_dim +
                               d->linear_num_v_heads * d->linear_value_dim);
    size_t vdim = (size_t)d->linear_num_v_heads * d->linear_value_dim;
    size_t hv = (size_t)d->linear_num_v_heads;
    for (int t = 0; t < n; t++) {
        fmr_gdn_step(d, conv_state, ssm_state, qkv + t * conv_dim, z + t * vdim, beta + t * hv,
                     alpha + t * hv, conv_w, A_log, dt_bias, norm_w, out + t * vdim, threads);
    }
    return 0;
}
