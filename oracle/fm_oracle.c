/* Plain-C restatement of the reference's CPU attention / GatedDeltaNet step.
 * TEST INFRASTRUCTURE ONLY -- see fm_oracle.h.  Nothing in the product path
 * links or loads this file.
 *
 * Parity pin: this restatement is checked bit-for-bit against the reference's
 * own CPU code (ref_harness.c over line ranges of the reference checkout) by
 * tests/test_oracle.py, and both are checked against the vectors committed
 * under tests/golden/ (which were produced by the reference build).  The
 * reference itself ships no golden vectors or unit tests for this path.
 *
 * Every routine keeps the reference's operation order (sequential fp32 sums,
 * max-subtracted three-pass softmax) so that results round identically.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "fm_oracle.h"

/* bf16 -> fp32 by shifting into the high half (metal_infer/weights.h:9-14) */
static inline float bf16f(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* fp32 -> nearest-even bf16 -> fp32 */
static inline float round_bf16f(float x) {
    uint32_t u;
    memcpy(&u, &x, sizeof u);
    u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;
    memcpy(&x, &u, sizeof x);
    return x;
}

/* ------------------------------------------------------------------------ */
/* RoPE frequency with the scaling modes of metal_infer/layer_forward.h:22-63 */
static float rope_freq(const FmoDims *d, int i) {
    const float base = d->rope_theta;
    const int rot = d->rotary_dim;
    const int mode = d->rope_scaling_mode;
    const float s = d->rope_scale_factor;
    const float expo = (float)(2 * i) / rot;
    if (mode == 0 || s <= 1.0f || mode == 1) return 1.0f / powf(base, expo);
    const float base_ntk = base * powf(s, (float)rot / (rot - 2));
    if (mode == 2) return 1.0f / powf(base_ntk, expo);
    /* YaRN: keep short wavelengths, NTK-scale long ones, ramp in between */
    const float f_orig = 1.0f / powf(base, expo);
    const float f_ntk = 1.0f / powf(base_ntk, expo);
    const float wavelength = 2.0f * M_PI / f_orig;
    const float lo = (float)d->max_seq_len;
    const float hi = lo / 32.0f;
    if (wavelength < hi) return f_orig;
    if (wavelength > lo) return f_ntk;
    const float ramp = (wavelength - hi) / (lo - hi);
    return f_orig * (1.0f - ramp) + f_ntk * ramp;
}

/* softmax logit temperature under YaRN (metal_infer/layer_forward.h:67-70) */
static float yarn_logit_factor(const FmoDims *d) {
    if (d->rope_scaling_mode != 3 || d->rope_scale_factor <= 1.0f) return 1.0f;
    return sqrtf(0.1f * logf(d->rope_scale_factor) + 1.0f);
}

/* rotate pairs (x[i], x[i+rot/2]) of each head (metal_infer/layer_forward.h:72-115) */
static void rope_heads(const FmoDims *d, float *x, int heads, int pos) {
    const int half = d->rotary_dim / 2;
    float p = (float)pos;
    if (d->rope_scaling_mode == 1 && d->rope_scale_factor > 1.0f) p = (float)pos / d->rope_scale_factor;
    for (int h = 0; h < heads; h++) {
        float *xh = x + (size_t)h * d->head_dim;
        for (int i = 0; i < half; i++) {
            const float ang = p * rope_freq(d, i);
            const float c = cosf(ang), s = sinf(ang);
            const float a = xh[i], b = xh[i + half];
            xh[i] = a * c - b * s;
            xh[i + half] = a * s + b * c;
        }
    }
}

/* per-head RMS-norm with bf16 weight (metal_infer/layer_forward.h:562-585) */
static void head_rms_norm(float *x, int heads, int dim, const uint16_t *w, float eps) {
    if (!w) return;
    for (int h = 0; h < heads; h++) {
        float *xh = x + (size_t)h * dim;
        float ss = 0.0f;
        for (int i = 0; i < dim; i++) ss += xh[i] * xh[i];
        const float inv = 1.0f / sqrtf(ss / dim + eps);
        for (int i = 0; i < dim; i++) xh[i] = xh[i] * inv * bf16f(w[i]);
    }
}

/* max-subtracted softmax (metal_infer/cpu_kernels.h:263-277) */
static void softmax_inplace(float *x, int n) {
    float m = x[0];
    for (int i = 1; i < n; i++)
        if (x[i] > m) m = x[i];
    float sum = 0.0f;
    for (int i = 0; i < n; i++) {
        x[i] = expf(x[i] - m);
        sum += x[i];
    }
    const float inv = 1.0f / sum;
    for (int i = 0; i < n; i++) x[i] *= inv;
}

int fmo_attn_step(const FmoDims *d, float *k_cache, float *v_cache, int *len, int capacity,
                  const float *q_in, const float *gate, const float *k_in, const float *v_in,
                  const uint16_t *q_norm_w, const uint16_t *k_norm_w, int pos, float *out,
                  int threads) {
    const int H = d->num_attn_heads, Hkv = d->num_kv_heads, D = d->head_dim;
    const int q_dim = H * D, kv_dim = Hkv * D;
    const int W = d->sliding_window;
    if (W > 0 && capacity != W) return -1;        /* metal_infer/layer_forward.h:154-161 */
    if (W == 0 && *len >= capacity) return -1;     /* metal_infer/layer_forward.h:603-607 */
    const int cache_pos = W > 0 ? *len % capacity : *len; /* :600-601 circular write */

    float *q = malloc((size_t)q_dim * sizeof(float));
    float *k = malloc((size_t)kv_dim * sizeof(float));
    memcpy(q, q_in, (size_t)q_dim * sizeof(float));
    memcpy(k, k_in, (size_t)kv_dim * sizeof(float));

    head_rms_norm(q, H, D, q_norm_w, d->rms_norm_eps);
    head_rms_norm(k, Hkv, D, k_norm_w, d->rms_norm_eps);
    rope_heads(d, q, H, pos);
    rope_heads(d, k, Hkv, pos);

    /* append, then attend over the cache including the new row
       (metal_infer/layer_forward.h:591-646) */
    memcpy(k_cache + (size_t)cache_pos * kv_dim, k, (size_t)kv_dim * sizeof(float));
    memcpy(v_cache + (size_t)cache_pos * kv_dim, v_in, (size_t)kv_dim * sizeof(float));
    if (d->store_bf16) {
        float *kr = k_cache + (size_t)cache_pos * kv_dim, *vr = v_cache + (size_t)cache_pos * kv_dim;
        for (int i = 0; i < kv_dim; i++) {
            kr[i] = round_bf16f(kr[i]);
            vr[i] = round_bf16f(vr[i]);
        }
    }
    *len += 1;
    /* rows attended and where row i of the window lives (metal_infer/layer_forward.h:649-650, 673-677) */
    const int wrapped = W > 0 && *len > W;
    const int L = wrapped ? W : *len;
    const int first = wrapped ? *len - W : 0;
    const int group = H / Hkv;
    const float scale = (1.0f / sqrtf((float)D)) * yarn_logit_factor(d);

    memset(out, 0, (size_t)q_dim * sizeof(float));
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static) if (threads > 1)
    for (int h = 0; h < H; h++) {
        const int kvh = h / group;
        const float *qh = q + (size_t)h * D;
        float *s = malloc((size_t)L * sizeof(float));
        for (int i = 0; i < L; i++) {
            const int p = wrapped ? (first + i) % capacity : i;
            const float *kp = k_cache + (size_t)p * kv_dim + (size_t)kvh * D;
            float dot = 0.0f;
            for (int e = 0; e < D; e++) dot += qh[e] * kp[e];
            s[i] = dot * scale;
        }
        softmax_inplace(s, L);
        float *oh = out + (size_t)h * D;
        for (int i = 0; i < L; i++) {
            const int p = wrapped ? (first + i) % capacity : i;
            const float *vp = v_cache + (size_t)p * kv_dim + (size_t)kvh * D;
            for (int e = 0; e < D; e++) oh[e] += s[i] * vp[e];
        }
        free(s);
    }
    /* sigmoid output gate (metal_infer/layer_forward.h:729-735) */
    for (int i = 0; i < q_dim; i++) {
        const float g = 1.0f / (1.0f + expf(-gate[i]));
        out[i] *= g;
    }
    free(q);
    free(k);
    return 0;
}

int fmo_attn_run(const FmoDims *d, float *k_cache, float *v_cache, int *len, int capacity,
                 const float *q, const float *gate, const float *k, const float *v,
                 const uint16_t *q_norm_w, const uint16_t *k_norm_w, int start_pos, int n,
                 float *out, int threads) {
    const size_t q_dim = (size_t)d->num_attn_heads * d->head_dim;
    const size_t kv_dim = (size_t)d->num_kv_heads * d->head_dim;
    for (int t = 0; t < n; t++) {
        int rc = fmo_attn_step(d, k_cache, v_cache, len, capacity, q + t * q_dim, gate + t * q_dim,
                               k + t * kv_dim, v + t * kv_dim, q_norm_w, k_norm_w, start_pos + t,
                               out + t * q_dim, threads);
        if (rc) return rc;
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
int fmo_gdn_step(const FmoDims *d, float *conv_state, float *ssm_state, const float *qkv,
                 const float *z, const float *beta, const float *alpha, const uint16_t *conv_w,
                 const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, float *out,
                 int threads) {
    const int Hv = d->linear_num_v_heads, Hk = d->linear_num_k_heads;
    const int dk = d->linear_key_dim, dv = d->linear_value_dim, ks = d->conv_kernel_size;
    const int total_k = Hk * dk, total_v = Hv * dv, C = 2 * total_k + total_v;

    /* depthwise conv over [history | new] then SiLU (metal_infer/cpu_kernels.h:364-387);
       skipped (zeros) when there is no conv weight, as the reference does */
    float *c = calloc((size_t)C, sizeof(float));
    if (conv_w) {
        for (int ch = 0; ch < C; ch++) {
            float acc = 0.0f;
            for (int t = 0; t < ks - 1; t++) acc += conv_state[(size_t)t * C + ch] * bf16f(conv_w[ch * ks + t]);
            acc += qkv[ch] * bf16f(conv_w[ch * ks + (ks - 1)]);
            c[ch] = acc;
        }
        for (int ch = 0; ch < C; ch++) c[ch] = c[ch] / (1.0f + expf(-c[ch]));
    }
    /* history: drop the oldest row, append the raw input (metal_infer/layer_forward.h:897-901) */
    memmove(conv_state, conv_state + C, (size_t)(ks - 2) * C * sizeof(float));
    memcpy(conv_state + (size_t)(ks - 2) * C, qkv, (size_t)C * sizeof(float));

    float *lq = c, *lk = c + total_k, *lv = c + 2 * total_k;

    /* q <- rmsnorm(q)/dk, k <- rmsnorm(k)/sqrt(dk), eps 1e-6 (metal_infer/layer_forward.h:917-929) */
    const float inv_scale = 1.0f / sqrtf((float)dk);
    for (int pass = 0; pass < 2; pass++) {
        float *base = pass == 0 ? lq : lk;
        const float mul = pass == 0 ? inv_scale * inv_scale : inv_scale;
        for (int h = 0; h < Hk; h++) {
            float *x = base + (size_t)h * dk;
            float ss = 0.0f;
            for (int i = 0; i < dk; i++) ss += x[i] * x[i];
            const float inv = 1.0f / sqrtf(ss / dk + 1e-6f);
            for (int i = 0; i < dk; i++) x[i] = x[i] * inv;
            for (int i = 0; i < dk; i++) x[i] *= mul;
        }
    }

    /* decay and beta per value head (metal_infer/layer_forward.h:955-965) */
    float *g_decay = malloc((size_t)Hv * sizeof(float));
    float *b_gate = malloc((size_t)Hv * sizeof(float));
    for (int vh = 0; vh < Hv; vh++) {
        const float bias = dt_bias ? bf16f(dt_bias[vh]) : 0.0f;
        const float A = A_log ? expf(A_log[vh]) : 1.0f;
        const float sp = logf(1.0f + expf(alpha[vh] + bias));
        g_decay[vh] = expf(-A * sp);
        b_gate[vh] = 1.0f / (1.0f + expf(-beta[vh]));
    }

    /* delta rule on S[vi][ki] (metal_infer/layer_forward.h:967-1009) */
    float *o = calloc((size_t)total_v, sizeof(float));
    const int rep = Hv / Hk;
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static) if (threads > 1)
    for (int vh = 0; vh < Hv; vh++) {
        const int kh = vh / rep;
        float *S = ssm_state + (size_t)vh * dv * dk;
        const float *kk = lk + (size_t)kh * dk, *qq = lq + (size_t)kh * dk, *vv = lv + (size_t)vh * dv;
        const float g = g_decay[vh], bg = b_gate[vh];
        for (int i = 0; i < dv * dk; i++) S[i] *= g;
        for (int vi = 0; vi < dv; vi++) {
            float *row = S + (size_t)vi * dk;
            float mem = 0.0f;
            for (int ki = 0; ki < dk; ki++) mem += row[ki] * kk[ki];
            const float delta = (vv[vi] - mem) * bg;
            for (int ki = 0; ki < dk; ki++) row[ki] += kk[ki] * delta;
        }
        for (int vi = 0; vi < dv; vi++) {
            const float *row = S + (size_t)vi * dk;
            float sum = 0.0f;
            for (int ki = 0; ki < dk; ki++) sum += row[ki] * qq[ki];
            o[(size_t)vh * dv + vi] = sum;
        }
    }

    /* gated RMS-norm: o * rsqrt(mean o^2 + eps) * w * silu(z) (metal_infer/layer_forward.h:787-797) */
    for (int vh = 0; vh < Hv; vh++) {
        const float *oh = o + (size_t)vh * dv, *zh = z + (size_t)vh * dv;
        float *gh = out + (size_t)vh * dv;
        if (!norm_w) {
            memcpy(gh, oh, (size_t)dv * sizeof(float));
            continue;
        }
        float ss = 0.0f;
        for (int i = 0; i < dv; i++) ss += oh[i] * oh[i];
        const float inv = 1.0f / sqrtf(ss / dv + d->rms_norm_eps);
        for (int i = 0; i < dv; i++) {
            const float w = bf16f(norm_w[i]);
            const float sz = zh[i] / (1.0f + expf(-zh[i]));
            gh[i] = oh[i] * inv * w * sz;
        }
    }
    free(c);
    free(g_decay);
    free(b_gate);
    free(o);
    return 0;
}

int fmo_gdn_run(const FmoDims *d, float *conv_state, float *ssm_state, const float *qkv,
                const float *z, const float *beta, const float *alpha, const uint16_t *conv_w,
                const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, int n,
                float *out, int threads) {
    const size_t conv_dim = (size_t)(2 * d->linear_num_k_heads * d->linear_key_dim +
                                     d->linear_num_v_heads * d->linear_value_dim);
    const size_t vdim = (size_t)d->linear_num_v_heads * d->linear_value_dim;
    const size_t hv = (size_t)d->linear_num_v_heads;
    for (int t = 0; t < n; t++) {
        fmo_gdn_step(d, conv_state, ssm_state, qkv + t * conv_dim, z + t * vdim, beta + t * hv,
                     alpha + t * hv, conv_w, A_log, dt_bias, norm_w, out + t * vdim, threads);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* FP8 E4M3 codec of the KV cache (metal_infer/fp8.h:19-118), restated: per-row scale = absmax / 240
   (1 for an all-zero row); 3-bit mantissa rounded half up; magnitudes below 2^-6 that are not below 2^-9 go
   through the normal-number branch with the exponent clamped to -6, whose negative mantissa term is OR-ed into
   the byte as a two's-complement int; the decoder knows 0x7F as the only NaN. */
static uint8_t e4m3_encode(float x, float inv_scale) {
    float scaled = x * inv_scale;
    if (scaled != scaled) return 0x7F;
    scaled = fminf(fmaxf(scaled, -448.0f), 448.0f);
    uint32_t bits;
    memcpy(&bits, &scaled, sizeof bits);
    const uint8_t sign = (bits >> 31) & 1;
    const float mag = fabsf(scaled);
    if (mag < 0.001953125f) {
        int m = (int)(mag / 0.001953125f + 0.5f);
        if (m > 7) m = 7;
        return (uint8_t)((sign << 7) | m);
    }
    int e = (int)floorf(log2f(mag));
    if (e < -6) e = -6;
    if (e > 8) e = 8;
    const float frac = mag / powf(2.0f, (float)e) - 1.0f;
    int mant = (int)(frac * 8.0f + 0.5f);
    if (mant > 7) { mant = 0; e++; }
    int eb = e + 7;
    if (eb < 0) { eb = 0; mant = 0; }
    if (eb > 15) { eb = 15; mant = 6; }
    if (eb == 15 && mant >= 7) mant = 6;
    return (uint8_t)((sign << 7) | (eb << 3) | mant);
}

static float e4m3_value(uint8_t x) { /* the byte's value before the scale (NaN for 0x7F) */
    if (x == 0x7F) return NAN;
    const int eb = (x >> 3) & 0xF, mant = x & 7;
    float val = eb == 0 ? (float)mant * 0.001953125f : (1.0f + (float)mant / 8.0f) * powf(2.0f, (float)eb - 7.0f);
    return (x & 0x80) ? -val : val;
}

void fmo_fp8_encode_rows(const float *src, int n, int kv_dim, uint8_t *dst, float *scales) {
    for (int i = 0; i < n; i++) {
        const float *r = src + (size_t)i * kv_dim;
        float amax = 0.0f;
        for (int j = 0; j < kv_dim; j++) {
            const float a = fabsf(r[j]);
            if (a > amax) amax = a;
        }
        const float scale = amax > 0.0f ? amax / 240.0f : 1.0f;
        const float inv = 1.0f / scale;
        for (int j = 0; j < kv_dim; j++) dst[(size_t)i * kv_dim + j] = e4m3_encode(r[j], inv);
        scales[i] = scale;
    }
}

void fmo_fp8_decode_rows(const uint8_t *src, const float *scales, int n, int kv_dim, float *dst) {
    for (int i = 0; i < n; i++)
        for (int j = 0; j < kv_dim; j++) dst[(size_t)i * kv_dim + j] = e4m3_value(src[(size_t)i * kv_dim + j]) * scales[i];
}

/* H2O eviction (metal_infer/layer_forward.h:265-383): keep the first `sinks` rows, the last `recent` rows and,
   of the rows between, the `budget - sinks - recent` with the largest accumulated attention mass (selection in
   the reference's order: repeated arg-max with strict >, so ties go to the earlier row), compacted in
   temporal order. */
static void h2o_evict(const FmoDims *d, FmoCache *c) {
    if (c->h2o_num_valid <= c->h2o_budget) return;
    const int num_valid = c->h2o_num_valid, budget = c->h2o_budget;
    int sinks = c->h2o_num_sinks, recent = c->h2o_num_recent;
    if (sinks > budget) sinks = budget;
    if (sinks + recent > budget) recent = budget - sinks;
    const int heavy = budget - sinks - recent;
    const int ev0 = sinks, ev1 = num_valid - recent, nev = ev1 - ev0;
    if (nev <= 0 || heavy >= nev) return;
    int *idx = malloc((size_t)nev * sizeof(int));
    float *sc = malloc((size_t)nev * sizeof(float));
    for (int i = 0; i < nev; i++) { idx[i] = ev0 + i; sc[i] = c->attn_scores_accum[ev0 + i]; }
    for (int i = 0; i < heavy && i < nev; i++) {
        int mi = i;
        for (int j = i + 1; j < nev; j++)
            if (sc[j] > sc[mi]) mi = j;
        if (mi != i) {
            const float ts = sc[i]; sc[i] = sc[mi]; sc[mi] = ts;
            const int ti = idx[i]; idx[i] = idx[mi]; idx[mi] = ti;
        }
    }
    int *keep = malloc((size_t)budget * sizeof(int));
    int nk = 0;
    for (int i = 0; i < sinks && i < num_valid; i++) keep[nk++] = i;
    for (int i = 0; i < heavy - 1; i++)          /* heavy hitters back in temporal order */
        for (int j = i + 1; j < heavy; j++)
            if (idx[j] < idx[i]) { const int t = idx[i]; idx[i] = idx[j]; idx[j] = t; }
    for (int i = 0; i < heavy; i++) keep[nk++] = idx[i];
    for (int i = num_valid - recent; i < num_valid; i++) keep[nk++] = i;
    const size_t kv_dim = (size_t)d->num_kv_heads * d->head_dim;
    for (int dst = 0; dst < nk; dst++) {
        const int src = keep[dst];
        if (src == dst) continue;
        if (c->use_fp8) {
            memmove(c->k8 + dst * kv_dim, c->k8 + src * kv_dim, kv_dim);
            memmove(c->v8 + dst * kv_dim, c->v8 + src * kv_dim, kv_dim);
            c->k_scales[dst] = c->k_scales[src];
            c->v_scales[dst] = c->v_scales[src];
        } else {
            memmove(c->k_cache + dst * kv_dim, c->k_cache + src * kv_dim, kv_dim * sizeof(float));
            memmove(c->v_cache + dst * kv_dim, c->v_cache + src * kv_dim, kv_dim * sizeof(float));
        }
        c->attn_scores_accum[dst] = c->attn_scores_accum[src];
        c->token_positions[dst] = c->token_positions[src];
    }
    c->h2o_num_valid = nk;
    free(idx); free(sc); free(keep);
}

/* One decode step with the cache policies of metal_infer/layer_forward.h:591-727: where the row goes (H2O: the
   next compacted slot; window: len % capacity; else len), FP8 quantisation of the appended row, rows attended,
   per-position softmax mass summed over heads for H2O, eviction after the step. */
int fmo_attn_step_cache(const FmoDims *d, FmoCache *c, const float *q_in, const float *gate, const float *k_in,
                        const float *v_in, const uint16_t *q_norm_w, const uint16_t *k_norm_w, int pos, float *out,
                        int threads) {
    const int H = d->num_attn_heads, Hkv = d->num_kv_heads, D = d->head_dim;
    const int q_dim = H * D, kv_dim = Hkv * D;
    const int h2o = c->h2o_budget > 0;
    const int W = h2o ? 0 : c->window_size;
    if (W > 0 && c->capacity != W) return -1;
    int cache_pos;
    if (h2o) {
        cache_pos = c->h2o_num_valid;
        if (cache_pos >= c->capacity) return -1;
    } else if (W > 0) {
        cache_pos = c->len % c->capacity;
    } else {
        cache_pos = c->len;
        if (cache_pos >= c->capacity) return -1;
    }
    float *q = malloc((size_t)q_dim * sizeof(float));
    float *k = malloc((size_t)kv_dim * sizeof(float));
    memcpy(q, q_in, (size_t)q_dim * sizeof(float));
    memcpy(k, k_in, (size_t)kv_dim * sizeof(float));
    head_rms_norm(q, H, D, q_norm_w, d->rms_norm_eps);
    head_rms_norm(k, Hkv, D, k_norm_w, d->rms_norm_eps);
    rope_heads(d, q, H, pos);
    rope_heads(d, k, Hkv, pos);
    if (c->use_fp8) {
        fmo_fp8_encode_rows(k, 1, kv_dim, c->k8 + (size_t)cache_pos * kv_dim, c->k_scales + cache_pos);
        fmo_fp8_encode_rows(v_in, 1, kv_dim, c->v8 + (size_t)cache_pos * kv_dim, c->v_scales + cache_pos);
    } else {
        float *kr = c->k_cache + (size_t)cache_pos * kv_dim, *vr = c->v_cache + (size_t)cache_pos * kv_dim;
        memcpy(kr, k, (size_t)kv_dim * sizeof(float));
        memcpy(vr, v_in, (size_t)kv_dim * sizeof(float));
        if (d->store_bf16)
            for (int i = 0; i < kv_dim; i++) { kr[i] = round_bf16f(kr[i]); vr[i] = round_bf16f(vr[i]); }
    }
    if (h2o) {
        c->token_positions[cache_pos] = c->len;
        c->attn_scores_accum[cache_pos] = 0.0f;
        c->h2o_num_valid++;
    }
    c->len++;
    const int wrapped = !h2o && W > 0 && c->len > W;
    const int L = h2o ? c->h2o_num_valid : (wrapped ? W : c->len);
    const int first = wrapped ? c->len - W : 0;
    const int group = H / Hkv;
    const float scale = (1.0f / sqrtf((float)D)) * yarn_logit_factor(d);
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = e4m3_value((uint8_t)i);

    memset(out, 0, (size_t)q_dim * sizeof(float));
    float *mass = h2o ? calloc((size_t)H * L, sizeof(float)) : NULL;  /* per head, summed in head order below */
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static) if (threads > 1)
    for (int h = 0; h < H; h++) {
        const int kvh = h / group;
        const float *qh = q + (size_t)h * D;
        float *s = malloc((size_t)L * sizeof(float));
        float *deq = c->use_fp8 ? malloc((size_t)D * sizeof(float)) : NULL;
        for (int i = 0; i < L; i++) {
            const int p = wrapped ? (first + i) % c->capacity : i;
            const float *kp;
            if (c->use_fp8) {
                const uint8_t *kb = c->k8 + (size_t)p * kv_dim + (size_t)kvh * D;
                const float sc = c->k_scales[p];
                for (int e = 0; e < D; e++) deq[e] = lut[kb[e]] * sc;
                kp = deq;
            } else {
                kp = c->k_cache + (size_t)p * kv_dim + (size_t)kvh * D;
            }
            float dot = 0.0f;
            for (int e = 0; e < D; e++) dot += qh[e] * kp[e];
            s[i] = dot * scale;
        }
        softmax_inplace(s, L);
        if (mass) memcpy(mass + (size_t)h * L, s, (size_t)L * sizeof(float));
        float *oh = out + (size_t)h * D;
        for (int i = 0; i < L; i++) {
            const int p = wrapped ? (first + i) % c->capacity : i;
            const float *vp;
            if (c->use_fp8) {
                const uint8_t *vb = c->v8 + (size_t)p * kv_dim + (size_t)kvh * D;
                const float sc = c->v_scales[p];
                for (int e = 0; e < D; e++) deq[e] = lut[vb[e]] * sc;
                vp = deq;
            } else {
                vp = c->v_cache + (size_t)p * kv_dim + (size_t)kvh * D;
            }
            for (int e = 0; e < D; e++) oh[e] += s[i] * vp[e];
        }
        free(s);
        free(deq);
    }
    if (h2o) {
        /* sum over heads in head order, then into the running totals (metal_infer/layer_forward.h:694-699, 256-261) */
        for (int i = 0; i < L && i < c->h2o_num_valid; i++) {
            float step = 0.0f;
            for (int h = 0; h < H; h++) step += mass[(size_t)h * L + i];
            c->attn_scores_accum[i] += step;
        }
        free(mass);
        h2o_evict(d, c);
    }
    for (int i = 0; i < q_dim; i++) {
        const float g = 1.0f / (1.0f + expf(-gate[i]));
        out[i] *= g;
    }
    free(q);
    free(k);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* 4-bit affine dequantising matvec (metal_infer/cpu_kernels.h:199-232), residual add (a + b, metal_infer/
   shaders.metal:873-882) and RMS-norm with a bf16 weight (metal_infer/cpu_kernels.h:235-246), in the reference's
   operation order: one fp32 accumulator per output row, groups and nibbles in ascending order. */
void fmo_out_proj_norm(const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int out_dim, int in_dim,
                       int group_size, const float *x, const float *residual, const uint16_t *norm_w, float eps,
                       float *h_mid, float *h_post) {
    const int num_groups = in_dim / group_size, packed_per_group = group_size / 8, packed_cols = in_dim / 8;
    for (int row = 0; row < out_dim; row++) {
        float acc = 0.0f;
        const uint32_t *w_row = w + (size_t)row * packed_cols;
        for (int g = 0; g < num_groups; g++) {
            const float scale = bf16f(scales[(size_t)row * num_groups + g]), bias = bf16f(biases[(size_t)row * num_groups + g]);
            for (int p = 0; p < packed_per_group; p++) {
                const uint32_t packed = w_row[g * packed_per_group + p];
                const float *xb = x + g * group_size + p * 8;
                for (int n = 0; n < 8; n++) acc += ((float)((packed >> (n * 4)) & 0xF) * scale + bias) * xb[n];
            }
        }
        h_mid[row] = acc;
    }
    if (residual)
        for (int i = 0; i < out_dim; i++) h_mid[i] = residual[i] + h_mid[i];
    if (h_post) {
        float ss = 0.0f;
        for (int i = 0; i < out_dim; i++) ss += h_mid[i] * h_mid[i];
        const float inv = 1.0f / sqrtf(ss / out_dim + eps);
        for (int i = 0; i < out_dim; i++) h_post[i] = h_mid[i] * inv * bf16f(norm_w[i]);
    }
}
