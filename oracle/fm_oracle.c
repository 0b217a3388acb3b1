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
