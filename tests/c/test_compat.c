/* C host program in the reference's calling style: a few decode steps of one full-attention layer
 * and one GatedDeltaNet layer through fm_compat.h, checked against the CPU checker (fm_oracle.c is
 * linked into this TEST program only).  Prints PASS/FAIL lines; exit code 0 on success. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "fm_compat.h"
#include "fm_oracle.h"

static unsigned long long rng_state = 88172645463325252ULL;
static float frand(void) { /* xorshift + Box-Muller */
    float u[2];
    for (int i = 0; i < 2; i++) {
        rng_state ^= rng_state << 13; rng_state ^= rng_state >> 7; rng_state ^= rng_state << 17;
        u[i] = ((rng_state >> 11) + 0.5f) * (1.0f / 9007199254740992.0f);
    }
    return sqrtf(-2.0f * logf(u[0])) * cosf(6.2831853f * u[1]);
}
static float bf16r(float x) { unsigned u; memcpy(&u, &x, 4); u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u; memcpy(&x, &u, 4); return x; }
static unsigned short bf16b(float x) { unsigned u; x = bf16r(x); memcpy(&u, &x, 4); return (unsigned short)(u >> 16); }
static double gated_err(const float *a, const float *r, int n) {
    double ss = 0, worst = 0;
    for (int i = 0; i < n; i++) ss += (double)r[i] * r[i];
    const double rms = sqrt(ss / n);
    for (int i = 0; i < n; i++) {
        const double den = fabs(r[i]) > rms ? fabs(r[i]) : rms, e = fabs((double)a[i] - r[i]) / den;
        if (e > worst) worst = e;
    }
    return worst;
}

int main(void) {
    enum { H = 32, HKV = 2, D = 256, CTX = 200, STEPS = 3, CAP = 256 };
    FmConfig cfg;
    fm_default_config(&cfg);
    cfg.num_full_layers = 1; cfg.num_linear_layers = 1; cfg.max_seq_len = CAP;
    if (fm_compat_init(&cfg) != 0) return 2;
    KVCache *kv = kv_cache_new();
    LinearAttnState *la = linear_attn_state_new();
    int fails = 0;

    /* ---- full attention: prefix through fm_kv_import, then decode steps ---- */
    const int kvd = HKV * D, qd = H * D;
    float *kc = calloc((size_t)CAP * kvd, 4), *vc = calloc((size_t)CAP * kvd, 4);
    for (int i = 0; i < CTX * kvd; i++) { kc[i] = bf16r(frand()); vc[i] = bf16r(frand()); }
    if (fm_kv_import(fm_compat_ctx(), 0, 0, kc, vc, CTX) != FM_OK) { fprintf(stderr, "ERROR: %s\n", fm_last_error(fm_compat_ctx())); return 2; }
    kv->len = CTX;
    unsigned short qn[D], kn[D];
    for (int i = 0; i < D; i++) { qn[i] = bf16b(1.0f + 0.1f * frand()); kn[i] = bf16b(1.0f + 0.1f * frand()); }
    FmoDims dims = {H, HKV, D, 64, 1e7f, 1e-6f, 0, 1.0f, 262144, 64, 16, 128, 128, 4, 1};
    int len = CTX;
    float *qp = malloc((size_t)H * 2 * D * 4), *q = malloc(qd * 4), *g = malloc(qd * 4), *k = malloc(kvd * 4), *v = malloc(kvd * 4);
    float *out = malloc(qd * 4), *ref = malloc(qd * 4);
    for (int s = 0; s < STEPS; s++) {
        for (int h = 0; h < H; h++)
            for (int d = 0; d < D; d++) {
                q[h * D + d] = frand(); g[h * D + d] = frand();
                qp[h * 2 * D + d] = q[h * D + d]; qp[h * 2 * D + D + d] = g[h * D + d];
            }
        for (int i = 0; i < kvd; i++) { k[i] = frand(); v[i] = bf16r(frand()); }
        full_attention_core(qp, k, v, qn, kn, kv, CTX + s, out);
        fmo_attn_step(&dims, kc, vc, &len, CAP, q, g, k, v, qn, kn, CTX + s, ref, 4);
        const double e = gated_err(out, ref, qd);
        printf("%s full_attention_core step %d: err %.3g, kv->len %d\n", e <= 2e-3 && kv->len == len ? "PASS" : "FAIL", s, e, kv->len);
        fails += !(e <= 2e-3 && kv->len == len);
    }
    /* overflow: the reference prints an error and returns; the cache is unchanged */
    kv->len = CAP;
    if (fm_kv_import(fm_compat_ctx(), 0, 0, kc, vc, CAP) != FM_OK) return 2;
    full_attention_core(qp, k, v, qn, kn, kv, CAP, out);
    printf("%s overflow leaves len at %d\n", fm_kv_len(fm_compat_ctx(), 0, 0) == CAP ? "PASS" : "FAIL", fm_kv_len(fm_compat_ctx(), 0, 0));
    fails += fm_kv_len(fm_compat_ctx(), 0, 0) != CAP;

    /* ---- GatedDeltaNet: zero state, a few steps ---- */
    enum { HV = 64, HK = 16, DK = 128, CONV = 2 * HK * DK + HV * DK };
    float *conv_state = calloc(3 * CONV, 4), *ssm = calloc((size_t)HV * DK * DK, 4);
    unsigned short *cw = malloc(CONV * 4 * 2), dtb[HV], nw[DK];
    float Alog[HV];
    for (int i = 0; i < CONV * 4; i++) cw[i] = bf16b(0.1f * frand());
    for (int i = 0; i < HV; i++) { dtb[i] = bf16b(0.3f * frand()); Alog[i] = -1.0f + 0.5f * frand(); }
    for (int i = 0; i < DK; i++) nw[i] = bf16b(1.0f + 0.1f * frand());
    float *qkv = malloc(CONV * 4), *z = malloc(HV * DK * 4), be[HV], al[HV], *go = malloc(HV * DK * 4), *gr = malloc(HV * DK * 4);
    for (int s = 0; s < 5; s++) {
        for (int i = 0; i < CONV; i++) qkv[i] = frand();
        for (int i = 0; i < HV * DK; i++) z[i] = frand();
        for (int i = 0; i < HV; i++) { be[i] = frand(); al[i] = frand(); }
        linear_attention_core(qkv, z, be, al, cw, Alog, dtb, nw, la, go);
        fmo_gdn_step(&dims, conv_state, ssm, qkv, z, be, al, cw, Alog, dtb, nw, gr, 4);
        const double e = gated_err(go, gr, HV * DK);
        printf("%s linear_attention_core step %d: err %.3g\n", e <= 5e-3 ? "PASS" : "FAIL", s, e);
        fails += !(e <= 5e-3);
    }
    /* ---- batched prefill: a prompt in chunks of 32 tokens (the reference's MAX_PFB_GPU), both layer kinds, against
     *      sequential checker steps ---- */
    {
        enum { NP = 80, CH = 32 };
        reset_delta_net_state();
        kv->len = 0;
        memset(kc, 0, (size_t)CAP * kvd * 4); memset(vc, 0, (size_t)CAP * kvd * 4);
        memset(conv_state, 0, 3 * CONV * 4); memset(ssm, 0, (size_t)HV * DK * DK * 4);
        float *pq = malloc((size_t)NP * H * 2 * D * 4), *pk = malloc((size_t)NP * kvd * 4), *pv = malloc((size_t)NP * kvd * 4);
        float *po = malloc((size_t)NP * qd * 4), *pr = malloc((size_t)NP * qd * 4), *tq = malloc(qd * 4), *tg = malloc(qd * 4);
        float *lq = malloc((size_t)NP * CONV * 4), *lz = malloc((size_t)NP * HV * DK * 4), *lb = malloc(NP * HV * 4), *la_ = malloc(NP * HV * 4);
        float *lo = malloc((size_t)NP * HV * DK * 4), *lr = malloc((size_t)NP * HV * DK * 4);
        for (size_t i = 0; i < (size_t)NP * H * 2 * D; i++) pq[i] = bf16r(frand());
        for (size_t i = 0; i < (size_t)NP * kvd; i++) { pk[i] = bf16r(frand()); pv[i] = bf16r(frand()); }
        for (size_t i = 0; i < (size_t)NP * CONV; i++) lq[i] = bf16r(frand());
        for (size_t i = 0; i < (size_t)NP * HV * DK; i++) lz[i] = bf16r(frand());
        for (int i = 0; i < NP * HV; i++) { lb[i] = frand(); la_[i] = frand(); }
        int plen = 0;
        for (int t = 0; t < NP; t++) {  /* the checker, token by token */
            for (int h = 0; h < H; h++)
                for (int d = 0; d < D; d++) { tq[h * D + d] = pq[((size_t)t * H + h) * 2 * D + d]; tg[h * D + d] = pq[((size_t)t * H + h) * 2 * D + D + d]; }
            fmo_attn_step(&dims, kc, vc, &plen, CAP, tq, tg, pk + (size_t)t * kvd, pv + (size_t)t * kvd, qn, kn, t, pr + (size_t)t * qd, 4);
            fmo_gdn_step(&dims, conv_state, ssm, lq + (size_t)t * CONV, lz + (size_t)t * HV * DK, lb + t * HV, la_ + t * HV, cw, Alog, dtb, nw,
                         lr + (size_t)t * HV * DK, 4);
        }
        for (int t = 0; t < NP; t += CH) {
            const int n = NP - t < CH ? NP - t : CH;
            batched_prefill_full_attention(pq + (size_t)t * H * 2 * D, pk + (size_t)t * kvd, pv + (size_t)t * kvd, qn, kn, kv, t, n, po + (size_t)t * qd);
            batched_prefill_linear_attention(lq + (size_t)t * CONV, lz + (size_t)t * HV * DK, lb + t * HV, la_ + t * HV, cw, Alog, dtb, nw, la, n,
                                             lo + (size_t)t * HV * DK);
        }
        const double ea = gated_err(po, pr, NP * qd), el = gated_err(lo, lr, NP * HV * DK);
        printf("%s batched_prefill_full_attention: err %.3g, kv->len %d\n", ea <= 2e-3 && kv->len == NP ? "PASS" : "FAIL", ea, kv->len);
        printf("%s batched_prefill_linear_attention: err %.3g\n", el <= 5e-3 ? "PASS" : "FAIL", el);
        fails += !(ea <= 2e-3 && kv->len == NP) + !(el <= 5e-3);
    }
    reset_delta_net_state();
    printf("%s reset_delta_net_state: kv len %d\n", fm_kv_len(fm_compat_ctx(), 0, 0) == 0 ? "PASS" : "FAIL", fm_kv_len(fm_compat_ctx(), 0, 0));
    fails += fm_kv_len(fm_compat_ctx(), 0, 0) != 0;
    kv_cache_free(kv); linear_attn_state_free(la);
    fm_compat_shutdown();
    printf(fails ? "FAILED %d\n" : "ALL PASS\n", fails);
    return fails ? 1 : 0;
}
