// GatedDeltaNet over a run of n tokens of one sequence, in chunked (WY / UT-transform) form.
//
// The recurrence of metal_infer/layer_forward.h:967-1009, per value head and token t,
//     S <- g_t S ;  d_t = beta_t (v_t - S k_t) ;  S <- S + d_t k_t^T ;  o_t = S q_t ,
// is evaluated 64 tokens at a time.  With c_t the running sum of ln g inside a chunk,
// A[t][i] = beta_t e^{c_t-c_i} (k_t . k_i) for i < t and T = (I + A)^-1 (unit lower triangular):
//     U = T diag(beta) V ,   W = T diag(beta e^{c}) K                       (independent of S)
//     D = U - W S0^T ,       O = diag(e^{c}) Q S0^T + (M o Q K^T) D ,  M[t][i] = e^{c_t-c_i}, i <= t
//     S1 = e^{c_C} S0 + D^T diag(e^{c_C-c}) K .
// The reference has no such form (its batched kernel walks the tokens one by one,
// metal_infer/shaders.metal:2763-2815); results are checked against sequential CPU steps.
//
// Launch sequence:
//   gdn_prep_kernel    per token   : conv + SiLU, q/k normalisation, ln(decay), beta  -> workspace
//   gdn_ring_kernel                : last three raw inputs -> conv history ring
//   gdn_chunk_kernel   per (head, chunk), all chunks in parallel: K K^T, Q K^T, A, then U and W by
//                      forward substitution -> workspace
//   gdn_scan_kernel    per (head, 64-row slice of the state), chunks in sequence: D, O, S
//   gdn_norm_kernel    per (token, head): gated RMS-norm in place
// Contractions run on tensor cores as split tf32 (m16n8k8, two terms per operand, fp32 accumulate);
// the triangular solve, the decay exponentials and the state stay fp32.
#include "fm_device.cuh"
#include "fm_internal.h"
#include "fm_tc.cuh"
#include <cstdlib>

namespace fm {

constexpr int kC = 64;    // chunk length
constexpr int kDH = 128;  // dk = dv

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm volatile("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// acc[16 x 8*NT] += A[16 x K] B[K x 8*NT] for one warp; fa(m, k) and fb(k, n) fetch operands.
// Each operand is split into two tf32 terms (x = hi + lo) and the product taken as
// lo*hi + hi*lo + hi*hi ("3xTF32"): plain tf32 (10 mantissa bits) left the state 5e-3 off the
// sequential fp32 recurrence, this keeps ~21 bits.
__device__ __forceinline__ void split_tf32(float x, uint32_t &hi, uint32_t &lo) {
    hi = to_tf32(x);
    lo = to_tf32(x - __uint_as_float(hi));
}
template <int NT, class FA, class FB>
__device__ __forceinline__ void warp_gemm_tf32(float (&acc)[NT][4], int K, FA fa, FB fb, int lane) {
    const int g = lane >> 2, t = lane & 3;
    for (int k0 = 0; k0 < K; k0 += 8) {
        uint32_t ah[4], al[4];
        split_tf32(fa(g, k0 + t), ah[0], al[0]);
        split_tf32(fa(g + 8, k0 + t), ah[1], al[1]);
        split_tf32(fa(g, k0 + t + 4), ah[2], al[2]);
        split_tf32(fa(g + 8, k0 + t + 4), ah[3], al[3]);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            uint32_t bh0, bl0, bh1, bl1;
            split_tf32(fb(k0 + t, nt * 8 + g), bh0, bl0);
            split_tf32(fb(k0 + t + 4, nt * 8 + g), bh1, bl1);
            mma_tf32(acc[nt], al[0], al[1], al[2], al[3], bh0, bh1);
            mma_tf32(acc[nt], ah[0], ah[1], ah[2], ah[3], bl0, bl1);
            mma_tf32(acc[nt], ah[0], ah[1], ah[2], ah[3], bh0, bh1);
        }
    }
}

struct GdnWork {  // workspace carved by the host
    float *qn, *kn, *vn;  // [n][Hk*128], [n][Hk*128], [n][Hv*128]
    float *lg, *bt;       // [n][Hv]  ln(decay), beta
    float *U, *W;         // [Hv][nchunks][64][128]
    float *QK;            // [Hv][nchunks][64][64]
    float *cv;            // [Hv][nchunks][64]  inclusive running sum of ln(decay)
    float *KT;            // [Hk][nchunks][128][64]  normalised k of each chunk, transposed (key dim major)
};

// ---- per token: conv + SiLU, q/k normalisation, decay, beta ------------------------------------
// grid (n), 512 threads
__global__ void __launch_bounds__(512)
gdn_prep_kernel(GdnDims g, int n, int step0, const float *__restrict__ ring, const float *__restrict__ qkv,
                const float *__restrict__ beta, const float *__restrict__ alpha,
                const uint16_t *__restrict__ conv_w, const float *__restrict__ A_log,
                const uint16_t *__restrict__ dt_bias, GdnWork w) {
    extern __shared__ float s_c[];  // conv output, [conv_dim]
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int C = g.conv_dim, total_k = g.Hk * kDH;
    for (int ch = tid; ch < C; ch += blockDim.x) {
        float acc = 0.f;
        if (conv_w != nullptr) {
#pragma unroll
            for (int j = 0; j < 3; j++) {
                const int tt = t - 3 + j;  // token inside this run, or history before it
                float h;
                if (tt >= 0)
                    h = qkv[(size_t)tt * C + ch];
                else {
                    const int tokidx = step0 + tt;
                    h = tokidx >= 0 ? ring[(size_t)(tokidx & 3) * C + ch] : 0.f;
                }
                acc += h * bf16_bits_to_float(conv_w[ch * 4 + j]);
            }
            acc += qkv[(size_t)t * C + ch] * bf16_bits_to_float(conv_w[ch * 4 + 3]);
            acc = acc / (1.0f + expf(-acc));
        }
        s_c[ch] = acc;
    }
    __syncthreads();
    // q and k heads: one warp per head, 4 channels per lane
    const float inv_scale = 1.0f / sqrtf((float)kDH);
    for (int hh = warp; hh < 2 * g.Hk; hh += blockDim.x / 32) {
        const bool is_q = hh < g.Hk;
        const float *src = s_c + (size_t)hh * kDH;  // q heads then k heads are contiguous in conv_out
        const float4 x = *reinterpret_cast<const float4 *>(src + lane * 4);
        const float ss = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
        const float inv = 1.0f / sqrtf(ss / kDH + 1e-6f);
        const float mul = is_q ? inv_scale * inv_scale : inv_scale;
        float4 y = make_float4(x.x * inv * mul, x.y * inv * mul, x.z * inv * mul, x.w * inv * mul);
        float *dst = (is_q ? w.qn : w.kn) + (size_t)t * total_k + (size_t)(is_q ? hh : hh - g.Hk) * kDH;
        *reinterpret_cast<float4 *>(dst + lane * 4) = y;
    }
    const int total_v = g.Hv * kDH;
    for (int i = tid * 4; i < total_v; i += blockDim.x * 4)
        *reinterpret_cast<float4 *>(w.vn + (size_t)t * total_v + i) = *reinterpret_cast<const float4 *>(s_c + 2 * total_k + i);
    for (int vh = tid; vh < g.Hv; vh += blockDim.x) {
        const float bias = dt_bias ? bf16_bits_to_float(dt_bias[vh]) : 0.f;
        const float A = A_log ? expf(A_log[vh]) : 1.0f;
        const float sp = logf(1.0f + expf(alpha[(size_t)t * g.Hv + vh] + bias));
        w.lg[(size_t)t * g.Hv + vh] = -A * sp;  // ln of the decay
        w.bt[(size_t)t * g.Hv + vh] = 1.0f / (1.0f + expf(-beta[(size_t)t * g.Hv + vh]));
    }
}

// raw inputs of the last min(n, 3) tokens -> ring slots (token count & 3)
__global__ void gdn_ring_kernel(int C, int n, int step0, float *__restrict__ ring, const float *__restrict__ qkv) {
    const int first = n > 3 ? n - 3 : 0;
    for (int t = first + blockIdx.y; t < n; t += gridDim.y)
        for (int ch = blockIdx.x * blockDim.x + threadIdx.x; ch < C; ch += gridDim.x * blockDim.x)
            ring[(size_t)((step0 + t) & 3) * C + ch] = qkv[(size_t)t * C + ch];
}

// ---- per (head, chunk): everything that does not depend on the state ---------------------------
constexpr int kLdK = kDH + 4;   // [row][k] operands read as (row g, k t): stride = 4 mod 32
constexpr int kLdT = kC + 4;
constexpr int kChunkSmem = (3 * kC * kLdK + 2 * kC * kLdT + 2 * kC) * 4;

// grid (nchunks, Hv), 256 threads
__global__ void __launch_bounds__(256, 1)
gdn_chunk_kernel(GdnDims g, int n, GdnWork w, int nchunks) {
    extern __shared__ __align__(16) float sm[];
    float *sK = sm, *sQ = sK + kC * kLdK, *sV = sQ + kC * kLdK;
    float *sA = sV + kC * kLdK, *sT = sA + kC * kLdT;
    float *sc = sT + kC * kLdT, *sb = sc + kC;
    const int chunk = blockIdx.x, vh = blockIdx.y, kh = vh / (g.Hv / g.Hk);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = chunk * kC;
    const int total_k = g.Hk * kDH, total_v = g.Hv * kDH;

    // rows past the end of the run are zero (beta 0, decay 1: they leave the state alone)
    for (int i = tid; i < kC * (kDH / 4); i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), q4 = k4, v4 = k4;
        if (t0 + r < n) {
            k4 = *reinterpret_cast<const float4 *>(w.kn + (size_t)(t0 + r) * total_k + (size_t)kh * kDH + c4);
            q4 = *reinterpret_cast<const float4 *>(w.qn + (size_t)(t0 + r) * total_k + (size_t)kh * kDH + c4);
            v4 = *reinterpret_cast<const float4 *>(w.vn + (size_t)(t0 + r) * total_v + (size_t)vh * kDH + c4);
        }
        *reinterpret_cast<float4 *>(sK + r * kLdK + c4) = k4;
        *reinterpret_cast<float4 *>(sQ + r * kLdK + c4) = q4;
        *reinterpret_cast<float4 *>(sV + r * kLdK + c4) = v4;
    }
    if (warp == 0) {  // inclusive scan of ln(decay) over the 64 rows, two per lane
        float a = (t0 + lane < n) ? w.lg[(size_t)(t0 + lane) * g.Hv + vh] : 0.f;
        float b = (t0 + 32 + lane < n) ? w.lg[(size_t)(t0 + 32 + lane) * g.Hv + vh] : 0.f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) { a += ua; b += ub; }
        }
        b += __shfl_sync(0xffffffffu, a, 31);
        sc[lane] = a; sc[32 + lane] = b;
        sb[lane] = (t0 + lane < n) ? w.bt[(size_t)(t0 + lane) * g.Hv + vh] : 0.f;
        sb[32 + lane] = (t0 + 32 + lane < n) ? w.bt[(size_t)(t0 + 32 + lane) * g.Hv + vh] : 0.f;
        float *cv = w.cv + ((size_t)vh * nchunks + chunk) * kC;
        cv[lane] = a; cv[32 + lane] = b;
    }
    __syncthreads();
    if (vh % (g.Hv / g.Hk) == 0) {  // one CTA per key head leaves the chunk's k transposed for the scan
        float *kt = w.KT + ((size_t)kh * nchunks + chunk) * kDH * kC;
        for (int i = tid; i < kDH * kC; i += 256) kt[i] = sK[(i & (kC - 1)) * kLdK + (i >> 6)];
    }

    // K K^T and Q K^T (64 x 64 x 128): warp = (16-row tile, 32-column half)
    {
        const int mt = warp & 3, nh = warp >> 2;
        float akk[4][4] = {}, aqk[4][4] = {};
        const float *Ka = sK + (mt * 16) * kLdK, *Qa = sQ + (mt * 16) * kLdK, *Kb = sK + (nh * 32) * kLdK;
        auto fb = [&](int k, int nn) { return Kb[nn * kLdK + k]; };
        warp_gemm_tf32<4>(akk, kDH, [&](int m, int k) { return Ka[m * kLdK + k]; }, fb, lane);
        warp_gemm_tf32<4>(aqk, kDH, [&](int m, int k) { return Qa[m * kLdK + k]; }, fb, lane);
        float *qk_out = w.QK + ((size_t)vh * nchunks + chunk) * kC * kC;
        const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int r = mt * 16 + gq + (e >> 1) * 8, c = nh * 32 + nt * 8 + 2 * tq + (e & 1);
                const float dec = c <= r ? expf(sc[r] - sc[c]) : 0.f;
                sA[r * kLdT + c] = c < r ? sb[r] * dec * akk[nt][e] : 0.f;
                qk_out[r * kC + c] = dec * aqk[nt][e];
            }
    }
    __syncthreads();
    // (I + A) X = [beta V | beta e^c K] by forward substitution: thread c owns column c of X (a column
    // of U for c < 128, of W otherwise) and keeps its 64 entries in registers; A is read as broadcast
    // 128-bit loads and four partial sums shorten the dependent chain.  This replaces forming
    // T = (I + A)^-1 and multiplying by it.
    if (tid < kC) sT[tid] = sb[tid] * expf(sc[tid]);  // row scale of the K block
    __syncthreads();
    {
        const int c = tid;
        const bool is_u = c < kDH;
        const float *src = is_u ? sV + c : sK + (c - kDH);
        const float *scale = is_u ? sb : sT;
        float x[kC];
#pragma unroll
        for (int r = 0; r < kC; r++) x[r] = src[r * kLdK] * scale[r];
#pragma unroll
        for (int r = 1; r < kC; r++) {
            const float *Ar = sA + r * kLdT;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
            for (int i = 0; i + 3 < r; i += 4) {
                const float4 a = *reinterpret_cast<const float4 *>(Ar + i);
                a0 += a.x * x[i]; a1 += a.y * x[i + 1]; a2 += a.z * x[i + 2]; a3 += a.w * x[i + 3];
            }
#pragma unroll
            for (int i = r & ~3; i < r; i++) a0 += Ar[i] * x[i];
            x[r] -= (a0 + a1) + (a2 + a3);
        }
        float *dst = (is_u ? w.U : w.W) + ((size_t)vh * nchunks + chunk) * kC * kDH + (is_u ? c : c - kDH);
#pragma unroll
        for (int r = 0; r < kC; r++) dst[r * kDH] = x[r];
    }
}

// ---- per (head, 64-row slice of the state): walk the chunks ------------------------------------
constexpr int kSl = 64;           // state rows (value dims) per CTA: 64 heads x 2 slices = 128 CTAs, one wave
constexpr int kLdS = kDH + 4;     // S[vi][ki] read as B[n = vi][k = ki]
constexpr int kLdKs = kDH + 8;    // scaled K read as B[k = i][n = ki]
constexpr int kLdD = kSl + 8;     // D[i][vi] read as B[k = i][n = vi] and as A[m = vi][k = i]
constexpr int kScanSmem = (kSl * kLdS + 2 * kC * kLdK + kC * kLdKs + kC * kLdT + kC * kLdD + 2 * kC) * 4;

// grid (128 / kSl, Hv), 256 threads
__global__ void __launch_bounds__(256, 1)
gdn_scan_kernel(GdnDims g, int n, GdnWork w, int nchunks, float *__restrict__ ssm, float *__restrict__ out) {
    extern __shared__ __align__(16) float sm[];
    float *sS = sm, *sW = sS + kSl * kLdS, *sQ = sW + kC * kLdK, *sKs = sQ + kC * kLdK;
    float *sQK = sKs + kC * kLdKs, *sD = sQK + kC * kLdT, *sc = sD + kC * kLdD, *se = sc + kC;
    const int slice = blockIdx.x, vh = blockIdx.y, kh = vh / (g.Hv / g.Hk);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gq = lane >> 2, tq = lane & 3;
    const int total_k = g.Hk * kDH, total_v = g.Hv * kDH;
    float *Sg = ssm + ((size_t)vh * kDH + slice * kSl) * kDH;
    for (int i = tid; i < kSl * (kDH / 4); i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        *reinterpret_cast<float4 *>(sS + r * kLdS + c4) = *reinterpret_cast<const float4 *>(Sg + (size_t)r * kDH + c4);
    }
    for (int chunk = 0; chunk < nchunks; chunk++) {
        const int t0 = chunk * kC;
        const size_t hc = (size_t)vh * nchunks + chunk;
        __syncthreads();  // previous chunk's readers are done with every buffer
        if (tid < kC) {
            const float c = w.cv[hc * kC + tid];
            sc[tid] = c;
        }
        {
            const float *Wg = w.W + hc * kC * kDH, *QKg = w.QK + hc * kC * kC;
            for (int i = tid; i < kC * (kDH / 4); i += 256) {
                const int r = i >> 5, c4 = (i & 31) * 4;
                cp_async16(smem_u32(sW + r * kLdK + c4), Wg + (size_t)r * kDH + c4);
                if (t0 + r < n) {
                    cp_async16(smem_u32(sQ + r * kLdK + c4), w.qn + (size_t)(t0 + r) * total_k + (size_t)kh * kDH + c4);
                    cp_async16(smem_u32(sKs + r * kLdKs + c4), w.kn + (size_t)(t0 + r) * total_k + (size_t)kh * kDH + c4);
                } else {
                    *reinterpret_cast<float4 *>(sQ + r * kLdK + c4) = make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4 *>(sKs + r * kLdKs + c4) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            for (int i = tid; i < kC * (kC / 4); i += 256) {
                const int r = i >> 4, c4 = (i & 15) * 4;
                cp_async16(smem_u32(sQK + r * kLdT + c4), QKg + (size_t)r * kC + c4);
            }
            cp_async_commit();
            cp_async_wait<0>();
        }
        __syncthreads();
        const float cC = sc[kC - 1];
        if (tid < kC) se[tid] = expf(cC - sc[tid]);
        __syncthreads();
        for (int i = tid; i < kC * kDH; i += 256) {  // K rows scaled for the state update
            const int r = i >> 7, c = i & 127;
            sKs[r * kLdKs + c] *= se[r];
        }
        // D = U - W S^T and Q S^T: warp = (16 token rows, 32 of the slice's 64 state rows)
        const int mtok = warp & 3, nhs = warp >> 2;
        float ad[4][4] = {}, aq[4][4] = {};
        {
            const float *Wa = sW + (mtok * 16) * kLdK, *Qa = sQ + (mtok * 16) * kLdK;
            auto fb = [&](int k, int nn) { return sS[(nhs * 32 + nn) * kLdS + k]; };
            warp_gemm_tf32<4>(ad, kDH, [&](int m, int k) { return Wa[m * kLdK + k]; }, fb, lane);
            warp_gemm_tf32<4>(aq, kDH, [&](int m, int k) { return Qa[m * kLdK + k]; }, fb, lane);
            const float *Ug = w.U + hc * kC * kDH + slice * kSl;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int r = mtok * 16 + gq, c = nhs * 32 + nt * 8 + 2 * tq;
                const float2 u0 = *reinterpret_cast<const float2 *>(Ug + (size_t)r * kDH + c);
                const float2 u1 = *reinterpret_cast<const float2 *>(Ug + (size_t)(r + 8) * kDH + c);
                sD[r * kLdD + c] = u0.x - ad[nt][0];
                sD[r * kLdD + c + 1] = u0.y - ad[nt][1];
                sD[(r + 8) * kLdD + c] = u1.x - ad[nt][2];
                sD[(r + 8) * kLdD + c + 1] = u1.y - ad[nt][3];
                const float e0 = expf(sc[r]), e1 = expf(sc[r + 8]);
                aq[nt][0] *= e0; aq[nt][1] *= e0; aq[nt][2] *= e1; aq[nt][3] *= e1;
            }
        }
        __syncthreads();  // D complete; S fully read
        // O = e^{c} Q S^T + (M o Q K^T) D
        {
            const float *QKa = sQK + (mtok * 16) * kLdT;
            warp_gemm_tf32<4>(aq, kC, [&](int m, int k) { return QKa[m * kLdT + k]; },
                              [&](int k, int nn) { return sD[k * kLdD + nhs * 32 + nn]; }, lane);
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int r = mtok * 16 + gq, c = slice * kSl + nhs * 32 + nt * 8 + 2 * tq;
                if (t0 + r < n)
                    *reinterpret_cast<float2 *>(out + (size_t)(t0 + r) * total_v + (size_t)vh * kDH + c) = make_float2(aq[nt][0], aq[nt][1]);
                if (t0 + r + 8 < n)
                    *reinterpret_cast<float2 *>(out + (size_t)(t0 + r + 8) * total_v + (size_t)vh * kDH + c) = make_float2(aq[nt][2], aq[nt][3]);
            }
        }
        // S <- e^{c_C} S + D^T (e^{c_C - c} K): warp = (16 state rows, 64 key columns)
        {
            const int mt = warp & 3, nh = warp >> 2;
            const float eC = expf(cC);
            float as[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const int r = mt * 16 + gq, c = nh * 64 + nt * 8 + 2 * tq;
                as[nt][0] = eC * sS[r * kLdS + c]; as[nt][1] = eC * sS[r * kLdS + c + 1];
                as[nt][2] = eC * sS[(r + 8) * kLdS + c]; as[nt][3] = eC * sS[(r + 8) * kLdS + c + 1];
            }
            warp_gemm_tf32<8>(as, kC, [&](int m, int k) { return sD[k * kLdD + mt * 16 + m]; },
                              [&](int k, int nn) { return sKs[k * kLdKs + nh * 64 + nn]; }, lane);
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                const int r = mt * 16 + gq, c = nh * 64 + nt * 8 + 2 * tq;
                sS[r * kLdS + c] = as[nt][0]; sS[r * kLdS + c + 1] = as[nt][1];
                sS[(r + 8) * kLdS + c] = as[nt][2]; sS[(r + 8) * kLdS + c + 1] = as[nt][3];
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < kSl * (kDH / 4); i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        *reinterpret_cast<float4 *>(Sg + (size_t)r * kDH + c4) = *reinterpret_cast<const float4 *>(sS + r * kLdS + c4);
    }
}

// ---- the scan on the 5th-generation tensor cores ------------------------------------------------
// One CTA per value head walks the chunks with the state in tensor memory, transposed so that the
// state row (value dim v) is the TMEM lane and every product has its A operand in TMEM and a K-major
// B tile brought by TMA:
//     Dt[v][t]  = U[t][v] - sum_k S[v][k] W[t][k]                     (M128 N64  K128)
//     O1[v][t]  = sum_k S[v][k] Q[t][k]                                (M128 N64  K128)
//     O2[v][t]  = sum_i Dt[v][i] QKm[t][i]                             (M128 N64  K64)
//     S[v][k]   = e^{cC} S[v][k] + sum_i Dt[v][i] e^{cC-c_i} K[i][k]   (M128 N128 K64, B = scaled K^T)
//     out[t][v] = e^{c_t} O1[v][t] + O2[v][t]
// kind::tf32 reads 19 bits of each operand, so the recurrent operands enter as two terms: the TMEM
// operands S and Dt keep a second copy of their truncated remainder (x - tf32(x)), and W and the
// B tiles (W, Q, QKm, scaled K) get a remainder tile in shared memory; the cross terms hi*lo and lo*hi
// are extra MMAs into the same accumulator ("3xTF32").
//   warps 0-3   one state row per thread: initial S -> TMEM, per chunk U - acc -> Dt (+ remainder),
//               S *= e^{cC}, remainder of the new S, output rows
//   warp 4      TMA producer (single-buffered tiles: W, Q are free again after the first product
//               group, QKm, K^T after the second)
//   warp 5      MMA issuer
//   warps 6-9   operand preparation in shared memory: decay tables, remainder tiles, scaled K^T
// TMEM: S 128 + S remainder 128 + Dt 64 + Dt remainder 64 + O1 64 + O2 64 = 512 columns.
// Every mbarrier wait is bounded; on expiry the CTA records an error code and winds down.
constexpr int kScThreads = 320;
constexpr uint32_t kTcS = 0, kTcSl = 128, kTcD = 256, kTcDl = 320, kTcO1 = 384, kTcO2 = 448;
constexpr int kSlab64 = 64 * 128;    // bytes of one 32-float-wide slab of a 64-row tile
constexpr int kSlab128 = 128 * 128;  // ... of a 128-row tile
constexpr int kOffW = 0, kOffWl = 32768, kOffQ = 65536, kOffQl = 98304, kOffQK = 131072, kOffQKl = 147456, kOffKT = 163840,
              kOffKTl = 196608;
constexpr int kOffTab = 229376;      // 2 x [64 K-row scales | 64 output scales | e^{cC} ...] floats
constexpr int kTabFloats = 144;
constexpr int kOffBar = kOffTab + 2 * kTabFloats * 4;
enum ScBar { SB_SREADY = 0, SB_WQFULL, SB_WLFULL, SB_KQKFULL, SB_KSFULL, SB_CVFULL, SB_DACC, SB_QDONE, SB_WEMPTY, SB_DFULL,
             SB_SSCALED, SB_CDONE, SB_KEMPTY, SB_OFREE, SB_COUNT };
constexpr int kScSmem = kOffBar + SB_COUNT * 8 + 1024 /*alignment slack*/;

__device__ __forceinline__ float tf32_rest(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

struct ScanParams {
    int n, nchunks, Hv, Hk;
    const float *U, *cv;
    float *ssm, *out;
    int *err;
};

__global__ void __launch_bounds__(kScThreads, 1)
gdn_scan_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_qk, const __grid_constant__ CUtensorMap map_kt, ScanParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *gbase = smem_raw + (base - smem_u32(smem_raw));
    auto bar = [&](int i) { return base + kOffBar + 8u * (uint32_t)i; };
    float *tabs = reinterpret_cast<float *>(gbase + kOffTab);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vh = blockIdx.x, kh = vh / (p.Hv / p.Hk);
    const int nchunks = p.nchunks;

    if (tid == 0) {
        s_abort = 0;
        mbar_init(bar(SB_SREADY), 128);
        mbar_init(bar(SB_WQFULL), 1);
        mbar_init(bar(SB_WLFULL), 128);
        mbar_init(bar(SB_KQKFULL), 1);
        mbar_init(bar(SB_KSFULL), 128);
        mbar_init(bar(SB_CVFULL), 128);
        mbar_init(bar(SB_DACC), 1);
        mbar_init(bar(SB_QDONE), 1);
        mbar_init(bar(SB_WEMPTY), 1);
        mbar_init(bar(SB_DFULL), 128);
        mbar_init(bar(SB_SSCALED), 128);
        mbar_init(bar(SB_CDONE), 1);
        mbar_init(bar(SB_KEMPTY), 1);
        mbar_init(bar(SB_OFREE), 128);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    volatile int *abortp = &s_abort;

    if (warp == 4) {
        // ================= TMA producer =================
        if (lane == 0) {
            for (int j = 0; j < nchunks; j++) {
                const int hc = vh * nchunks + j;
                if (j > 0 && !mbar_wait(bar(SB_WEMPTY), (j - 1) & 1, abortp)) break;
                mbar_expect_tx(bar(SB_WQFULL), 65536);
                for (int s = 0; s < 4; s++) tma_load_2d(base + kOffW + s * kSlab64, &map_w, s * 32, hc * kC, bar(SB_WQFULL));
                for (int s = 0; s < 4; s++) tma_load_2d(base + kOffQ + s * kSlab64, &map_q, kh * kDH + s * 32, j * kC, bar(SB_WQFULL));
                if (j > 0 && !mbar_wait(bar(SB_KEMPTY), (j - 1) & 1, abortp)) break;
                mbar_expect_tx(bar(SB_KQKFULL), 16384 + 32768);
                for (int s = 0; s < 2; s++) tma_load_2d(base + kOffQK + s * kSlab64, &map_qk, s * 32, hc * kC, bar(SB_KQKFULL));
                for (int s = 0; s < 2; s++)
                    tma_load_2d(base + kOffKT + s * kSlab128, &map_kt, s * 32, (kh * nchunks + j) * kDH, bar(SB_KQKFULL));
            }
        }
    } else if (warp == 5) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t id64 = idesc_dense(128, 64, false, 2), id128 = idesc_dense(128, 128, false, 2);
            const uint64_t dW = smem_desc(base + kOffW, 16, 1024), dWl = smem_desc(base + kOffWl, 16, 1024);
            const uint64_t dQ = smem_desc(base + kOffQ, 16, 1024), dQK = smem_desc(base + kOffQK, 16, 1024);
            const uint64_t dQl = smem_desc(base + kOffQl, 16, 1024), dQKl = smem_desc(base + kOffQKl, 16, 1024);
            const uint64_t dKT = smem_desc(base + kOffKT, 16, 1024), dKTl = smem_desc(base + kOffKTl, 16, 1024);
            auto k64 = [](int ks) { return (uint64_t)((((ks >> 2) * kSlab64) + (ks & 3) * 32) >> 4); };
            auto k128 = [](int ks) { return (uint64_t)((((ks >> 2) * kSlab128) + (ks & 3) * 32) >> 4); };
            for (int j = 0; j < nchunks; j++) {
                const uint32_t ph = j & 1;
                bool ok = mbar_wait(bar(SB_SREADY), ph, abortp) && mbar_wait(bar(SB_WQFULL), ph, abortp) && mbar_wait(bar(SB_WLFULL), ph, abortp);
                if (!ok) break;
                tc_fence_after();
                // Dt = S W^T, three terms
#pragma unroll
                for (int ks = 0; ks < 16; ks++) tc_mma_tf32_ta(tmem + kTcD, tmem + kTcS + ks * 8, dW + k64(ks), id64, ks > 0);
#pragma unroll
                for (int ks = 0; ks < 16; ks++) tc_mma_tf32_ta(tmem + kTcD, tmem + kTcSl + ks * 8, dW + k64(ks), id64, 1);
#pragma unroll
                for (int ks = 0; ks < 16; ks++) tc_mma_tf32_ta(tmem + kTcD, tmem + kTcS + ks * 8, dWl + k64(ks), id64, 1);
                tc_commit(bar(SB_DACC));
                // O1 = S Q^T: the output accumulators of the previous chunk must have been read out
                if (j > 0 && !mbar_wait(bar(SB_OFREE), (j - 1) & 1, abortp)) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 16; ks++) tc_mma_tf32_ta(tmem + kTcO1, tmem + kTcS + ks * 8, dQ + k64(ks), id64, ks > 0);
#pragma unroll
                for (int ks = 0; ks < 16; ks++) tc_mma_tf32_ta(tmem + kTcO1, tmem + kTcSl + ks * 8, dQ + k64(ks), id64, 1);
#pragma unroll
                for (int ks = 0; ks < 16; ks++) tc_mma_tf32_ta(tmem + kTcO1, tmem + kTcS + ks * 8, dQl + k64(ks), id64, 1);
                tc_commit(bar(SB_QDONE));
                tc_commit(bar(SB_WEMPTY));
                // O2 = Dt QKm^T
                ok = mbar_wait(bar(SB_DFULL), ph, abortp) && mbar_wait(bar(SB_KQKFULL), ph, abortp) && mbar_wait(bar(SB_KSFULL), ph, abortp);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_tf32_ta(tmem + kTcO2, tmem + kTcD + ks * 8, dQK + k64(ks), id64, ks > 0);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_tf32_ta(tmem + kTcO2, tmem + kTcDl + ks * 8, dQK + k64(ks), id64, 1);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_tf32_ta(tmem + kTcO2, tmem + kTcD + ks * 8, dQKl + k64(ks), id64, 1);
                // S = e^{cC} S + Dt (scaled K^T)^T, three terms
                ok = mbar_wait(bar(SB_SSCALED), ph, abortp);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_tf32_ta(tmem + kTcS, tmem + kTcD + ks * 8, dKT + k128(ks), id128, 1);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_tf32_ta(tmem + kTcS, tmem + kTcDl + ks * 8, dKT + k128(ks), id128, 1);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_tf32_ta(tmem + kTcS, tmem + kTcD + ks * 8, dKTl + k128(ks), id128, 1);
                tc_commit(bar(SB_CDONE));
                tc_commit(bar(SB_KEMPTY));
            }
        }
    } else if (warp >= 6) {
        // ================= operand preparation in shared memory =================
        const int q = tid - 192;  // 0..127
        for (int j = 0; j < nchunks; j++) {
            const uint32_t ph = j & 1;
            const float *cvp = p.cv + ((size_t)vh * nchunks + j) * kC;
            float *tab = tabs + (j & 1) * kTabFloats;
            const float cC = __ldg(cvp + kC - 1);
            if (q < kC) {
                const float c = __ldg(cvp + q);
                tab[q] = expf(cC - c);   // scale of K row q in the state update
                tab[kC + q] = expf(c);   // scale of the S q term of output row q
            }
            if (q == 0) tab[2 * kC] = expf(cC);
            // the table is complete for the preparation threads once all of them have arrived; the state
            // threads read it only after the chunk's first products (which wait for SB_WLFULL below) are done
            mbar_arrive(bar(SB_CVFULL));
            if (!mbar_wait(bar(SB_CVFULL), ph, abortp)) break;
            // remainder tile of W
            if (!mbar_wait(bar(SB_WQFULL), ph, abortp)) break;
            for (int i = q; i < 4096; i += 128) {  // W | Wl | Q | Ql are consecutive 32 KB tiles
                const int o = (i & 2047) * 16 + (i >> 11) * 65536;
                const float4 v = *reinterpret_cast<const float4 *>(gbase + kOffW + o);
                *reinterpret_cast<float4 *>(gbase + kOffWl + o) = make_float4(tf32_rest(v.x), tf32_rest(v.y), tf32_rest(v.z), tf32_rest(v.w));
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            mbar_arrive(bar(SB_WLFULL));
            // K^T tile: column i scaled by e^{cC - c_i}, and its remainder tile
            if (!mbar_wait(bar(SB_KQKFULL), ph, abortp)) break;
            for (int i = q; i < 2048; i += 128) {
                const int o = i * 16, slab = o >> 14, row = (o & 16383) >> 7, lc = ((o >> 4) & 7) ^ (row & 7);
                const float *sc4 = tab + slab * 32 + lc * 4;
                float4 v = *reinterpret_cast<const float4 *>(gbase + kOffKT + o);
                v.x *= sc4[0]; v.y *= sc4[1]; v.z *= sc4[2]; v.w *= sc4[3];
                *reinterpret_cast<float4 *>(gbase + kOffKT + o) = v;
                *reinterpret_cast<float4 *>(gbase + kOffKTl + o) = make_float4(tf32_rest(v.x), tf32_rest(v.y), tf32_rest(v.z), tf32_rest(v.w));
            }
            for (int i = q; i < 1024; i += 128) {  // remainder tile of QKm
                const float4 v = *reinterpret_cast<const float4 *>(gbase + kOffQK + i * 16);
                *reinterpret_cast<float4 *>(gbase + kOffQKl + i * 16) = make_float4(tf32_rest(v.x), tf32_rest(v.y), tf32_rest(v.z), tf32_rest(v.w));
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            // the table of chunk j - 1 is rewritten at the top of chunk j + 1: its last readers (the output
            // rows of chunk j - 1) must be done before this chunk can complete
            if (j > 0 && !mbar_wait(bar(SB_OFREE), (j - 1) & 1, abortp)) break;
            mbar_arrive(bar(SB_KSFULL));
        }
    } else {
        // ================= state rows: one value dim per thread =================
        const int r = tid;  // state row = TMEM lane
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        float *Srow = p.ssm + ((size_t)vh * kDH + r) * kDH;
        const int total_v = p.Hv * kDH;
#pragma unroll 1
        for (int c = 0; c < kDH; c += 32) {
            uint32_t hi[32], lo[32];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 v = *reinterpret_cast<const float4 *>(Srow + c + 4 * i);
                hi[4 * i] = __float_as_uint(v.x); hi[4 * i + 1] = __float_as_uint(v.y);
                hi[4 * i + 2] = __float_as_uint(v.z); hi[4 * i + 3] = __float_as_uint(v.w);
            }
#pragma unroll
            for (int i = 0; i < 32; i++) lo[i] = __float_as_uint(tf32_rest(__uint_as_float(hi[i])));
            tc_st32(tmem + lane_base + kTcS + c, hi);
            tc_st32(tmem + lane_base + kTcSl + c, lo);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(SB_SREADY));
        bool ok = true;
        for (int j = 0; j < nchunks; j++) {
            const uint32_t ph = j & 1;
            const int t0 = j * kC;
            const float *Ug = p.U + ((size_t)vh * nchunks + j) * kC * kDH + r;
            const float *tab = tabs + (j & 1) * kTabFloats;
            // Dt = U - acc, and its remainder
            {
                uint32_t a0[32], a1[32];
                float u[kC];
#pragma unroll
                for (int t = 0; t < kC; t++) u[t] = __ldg(Ug + (size_t)t * kDH);
                ok = __all_sync(0xffffffffu, mbar_wait(bar(SB_DACC), ph, abortp));
                if (!ok) break;
                tc_fence_after();
                tc_ld32(tmem + lane_base + kTcD, a0);
                tc_ld32(tmem + lane_base + kTcD + 32, a1);
                tc_wait_ld();
                uint32_t l0[32], l1[32];
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float d0 = u[i] - __uint_as_float(a0[i]), d1 = u[32 + i] - __uint_as_float(a1[i]);
                    a0[i] = __float_as_uint(d0); a1[i] = __float_as_uint(d1);
                    l0[i] = __float_as_uint(tf32_rest(d0)); l1[i] = __float_as_uint(tf32_rest(d1));
                }
                tc_st32(tmem + lane_base + kTcD, a0);
                tc_st32(tmem + lane_base + kTcD + 32, a1);
                tc_st32(tmem + lane_base + kTcDl, l0);
                tc_st32(tmem + lane_base + kTcDl + 32, l1);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(bar(SB_DFULL));
            }
            // S *= e^{cC}, once every product that reads the old S has completed
            ok = __all_sync(0xffffffffu, mbar_wait(bar(SB_QDONE), ph, abortp));
            if (!ok) break;
            tc_fence_after();
            {
                const float eC = tab[2 * kC];
#pragma unroll 1
                for (int c = 0; c < kDH; c += 32) {
                    uint32_t x[32];
                    tc_ld32(tmem + lane_base + kTcS + c, x);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) x[i] = __float_as_uint(__uint_as_float(x[i]) * eC);
                    tc_st32(tmem + lane_base + kTcS + c, x);
                }
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(bar(SB_SSCALED));
            }
            // the new state: remainder copy for the next chunk's products
            ok = __all_sync(0xffffffffu, mbar_wait(bar(SB_CDONE), ph, abortp));
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < kDH; c += 32) {
                uint32_t x[32];
                tc_ld32(tmem + lane_base + kTcS + c, x);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) x[i] = __float_as_uint(tf32_rest(__uint_as_float(x[i])));
                tc_st32(tmem + lane_base + kTcSl + c, x);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(SB_SREADY));
            // output rows of this chunk (off the critical path: the next chunk's first products run meanwhile)
            {
                uint32_t o1[32], o2[32];
#pragma unroll 1
                for (int c = 0; c < kC; c += 32) {
                    tc_ld32(tmem + lane_base + kTcO1 + c, o1);
                    tc_ld32(tmem + lane_base + kTcO2 + c, o2);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int t = t0 + c + i;
                        if (t < p.n) p.out[(size_t)t * total_v + (size_t)vh * kDH + r] = tab[kC + c + i] * __uint_as_float(o1[i]) + __uint_as_float(o2[i]);
                    }
                }
                tc_fence_before();
                mbar_arrive(bar(SB_OFREE));
            }
        }
        if (ok) {  // final state back to memory
#pragma unroll 1
            for (int c = 0; c < kDH; c += 32) {
                uint32_t x[32];
                tc_ld32(tmem + lane_base + kTcS + c, x);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 8; i++)
                    *reinterpret_cast<float4 *>(Srow + c + 4 * i) = make_float4(__uint_as_float(x[4 * i]), __uint_as_float(x[4 * i + 1]),
                                                                                __uint_as_float(x[4 * i + 2]), __uint_as_float(x[4 * i + 3]));
            }
        }
    }
    // ---- wind down: everyone meets, TMEM goes back ----
    tc_fence_before();
    __syncthreads();
    if (s_abort && tid == 0) atomicCAS(p.err, 0, (3 << 16) | (blockIdx.x & 0xffff));
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---- gated RMS-norm in place: o * rsqrt(mean o^2 + eps) * w * silu(z) --------------------------
// grid (Hv, n), 32 threads (4 dims per lane)
__global__ void gdn_norm_kernel(GdnDims g, const float *__restrict__ z, const uint16_t *__restrict__ norm_w,
                                float *__restrict__ out) {
    const int vh = blockIdx.x, t = blockIdx.y, lane = threadIdx.x;
    const size_t o = (size_t)t * g.Hv * kDH + (size_t)vh * kDH + lane * 4;
    float4 x = *reinterpret_cast<const float4 *>(out + o);
    const float ss = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
    const float inv = 1.0f / sqrtf(ss / kDH + g.eps);
    const float4 zz = *reinterpret_cast<const float4 *>(z + o);
    auto f = [&](float v, float zv, int d) {
        return v * inv * bf16_bits_to_float(norm_w[d]) * (zv / (1.0f + expf(-zv)));
    };
    x.x = f(x.x, zz.x, lane * 4); x.y = f(x.y, zz.y, lane * 4 + 1);
    x.z = f(x.z, zz.z, lane * 4 + 2); x.w = f(x.w, zz.w, lane * 4 + 3);
    *reinterpret_cast<float4 *>(out + o) = x;
}

// ---- host side ---------------------------------------------------------------------------------
static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

static size_t carve(const GdnDims &g, int n, void *base, GdnWork *w) {
    const int nchunks = (n + kC - 1) / kC;
    size_t off = 0;
    auto take = [&](size_t floats) {
        float *p = base ? reinterpret_cast<float *>(static_cast<char *>(base) + off) : nullptr;
        off += align256(floats * sizeof(float));
        return p;
    };
    GdnWork t;
    t.qn = take((size_t)n * g.Hk * kDH);
    t.kn = take((size_t)n * g.Hk * kDH);
    t.vn = take((size_t)n * g.Hv * kDH);
    t.lg = take((size_t)n * g.Hv);
    t.bt = take((size_t)n * g.Hv);
    t.U = take((size_t)g.Hv * nchunks * kC * kDH);
    t.W = take((size_t)g.Hv * nchunks * kC * kDH);
    t.QK = take((size_t)g.Hv * nchunks * kC * kC);
    t.cv = take((size_t)g.Hv * nchunks * kC);
    t.KT = take((size_t)g.Hk * nchunks * kDH * kC);
    if (w) *w = t;
    return off;
}

size_t gdn_prefill_work_bytes(const GdnDims &g, int max_tokens, int chunk) {
    (void)chunk;
    return carve(g, max_tokens, nullptr, nullptr);
}

int launch_gdn_prefill(const GdnDims &g, int n, int chunk, int step0, float *conv_state, float *ssm_state,
                       const float *qkv, const float *z, const float *beta, const float *alpha,
                       const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                       const uint16_t *norm_w, float *out, void *work, size_t work_bytes, int *err, cudaStream_t st) {
    (void)chunk;
    GdnWork w;
    if (carve(g, n, work, &w) > work_bytes) return -1;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gdn_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g.conv_dim * 4) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kChunkSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScSmem) != cudaSuccess)
            return -1;
        configured = true;
    }
    const int nchunks = (n + kC - 1) / kC;
    gdn_prep_kernel<<<n, 512, g.conv_dim * 4, st>>>(g, n, step0, conv_state, qkv, beta, alpha, conv_w, A_log, dt_bias, w);
    gdn_ring_kernel<<<dim3(12, 3), 256, 0, st>>>(g.conv_dim, n, step0, conv_state, qkv);
    gdn_chunk_kernel<<<dim3(nchunks, g.Hv), 256, kChunkSmem, st>>>(g, n, w, nchunks);
    static const bool legacy_scan = getenv("FM_GDN_SCAN_MMA_SYNC") != nullptr;  // development switch
    if (legacy_scan) {
        gdn_scan_kernel<<<dim3(kDH / kSl, g.Hv), 256, kScanSmem, st>>>(g, n, w, nchunks, ssm_state, out);
    } else {
        CUtensorMap mw, mq, mqk, mkt;
        if (!make_map_2d(&mw, w.W, (uint64_t)g.Hv * nchunks * kC, kDH, kC, true) ||
            !make_map_2d(&mq, w.qn, (uint64_t)n, (uint64_t)g.Hk * kDH, kC, true) ||
            !make_map_2d(&mqk, w.QK, (uint64_t)g.Hv * nchunks * kC, kC, kC, true) ||
            !make_map_2d(&mkt, w.KT, (uint64_t)g.Hk * nchunks * kDH, kC, kDH, true))
            return -1;
        ScanParams sp;
        sp.n = n; sp.nchunks = nchunks; sp.Hv = g.Hv; sp.Hk = g.Hk;
        sp.U = w.U; sp.cv = w.cv; sp.ssm = ssm_state; sp.out = out; sp.err = err;
        gdn_scan_tc_kernel<<<g.Hv, kScThreads, kScSmem, st>>>(mw, mq, mqk, mkt, sp);
    }
    int launches = 4;
    if (norm_w != nullptr) {
        gdn_norm_kernel<<<dim3(g.Hv, n), 32, 0, st>>>(g, z, norm_w, out);
        launches++;
    }
    return cudaGetLastError() == cudaSuccess ? launches : -1;
}

}  // namespace fm
