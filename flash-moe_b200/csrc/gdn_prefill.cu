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
//   gdn_kk_kernel      per (key head, chunk): K K^T and Q K^T
//   gdn_chunk_kernel   per (value head, chunk), all chunks in parallel: A, then U and W by forward
//                      substitution, and the scan's operands as fp16 pairs -> workspace
//   gdn_scan_kernel    per head, chunks in sequence: D, O, S on tcgen05 with the state in tensor memory
//   gdn_norm_kernel    per token: gated RMS-norm in place
// The chunk kernel's contractions run as split tf32 (mma.sync m16n8k8, two terms per operand), the
// scan's as split fp16 (tcgen05 kind::f16, two terms per operand), both with fp32 accumulation; the
// triangular solve, the decay exponentials and the state stay fp32.
#include "fm_device.cuh"
#include "fm_internal.h"
#include <cuda_fp16.h>

#include "fm_tc.cuh"

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
    float *U;             // [Hv][nchunks][64][128]
    float *cv;            // [Hv][nchunks][64]  inclusive running sum of ln(decay)
    float *KKr, *QKr;     // [Hk][nchunks][64][64]  k k^T and q k^T of a chunk (shared by the value heads of a key head)
    // operands of the scan, each value as two fp16 terms laid side by side (hi | lo):
    __half *q16;          // [n][Hk][128 | 128]             normalised, scaled q
    __half *W16;          // [Hv][nchunks][64][128 | 128]
    __half *QK16;         // [Hv][nchunks][64][64 | 64]     decay-masked q k^T
    __half *KT16;         // [Hv][nchunks][128][64 | 64]    k transposed, column i scaled by e^{cC - c_i}
};

// x -> (hi, lo) fp16 with hi + lo = x to 22 bits; two values per 32-bit word (first value in the low half)
__device__ __forceinline__ void split2_f16(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    const __half2 hh = __floats2half2_rn(x0, x1);
    const float2 hf = __half22float2(hh);
    const __half2 ll = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&hh);
    lo = *reinterpret_cast<const uint32_t *>(&ll);
}

__device__ __forceinline__ void split_f16(float x, __half &hi, __half &lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}

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
    // four channels per thread: 16-byte loads of the four input rows, 32 bytes of bf16 taps
    for (int ch = tid * 4; ch < C; ch += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (conv_w != nullptr) {
            float4 x[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int tt = t - 3 + j;  // token inside this run, or history before it
                if (tt >= 0)
                    x[j] = __ldg(reinterpret_cast<const float4 *>(qkv + (size_t)tt * C + ch));
                else {
                    const int tokidx = step0 + tt;
                    x[j] = tokidx >= 0 ? *reinterpret_cast<const float4 *>(ring + (size_t)(tokidx & 3) * C + ch) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            const uint4 wa = __ldg(reinterpret_cast<const uint4 *>(conv_w + (size_t)ch * 4));      // channels ch, ch+1
            const uint4 wb = __ldg(reinterpret_cast<const uint4 *>(conv_w + (size_t)ch * 4 + 8));  // channels ch+2, ch+3
            auto lo16 = [](uint32_t u) { return __uint_as_float(u << 16); };
            auto hi16 = [](uint32_t u) { return __uint_as_float(u & 0xffff0000u); };
            // same order of operations as the scalar form: ((h0 w0 + h1 w1) + h2 w2) + x w3
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            a0 += x[0].x * lo16(wa.x); a0 += x[1].x * hi16(wa.x); a0 += x[2].x * lo16(wa.y); a0 += x[3].x * hi16(wa.y);
            a1 += x[0].y * lo16(wa.z); a1 += x[1].y * hi16(wa.z); a1 += x[2].y * lo16(wa.w); a1 += x[3].y * hi16(wa.w);
            a2 += x[0].z * lo16(wb.x); a2 += x[1].z * hi16(wb.x); a2 += x[2].z * lo16(wb.y); a2 += x[3].z * hi16(wb.y);
            a3 += x[0].w * lo16(wb.z); a3 += x[1].w * hi16(wb.z); a3 += x[2].w * lo16(wb.w); a3 += x[3].w * hi16(wb.w);
            acc = make_float4(a0 / (1.0f + expf(-a0)), a1 / (1.0f + expf(-a1)), a2 / (1.0f + expf(-a2)), a3 / (1.0f + expf(-a3)));
        }
        *reinterpret_cast<float4 *>(s_c + ch) = acc;
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
        if (is_q) {  // the scan's copy of q: hi | lo
            __half h[4], l[4];
            split_f16(y.x, h[0], l[0]); split_f16(y.y, h[1], l[1]); split_f16(y.z, h[2], l[2]); split_f16(y.w, h[3], l[3]);
            __half *d16 = w.q16 + ((size_t)t * g.Hk + hh) * 2 * kDH + lane * 4;
            *reinterpret_cast<uint2 *>(d16) = *reinterpret_cast<const uint2 *>(h);
            *reinterpret_cast<uint2 *>(d16 + kDH) = *reinterpret_cast<const uint2 *>(l);
        }
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


// ---- per (key head, chunk): K K^T and Q K^T (64 x 64 x 128), shared by the value heads -------------
constexpr int kLdK = kDH + 4;   // [row][k] operands read as (row g, k t): stride = 4 mod 32
constexpr int kKkSmem = 2 * kC * kLdK * 4;

// grid (nchunks, Hk), 256 threads: warp = (16-row tile, 32-column half)
__global__ void __launch_bounds__(256)
gdn_kk_kernel(GdnDims g, int n, GdnWork w, int nchunks) {
    extern __shared__ __align__(16) float sm[];
    float *sK = sm, *sQ = sK + kC * kLdK;
    const int chunk = blockIdx.x, kh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = chunk * kC, total_k = g.Hk * kDH;
    for (int i = tid; i < kC * (kDH / 4); i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), q4 = k4;
        if (t0 + r < n) {
            k4 = __ldg(reinterpret_cast<const float4 *>(w.kn + (size_t)(t0 + r) * total_k + (size_t)kh * kDH + c4));
            q4 = __ldg(reinterpret_cast<const float4 *>(w.qn + (size_t)(t0 + r) * total_k + (size_t)kh * kDH + c4));
        }
        *reinterpret_cast<float4 *>(sK + r * kLdK + c4) = k4;
        *reinterpret_cast<float4 *>(sQ + r * kLdK + c4) = q4;
    }
    __syncthreads();
    const int mt = warp & 3, nh = warp >> 2;
    float akk[4][4] = {}, aqk[4][4] = {};
    const float *Ka = sK + (mt * 16) * kLdK, *Qa = sQ + (mt * 16) * kLdK, *Kb = sK + (nh * 32) * kLdK;
    auto fb = [&](int k, int nn) { return Kb[nn * kLdK + k]; };
    warp_gemm_tf32<4>(akk, kDH, [&](int m, int k) { return Ka[m * kLdK + k]; }, fb, lane);
    warp_gemm_tf32<4>(aqk, kDH, [&](int m, int k) { return Qa[m * kLdK + k]; }, fb, lane);
    float *kk_out = w.KKr + ((size_t)kh * nchunks + chunk) * kC * kC, *qk_out = w.QKr + ((size_t)kh * nchunks + chunk) * kC * kC;
    const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 4; nt++) {
        const int r = mt * 16 + gq, c = nh * 32 + nt * 8 + 2 * tq;
        *reinterpret_cast<float2 *>(kk_out + r * kC + c) = make_float2(akk[nt][0], akk[nt][1]);
        *reinterpret_cast<float2 *>(kk_out + (r + 8) * kC + c) = make_float2(akk[nt][2], akk[nt][3]);
        *reinterpret_cast<float2 *>(qk_out + r * kC + c) = make_float2(aqk[nt][0], aqk[nt][1]);
        *reinterpret_cast<float2 *>(qk_out + (r + 8) * kC + c) = make_float2(aqk[nt][2], aqk[nt][3]);
    }
}

// ---- per (head, chunk): everything that does not depend on the state ---------------------------
constexpr int kLdT = kC + 4;
constexpr int kChunkSmem = (kC * kLdK + kC * kLdT + 3 * kC) * 4;  // 51 KB: several CTAs per SM overlap their phases

// grid (nchunks, Hv), 256 threads
__global__ void __launch_bounds__(256, 2)
gdn_chunk_kernel(GdnDims g, int n, GdnWork w, int nchunks) {
    extern __shared__ __align__(16) float sm[];
    float *sK = sm;
    float *sA = sK + kC * kLdK, *sT = sA + kC * kLdT;
    float *sc = sT + kC, *sb = sc + kC;
    const int chunk = blockIdx.x, vh = blockIdx.y, kh = vh / (g.Hv / g.Hk);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = chunk * kC;
    const int total_k = g.Hk * kDH, total_v = g.Hv * kDH;

    // rows past the end of the run are zero (beta 0, decay 1: they leave the state alone)
    for (int i = tid; i < kC * (kDH / 4); i += 256) {
        const int r = i >> 5, c4 = (i & 31) * 4;
        float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t0 + r < n) k4 = __ldg(reinterpret_cast<const float4 *>(w.kn + (size_t)(t0 + r) * total_k + (size_t)kh * kDH + c4));
        *reinterpret_cast<float4 *>(sK + r * kLdK + c4) = k4;
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
    {   // k transposed and scaled for the state update of the scan: Ks[k][i] = e^{cC - c_i} k_i[k], hi | lo
        __half *kt = w.KT16 + ((size_t)vh * nchunks + chunk) * kDH * 2 * kC;
        const float cC = sc[kC - 1];
        for (int i = tid; i < kDH * kC; i += 256) {
            const int kk = i >> 6, r = i & (kC - 1);
            __half h, l;
            split_f16(sK[r * kLdK + kk] * expf(cC - sc[r]), h, l);
            kt[kk * 2 * kC + r] = h;
            kt[kk * 2 * kC + kC + r] = l;
        }
    }

    // A = beta_t e^{c_t - c_i} (k_t . k_i) below the diagonal, and the decay-masked q k^T for the scan, from the
    // key head's products: a thread takes 4 consecutive columns of a row
    {
        const float *kk = w.KKr + ((size_t)kh * nchunks + chunk) * kC * kC, *qk = w.QKr + ((size_t)kh * nchunks + chunk) * kC * kC;
        __half *qk_out = w.QK16 + ((size_t)vh * nchunks + chunk) * kC * 2 * kC;
        for (int i = tid; i < kC * (kC / 4); i += 256) {
            const int r = i >> 4, c = (i & 15) * 4;
            const float4 a = __ldg(reinterpret_cast<const float4 *>(kk + r * kC + c));
            const float4 q = __ldg(reinterpret_cast<const float4 *>(qk + r * kC + c));
            const float av[4] = {a.x, a.y, a.z, a.w}, qv[4] = {q.x, q.y, q.z, q.w};
            __half h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float dec = c + e <= r ? expf(sc[r] - sc[c + e]) : 0.f;
                sA[r * kLdT + c + e] = c + e < r ? sb[r] * dec * av[e] : 0.f;
                split_f16(dec * qv[e], h[e], l[e]);
            }
            *reinterpret_cast<uint2 *>(qk_out + r * 2 * kC + c) = *reinterpret_cast<const uint2 *>(h);
            *reinterpret_cast<uint2 *>(qk_out + r * 2 * kC + kC + c) = *reinterpret_cast<const uint2 *>(l);
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
        const bool is_u = c < kDH;  // warp-uniform: warps 0-3 solve for U, 4-7 for W
        float x[kC];
        if (is_u) {  // the v rows come straight from memory (a warp reads 128 consecutive bytes per row)
            const float *vsrc = w.vn + (size_t)t0 * total_v + (size_t)vh * kDH + c;
#pragma unroll
            for (int r = 0; r < kC; r++) x[r] = (t0 + r < n ? __ldg(vsrc + (size_t)r * total_v) : 0.f) * sb[r];
        } else {
            const float *src = sK + (c - kDH);
#pragma unroll
            for (int r = 0; r < kC; r++) x[r] = src[r * kLdK] * sT[r];
        }
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
        if (is_u) {
            float *dst = w.U + ((size_t)vh * nchunks + chunk) * kC * kDH + c;
#pragma unroll
            for (int r = 0; r < kC; r++) dst[r * kDH] = x[r];
        } else {
            __half *dst = w.W16 + ((size_t)vh * nchunks + chunk) * kC * 2 * kDH + (c - kDH);
#pragma unroll
            for (int r = 0; r < kC; r++) {
                __half h, l;
                split_f16(x[r], h, l);
                dst[r * 2 * kDH] = h;
                dst[r * 2 * kDH + kDH] = l;
            }
        }
    }
}

// ---- the chunk scan on the 5th-generation tensor cores ------------------------------------------
// One CTA per value head walks the chunks with the state in tensor memory, transposed so that the
// state row (value dim v) is the TMEM lane; every product has its A operand in TMEM and a K-major
// B tile brought by TMA:
//     acc[v][t] = sum_k S[v][k] W[t][k]              Dt = U^T - acc   }  one product M128 N128 K128 with
//     O1[v][t]  = sum_k S[v][k] Q[t][k]                               }  B = [W ; Q] stacked along N
//     O2[v][t]  = sum_i Dt[v][i] QKm[t][i]                            }  one product M128 N192 K64 with
//     S[v][k]   = e^{cC} S[v][k] + sum_i Dt[v][i] Ks[k][i]            }  B = [Ks ; QKm] stacked along N
//     out[t][v] = e^{c_t} O1[v][t] + O2[v][t]
// (an M128 MMA costs about the same ~60 cycles for N = 64 as for N = 128, so the products that share their
// A operand are stacked: 36 MMAs per chunk instead of 72; their accumulators are adjacent TMEM columns, and
// O2, which must start from zero next to the accumulating S, is zeroed by the state threads beforehand)
// Precision: fp16 has 11 significant bits, so every operand enters as two fp16 terms (x = hi + lo,
// 22 bits) and every product as three MMAs into the same fp32 accumulator (hi*hi, lo*hi, hi*lo):
// the B tiles arrive from the chunk kernel already split (hi | lo side by side), the TMEM operands S
// and Dt are split by the state threads.  The fp32 state itself only ever lives in its accumulator
// columns; after each update one pass writes its two-term copy for the next chunk's products and
// scales the accumulator by the next chunk's total decay, so the next update accumulates on top.
//   warps 0-7   state threads, two per state row (each takes half of the columns of every pass):
//               S -> TMEM, per chunk Dt = U - acc (split), the pass over the new S, the output rows
//   warp 8      TMA producer (single-buffered tiles: [W ; Q] is free again after the first product, U after
//               Dt is formed, [Ks ; QKm] after the second)
//   warp 9      MMA issuer
// TMEM: S 128 | O2 64 | S hi 64 | S lo 64 | acc 64 | O1 64 | Dt hi 32 | Dt lo 32 = 512 columns.
// Every mbarrier wait is bounded; on expiry the CTA records an error code and winds down.
constexpr int kScThreads = 320;
constexpr uint32_t kTcS = 0, kTcO2 = 128, kTcSh = 192, kTcSl = 256, kTcAcc = 320, kTcO1 = 384, kTcDh = 448, kTcDl = 480;
constexpr int kSlab64 = 64 * 128;    // bytes of one 64-element-wide slab of a 64-row fp16 tile
constexpr int kSlab128 = 128 * 128;  // ... of a 128-row tile ([W ; Q])
constexpr int kSlab192 = 192 * 128;  // ... of a 192-row tile ([Ks ; QKm])
// shared-memory tiles (fp16, 128-byte swizzle): [hi | lo] pairs
// [W ; Q]: 4 slabs (hi k 0-63, hi k 64-127, lo, lo) of 128 rows, W in rows 0-63; [Ks ; QKm]: 2 slabs (hi, lo) of 192
// rows, Ks in rows 0-127
constexpr int kOffWQ = 0, kOffKQ = 65536, kOffU = 114688 /*fp32 [64][128], unswizzled slabs*/, kOffBar = 147456;
enum ScBar { SB_SREADY = 0, SB_WQFULL, SB_UFULL, SB_KQKFULL, SB_DACC, SB_WEMPTY, SB_DFULL, SB_CDONE, SB_KEMPTY, SB_COUNT };
constexpr int kScSmem = kOffBar + SB_COUNT * 8 + 1024 /*alignment slack*/;


struct ScanParams {
    int n, nchunks, Hv, Hk;
    const float *U, *cv;
    float *ssm, *out;
    int *err;
};

__global__ void __launch_bounds__(kScThreads, 1)
gdn_scan_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
                const __grid_constant__ CUtensorMap map_qk, const __grid_constant__ CUtensorMap map_kt,
                const __grid_constant__ CUtensorMap map_u, ScanParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const float *sU = reinterpret_cast<const float *>(smem_raw + (base - smem_u32(smem_raw)) + kOffU);
    auto bar = [&](int i) { return base + kOffBar + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int vh = blockIdx.x, kh = vh / (p.Hv / p.Hk);
    const int nchunks = p.nchunks;

    if (tid == 0) {
        s_abort = 0;
        mbar_init(bar(SB_SREADY), 256);
        mbar_init(bar(SB_WQFULL), 1);
        mbar_init(bar(SB_UFULL), 1);
        mbar_init(bar(SB_KQKFULL), 1);
        mbar_init(bar(SB_DACC), 1);
        mbar_init(bar(SB_WEMPTY), 1);
        mbar_init(bar(SB_DFULL), 256);
        mbar_init(bar(SB_CDONE), 1);
        mbar_init(bar(SB_KEMPTY), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    volatile int *abortp = &s_abort;

    if (warp == 8) {
        // ================= TMA producer =================
        if (lane == 0) {
            for (int j = 0; j < nchunks; j++) {
                const int hc = vh * nchunks + j;
                if (j > 0 && !mbar_wait(bar(SB_WEMPTY), (j - 1) & 1, abortp)) break;
                mbar_expect_tx(bar(SB_WQFULL), 65536);
                for (int s = 0; s < 4; s++) tma_load_2d(base + kOffWQ + s * kSlab128, &map_w, s * 64, hc * kC, bar(SB_WQFULL));
                for (int s = 0; s < 4; s++)
                    tma_load_2d(base + kOffWQ + s * kSlab128 + kSlab64, &map_q, kh * 2 * kDH + s * 64, j * kC, bar(SB_WQFULL));
                if (j > 0 && !mbar_wait(bar(SB_DFULL), (j - 1) & 1, abortp)) break;  // U of the previous chunk has been read
                mbar_expect_tx(bar(SB_UFULL), 32768);
                for (int s = 0; s < 4; s++) tma_load_2d(base + kOffU + s * kSlab64, &map_u, s * 32, hc * kC, bar(SB_UFULL));
                if (j > 0 && !mbar_wait(bar(SB_KEMPTY), (j - 1) & 1, abortp)) break;
                mbar_expect_tx(bar(SB_KQKFULL), 16384 + 32768);
                for (int s = 0; s < 2; s++) tma_load_2d(base + kOffKQ + s * kSlab192, &map_kt, s * 64, hc * kDH, bar(SB_KQKFULL));
                for (int s = 0; s < 2; s++) tma_load_2d(base + kOffKQ + s * kSlab192 + kSlab128, &map_qk, s * 64, hc * kC, bar(SB_KQKFULL));
            }
        }
    } else if (warp == 9) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t id128 = idesc_dense(128, 128, false, 0), id192 = idesc_dense(128, 192, false, 0);
            const uint64_t dWQh = smem_desc(base + kOffWQ, 16, 1024), dWQl = smem_desc(base + kOffWQ + 2 * kSlab128, 16, 1024);
            const uint64_t dKQh = smem_desc(base + kOffKQ, 16, 1024), dKQl = smem_desc(base + kOffKQ + kSlab192, 16, 1024);
            // k-step of 16 elements = 32 bytes inside a 64-element slab, then the next slab
            auto k128 = [](int ks) { return (uint64_t)((((ks >> 2) * kSlab128) + (ks & 3) * 32) >> 4); };
            auto kin = [](int ks) { return (uint64_t)((ks * 32) >> 4); };
            for (int j = 0; j < nchunks; j++) {
                const uint32_t ph = j & 1;
                // S (two-term copy) is ready, the previous chunk's output accumulators have been read out
                bool ok = mbar_wait(bar(SB_SREADY), ph, abortp) && mbar_wait(bar(SB_WQFULL), ph, abortp);
                if (!ok) break;
                tc_fence_after();
                // [acc | O1] = S [W ; Q]^T, three terms
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_f16_ta(tmem + kTcAcc, tmem + kTcSh + ks * 8, dWQh + k128(ks), id128, ks > 0);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_f16_ta(tmem + kTcAcc, tmem + kTcSl + ks * 8, dWQh + k128(ks), id128, 1);
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc_mma_f16_ta(tmem + kTcAcc, tmem + kTcSh + ks * 8, dWQl + k128(ks), id128, 1);
                tc_commit(bar(SB_DACC));
                tc_commit(bar(SB_WEMPTY));
                // [S | O2] += Dt [Ks ; QKm]^T, three terms (S pre-scaled, O2 zeroed by the state threads)
                ok = mbar_wait(bar(SB_DFULL), ph, abortp) && mbar_wait(bar(SB_KQKFULL), ph, abortp);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 4; ks++) tc_mma_f16_ta(tmem + kTcS, tmem + kTcDh + ks * 8, dKQh + kin(ks), id192, 1);
#pragma unroll
                for (int ks = 0; ks < 4; ks++) tc_mma_f16_ta(tmem + kTcS, tmem + kTcDl + ks * 8, dKQh + kin(ks), id192, 1);
#pragma unroll
                for (int ks = 0; ks < 4; ks++) tc_mma_f16_ta(tmem + kTcS, tmem + kTcDh + ks * 8, dKQl + kin(ks), id192, 1);
                tc_commit(bar(SB_CDONE));
                tc_commit(bar(SB_KEMPTY));
            }
        }
    } else {
        // ================= state threads: row r = TMEM lane, half h of the columns =================
        const int r = tid & 127, h = tid >> 7;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        float *Srow = p.ssm + ((size_t)vh * kDH + r) * kDH + h * 64;  // this thread's 64 state columns
        const int total_v = p.Hv * kDH;
        const float *cv0 = p.cv + (size_t)vh * nchunks * kC;
        const float *sUcol = sU + (r >> 5) * (kSlab64 / 4) + (r & 31);  // U[t][r] at sUcol[t * 32]
        // decay sums of the chunk at hand: lane l holds c_l and c_{32+l}
        float c_lo = __ldg(cv0 + lane), c_hi = __ldg(cv0 + 32 + lane);
        {
            // S -> its two-term copy; the accumulator starts scaled by the first chunk's total decay
            const float eC = expf(__shfl_sync(0xffffffffu, c_hi, 31));
#pragma unroll 1
            for (int c = 0; c < 64; c += 32) {
                uint32_t x[32], hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float4 v = *reinterpret_cast<const float4 *>(Srow + c + 4 * i);
                    split2_f16(v.x, v.y, hi[2 * i], lo[2 * i]);
                    split2_f16(v.z, v.w, hi[2 * i + 1], lo[2 * i + 1]);
                    x[4 * i] = __float_as_uint(v.x * eC); x[4 * i + 1] = __float_as_uint(v.y * eC);
                    x[4 * i + 2] = __float_as_uint(v.z * eC); x[4 * i + 3] = __float_as_uint(v.w * eC);
                }
                tc_st32(tmem + lane_base + kTcS + h * 64 + c, x);
                tc_st16(tmem + lane_base + kTcSh + h * 32 + (c >> 1), hi);
                tc_st16(tmem + lane_base + kTcSl + h * 32 + (c >> 1), lo);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(SB_SREADY));
        }
        bool ok = true;
        for (int j = 0; j < nchunks; j++) {
            const uint32_t ph = j & 1;
            const int t0 = j * kC + h * 32;  // this thread's 32 tokens of the chunk
            // output scales e^{c_t} of this chunk, and the decay sums of the next one
            const float ev = expf(h == 0 ? c_lo : c_hi);
            float eC_next = 1.0f;  // the last update leaves the state unscaled
            if (j + 1 < nchunks) {
                c_lo = __ldg(cv0 + (size_t)(j + 1) * kC + lane);
                c_hi = __ldg(cv0 + (size_t)(j + 1) * kC + 32 + lane);
                eC_next = expf(__shfl_sync(0xffffffffu, c_hi, 31));
            }
            // Dt = U - acc for tokens h*32 .. h*32+31, as two fp16 terms
            {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(SB_UFULL), ph, abortp) && mbar_wait(bar(SB_DACC), ph, abortp));
                if (!ok) break;
                tc_fence_after();
                uint32_t a0[32];
                tc_ld32(tmem + lane_base + kTcAcc + h * 32, a0);
                float u[32];
#pragma unroll
                for (int t = 0; t < 32; t++) u[t] = sUcol[(h * 32 + t) * 32];
                tc_wait_ld();
                uint32_t dh[16], dl[16];
#pragma unroll
                for (int i = 0; i < 16; i++)
                    split2_f16(u[2 * i] - __uint_as_float(a0[2 * i]), u[2 * i + 1] - __uint_as_float(a0[2 * i + 1]), dh[i], dl[i]);
                tc_st16(tmem + lane_base + kTcDh + h * 16, dh);
                tc_st16(tmem + lane_base + kTcDl + h * 16, dl);
                {   // O2 starts from zero (its product accumulates next to S)
                    uint32_t zz[32];
#pragma unroll
                    for (int i = 0; i < 32; i++) zz[i] = 0u;
                    tc_st32(tmem + lane_base + kTcO2 + h * 32, zz);
                }
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(bar(SB_DFULL));
            }
            // the new state: two-term copy for the next chunk's products, accumulator pre-scaled for its update
            ok = __all_sync(0xffffffffu, mbar_wait(bar(SB_CDONE), ph, abortp));
            if (!ok) break;
            tc_fence_after();
            // the output accumulators go to registers first: the next chunk's first product overwrites O1
            uint32_t o1[32], o2[32];
            tc_ld32(tmem + lane_base + kTcO1 + h * 32, o1);
            tc_ld32(tmem + lane_base + kTcO2 + h * 32, o2);
#pragma unroll 1
            for (int c = 0; c < 64; c += 32) {
                uint32_t x[32], hi[16], lo[16];
                tc_ld32(tmem + lane_base + kTcS + h * 64 + c, x);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float v0 = __uint_as_float(x[2 * i]), v1 = __uint_as_float(x[2 * i + 1]);
                    split2_f16(v0, v1, hi[i], lo[i]);
                    x[2 * i] = __float_as_uint(v0 * eC_next);
                    x[2 * i + 1] = __float_as_uint(v1 * eC_next);
                }
                tc_st16(tmem + lane_base + kTcSh + h * 32 + (c >> 1), hi);
                tc_st16(tmem + lane_base + kTcSl + h * 32 + (c >> 1), lo);
                if (j + 1 < nchunks) tc_st32(tmem + lane_base + kTcS + h * 64 + c, x);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(SB_SREADY));
            // output rows of this chunk (off the critical path: the next chunk's first product runs meanwhile)
            {
                float *orow = p.out + (size_t)t0 * total_v + (size_t)vh * kDH + r;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float sc = __shfl_sync(0xffffffffu, ev, i);
                    if (t0 + i < p.n) orow[(size_t)i * total_v] = sc * __uint_as_float(o1[i]) + __uint_as_float(o2[i]);
                }
            }
        }
        if (ok) {  // final state back to memory
#pragma unroll 1
            for (int c = 0; c < 64; c += 32) {
                uint32_t x[32];
                tc_ld32(tmem + lane_base + kTcS + h * 64 + c, x);
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
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---- gated RMS-norm in place: o * rsqrt(mean o^2 + eps) * w * silu(z) --------------------------
// grid (n), 256 threads: a warp walks heads, 4 dims per lane
__global__ void __launch_bounds__(256)
gdn_norm_kernel(GdnDims g, const float *__restrict__ z, const uint16_t *__restrict__ norm_w, float *__restrict__ out) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint2 wq = __ldg(reinterpret_cast<const uint2 *>(norm_w + lane * 4));
    const float w0 = __uint_as_float(wq.x << 16), w1 = __uint_as_float(wq.x & 0xffff0000u);
    const float w2 = __uint_as_float(wq.y << 16), w3 = __uint_as_float(wq.y & 0xffff0000u);
    for (int vh = warp; vh < g.Hv; vh += 8) {
        const size_t o = (size_t)t * g.Hv * kDH + (size_t)vh * kDH + lane * 4;
        float4 x = *reinterpret_cast<const float4 *>(out + o);
        const float4 zz = __ldg(reinterpret_cast<const float4 *>(z + o));
        const float ss = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
        const float inv = 1.0f / sqrtf(ss / kDH + g.eps);
        auto f = [&](float v, float zv, float wv) { return v * inv * wv * (zv / (1.0f + expf(-zv))); };
        x.x = f(x.x, zz.x, w0); x.y = f(x.y, zz.y, w1);
        x.z = f(x.z, zz.z, w2); x.w = f(x.w, zz.w, w3);
        *reinterpret_cast<float4 *>(out + o) = x;
    }
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
    t.cv = take((size_t)g.Hv * nchunks * kC);
    t.KKr = take((size_t)g.Hk * nchunks * kC * kC);
    t.QKr = take((size_t)g.Hk * nchunks * kC * kC);
    // fp16 pairs: two halves per value = one float's worth of bytes
    t.q16 = reinterpret_cast<__half *>(take((size_t)n * g.Hk * kDH));
    t.W16 = reinterpret_cast<__half *>(take((size_t)g.Hv * nchunks * kC * kDH));
    t.QK16 = reinterpret_cast<__half *>(take((size_t)g.Hv * nchunks * kC * kC));
    t.KT16 = reinterpret_cast<__half *>(take((size_t)g.Hv * nchunks * kDH * kC));
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
    // the prep kernel's shared memory grows with conv_dim: the limit is raised whenever a context needs more than
    // any earlier one on the same device did
    static int prep_smem_set[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (g.conv_dim * 4 > prep_smem_set[dev]) {
        if (cudaFuncSetAttribute(gdn_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g.conv_dim * 4) != cudaSuccess) return -1;
        prep_smem_set[dev] = g.conv_dim * 4;
    }
    static unsigned long long configured = 0;  // one bit per device
    if (first_use_on_device(&configured)) {
        if (cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kChunkSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_kk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kKkSmem) != cudaSuccess ||
            cudaFuncSetAttribute(gdn_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScSmem) != cudaSuccess)
            return -1;
    }
    const int nchunks = (n + kC - 1) / kC;
    gdn_prep_kernel<<<n, 512, g.conv_dim * 4, st>>>(g, n, step0, conv_state, qkv, beta, alpha, conv_w, A_log, dt_bias, w);
    gdn_ring_kernel<<<dim3(12, 3), 256, 0, st>>>(g.conv_dim, n, step0, conv_state, qkv);
    gdn_kk_kernel<<<dim3(nchunks, g.Hk), 256, kKkSmem, st>>>(g, n, w, nchunks);
    gdn_chunk_kernel<<<dim3(nchunks, g.Hv), 256, kChunkSmem, st>>>(g, n, w, nchunks);
    {
        CUtensorMap mw, mq, mqk, mkt, mu;
        if (!make_map_2d(&mw, w.W16, (uint64_t)g.Hv * nchunks * kC, 2 * kDH, kC, false) ||
            !make_map_2d(&mq, w.q16, (uint64_t)n, (uint64_t)g.Hk * 2 * kDH, kC, false) ||
            !make_map_2d(&mqk, w.QK16, (uint64_t)g.Hv * nchunks * kC, 2 * kC, kC, false) ||
            !make_map_2d(&mkt, w.KT16, (uint64_t)g.Hv * nchunks * kDH, 2 * kC, kDH, false) ||
            !make_map_2d(&mu, w.U, (uint64_t)g.Hv * nchunks * kC, kDH, kC, true, /*swizzle=*/false))
            return -1;
        ScanParams sp;
        sp.n = n; sp.nchunks = nchunks; sp.Hv = g.Hv; sp.Hk = g.Hk;
        sp.U = w.U; sp.cv = w.cv; sp.ssm = ssm_state; sp.out = out; sp.err = err;
        gdn_scan_kernel<<<g.Hv, kScThreads, kScSmem, st>>>(mw, mq, mqk, mkt, mu, sp);
    }
    int launches = 5;
    if (norm_w != nullptr) {
        gdn_norm_kernel<<<n, 256, 0, st>>>(g, z, norm_w, out);
        launches++;
    }
    return cudaGetLastError() == cudaSuccess ? launches : -1;
}

}  // namespace fm
