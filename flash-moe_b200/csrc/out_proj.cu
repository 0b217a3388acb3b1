// The step behind the token-mixing kernels: output projection (o_proj of a full-attention layer, out_proj of a
// GatedDeltaNet layer) from the reference's 4-bit weight format, residual add and post-attention RMS-norm.
//
// Reference: cpu_dequant_matvec (metal_infer/cpu_kernels.h:199-232; Metal dequant_matvec_4bit*), then residual_add,
// rms_norm_sum_sq and rms_norm_apply_bf16 (metal_infer/shaders.metal:792-882) as encoded after attention in
// fused_layer_forward (metal_infer/layer_forward.h:3369-3450):
//     y[r]      = sum_k (nibble[r][k] * scale[r][k / 64] + bias[r][k / 64]) * x[k]
//     h_mid     = residual + y
//     h_post    = h_mid * rsqrt(mean(h_mid^2) + eps) * w_bf16
// Weights: uint32 [out_dim][in_dim / 8], eight 4-bit values per word, lowest nibble first; scale and bias bf16 per
// (row, group of 64 inputs).
//
// At decode the projection is a stream over the weights (18.9 MB for 4096 x 8192) with a handful of tokens riding
// along, so the kernel is built around that stream: a CTA owns 28 output rows (147 CTAs for 4096 rows: one per SM),
// its 16 warps are 2 row tiles x 8 groups side by side, every lane fetches 8 bytes of a row group straight into registers (a full 32-byte sector per
// row and quad, several groups ahead) and widens the nibbles in place with the OR-in-a-magic-exponent trick
// (nibble | 0x6400 is the fp16 number 1024 + nibble).  The words a lane holds fix which inputs land in which
// k-slot of its mma.sync A fragment; the activations are staged in shared memory, as fp16, in exactly that order,
// so no weight byte is ever moved between lanes.  Tokens are the N dimension: 8 per launch (more tokens take more
// launches, which find the weights in L2; a prompt-sized batch wants a GEMM tiling instead, which this is not).
// Residual add and the sum of squares ride in the epilogue; the normalisation needs whole rows, which no CTA has,
// so it is a second, tiny launch that starts (programmatic dependent launch) while the projection drains.
#include <cuda_fp16.h>

#include <algorithm>

#include "fm_device.cuh"
#include "fm_internal.h"

namespace fm {

constexpr int kPjRows = 28;          // output rows per CTA: 4096 rows make 147 CTAs, one per SM of a 148-SM part
constexpr int kPjWarps = 16;         // 2 row tiles (16 + 12 rows) x 8 groups in flight
constexpr int kPjThreads = 32 * kPjWarps;
constexpr int kPjTok = 8;            // tokens per launch: the N of one mma.sync
constexpr int kPjChunkGroups = 8;    // weight groups (of 64 inputs) the 8 warps of a row tile take side by side
constexpr int kPjChunkK = 64 * kPjChunkGroups;
constexpr int kPjTokStride = kPjChunkK / 2 + 1;  // half2 words per token and chunk, +1 keeps the fragment loads off each other's banks
constexpr int kPjDepth = 8;          // weight groups a warp has in flight

__device__ __forceinline__ void mma_f16_f32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (nibble q, nibble q + 4) of a weight word as two fp16 weights nibble * s + b.
// The word with 0x6400 OR-ed into each half is (1024 + n_lo, 1024 + n_hi) for the nibbles at bits 0..3 / 16..19,
// and 1024 + 16 n for those at bits 4..7 / 20..23; subtracting 1024 is exact, the scale of the second kind is s / 16.
__device__ __forceinline__ uint32_t q4_pair(uint32_t word, int q, __half2 s, __half2 s16, __half2 b) {
    const uint32_t v = (q & 2) ? word >> 8 : word;
    const uint32_t m = (q & 1) ? (v & 0x00F000F0u) | 0x64006400u : (v & 0x000F000Fu) | 0x64006400u;
    const __half2 n = __hsub2(*reinterpret_cast<const __half2 *>(&m), __half2half2(__ushort_as_half(0x6400)));
    const __half2 w = __hfma2(n, (q & 1) ? s16 : s, b);
    return *reinterpret_cast<const uint32_t *>(&w);
}

struct ProjParams {
    const uint32_t *w;
    const uint16_t *scales, *biases;
    int out_dim, in_dim;
    int n;                  // tokens (<= 8)
    const float *x;         // [n][in_dim]
    const float *residual;  // [n][out_dim] or null
    float *h_mid;           // [n][out_dim]
    float *ssq;             // [8] sum of squares of h_mid rows, accumulated with atomics (zero on entry)
};

// grid (ceil(out_dim / 28)), 512 threads, dynamic shared memory: the activations of up to 8 tokens as fp16
__global__ void __launch_bounds__(kPjThreads, 1)
out_proj_q4_kernel(ProjParams p) {
    extern __shared__ uint32_t s_x[];  // [chunk][8 tokens][kPjTokStride] half2 words
    __shared__ float s_ssq[kPjTok];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int mt = warp & 1, ks = warp >> 1;
    const int words_per_row = p.in_dim / 8, groups_per_row = p.in_dim / 64;
    const int nchunks = p.in_dim / kPjChunkK;
    const int row_base = blockIdx.x * kPjRows;
    const int l0 = mt * 16 + g, l1 = l0 + 8;  // rows of this lane within the CTA's 28
    const bool ok0 = l0 < kPjRows && row_base + l0 < p.out_dim, ok1 = l1 < kPjRows && row_base + l1 < p.out_dim;
    const int r0 = ok0 ? row_base + l0 : 0, r1 = ok1 ? row_base + l1 : 0;  // rows without a place read row 0 and are dropped at the end
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (tid < kPjTok) s_ssq[tid] = 0.f;

    // this warp's weight groups: ks, ks + 8, ... of the row; kPjDepth of them in flight
    uint2 wq0[kPjDepth], wq1[kPjDepth];
    uint32_t sb0[kPjDepth], sb1[kPjDepth];  // scale | bias << 16 (bf16 bits) of rows r0, r1
    auto fetch = [&](int c, int slot) {
        const int grp = c * kPjChunkGroups + ks;
        wq0[slot] = __ldg(reinterpret_cast<const uint2 *>(p.w + (size_t)r0 * words_per_row + grp * 8) + t);
        wq1[slot] = __ldg(reinterpret_cast<const uint2 *>(p.w + (size_t)r1 * words_per_row + grp * 8) + t);
        sb0[slot] = (uint32_t)__ldg(p.scales + (size_t)r0 * groups_per_row + grp) | ((uint32_t)__ldg(p.biases + (size_t)r0 * groups_per_row + grp) << 16);
        sb1[slot] = (uint32_t)__ldg(p.scales + (size_t)r1 * groups_per_row + grp) | ((uint32_t)__ldg(p.biases + (size_t)r1 * groups_per_row + grp) << 16);
    };
#pragma unroll
    for (int c = 0; c < kPjDepth; c++)
        if (c < nchunks) fetch(c, c);

    // All activations -> shared memory as fp16, once, the inputs of a group reordered to the k-slots of the fragments:
    // chunk c, group gi, lane quad t, word wi (0, 1), type q: half2 (x[512 c + 64 gi + 8 (2t + wi) + q], x[... + q + 4])
    // at word ((gi * 4 + t) * 8 + wi * 4 + q) of (chunk, token).  One thread converts the eight inputs under one
    // weight word; every load of the pass is in flight before the first is used.
    // (token columns beyond n are never read back, so their slots stay as they are)
#pragma unroll 4
    for (int e = tid; e < p.n * (p.in_dim / 8); e += kPjThreads) {
        const int tok = e / (p.in_dim / 8), w8 = e - tok * (p.in_dim / 8);  // w8: which 8 inputs of the row
        const float4 *src = reinterpret_cast<const float4 *>(p.x + (size_t)tok * p.in_dim + (size_t)w8 * 8);
        const float4 a = __ldg(src), b = __ldg(src + 1);
        const int c = w8 >> 6, gi = (w8 >> 3) & 7, w = w8 & 7;
        uint32_t *o = s_x + ((size_t)c * kPjTok + tok) * kPjTokStride + ((gi * 4 + (w >> 1)) * 8 + (w & 1) * 4);
        const __half2 h0 = __floats2half2_rn(a.x, b.x), h1 = __floats2half2_rn(a.y, b.y), h2 = __floats2half2_rn(a.z, b.z), h3 = __floats2half2_rn(a.w, b.w);
        o[0] = *reinterpret_cast<const uint32_t *>(&h0); o[1] = *reinterpret_cast<const uint32_t *>(&h1);
        o[2] = *reinterpret_cast<const uint32_t *>(&h2); o[3] = *reinterpret_cast<const uint32_t *>(&h3);
    }
    __syncthreads();

    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of dependent MMAs instead of one
    for (int c0 = 0; c0 < nchunks; c0 += kPjDepth) {
#pragma unroll
        for (int slot = 0; slot < kPjDepth; slot++) {  // unrolled so that the in-flight weight registers are indexed statically
            const int c = c0 + slot;
            if (c >= nchunks) break;
            // weights of this warp's group: widen, scale, shift
            uint32_t a[4][4];  // [type q][fragment register]
            {
                const float s0 = bf16_bits_to_float((uint16_t)(sb0[slot] & 0xffff)), b0 = bf16_bits_to_float((uint16_t)(sb0[slot] >> 16));
                const float s1 = bf16_bits_to_float((uint16_t)(sb1[slot] & 0xffff)), b1 = bf16_bits_to_float((uint16_t)(sb1[slot] >> 16));
                const __half2 hs0 = __float2half2_rn(s0), hs0b = __float2half2_rn(s0 * 0.0625f), hb0 = __float2half2_rn(b0);
                const __half2 hs1 = __float2half2_rn(s1), hs1b = __float2half2_rn(s1 * 0.0625f), hb1 = __float2half2_rn(b1);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    a[q][0] = q4_pair(wq0[slot].x, q, hs0, hs0b, hb0);
                    a[q][1] = q4_pair(wq1[slot].x, q, hs1, hs1b, hb1);
                    a[q][2] = q4_pair(wq0[slot].y, q, hs0, hs0b, hb0);
                    a[q][3] = q4_pair(wq1[slot].y, q, hs1, hs1b, hb1);
                }
            }
            if (c + kPjDepth < nchunks) fetch(c + kPjDepth, slot);
            const uint32_t *xt = s_x + ((size_t)c * kPjTok + g) * kPjTokStride + (ks * 4 + t) * 8;
            mma_f16_f32(acc, a[0][0], a[0][1], a[0][2], a[0][3], xt[0], xt[4]);
            mma_f16_f32(acc2, a[1][0], a[1][1], a[1][2], a[1][3], xt[1], xt[5]);
            mma_f16_f32(acc, a[2][0], a[2][1], a[2][2], a[2][3], xt[2], xt[6]);
            mma_f16_f32(acc2, a[3][0], a[3][1], a[3][2], a[3][3], xt[3], xt[7]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) acc[i] += acc2[i];
    __syncthreads();  // the activations are dead; their space takes the partial sums

    // ---- the eight group-phases of a row tile meet in shared memory ----
    float *red = reinterpret_cast<float *>(s_x);  // [8 phases][32 rows][8 tokens]
    {
        float *o = red + ((size_t)ks * 32 + mt * 16) * kPjTok + 2 * t;
        o[(size_t)g * kPjTok] = acc[0]; o[(size_t)g * kPjTok + 1] = acc[1];
        o[(size_t)(g + 8) * kPjTok] = acc[2]; o[(size_t)(g + 8) * kPjTok + 1] = acc[3];
    }
    __syncthreads();
    // h_mid = residual + y, and the rows' share of each token's sum of squares: warp w takes token w
    if (warp < p.n) {
        const int tok = warp, r = lane;
        float h = 0.f;
        if (r < kPjRows && row_base + r < p.out_dim) {
            float y = 0.f;
#pragma unroll
            for (int ph = 0; ph < 8; ph++) y += red[((size_t)ph * 32 + r) * kPjTok + tok];
            const size_t o = (size_t)tok * p.out_dim + row_base + r;
            h = (p.residual ? p.residual[o] : 0.f) + y;
            p.h_mid[o] = h;
        }
        const float sq = warp_sum(h * h);
        if (lane == 0) atomicAdd(p.ssq + tok, sq);
    }
}

// h_post = h_mid * rsqrt(ssq / dim + eps) * w; grid (tokens, dim / 1024), 256 threads x float4.  It also clears the
// sums the NEXT projection launch will accumulate into (`ssq_next`: the two sets alternate between calls).
__global__ void __launch_bounds__(256)
rms_norm_apply_kernel(const float *__restrict__ h_mid, const float *__restrict__ ssq, float *__restrict__ ssq_next, const uint16_t *__restrict__ w,
                      float eps, int dim, float *__restrict__ h_post) {
    const int tok = blockIdx.x, i = (blockIdx.y * 256 + threadIdx.x) * 4;
    uint2 wb = make_uint2(0x3f803f80u, 0x3f803f80u);
    if (i < dim && w != nullptr) wb = __ldg(reinterpret_cast<const uint2 *>(w + i));
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (blockIdx.y == 0 && threadIdx.x == 0) ssq_next[tok] = 0.f;
    if (i >= dim) return;
    const float inv = 1.0f / sqrtf(__ldcg(ssq + tok) / dim + eps);
    const float4 h = __ldcg(reinterpret_cast<const float4 *>(h_mid + (size_t)tok * dim + i));
    *reinterpret_cast<float4 *>(h_post + (size_t)tok * dim + i) =
        make_float4(h.x * inv * __uint_as_float(wb.x << 16), h.y * inv * __uint_as_float(wb.x & 0xffff0000u),
                    h.z * inv * __uint_as_float(wb.y << 16), h.w * inv * __uint_as_float(wb.y & 0xffff0000u));
}

// ssq: two sets of 8 floats, both zero when the context is created; *parity says which one this call uses.
int launch_out_proj_q4(const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int out_dim, int in_dim, int n, const float *x,
                       const float *residual, const uint16_t *norm_w, float eps, float *h_mid, float *h_post, float *ssq, int *parity,
                       cudaStream_t st) {
    if (n < 1 || n > kPjTok || in_dim % kPjChunkK) return -1;
    const size_t smem = (size_t)(in_dim / kPjChunkK) * kPjTok * kPjTokStride * 4;
    static unsigned long long configured = 0;
    if (first_use_on_device(&configured)) {
        if (cudaFuncSetAttribute(out_proj_q4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return -1;
    }
    if (smem > 200 * 1024 || smem < (size_t)8 * 32 * kPjTok * 4) return -1;
    float *mine = ssq + (*parity) * kPjTok, *next = ssq + ((*parity) ^ 1) * kPjTok;
    ProjParams p;
    p.w = w; p.scales = scales; p.biases = biases; p.out_dim = out_dim; p.in_dim = in_dim; p.n = n; p.x = x; p.residual = residual;
    p.h_mid = h_mid; p.ssq = mine;
    out_proj_q4_kernel<<<(out_dim + kPjRows - 1) / kPjRows, kPjThreads, smem, st>>>(p);
    if (cudaGetLastError() != cudaSuccess) return -1;
    if (h_post == nullptr)  // nobody reads the sums: clear them for the call after this one
        return cudaMemsetAsync(mine, 0, kPjTok * sizeof(float), st) == cudaSuccess ? 1 : -1;
    *parity ^= 1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(n, (out_dim + 1023) / 1024); lc.blockDim = dim3(256); lc.dynamicSmemBytes = 0; lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, rms_norm_apply_kernel, (const float *)h_mid, (const float *)mine, next, norm_w, eps, out_dim, h_post) == cudaSuccess ? 2 : -1;
}

}  // namespace fm
