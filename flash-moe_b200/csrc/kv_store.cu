// Paged bf16 KV store: fused k-RMS-norm + partial RoPE + append, and export / import in the
// reference's fp32 [row][Hkv*D] layout.
//
// Follows the CPU append of metal_infer/layer_forward.h:574-629 and the Metal kernel
// prefill_kv_cache_bf16 (metal_infer/shaders.metal:2405-2482): normalise k per head with the bf16
// weight, rotate pairs (i, i + rotary_dim/2) by pos * inv_freq[i], write k and the untouched v at
// the row's place.
#include "fm_device.cuh"
#include "fm_internal.h"

namespace fm {

// Address of element (row, kvh, 0) of K (which = 0) or V (which = 1); nullptr if this context does
// not hold the row's page.
__device__ __forceinline__ __nv_bfloat16 *kv_row_ptr(const KvView &kv, int seq, int row, int kvh,
                                                     int which) {
    const int gpage = row / kv.page_size;
    if (gpage % kv.shard_count != kv.shard_rank) return nullptr;
    const int slot = gpage / kv.shard_count;
    const int page = kv.page_table[(size_t)seq * kv.max_slots + slot];
    const int r = row - gpage * kv.page_size;
    const size_t page_elems = (size_t)2 * kv.Hkv * kv.page_size * kv.D;
    return kv.pool + (size_t)page * page_elems +
           ((size_t)(which * kv.Hkv + kvh) * kv.page_size + r) * kv.D;
}

// grid (Hkv, tokens), block D threads (one per dim)
__global__ void kv_append_kernel(KvView kv, RopeParams rope, TokSpec toks, const float *__restrict__ k,
                                 const float *__restrict__ v, const uint16_t *__restrict__ knw,
                                 float eps) {
    __shared__ float sx[256];
    __shared__ float sred[8];
    const int kvh = blockIdx.x, t = blockIdx.y, d = threadIdx.x, D = kv.D;
    int seq, pos, row;
    tok_get(toks, t, seq, pos, row);
    __nv_bfloat16 *kdst = kv_row_ptr(kv, seq, row, kvh, 0);
    if (kdst == nullptr) return;  // another context owns this row
    __nv_bfloat16 *vdst = kv_row_ptr(kv, seq, row, kvh, 1);

    const size_t src = ((size_t)t * kv.Hkv + kvh) * D + d;
    float x = k[src];
    if (knw != nullptr) {
        float ss = warp_sum(x * x);
        if ((d & 31) == 0) sred[d >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < D / 32; w++) tot += sred[w];
        const float inv = 1.0f / sqrtf(tot / D + eps);
        x = x * inv * bf16_bits_to_float(knw[d]);
    }
    sx[d] = x;
    __syncthreads();
    const int half = rope.rotary_dim / 2;
    if (d < rope.rotary_dim) {
        const int i = d < half ? d : d - half;
        float c, s;
        sincos_reduced(((float)pos / rope.pos_div) * rope.inv_freq[i], s, c);
        if (d < half)
            x = x * c - sx[d + half] * s;
        else
            x = sx[d - half] * s + x * c;
    }
    kdst[d] = __float2bfloat16_rn(x);
    vdst[d] = __float2bfloat16_rn(v[src]);
}

int launch_kv_append(const KvView &kv, const RopeParams &rope, const TokSpec &toks, const float *k,
                     const float *v, const uint16_t *k_norm_w, float eps, cudaStream_t st) {
    if (toks.n <= 0) return 0;
    dim3 grid(kv.Hkv, toks.n);
    kv_append_kernel<<<grid, kv.D, 0, st>>>(kv, rope, toks, k, v, k_norm_w, eps);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// grid (rows), block Hkv*D/4 threads... one thread per 2 elements; rows not held locally are skipped
template <bool kImport>
__global__ void kv_copy_kernel(KvView kv, int seq, int len, float *__restrict__ k,
                               float *__restrict__ v) {
    const int row = blockIdx.x;
    if (row >= len) return;
    const int kv_dim = kv.Hkv * kv.D;
    for (int e = threadIdx.x; e < kv_dim; e += blockDim.x) {
        const int kvh = e / kv.D, d = e - kvh * kv.D;
        __nv_bfloat16 *kp = kv_row_ptr(kv, seq, row, kvh, 0);
        if (kp == nullptr) return;
        __nv_bfloat16 *vp = kv_row_ptr(kv, seq, row, kvh, 1);
        const size_t o = (size_t)row * kv_dim + e;
        if (kImport) {
            kp[d] = __float2bfloat16_rn(k[o]);
            vp[d] = __float2bfloat16_rn(v[o]);
        } else {
            k[o] = __bfloat162float(kp[d]);
            v[o] = __bfloat162float(vp[d]);
        }
    }
}

int launch_kv_export(const KvView &kv, int seq, int len, float *k, float *v, cudaStream_t st) {
    if (len <= 0) return 0;
    kv_copy_kernel<false><<<len, 256, 0, st>>>(kv, seq, len, k, v);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}
int launch_kv_import(const KvView &kv, int seq, int len, const float *k, const float *v,
                     cudaStream_t st) {
    if (len <= 0) return 0;
    kv_copy_kernel<true><<<len, 256, 0, st>>>(kv, seq, len, const_cast<float *>(k),
                                              const_cast<float *>(v));
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace fm
