// Paged KV store (bf16, or FP8 E4M3 with per-row scales): fused k-RMS-norm + partial RoPE + append, and
// export / import in the reference's layouts.
//
// Follows the CPU append of metal_infer/layer_forward.h:574-629 and the Metal kernel
// prefill_kv_cache_bf16 (metal_infer/shaders.metal:2405-2482): normalise k per head with the bf16
// weight, rotate pairs (i, i + rotary_dim/2) by pos * inv_freq[i], write k and the untouched v at
// the row's place -- rounded to bf16, or quantised the way fp8_encode_vec does (metal_infer/fp8.h:100-108).
#include "fm_device.cuh"
#include "fm_fp8.cuh"
#include "fm_internal.h"

namespace fm {

// Page base and row-in-page of a store row; nullptr if this context does not hold the row's page.
__device__ __forceinline__ unsigned char *kv_row_page(const KvView &kv, int seq, int row, int &r) {
    const int gpage = row / kv.page_size;
    if (gpage % kv.shard_count != kv.shard_rank) return nullptr;
    const int slot = gpage / kv.shard_count;
    r = row - gpage * kv.page_size;
    return kv_page(kv, kv.page_table[(size_t)seq * kv.max_slots + slot]);
}

// Largest |x| over the block's threads (blockDim.x a multiple of 32, at most 1024); NaNs are skipped like the
// reference's `a > amax` test does.  `red` holds 32 floats.
__device__ __forceinline__ float block_absmax(float a, float *red) {
    a = warp_max(a);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
    __syncthreads();
    float m = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) m = fmaxf(m, red[w]);
    return m;
}

// grid (tokens), block D threads (one per dim); a block walks the KV heads of its token (the FP8 scale of a row
// spans all of them)
__global__ void kv_append_kernel(KvView kv, RopeParams rope, TokSpec toks, const float *__restrict__ k,
                                 const float *__restrict__ v, const uint16_t *__restrict__ knw,
                                 float eps) {
    __shared__ float sx[256];
    __shared__ float sred[32];
    const int t = blockIdx.x, d = threadIdx.x, D = kv.D;
    int seq, pos, row, r = 0;
    tok_get(toks, t, seq, pos, row);
    unsigned char *pg = kv_row_page(kv, seq, row, r);
    if (pg == nullptr) return;  // another context owns this row
    const int half = rope.rotary_dim / 2;
    float c = 1.f, s = 0.f;
    if (d < rope.rotary_dim) sincos_reduced(((float)pos / rope.pos_div) * rope.inv_freq[d < half ? d : d - half], s, c);
    float kx[8], vx[8];  // up to 8 KV heads per context
    float ak = 0.f, av = 0.f;
    for (int h = 0; h < kv.Hkv; h++) {
        const size_t src = ((size_t)t * kv.Hkv + h) * D + d;
        float x = k[src];
        if (knw != nullptr) {
            const float ss = warp_sum(x * x);
            __syncthreads();
            if ((d & 31) == 0) sred[d >> 5] = ss;
            __syncthreads();
            float tot = 0.f;
            for (int w = 0; w < D / 32; w++) tot += sred[w];
            x = x * (1.0f / sqrtf(tot / D + eps)) * bf16_bits_to_float(knw[d]);
        }
        __syncthreads();
        sx[d] = x;
        __syncthreads();
        if (d < rope.rotary_dim) x = d < half ? x * c - sx[d + half] * s : sx[d - half] * s + x * c;
        const float vv = v[src];
        if (!kv.fp8) {
            reinterpret_cast<__nv_bfloat16 *>(pg + kv_tile_offset(kv, 0, h))[(size_t)r * D + d] = __float2bfloat16_rn(x);
            reinterpret_cast<__nv_bfloat16 *>(pg + kv_tile_offset(kv, 1, h))[(size_t)r * D + d] = __float2bfloat16_rn(vv);
        } else {
            kx[h] = x; vx[h] = vv;
            ak = fmaxf(ak, fabsf(x)); av = fmaxf(av, fabsf(vv));
        }
    }
    if (!kv.fp8) return;
    ak = block_absmax(ak, sred);
    av = block_absmax(av, sred);
    const float ksc = ak > 0.f ? ak / 240.0f : 1.0f, vsc = av > 0.f ? av / 240.0f : 1.0f;
    const float kinv = 1.0f / ksc, vinv = 1.0f / vsc;
    for (int h = 0; h < kv.Hkv; h++) {
        (pg + kv_tile_offset(kv, 0, h))[(size_t)r * D + d] = fp8_e4m3_encode_ref(kx[h], kinv);
        (pg + kv_tile_offset(kv, 1, h))[(size_t)r * D + d] = fp8_e4m3_encode_ref(vx[h], vinv);
    }
    if (d == 0) {
        kv_page_scales(kv, pg, 0)[r] = ksc;
        kv_page_scales(kv, pg, 1)[r] = vsc;
    }
}

int launch_kv_append(const KvView &kv, const RopeParams &rope, const TokSpec &toks, const float *k,
                     const float *v, const uint16_t *k_norm_w, float eps, cudaStream_t st) {
    if (toks.n <= 0) return 0;
    if (kv.Hkv > 8) return -1;
    kv_append_kernel<<<toks.n, kv.D, 0, st>>>(kv, rope, toks, k, v, k_norm_w, eps);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// Export / import of rows [row0, row0 + n) in fp32 [n][Hkv*D] (the buffers start at row0): grid (n rows), 256
// threads; rows not held locally are skipped.  An FP8 store decodes (value * scale) on export and quantises the
// row the reference's way on import.
template <bool kImport>
__global__ void kv_copy_kernel(KvView kv, int seq, int row0, float *__restrict__ k, float *__restrict__ v, const int *__restrict__ order) {
    __shared__ float sred[32];
    const int i = blockIdx.x, row = order ? order[row0 + i] : row0 + i, kv_dim = kv.Hkv * kv.D;
    int r = 0;
    unsigned char *pg = kv_row_page(kv, seq, row, r);
    if (pg == nullptr) return;
    float *kr = k + (size_t)i * kv_dim, *vr = v + (size_t)i * kv_dim;
    float kinv = 1.f, vinv = 1.f, ksc = 1.f, vsc = 1.f;
    if (kv.fp8) {
        if (kImport) {
            float ak = 0.f, av = 0.f;
            for (int e = threadIdx.x; e < kv_dim; e += blockDim.x) { ak = fmaxf(ak, fabsf(kr[e])); av = fmaxf(av, fabsf(vr[e])); }
            ak = block_absmax(ak, sred);
            av = block_absmax(av, sred);
            ksc = ak > 0.f ? ak / 240.0f : 1.0f; vsc = av > 0.f ? av / 240.0f : 1.0f;
            kinv = 1.0f / ksc; vinv = 1.0f / vsc;
            if (threadIdx.x == 0) { kv_page_scales(kv, pg, 0)[r] = ksc; kv_page_scales(kv, pg, 1)[r] = vsc; }
        } else {
            ksc = kv_page_scales(kv, pg, 0)[r]; vsc = kv_page_scales(kv, pg, 1)[r];
        }
    }
    for (int e = threadIdx.x; e < kv_dim; e += blockDim.x) {
        const int kvh = e / kv.D, d = e - kvh * kv.D;
        unsigned char *kt = pg + kv_tile_offset(kv, 0, kvh), *vt = pg + kv_tile_offset(kv, 1, kvh);
        const size_t o = (size_t)r * kv.D + d;
        if (!kv.fp8) {
            __nv_bfloat16 *kp = reinterpret_cast<__nv_bfloat16 *>(kt) + o, *vp = reinterpret_cast<__nv_bfloat16 *>(vt) + o;
            if (kImport) { *kp = __float2bfloat16_rn(kr[e]); *vp = __float2bfloat16_rn(vr[e]); }
            else { kr[e] = __bfloat162float(*kp); vr[e] = __bfloat162float(*vp); }
        } else if (kImport) {
            kt[o] = fp8_e4m3_encode_ref(kr[e], kinv);
            vt[o] = fp8_e4m3_encode_ref(vr[e], vinv);
        } else {
            kr[e] = fp8_e4m3_decode_ref(kt[o], ksc);
            vr[e] = fp8_e4m3_decode_ref(vt[o], vsc);
        }
    }
}

int launch_kv_export(const KvView &kv, int seq, int row0, int n, float *k, float *v, const int *order, cudaStream_t st) {
    if (n <= 0) return 0;
    kv_copy_kernel<false><<<n, 256, 0, st>>>(kv, seq, row0, k, v, order);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}
int launch_kv_import(const KvView &kv, int seq, int row0, int n, const float *k, const float *v, cudaStream_t st) {
    if (n <= 0) return 0;
    kv_copy_kernel<true><<<n, 256, 0, st>>>(kv, seq, row0, const_cast<float *>(k), const_cast<float *>(v), nullptr);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// The stored bytes and scales themselves, in the layout of KVCache.k_cache_fp8 / v_cache_fp8 / k_scales / v_scales
// (metal_infer/layer_forward.h:124-127): bytes [n][Hkv*D], scales [n].  grid (n rows), 128 threads x 4 bytes.
template <bool kImport>
__global__ void kv_copy_fp8_kernel(KvView kv, int seq, int row0, uint8_t *__restrict__ k, uint8_t *__restrict__ v,
                                   float *__restrict__ ks, float *__restrict__ vs, const int *__restrict__ order) {
    const int i = blockIdx.x, row = order ? order[row0 + i] : row0 + i, kv_dim = kv.Hkv * kv.D;
    int r = 0;
    unsigned char *pg = kv_row_page(kv, seq, row, r);
    if (pg == nullptr) return;
    for (int e = threadIdx.x * 4; e < kv_dim; e += blockDim.x * 4) {
        const int kvh = e / kv.D, d = e - kvh * kv.D;
        uint32_t *kp = reinterpret_cast<uint32_t *>(pg + kv_tile_offset(kv, 0, kvh) + (size_t)r * kv.D + d);
        uint32_t *vp = reinterpret_cast<uint32_t *>(pg + kv_tile_offset(kv, 1, kvh) + (size_t)r * kv.D + d);
        uint32_t *ku = reinterpret_cast<uint32_t *>(k + (size_t)i * kv_dim + e), *vu = reinterpret_cast<uint32_t *>(v + (size_t)i * kv_dim + e);
        if (kImport) { *kp = *ku; *vp = *vu; } else { *ku = *kp; *vu = *vp; }
    }
    if (threadIdx.x == 0) {
        float *pk = kv_page_scales(kv, pg, 0) + r, *pv = kv_page_scales(kv, pg, 1) + r;
        if (kImport) { *pk = ks[i]; *pv = vs[i]; } else { ks[i] = *pk; vs[i] = *pv; }
    }
}

int launch_kv_copy_fp8(const KvView &kv, int seq, int row0, int n, uint8_t *k, uint8_t *v, float *ks, float *vs, bool import,
                       const int *order, cudaStream_t st) {
    if (n <= 0) return 0;
    if (import)
        kv_copy_fp8_kernel<true><<<n, 128, 0, st>>>(kv, seq, row0, k, v, ks, vs, nullptr);
    else
        kv_copy_fp8_kernel<false><<<n, 128, 0, st>>>(kv, seq, row0, k, v, ks, vs, order);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace fm
