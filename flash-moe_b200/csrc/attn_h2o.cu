// Heavy-hitter (H2O) eviction of the KV store at decode.
//
// The reference (metal_infer/layer_forward.h:248-383 and its use in the decode step, :591-727) keeps per cache row the
// attention mass it has received -- after every step, the softmax weight of the row summed over the query heads is
// added -- and, once the cache holds more than `budget` rows, drops rows from the unprotected middle (everything but
// the first `sinks` and the last `recent` rows) with the smallest accumulated mass, compacting the cache in place.
//
// Here the rows of a sequence never move.  A sequence owns budget + 1 physical rows; `order[i]` is the physical row of
// the i-th row in cache order (what the reference's compaction keeps contiguous), and the row an eviction frees is
// where the next token goes.  Attention does not care about row order, so the decode kernel runs unchanged over the
// dense physical rows; only export (and the protection of sinks / recent rows, which is by cache order) goes through
// `order`.  One decode step appends one row, so at most one row is evicted per step.
//
// After the decode launch of a step, h2o_mass_kernel
//   * recomputes the scores of the step's q against the K rows (a budget-sized read, K only), turns them into
//     softmax weights with the (max, sum) the decode kernel produced for every head, and adds the head-sum to the
//     row's accumulated mass;
//   * the last CTA to finish records the new row in `order` / token positions and, if the rows now exceed the
//     budget, removes the lightest unprotected row from `order` (ties: the later row, which is what the reference's
//     strict `>` selection of the rows to KEEP leaves out) and publishes its physical row as the next free slot.
// Nothing comes back to the host: the row count per step is a function of the token count alone.
#include "fm_device.cuh"
#include "fm_fp8.cuh"
#include "fm_internal.h"

namespace fm {

constexpr int kH2oRowsPerCta = 64;
constexpr int kH2oThreads = 256;

struct H2oParams {
    H2oView h;           // this layer's arrays, indexed [seq][cap]
    int budget, sinks, recent;
    int H;
    const float *q_proj_out, *q_in;  // the step's q, as given to the decode entry point
    const uint16_t *qnw;
    float eps;
    const float *ml;     // [tokens][H][2] (max in log2 units, sum) from the decode launch
    int token_index[kMaxList];  // how many tokens the sequence had seen before this one (KVCache.len at the append)
};

// grid (row chunks, tokens), 256 threads, dynamic shared memory: H * 256 floats (prepared q)
__global__ void __launch_bounds__(kH2oThreads)
h2o_mass_kernel(KvView kv, RopeParams rope, TokSpec toks, H2oParams p) {
    extern __shared__ float s_q[];  // [H][256], scaled so that q . k is the score in log2 units
    __shared__ float s_rc[64], s_rs[64];
    __shared__ int s_last;
    __shared__ float s_val[kH2oThreads / 32];
    __shared__ int s_idx[kH2oThreads / 32];
    constexpr int D = 256;
    const int tok = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int seq, pos, row_unused;
    tok_get(toks, tok, seq, pos, row_unused);
    const int n = tok_rows(toks, tok);  // rows attended this step, the new one included
    const int cap = p.h.cap;
    const int row_new = p.h.slot[seq];
    float *accum = p.h.accum + (size_t)seq * cap;
    int *order = p.h.order + (size_t)seq * cap;
    int *tokpos = p.h.tokpos + (size_t)seq * cap;
    const int group = p.H / kv.Hkv;

    // ---- q of every head: RMS-norm, partial RoPE, logit scale (as the decode kernel prepares it) ----
    if (tid < rope.rotary_dim / 2) sincos_reduced(((float)pos / rope.pos_div) * rope.inv_freq[tid], s_rs[tid], s_rc[tid]);
    __syncthreads();
    const int half = rope.rotary_dim / 2;
    const float qscale = rope.logit_scale * kLog2e;
    for (int h = warp; h < p.H; h += kH2oThreads / 32) {
        const float *src = p.q_proj_out ? p.q_proj_out + ((size_t)tok * p.H + h) * 2 * D : p.q_in + ((size_t)tok * p.H + h) * D;
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = src[lane * 8 + j];
        if (p.qnw != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) ss += x[j] * x[j];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / D + p.eps);
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = x[j] * inv * bf16_bits_to_float(p.qnw[lane * 8 + j]);
        }
        float *dst = s_q + (size_t)h * D;
#pragma unroll
        for (int j = 0; j < 8; j++) dst[lane * 8 + j] = x[j];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int d = lane * 8 + j;
            if (d < rope.rotary_dim) {
                const int i = d < half ? d : d - half;
                x[j] = d < half ? x[j] * s_rc[i] - dst[d + half] * s_rs[i] : dst[d - half] * s_rs[i] + x[j] * s_rc[i];
            }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; j++) dst[lane * 8 + j] = x[j] * qscale;
    }
    __syncthreads();

    // ---- this CTA's rows: a warp per row ----
    const int r0 = blockIdx.x * kH2oRowsPerCta;
    for (int r = r0 + warp; r < min(n, r0 + kH2oRowsPerCta); r += kH2oThreads / 32) {
        const unsigned char *pg = kv_page(kv, kv.page_table[(size_t)seq * kv.max_slots + r / kv.page_size]);
        const int rr = r % kv.page_size;
        float mass = 0.f;
        for (int kvh = 0; kvh < kv.Hkv; kvh++) {
            float k[8];
            if (!kv.fp8) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(pg + kv_tile_offset(kv, 0, kvh) + ((size_t)rr * D + lane * 8) * 2);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    k[2 * j] = __uint_as_float(w[j] << 16);
                    k[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                }
            } else {
                const uint2 raw = *reinterpret_cast<const uint2 *>(pg + kv_tile_offset(kv, 0, kvh) + (size_t)rr * D + lane * 8);
                const float sc = kv_page_scales(kv, const_cast<unsigned char *>(pg), 0)[rr];
#pragma unroll
                for (int j = 0; j < 8; j++) k[j] = fp8_e4m3_decode_ref((uint8_t)(((j < 4 ? raw.x : raw.y) >> (8 * (j & 3))) & 0xff), sc);
            }
            for (int g = 0; g < group; g++) {
                const int h = kvh * group + g;
                const float4 qa = *reinterpret_cast<const float4 *>(s_q + (size_t)h * D + lane * 8);
                const float4 qb = *reinterpret_cast<const float4 *>(s_q + (size_t)h * D + lane * 8 + 4);
                float dot = k[0] * qa.x + k[1] * qa.y + k[2] * qa.z + k[3] * qa.w + k[4] * qb.x + k[5] * qb.y + k[6] * qb.z + k[7] * qb.w;
                dot = warp_sum(dot);
                const float2 ml = *reinterpret_cast<const float2 *>(p.ml + ((size_t)tok * p.H + h) * 2);
                mass += ml.y > 0.f ? fast_exp2(dot - ml.x) / ml.y : 0.f;
            }
        }
        if (lane == 0) accum[r] = (r == row_new ? 0.f : accum[r]) + mass;  // the new row starts from zero (layer_forward.h:621)
    }

    // ---- the last CTA of this token finishes the bookkeeping ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int old = atomicAdd(p.h.counter + seq, 1u);
        s_last = old == gridDim.x - 1;
        if (s_last) p.h.counter[seq] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) {
        order[n - 1] = row_new;
        tokpos[row_new] = p.token_index[tok];
    }
    __syncthreads();
    int next_slot = n;  // no eviction: the next row extends the dense range
    if (n > p.budget) {
        // cache rows [sinks, n - recent) may go; the lightest goes, the later one among equals
        int sinks = min(p.sinks, p.budget), recent = p.recent;
        if (sinks + recent > p.budget) recent = p.budget - sinks;
        const int ev0 = sinks, ev1 = n - recent;
        const int heavy = p.budget - sinks - recent;
        if (ev1 - ev0 > 0 && heavy < ev1 - ev0) {
            float best = 3.0e38f;
            int bi = -1;
            for (int i = ev0 + tid; i < ev1; i += kH2oThreads) {
                const float a = __ldcg(accum + order[i]);
                if (a < best || (a == best && i > bi)) { best = a; bi = i; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi >= 0 && (bi < 0 || ob < best || (ob == best && oi > bi))) { best = ob; bi = oi; }
            }
            if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
            __syncthreads();
            if (tid == 0) {
                for (int w = 1; w < kH2oThreads / 32; w++)
                    if (s_idx[w] >= 0 && (s_idx[0] < 0 || s_val[w] < s_val[0] || (s_val[w] == s_val[0] && s_idx[w] > s_idx[0]))) {
                        s_val[0] = s_val[w];
                        s_idx[0] = s_idx[w];
                    }
            }
            __syncthreads();
            const int e = s_idx[0];
            next_slot = order[e];
            __syncthreads();
            // close the gap in cache order: every thread reads its entries, all meet, then all write
            for (int base = e; base < n - 1; base += kH2oThreads) {
                const int i = base + tid;
                const int v = i < n - 1 ? order[i + 1] : 0;
                __syncthreads();
                if (i < n - 1) order[i] = v;
                __syncthreads();
            }
        }
    }
    if (tid == 0) p.h.slot[seq] = next_slot;
}

int launch_h2o_mass(const KvView &kv, const RopeParams &rope, const TokSpec &toks, const int *token_index, const H2oView &h, int budget, int sinks,
                    int recent, int H, const float *q_proj_out, const float *q, const uint16_t *q_norm_w, float eps, const float *ml, int max_rows,
                    cudaStream_t st) {
    static unsigned long long configured = 0;
    const int smem = H * 256 * (int)sizeof(float);
    if (first_use_on_device(&configured) && smem > 48 * 1024) {
        if (cudaFuncSetAttribute(h2o_mass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) return -1;
    }
    if (smem > 96 * 1024) return -1;
    H2oParams p;
    p.h = h; p.budget = budget; p.sinks = sinks; p.recent = recent; p.H = H;
    p.q_proj_out = q_proj_out; p.q_in = q; p.qnw = q_norm_w; p.eps = eps; p.ml = ml;
    for (int i = 0; i < toks.n; i++) p.token_index[i] = token_index[i];
    dim3 grid((max_rows + kH2oRowsPerCta - 1) / kH2oRowsPerCta, toks.n);
    h2o_mass_kernel<<<grid, kH2oThreads, smem, st>>>(kv, rope, toks, p);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// accum / token positions in cache order: out[i] = in[order[i]]
__global__ void h2o_gather_kernel(H2oView h, int seq, int n, float *__restrict__ accum_out, int *__restrict__ tokpos_out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int phys = h.order[(size_t)seq * h.cap + i];
    if (accum_out) accum_out[i] = h.accum[(size_t)seq * h.cap + phys];
    if (tokpos_out) tokpos_out[i] = h.tokpos[(size_t)seq * h.cap + phys];
}

int launch_h2o_gather(const H2oView &h, int seq, int n, float *accum_out, int *tokpos_out, cudaStream_t st) {
    if (n <= 0) return 0;
    h2o_gather_kernel<<<(n + 255) / 256, 256, 0, st>>>(h, seq, n, accum_out, tokpos_out);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// identity order and token positions for rows [0, n) of a sequence (after an import), zero mass
__global__ void h2o_init_kernel(H2oView h, int seq, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < h.cap) {
        h.order[(size_t)seq * h.cap + i] = i;
        h.tokpos[(size_t)seq * h.cap + i] = i;
        h.accum[(size_t)seq * h.cap + i] = 0.f;
    }
    if (i == 0) { h.slot[seq] = n; h.counter[seq] = 0; }
}

int launch_h2o_init(const H2oView &h, int seq, int n, cudaStream_t st) {
    h2o_init_kernel<<<(h.cap + 255) / 256, 256, 0, st>>>(h, seq, n);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace fm
