// GatedDeltaNet decode step: one launch does conv + SiLU, q/k normalisation, decay / beta, the
// delta-rule update of the per-head [dv][dk] fp32 state, and the gated RMS-norm.
//
// Math of metal_infer/layer_forward.h:886-1025 (CPU) / the Metal kernels conv1d_step, rms_norm_qk,
// compute_decay_beta, gated_delta_net_step_fused, gated_rms_norm (metal_infer/shaders.metal:
// 1648-1850).  Organisation for the GPU:
//   * the state is the only large operand (64 KB per head, read and written once per step); a
//     warp owns whole state rows, each lane holding a float4 of the row, so every access is a
//     coalesced 512-byte line (the reference kernel gives a thread a row: adjacent threads stride
//     512 B apart);
//   * the dv rows of a head are split over `S` CTAs of one thread-block cluster so that a
//     batch-1 step still fills the machine (64 heads x 4 = 256 CTAs); the only cross-CTA datum
//     is the sum of squares of the head's output, exchanged through distributed shared memory;
//   * the conv history is a ring of 4 rows per sequence indexed by the token count, so all CTAs
//     of a step read three rows and the owner writes the fourth: no shift, no read/write race.
#include <cooperative_groups.h>

#include "fm_device.cuh"
#include "fm_internal.h"

namespace cg = cooperative_groups;

namespace fm {

constexpr int kDk = 128, kDv = 128;
constexpr int kGdnThreads = 256;

// conv + SiLU for one channel at token index `step`; ring rows hold the raw inputs of tokens
// step-3..step-1 at slots (step-3)&3.. ; the caller that owns the channel stores x at slot step&3.
__device__ __forceinline__ float conv_silu(const float *ring, int conv_dim, int step, int ch, float x,
                                           const uint16_t *conv_w, bool has_w) {
    if (!has_w) return 0.f;
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < 3; t++) {
        const int tokidx = step - 3 + t;
        const float h = tokidx >= 0 ? ring[(size_t)(tokidx & 3) * conv_dim + ch] : 0.f;
        acc += h * bf16_bits_to_float(conv_w[ch * 4 + t]);
    }
    acc += x * bf16_bits_to_float(conv_w[ch * 4 + 3]);
    return acc / (1.0f + expf(-acc));
}

template <int S, int W>  // CTAs (row slices) per head; warps per CTA (8, or 16 for whole-head CTAs at large batch)
__global__ void __launch_bounds__(32 * W)
gdn_decode_kernel(GdnDims g, TokSpec toks, float *__restrict__ conv_ring, float *__restrict__ ssm,
                  long long conv_seq_stride, long long ssm_seq_stride, const float *__restrict__ qkv,
                  const float *__restrict__ z, const float *__restrict__ beta,
                  const float *__restrict__ alpha, const uint16_t *__restrict__ conv_w,
                  const float *__restrict__ A_log, const uint16_t *__restrict__ dt_bias,
                  const uint16_t *__restrict__ norm_w, float *__restrict__ out) {
    constexpr int kRows = kDv / S;          // state rows of this CTA
    constexpr int kRowsPerWarp = kRows / W;
    __shared__ __align__(16) float s_q[kDk];
    __shared__ __align__(16) float s_k[kDk];
    __shared__ float s_v[kRows];
    __shared__ float s_o[kRows];
    __shared__ float s_red[8 + W];
    __shared__ float s_share[8];  // sum(o^2) of every CTA of the cluster, each written by its owner into all copies

    const int slice = blockIdx.x, vh = blockIdx.y, tok = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rep = g.Hv / g.Hk, kh = vh / rep;
    const int total_k = g.Hk * kDk;
    int seq, step, unused;
    tok_get(toks, tok, seq, step, unused);

    // Launched as a programmatic dependent (the caller vouched that the previous launch in the stream does not touch
    // this layer's state, fm_set_layer_overlap): the next such launch may start, and this one requests its state before
    // it waits for the previous launch -- whose results its other inputs may be -- to complete.  Without the launch
    // attribute both instructions do nothing.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    // ---- start the state loads first: they are the long pole ----
    float *S0 = ssm + (size_t)seq * ssm_seq_stride + ((size_t)vh * kDv + slice * kRows) * kDk;
    float4 st[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; i++)
        st[i] = *reinterpret_cast<const float4 *>(S0 + (size_t)(warp * kRowsPerWarp + i) * kDk + lane * 4);

    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // first phase of the cluster barrier: arrive now, wait just before the first write into a peer's shared memory
    // (which is only legal once that peer has started); by then everyone has long arrived
    if (S > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // ---- everything else the step reads from global memory is requested now as well, so that one memory latency
    //      covers it all: the gate row, the head's decay / beta inputs, the norm weight ----
    const bool has_norm = norm_w != nullptr;
    float z_pre = 0.f, nw_pre = 1.f;
    if (tid < kRows && has_norm) {
        const int d = slice * kRows + tid;
        z_pre = __ldg(z + (size_t)tok * g.Hv * kDv + (size_t)vh * kDv + d);
        nw_pre = bf16_bits_to_float(__ldg(norm_w + d));
    }
    const float alpha_pre = __ldg(alpha + (size_t)tok * g.Hv + vh), beta_pre = __ldg(beta + (size_t)tok * g.Hv + vh);
    const float bias = dt_bias ? bf16_bits_to_float(__ldg(dt_bias + vh)) : 0.f;
    const float alog = A_log ? __ldg(A_log + vh) : 0.f;

    // ---- conv + SiLU for this head's q, k channels and this slice's v channels ----
    float *ring = conv_ring + (size_t)seq * conv_seq_stride;
    const float *x_in = qkv + (size_t)tok * g.conv_dim;
    const bool has_w = conv_w != nullptr;
    const bool own_qk = (slice == 0) && (vh % rep == 0);
    float my = 0.f;
    if (tid < 2 * kDk) {
        // threads 0..127: q channel, 128..255: k channel
        const int ch = (tid < kDk ? 0 : total_k) + kh * kDk + (tid & (kDk - 1));
        const float x = x_in[ch];
        my = conv_silu(ring, g.conv_dim, step, ch, x, conv_w, has_w);
        if (own_qk) ring[(size_t)(step & 3) * g.conv_dim + ch] = x;
        float ss = warp_sum(my * my);
        if (lane == 0) s_red[warp] = ss;
    }
    if (tid < kRows) {
        const int ch = 2 * total_k + vh * kDv + slice * kRows + tid;
        const float x = x_in[ch];
        s_v[tid] = conv_silu(ring, g.conv_dim, step, ch, x, conv_w, has_w);
        ring[(size_t)(step & 3) * g.conv_dim + ch] = x;
    }
    __syncthreads();
    {
        // q <- rmsnorm(q) / dk ; k <- rmsnorm(k) / sqrt(dk), eps 1e-6
        const int base = tid < kDk ? 0 : 4;
        const float tot = s_red[base] + s_red[base + 1] + s_red[base + 2] + s_red[base + 3];
        const float inv = 1.0f / sqrtf(tot / kDk + 1e-6f);
        const float inv_scale = 1.0f / sqrtf((float)kDk);
        if (tid < kDk)
            s_q[tid] = my * inv * (inv_scale * inv_scale);
        else if (tid < 2 * kDk)
            s_k[tid - kDk] = my * inv * inv_scale;
    }
    // decay and beta of this head
    const float A = A_log ? expf(alog) : 1.0f;
    const float sp = logf(1.0f + expf(alpha_pre + bias));
    const float decay = expf(-A * sp);
    const float bgate = 1.0f / (1.0f + expf(-beta_pre));
    __syncthreads();

    // ---- delta rule, one warp per row.  With S the row before the step: mem = decay (S k), delta = (v - mem) beta,
    // S' = decay S + delta k, o = S' q = decay (S q) + delta (k q).  S k and S q are reduced side by side (one pass of
    // shuffles over two independent sums instead of two passes one after the other) for all rows of the warp at once.
    const float4 k4 = *reinterpret_cast<const float4 *>(s_k + lane * 4);
    const float4 q4 = *reinterpret_cast<const float4 *>(s_q + lane * 4);
    const float kq = warp_sum(k4.x * q4.x + k4.y * q4.y + k4.z * q4.z + k4.w * q4.w);
    float sk[kRowsPerWarp], sq[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; i++) {
        const float4 s = st[i];
        sk[i] = s.x * k4.x + s.y * k4.y + s.z * k4.z + s.w * k4.w;
        sq[i] = s.x * q4.x + s.y * q4.y + s.z * q4.z + s.w * q4.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; i++) {
            sk[i] += __shfl_xor_sync(0xffffffffu, sk[i], o);
            sq[i] += __shfl_xor_sync(0xffffffffu, sq[i], o);
        }
    }
    float ss_local = 0.f;
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; i++) {
        const int r = warp * kRowsPerWarp + i;
        const float delta = (s_v[r] - decay * sk[i]) * bgate;
        float4 s = st[i];
        s.x = s.x * decay + k4.x * delta; s.y = s.y * decay + k4.y * delta;
        s.z = s.z * decay + k4.z * delta; s.w = s.w * decay + k4.w * delta;
        *reinterpret_cast<float4 *>(S0 + (size_t)r * kDk + lane * 4) = s;
        const float o = decay * sq[i] + delta * kq;
        if (lane == 0) s_o[r] = o;
        ss_local += o * o;  // the same value in every lane
    }
    if (lane == 0) s_red[8 + warp] = ss_local;
    __syncthreads();
    float total_ss = 0.f;
    if (S > 1) {
        // every CTA of the cluster puts its share of sum(o^2) into every peer's shared memory, then one cluster barrier:
        // after it each CTA reads only its own copy, so nobody depends on a peer that may already have exited
        cg::cluster_group cluster = cg::this_cluster();
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
        if (tid < S) {
            float t = 0.f;
            for (int w = 0; w < W; w++) t += s_red[8 + w];
            *cluster.map_shared_rank(&s_share[slice], tid) = t;
        }
        cluster.sync();
#pragma unroll
        for (int r = 0; r < S; r++) total_ss += s_share[r];
    } else {
        for (int w = 0; w < W; w++) total_ss += s_red[8 + w];
    }
    // ---- gated RMS-norm: o * rsqrt(mean o^2 + eps) * w * silu(z) ----
    if (tid < kRows) {
        const int d = slice * kRows + tid;
        const size_t oi = (size_t)tok * g.Hv * kDv + (size_t)vh * kDv + d;
        float o = s_o[tid];
        if (has_norm) {
            const float inv = 1.0f / sqrtf(total_ss / kDv + g.eps);
            o = o * inv * nw_pre * (z_pre / (1.0f + expf(-z_pre)));
        }
        out[oi] = o;
    }
}

template <int S, int W>
static int launch_gdn_decode_s(const GdnDims &g, const TokSpec &toks, float *conv_state, float *ssm_state,
                               long long conv_seq_stride, long long ssm_seq_stride, const float *qkv,
                               const float *z, const float *beta, const float *alpha,
                               const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                               const uint16_t *norm_w, float *out, bool overlap_prev, cudaStream_t st) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(S, g.Hv, toks.n);
    lc.blockDim = dim3(32 * W);
    lc.dynamicSmemBytes = 0;
    lc.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = overlap_prev ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, gdn_decode_kernel<S, W>, g, toks, conv_state, ssm_state,
                                       conv_seq_stride, ssm_seq_stride, qkv, z, beta, alpha, conv_w,
                                       A_log, dt_bias, norm_w, out);
    return e == cudaSuccess ? 1 : -1;
}

int launch_gdn_decode(const GdnDims &g, const TokSpec &toks, float *conv_state, float *ssm_state,
                      long long conv_seq_stride, long long ssm_seq_stride, const float *qkv,
                      const float *z, const float *beta, const float *alpha, const uint16_t *conv_w,
                      const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, float *out,
                      bool overlap_prev, cudaStream_t st) {
    if (toks.n <= 0) return 0;
    // enough CTAs to cover the machine at small batch, whole heads per CTA at large batch
    const int ctas_whole = g.Hv * toks.n;
    if (ctas_whole >= 512)
        return launch_gdn_decode_s<1, 16>(g, toks, conv_state, ssm_state, conv_seq_stride, ssm_seq_stride, qkv, z,
                                      beta, alpha, conv_w, A_log, dt_bias, norm_w, out, overlap_prev, st);
    if (ctas_whole >= 256)
        return launch_gdn_decode_s<2, 8>(g, toks, conv_state, ssm_state, conv_seq_stride, ssm_seq_stride, qkv, z,
                                      beta, alpha, conv_w, A_log, dt_bias, norm_w, out, overlap_prev, st);
    return launch_gdn_decode_s<4, 8>(g, toks, conv_state, ssm_state, conv_seq_stride, ssm_seq_stride, qkv, z,
                                  beta, alpha, conv_w, A_log, dt_bias, norm_w, out, overlap_prev, st);
}

}  // namespace fm
