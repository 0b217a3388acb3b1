// GatedDeltaNet decode step for many (head, sequence) pairs: a persistent kernel streams the recurrent states.
//
// Same math as gdn_decode.cu (metal_infer/layer_forward.h:886-1025; Metal kernels conv1d_step, rms_norm_qk,
// compute_decay_beta, gated_delta_net_step_fused, gated_rms_norm, metal_infer/shaders.metal:1648-1850), organised
// for the case where there are several (head, sequence) pairs per SM.  The step moves each pair's 64 KB state
// through the SM once in each direction and does a few flops per byte, so what matters is that the next pairs'
// states are already on their way while one is being updated:
//   * gdn_decode_prep_kernel does everything that is per token and small (conv + SiLU, ring update, q / k
//     normalisation, decay, beta) into a scratch record per (token, head);
//   * gdn_decode_stream_kernel runs one CTA per SM over pairs p = blockIdx.x, blockIdx.x + gridDim.x, ...  A ring of
//     three shared-memory stages holds the states; one thread fetches a pair's state and its scratch records with
//     bulk copies that complete on the stage's mbarrier, 16 warps update the rows in place (a warp owns 8 rows, a
//     lane a float4 of each), the same thread writes the stage back with a bulk store, and the extra warp finishes
//     the gated RMS-norm of the pair's output while the 16 warps are already on the next pair.  The warps never meet
//     at a CTA-wide barrier.
//   * The stream kernel is launched as a programmatic dependent of the prep kernel: its first three state fetches
//     do not depend on the prep kernel and start at once; only the scratch records wait for it.
// Every mbarrier wait is bounded; on expiry the CTA records an error code and winds down.
#include "fm_device.cuh"
#include "fm_internal.h"
#include "fm_tc.cuh"

namespace fm {

namespace {

constexpr int kSDk = 128, kSDv = 128;
constexpr int kStStages = 3;
constexpr int kStWarps = 16;                       // update warps; warp kStWarps is the copy / output warp
constexpr int kStThreads = 32 * (kStWarps + 1);
constexpr int kStRows = kSDv / kStWarps;            // state rows per warp
constexpr uint32_t kStateBytes = kSDv * kSDk * 4;   // 64 KB
// one stage: state | q k (1 KB) | v (512 B) | z (512 B) | decay, beta (16 B) | output rows (512 B) | sum-of-squares parts
constexpr uint32_t kOffQK = kStateBytes, kOffV = kOffQK + 1024, kOffZ = kOffV + 512, kOffDB = kOffZ + 512;
constexpr uint32_t kOffO = kOffDB + 128, kOffSS = kOffO + 512, kStageBytes = kOffSS + 128;
constexpr uint32_t kStSmem = kStStages * kStageBytes + 256;  // + barriers and the abort word

// scratch record sizes per token, in floats
__host__ __device__ inline size_t scr_qk_floats(int Hk) { return (size_t)Hk * 2 * kSDk; }
__host__ __device__ inline size_t scr_v_floats(int Hv) { return (size_t)Hv * kSDv; }
__host__ __device__ inline size_t scr_db_floats(int Hv) { return (size_t)Hv * 4; }

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ float conv_silu4(const float *ring, int conv_dim, int step, int ch, float x, const uint16_t *conv_w,
                                            bool has_w) {
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

}  // namespace

// grid (Hk, tokens), 256 threads: the q and k channels of k-head blockIdx.x and the v channels of its Hv/Hk value heads
__global__ void __launch_bounds__(256)
gdn_decode_prep_kernel(GdnDims g, TokSpec toks, float *__restrict__ conv_ring, long long conv_seq_stride,
                       const float *__restrict__ qkv, const float *__restrict__ beta, const float *__restrict__ alpha,
                       const uint16_t *__restrict__ conv_w, const float *__restrict__ A_log, const uint16_t *__restrict__ dt_bias,
                       float *__restrict__ scr_qk, float *__restrict__ scr_v, float *__restrict__ scr_db) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    __shared__ float s_red[8];
    const int kh = blockIdx.x, tok = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rep = g.Hv / g.Hk, total_k = g.Hk * kSDk;
    int seq, step, unused;
    tok_get(toks, tok, seq, step, unused);
    float *ring = conv_ring + (size_t)seq * conv_seq_stride;
    float *slot = ring + (size_t)(step & 3) * g.conv_dim;
    const float *x_in = qkv + (size_t)tok * g.conv_dim;
    const bool has_w = conv_w != nullptr;
    // threads 0..127: q channel, 128..255: k channel
    const int ch = (tid < kSDk ? 0 : total_k) + kh * kSDk + (tid & (kSDk - 1));
    const float x = x_in[ch];
    const float my = conv_silu4(ring, g.conv_dim, step, ch, x, conv_w, has_w);
    slot[ch] = x;
    const float ss = warp_sum(my * my);
    if (lane == 0) s_red[warp] = ss;
    // v channels of the value heads that share this k-head
    for (int c = tid; c < rep * kSDv; c += 256) {
        const int vch = 2 * total_k + kh * rep * kSDv + c;
        const float xv = x_in[vch];
        scr_v[(size_t)tok * scr_v_floats(g.Hv) + (size_t)kh * rep * kSDv + c] = conv_silu4(ring, g.conv_dim, step, vch, xv, conv_w, has_w);
        slot[vch] = xv;
    }
    if (tid < rep) {
        const int vh = kh * rep + tid;
        const float A = A_log ? expf(A_log[vh]) : 1.0f;
        const float bias = dt_bias ? bf16_bits_to_float(dt_bias[vh]) : 0.f;
        const float sp = logf(1.0f + expf(alpha[(size_t)tok * g.Hv + vh] + bias));
        float *db = scr_db + (size_t)tok * scr_db_floats(g.Hv) + (size_t)vh * 4;
        db[0] = expf(-A * sp);
        db[1] = 1.0f / (1.0f + expf(-beta[(size_t)tok * g.Hv + vh]));
        db[2] = 0.f;
        db[3] = 0.f;
    }
    __syncthreads();
    // q <- rmsnorm(q) / dk ; k <- rmsnorm(k) / sqrt(dk), eps 1e-6
    const int base = tid < kSDk ? 0 : 4;
    const float tot = s_red[base] + s_red[base + 1] + s_red[base + 2] + s_red[base + 3];
    const float inv = 1.0f / sqrtf(tot / kSDk + 1e-6f);
    const float inv_scale = 1.0f / sqrtf((float)kSDk);
    scr_qk[(size_t)tok * scr_qk_floats(g.Hk) + (size_t)kh * 2 * kSDk + tid] = tid < kSDk ? my * inv * (inv_scale * inv_scale) : my * inv * inv_scale;
}

__global__ void __launch_bounds__(kStThreads, 1)
gdn_decode_stream_kernel(GdnDims g, TokSpec toks, float *__restrict__ ssm, long long ssm_seq_stride, const float *__restrict__ z,
                         const uint16_t *__restrict__ norm_w, const float *__restrict__ scr_qk, const float *__restrict__ scr_v,
                         const float *__restrict__ scr_db, float *__restrict__ out, int *__restrict__ err) {
    extern __shared__ __align__(128) unsigned char st_smem[];
    const uint32_t sbase = smem_u32(st_smem);
    const uint32_t sbar = sbase + kStStages * kStageBytes;  // full[3], done[3]
    volatile int *abortp = reinterpret_cast<volatile int *>(st_smem + kStStages * kStageBytes + 64);
    auto full = [&](int s) { return sbar + 8 * s; };
    auto done = [&](int s) { return sbar + 8 * (kStStages + s); };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int items = g.Hv * toks.n;
    const int n_my = (int)blockIdx.x < items ? (items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int rep = g.Hv / g.Hk;
    const bool has_norm = norm_w != nullptr;
    const uint32_t tx = kStateBytes + 1024 + 512 + 16 + (has_norm ? 512u : 0u);
    if (tid == 0) {
        for (int s = 0; s < kStStages; s++) {
            mbar_init(full(s), 1);
            mbar_init(done(s), kStWarps);
        }
        *abortp = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    auto item_of = [&](int j, int &tok, int &vh) {
        const int it = (int)blockIdx.x + j * (int)gridDim.x;
        tok = it / g.Hv;
        vh = it - tok * g.Hv;
    };
    auto state_of = [&](int tok, int vh) {
        int seq, a, b;
        tok_get(toks, tok, seq, a, b);
        return ssm + (size_t)seq * ssm_seq_stride + (size_t)vh * kSDv * kSDk;
    };

    if (warp == kStWarps) {
        // ---- copy / output warp ----
        auto fetch_state = [&](int j) {
            int tok, vh;
            item_of(j, tok, vh);
            const int s = j % kStStages;
            mbar_expect_tx(full(s), tx);
            const float *src = state_of(tok, vh);
#pragma unroll
            for (int c = 0; c < 4; c++) bulk_g2s(sbase + s * kStageBytes + c * (kStateBytes / 4), src + c * (kStateBytes / 16), kStateBytes / 4, full(s));
        };
        auto fetch_small = [&](int j) {
            int tok, vh;
            item_of(j, tok, vh);
            const uint32_t sb = sbase + (j % kStStages) * kStageBytes, bar = full(j % kStStages);
            bulk_g2s(sb + kOffQK, scr_qk + (size_t)tok * scr_qk_floats(g.Hk) + (size_t)(vh / rep) * 2 * kSDk, 1024, bar);
            bulk_g2s(sb + kOffV, scr_v + (size_t)tok * scr_v_floats(g.Hv) + (size_t)vh * kSDv, 512, bar);
            bulk_g2s(sb + kOffDB, scr_db + (size_t)tok * scr_db_floats(g.Hv) + (size_t)vh * 4, 16, bar);
            if (has_norm) bulk_g2s(sb + kOffZ, z + ((size_t)tok * g.Hv + vh) * kSDv, 512, bar);
        };
        const int pre = n_my < kStStages ? n_my : kStStages;
        if (lane == 0)
            for (int j = 0; j < pre; j++) fetch_state(j);
        // the scratch records come from the launch this one depends on
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        if (lane == 0)
            for (int j = 0; j < pre; j++) fetch_small(j);
        float nw[4] = {1.f, 1.f, 1.f, 1.f};
        if (has_norm) {
#pragma unroll
            for (int e = 0; e < 4; e++) nw[e] = bf16_bits_to_float(norm_w[lane * 4 + e]);
        }
        int armed = pre;  // pairs whose fetch was issued
        bool ok = true;
        for (int j = 0; j < n_my && ok; j++) {
            const int s = j % kStStages;
            ok = __all_sync(0xffffffffu, mbar_wait(done(s), (j / kStStages) & 1, abortp));
            if (!ok) break;
            int tok, vh;
            item_of(j, tok, vh);
            const unsigned char *stg = st_smem + s * kStageBytes;
            // what the output needs leaves the stage first, so that the stage is written back and re-armed before the
            // output is computed (batch 64: 104.5 -> 97.7 us per layer)
            const float *ssp = reinterpret_cast<const float *>(stg + kOffSS);
            float total_ss = 0.f;
#pragma unroll
            for (int w = 0; w < kStWarps; w++) total_ss += ssp[w];
            float4 o = *reinterpret_cast<const float4 *>(stg + kOffO + lane * 16);
            float4 zz = make_float4(0.f, 0.f, 0.f, 0.f);
            if (has_norm) zz = *reinterpret_cast<const float4 *>(stg + kOffZ + lane * 16);
            __syncwarp();
            if (lane == 0) {
                float *dst = state_of(tok, vh);
#pragma unroll
                for (int c = 0; c < 4; c++) bulk_s2g(dst + c * (kStateBytes / 16), sbase + s * kStageBytes + c * (kStateBytes / 4), kStateBytes / 4);
                bulk_commit();
                if (j + kStStages < n_my) {
                    bulk_wait_read0();  // the store has read the stage
                    fetch_state(j + kStStages);
                    fetch_small(j + kStStages);
                    armed = j + kStStages + 1;
                }
            }
            // gated RMS-norm of the pair's output: o * rsqrt(mean o^2 + eps) * w * silu(z)
            if (has_norm) {
                const float inv = 1.0f / sqrtf(total_ss / kSDv + g.eps);
                o.x = o.x * inv * nw[0] * (zz.x / (1.0f + expf(-zz.x)));
                o.y = o.y * inv * nw[1] * (zz.y / (1.0f + expf(-zz.y)));
                o.z = o.z * inv * nw[2] * (zz.z / (1.0f + expf(-zz.z)));
                o.w = o.w * inv * nw[3] * (zz.w / (1.0f + expf(-zz.w)));
            }
            *reinterpret_cast<float4 *>(out + ((size_t)tok * g.Hv + vh) * kSDv + lane * 4) = o;
        }
        if (lane == 0) {
            if (!ok) {
                atomicCAS(err, 0, (3 << 16) | (blockIdx.x & 0xffff));
                // fetches still in flight land in this CTA's shared memory: give them a bounded time to finish
                for (int j = 0; j < armed; j++) {
                    const long long t0 = clock64();
                    while (!mbar_try(full(j % kStStages), (j / kStStages) & 1) && clock64() - t0 < 200000000LL) {
                    }
                }
            }
            bulk_wait0();
        }
        return;
    }

    // ---- update warps: rows warp*8 .. warp*8+7 of every pair ----
    for (int j = 0; j < n_my; j++) {
        const int s = j % kStStages;
        if (!__all_sync(0xffffffffu, mbar_wait(full(s), (j / kStStages) & 1, abortp))) return;
        unsigned char *stg = st_smem + s * kStageBytes;
        float *S0 = reinterpret_cast<float *>(stg) + (size_t)warp * kStRows * kSDk + lane * 4;
        const float4 q4 = *reinterpret_cast<const float4 *>(stg + kOffQK + lane * 16);
        const float4 k4 = *reinterpret_cast<const float4 *>(stg + kOffQK + 512 + lane * 16);
        const float decay = *reinterpret_cast<const float *>(stg + kOffDB), bgate = *reinterpret_cast<const float *>(stg + kOffDB + 4);
        const float *sv = reinterpret_cast<const float *>(stg + kOffV) + warp * kStRows;
        float4 st[kStRows];
        float sk[kStRows], sq[kStRows];
#pragma unroll
        for (int i = 0; i < kStRows; i++) {
            st[i] = *reinterpret_cast<const float4 *>(S0 + (size_t)i * kSDk);
            sk[i] = st[i].x * k4.x + st[i].y * k4.y + st[i].z * k4.z + st[i].w * k4.w;
            sq[i] = st[i].x * q4.x + st[i].y * q4.y + st[i].z * q4.z + st[i].w * q4.w;
        }
        float kq = k4.x * q4.x + k4.y * q4.y + k4.z * q4.z + k4.w * q4.w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kq += __shfl_xor_sync(0xffffffffu, kq, o);
#pragma unroll
            for (int i = 0; i < kStRows; i++) {
                sk[i] += __shfl_xor_sync(0xffffffffu, sk[i], o);
                sq[i] += __shfl_xor_sync(0xffffffffu, sq[i], o);
            }
        }
        // With S the row before the step: delta = (v - decay (S k)) beta, S' = decay S + delta k, o = decay (S q) + delta (k q)
        float ss_local = 0.f, o_mine = 0.f;
#pragma unroll
        for (int i = 0; i < kStRows; i++) {
            const float delta = (sv[i] - decay * sk[i]) * bgate;
            float4 r = st[i];
            r.x = r.x * decay + k4.x * delta; r.y = r.y * decay + k4.y * delta;
            r.z = r.z * decay + k4.z * delta; r.w = r.w * decay + k4.w * delta;
            *reinterpret_cast<float4 *>(S0 + (size_t)i * kSDk) = r;
            const float o = decay * sq[i] + delta * kq;
            if (lane == i) o_mine = o;
            ss_local += o * o;  // the same value in every lane
        }
        if (lane < kStRows) reinterpret_cast<float *>(stg + kOffO)[warp * kStRows + lane] = o_mine;
        if (lane == 0) reinterpret_cast<float *>(stg + kOffSS)[warp] = ss_local;
        fence_async_smem();  // the rows just written are read by the bulk store
        __syncwarp();
        if (lane == 0) mbar_arrive(done(s));
    }
}

size_t gdn_decode_scratch_bytes(const GdnDims &g, int tokens) {
    return (size_t)tokens * (scr_qk_floats(g.Hk) + scr_v_floats(g.Hv) + scr_db_floats(g.Hv)) * sizeof(float);
}

int launch_gdn_decode_stream(const GdnDims &g, const TokSpec &toks, float *conv_state, float *ssm_state, long long conv_seq_stride,
                             long long ssm_seq_stride, const float *qkv, const float *z, const float *beta, const float *alpha,
                             const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, float *out,
                             float *scratch, int sm_count, int *err, cudaStream_t st) {
    if (toks.n <= 0) return 0;
    if (g.dk != kSDk || g.dv != kSDv || g.Hk < 1 || g.Hv % g.Hk != 0 || (g.Hv / g.Hk) > 256) return -1;
    static unsigned long long configured = 0;
    if (first_use_on_device(&configured) &&
        cudaFuncSetAttribute(gdn_decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStSmem) != cudaSuccess)
        return -1;
    float *scr_qk = scratch, *scr_v = scr_qk + (size_t)toks.n * scr_qk_floats(g.Hk), *scr_db = scr_v + (size_t)toks.n * scr_v_floats(g.Hv);
    gdn_decode_prep_kernel<<<dim3(g.Hk, toks.n), 256, 0, st>>>(g, toks, conv_state, conv_seq_stride, qkv, beta, alpha, conv_w, A_log, dt_bias,
                                                               scr_qk, scr_v, scr_db);
    if (cudaGetLastError() != cudaSuccess) return -1;
    const int items = g.Hv * toks.n;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(items < sm_count ? items : sm_count);
    lc.blockDim = dim3(kStThreads);
    lc.dynamicSmemBytes = kStSmem;
    lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&lc, gdn_decode_stream_kernel, g, toks, ssm_state, ssm_seq_stride, z, norm_w, (const float *)scr_qk,
                                             (const float *)scr_v, (const float *)scr_db, out, err);
    return e == cudaSuccess ? 2 : -1;
}

}  // namespace fm
