// Split-KV decode attention over the paged bf16 KV store, and the log-sum-exp merge with the fused
// sigmoid output gate.
//
// Math of metal_infer/layer_forward.h:631-735 (scores = q.K/sqrt(D), max-subtracted softmax,
// weighted sum of V, times sigmoid(gate)), re-organised for a GPU:
//   * one CTA per (split of the sequence, KV head, sequence); the query heads that share the KV
//     head (up to 16) form the M dimension of bf16 tensor-core MMAs, so K and V are read from HBM
//     exactly once per step instead of once per query head;
//   * K/V pages (64 rows x 256 dims, 32 KB contiguous each) stream through a 3-stage shared-memory
//     ring filled by 16-byte asynchronous copies;
//   * online softmax in the exp2 domain with warp-shuffle row maxima; the running maximum is only
//     advanced when a row's maximum grew by more than 2^8, which keeps the rescaling of the
//     accumulators off the common path;
//   * q and the softmax weights enter the MMAs as two bf16 terms (hi + lo), which keeps ~16
//     mantissa bits: K and V are exact in bf16, so the result tracks the fp32 reference to ~1e-4;
//   * each CTA writes an un-normalised partial (O, max, sum); a second kernel merges the partials
//     and applies the gate.

#include "fm_device.cuh"
#include "fm_internal.h"


namespace fm {

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr int kD = 256;          // head dim the kernel is built for
constexpr int kPage = 64;        // rows per page
constexpr int kStages = 3;
constexpr int kTileBytes = kPage * kD * 2;  // one K or V tile: 32 KB
constexpr int kQBytes = 16 * kD * 2;        // 16 heads x 256 bf16
// Warp layout: 4 row-slices of 16 rows per tile x kNS warps per slice.  The warps of a slice split
// the head dim: each computes the partial scores over its 256/kNS dims, the partials are summed
// through shared memory (every warp of the slice then holds the same full scores), and each
// accumulates its own 256/kNS output dims.  More warps per scheduler hide the latency of the
// dependent MMA chains; the accumulator shrinks to 128/kNS registers per thread.
constexpr int kNS = 2;
constexpr int kDecWarps = 4 * kNS;
constexpr int kDecThreads = 32 * kDecWarps;
constexpr int kXchgBytes = 4 * kNS * 32 * 8 * 4;  // partial scores: [slice][split][lane][8] fp32
constexpr int kDecSmem = 2 * kQBytes + kXchgBytes + kStages * 2 * kTileBytes;
constexpr int kKSteps = (kD / 16) / kNS;   // k-steps of 16 dims a warp takes in Q K^T
constexpr int kNChunks = (kD / 16) / kNS;  // 16-dim output chunks a warp owns in P V

__device__ __forceinline__ void load_tile_async(uint32_t dst, const __nv_bfloat16 *src, int tid) {
    // 64 rows x 32 chunks of 16 B; consecutive threads take consecutive chunks (coalesced 512 B / warp)
#pragma unroll
    for (int i = 0; i < (kPage * 32) / kDecThreads; i++) {
        const int c = tid + i * kDecThreads;
        const int row = c >> 5, ch = c & 31;
        cp_async16(dst + swz_row512(row, ch), reinterpret_cast<const char *>(src) + (size_t)c * 16);
    }
}

// Programmatic dependent launch (griddepcontrol): both are no-ops unless the launch carries the
// programmatic-stream-serialization attribute.
__device__ __forceinline__ void dep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(nthreads) : "memory");
}

// What the fused form of the kernel does besides the split partials:
//   * append: the CTA whose last tile holds the step's new row forms that row itself (k: RMS-norm +
//     RoPE), stores it to the page and patches its shared-memory tile -- no separate append launch;
//   * tail: with one split per (KV head, sequence) the CTA finishes its rows itself; with several, the
//     last CTA to arrive at the unit's counter merges the splits (in two levels when there are many)
//     -- no separate merge launch, no grid barrier.  tail = 1: normalise, gate,
//     write the output; 2: un-normalised row and (max, sum) for the caller to exchange; 3: store the
//     row into every peer's exchange buffer and publish the step; 4: store the
//     rows of this (token, KV head) into every peer's buffer, publish that unit, wait -- bounded --
//     for every peer's rows of the same unit, merge them by log-sum-exp, gate, write the output: the
//     whole sequence-sharded step in this one kernel.
struct DecodeFused {
    const float *k_new, *v_new;  // [tokens][Hkv*D] or null
    const uint16_t *knw;
    int tail;
    const float *gate;  // [tokens][H*D] when q_proj_out is not given
    float *out;
    float *ml_out;
    XchgView x;
    uint32_t step;
    unsigned int *counters;  // [tokens*Hkv] arrivals per (token, KV head) + [1] finished units; self-resetting
    unsigned int *group_counters;  // [tokens*Hkv][kDecMaxGroups] arrivals per group of splits (many splits only)
    float *group_o, *group_ml;     // [tokens][H][kDecMaxGroups][D] / [..][2]: the groups' merged partials
    int *err;                // tail 4: device error word (a peer never published)
};


template <bool kFused>
__global__ void __launch_bounds__(kDecThreads, 1)
attn_decode_kernel(KvView kv, RopeParams rope, TokSpec toks, int H, const float *__restrict__ q_proj_out,
                   const float *__restrict__ q_in, const uint16_t *__restrict__ qnw, float eps,
                   float *__restrict__ part_o, float *__restrict__ part_ml, int nsplits, DecodeFused f) {
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t s_qhi = smem_u32(smem);
    const uint32_t s_qlo = s_qhi + kQBytes;
    float *s_x = reinterpret_cast<float *>(smem + 2 * kQBytes);
    const uint32_t s_kv = s_qlo + kQBytes + kXchgBytes;  // stage s: K at s_kv + s*2*kTileBytes, V right after
    unsigned char *kv_raw = smem + 2 * kQBytes + kXchgBytes;

    const int split = blockIdx.x, kvh = blockIdx.y, tok = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // A following launch marked as programmatically dependent (another layer's step) may start filling
    // free SMs now.
    if (kFused) dep_launch_dependents();
    const int pw = warp & 3;   // which 16 rows of the tile
    const int hs = warp >> 2;  // which share of the head dim
    const int group = H / kv.Hkv;  // query heads per KV head (<= 16)

    int seq, pos, row_new;
    tok_get(toks, tok, seq, pos, row_new);
    const int L = tok_rows(toks, tok);  // rows attended, the new one included (row_new + 1 unless the window wrapped)

    // ---- which page slots this CTA walks ----
    const int gpages = (L + kPage - 1) / kPage;
    const int nslots = gpages > kv.shard_rank ? (gpages - kv.shard_rank + kv.shard_count - 1) / kv.shard_count : 0;
    const int per = (nslots + nsplits - 1) / nsplits;
    const int slot_begin = split * per;
    const int slot_end = min(nslots, slot_begin + per);
    const int ntiles = max(0, slot_end - slot_begin);
    const int *ptab = kv.page_table + (size_t)seq * kv.max_slots;
    const size_t page_elems = (size_t)2 * kv.Hkv * kPage * kD;

    auto issue = [&](int t) {
        if (t < ntiles) {
            const int page = ptab[slot_begin + t];
            const __nv_bfloat16 *base = kv.pool + (size_t)page * page_elems;
            const uint32_t dst = s_kv + (uint32_t)(t % kStages) * 2 * kTileBytes;
            load_tile_async(dst, base + (size_t)kvh * kPage * kD, tid);
            load_tile_async(dst + kTileBytes, base + (size_t)(kv.Hkv + kvh) * kPage * kD, tid);
        }
        cp_async_commit();
    };
    issue(0);
    issue(1);

    // ---- q: RMS-norm, partial RoPE, scale, split into two bf16 terms -> shared memory ----
    // stage 2 of the ring is free until the first loop iteration: use it as fp32 scratch
    // rotation table of this token: one sincos per lane instead of eight per row on a few lanes (the
    // accurate sincosf is some hundred instructions, more beyond |x| ~ 1e5)
    __shared__ float s_rc[64], s_rs[64];
    if (tid < rope.rotary_dim / 2) {
        float sn, cs;
        sincos_reduced(((float)pos / rope.pos_div) * rope.inv_freq[tid], sn, cs);
        s_rc[tid] = cs;
        s_rs[tid] = sn;
    }
    __syncthreads();
    {
        float *scratch = reinterpret_cast<float *>(kv_raw + 2 * 2 * kTileBytes);  // [16][256]
        const float qscale = rope.logit_scale * kLog2e;
        const int half = rope.rotary_dim / 2;
        for (int r = warp; r < 16; r += kDecWarps) {
            float x[8];
            if (r < group) {
                const int head = kvh * group + r;
                const float *src = q_proj_out ? q_proj_out + ((size_t)tok * H + head) * 2 * kD
                                              : q_in + ((size_t)tok * H + head) * kD;
                const float4 a = *reinterpret_cast<const float4 *>(src + lane * 8);
                const float4 b = *reinterpret_cast<const float4 *>(src + lane * 8 + 4);
                x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
                x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
                if (qnw != nullptr) {
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++) ss += x[j] * x[j];
                    ss = warp_sum(ss);
                    const float inv = 1.0f / sqrtf(ss / kD + eps);
#pragma unroll
                    for (int j = 0; j < 8; j++) x[j] = x[j] * inv * bf16_bits_to_float(qnw[lane * 8 + j]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] = 0.f;
            }
            float *srow = scratch + r * kD;
#pragma unroll
            for (int j = 0; j < 8; j++) srow[lane * 8 + j] = x[j];
            __syncwarp();
            if (r < group) {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int d = lane * 8 + j;
                    if (d < rope.rotary_dim) {
                        const int i = d < half ? d : d - half;
                        const float c = s_rc[i], s = s_rs[i];
                        x[j] = d < half ? x[j] * c - srow[d + half] * s : srow[d - half] * s + x[j] * c;
                    }
                }
            }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 4; j++) split_pack_bf16(x[2 * j] * qscale, x[2 * j + 1] * qscale, hi[j], lo[j]);
            const uint32_t off = swz_row512(r, lane);
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(s_qhi + off), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]));
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(s_qlo + off), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]));
        }
    }

    // ---- main loop ----
    float o[2 * kNChunks][4];
#pragma unroll
    for (int i = 0; i < 2 * kNChunks; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_ref[2] = {kNegBig, kNegBig};  // rows lane/4 and lane/4 + 8
    float l_sum[2] = {0.f, 0.f};

    const int lm = lane >> 3, lr = lane & 7;  // ldmatrix: matrix index and row within it
    // partial-score exchange buffer, [slice][split][2 float4 planes][lane]: lanes 16 B apart, no bank conflicts
    float4 *xmine = reinterpret_cast<float4 *>(s_x) + (size_t)(pw * kNS + hs) * 64 + lane;
    const float4 *xslice = reinterpret_cast<const float4 *>(s_x) + (size_t)(pw * kNS) * 64 + lane;
    // this warp's q fragments (its share of the head dim, hi and lo terms) stay in registers
    __syncthreads();
    uint32_t qh[kKSteps][4], ql[kKSteps][4];
#pragma unroll
    for (int k8 = 0; k8 < kKSteps; k8++) {
        const uint32_t qoff = swz_row512(lr + (lm & 1) * 8, 2 * (hs * kKSteps + k8) + (lm >> 1));
        ldmatrix_x4(qh[k8][0], qh[k8][1], qh[k8][2], qh[k8][3], s_qhi + qoff);
        ldmatrix_x4(ql[k8][0], ql[k8][1], ql[k8][2], ql[k8][3], s_qlo + qoff);
    }
    for (int t = 0; t < ntiles; t++) {
        cp_async_wait<1>();
        __syncthreads();  // tile t landed for everyone; everyone is done with tile t-1 (and with q)
        issue(t + 2);

        const int gpage = (slot_begin + t) * kv.shard_count + kv.shard_rank;
        if (kFused && f.k_new != nullptr && gpage == row_new / kPage) {
            // this tile holds the step's new row: form it, store it to the page, patch the tile
            const int rn = row_new - gpage * kPage, d = tid;  // 256 threads = 256 dims
            float *red = s_x, *xs = s_x + 8;               // the score-exchange buffer is idle here
            float x = f.k_new[((size_t)tok * kv.Hkv + kvh) * kD + d];
            if (f.knw != nullptr) {
                const float ss = warp_sum(x * x);
                if (lane == 0) red[warp] = ss;
                __syncthreads();
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kDecWarps; w++) tot += red[w];
                x = x * (1.0f / sqrtf(tot / kD + eps)) * bf16_bits_to_float(f.knw[d]);
            }
            xs[d] = x;
            __syncthreads();
            const int half = rope.rotary_dim / 2;
            if (d < rope.rotary_dim) {
                const int i = d < half ? d : d - half;
                const float c = s_rc[i], sn = s_rs[i];
                x = d < half ? x * c - xs[d + half] * sn : xs[d - half] * sn + x * c;
            }
            const __nv_bfloat16 kb = __float2bfloat16_rn(x);
            const __nv_bfloat16 vb = __float2bfloat16_rn(f.v_new[((size_t)tok * kv.Hkv + kvh) * kD + d]);
            __nv_bfloat16 *pg = kv.pool + (size_t)ptab[slot_begin + t] * page_elems;
            pg[((size_t)kvh * kPage + rn) * kD + d] = kb;
            pg[((size_t)(kv.Hkv + kvh) * kPage + rn) * kD + d] = vb;
            const uint32_t tile = s_kv + (uint32_t)(t % kStages) * 2 * kTileBytes;
            const uint32_t off = swz_row512(rn, d >> 3) + (d & 7) * 2;
            asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(tile + off), "h"(*reinterpret_cast<const unsigned short *>(&kb)) : "memory");
            asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(tile + kTileBytes + off), "h"(*reinterpret_cast<const unsigned short *>(&vb)) : "memory");
            __syncthreads();
        }
        const int p0 = gpage * kPage + pw * 16;  // first row of this slice's 16
        if (p0 >= L) continue;                   // the whole slice skips together
        const uint32_t sk = s_kv + (uint32_t)(t % kStages) * 2 * kTileBytes;
        const uint32_t sv = sk + kTileBytes;

        // partial S = Q K^T over this warp's dims; hi and lo terms in separate accumulators
        float sh[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float sl[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int k8 = 0; k8 < kKSteps; k8++) {
            const int kk = hs * kKSteps + k8;
            uint32_t b[4];
            ldmatrix_x4(b[0], b[1], b[2], b[3], sk + swz_row512(pw * 16 + (lm >> 1) * 8 + lr, 2 * kk + (lm & 1)));
            mma_bf16(sh[0], qh[k8][0], qh[k8][1], qh[k8][2], qh[k8][3], b[0], b[1]);
            mma_bf16(sh[1], qh[k8][0], qh[k8][1], qh[k8][2], qh[k8][3], b[2], b[3]);
            mma_bf16(sl[0], ql[k8][0], ql[k8][1], ql[k8][2], ql[k8][3], b[0], b[1]);
            mma_bf16(sl[1], ql[k8][0], ql[k8][1], ql[k8][2], ql[k8][3], b[2], b[3]);
        }
        // exchange: every warp of the slice sums the kNS partials in the same order
        xmine[0] = make_float4(sh[0][0] + sl[0][0], sh[0][1] + sl[0][1], sh[0][2] + sl[0][2], sh[0][3] + sl[0][3]);
        xmine[32] = make_float4(sh[1][0] + sl[1][0], sh[1][1] + sl[1][1], sh[1][2] + sl[1][2], sh[1][3] + sl[1][3]);
        named_barrier(1 + pw, 32 * kNS);
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int j = 0; j < kNS; j++) {
            const float4 a = xslice[j * 64];
            const float4 c = xslice[j * 64 + 32];
            s[0][0] += a.x; s[0][1] += a.y; s[0][2] += a.z; s[0][3] += a.w;
            s[1][0] += c.x; s[1][1] += c.y; s[1][2] += c.z; s[1][3] += c.w;
        }
        // mask rows beyond the sequence
        if (p0 + 16 > L) {
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int p = p0 + nt * 8 + 2 * (lane & 3) + (e & 1);
                    if (p >= L) s[nt][e] = kNegBig;
                }
        }
        // row maxima (rows g and g+8), shared by the 4 lanes of a quad
        float mx[2];
        mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        const bool grow = (mx[0] > m_ref[0] + 8.f) || (mx[1] > m_ref[1] + 8.f);
        if (__any_sync(0xffffffffu, grow)) {
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const float mn = fmaxf(m_ref[r], mx[r]);
                corr[r] = fast_exp2(m_ref[r] - mn);
                m_ref[r] = mn;
                l_sum[r] *= corr[r];
            }
#pragma unroll
            for (int i = 0; i < 2 * kNChunks; i++) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
        }
        // weights, as two bf16 terms
        uint32_t ph[4], pl[4];
        {
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                p[nt][0] = fast_exp2(s[nt][0] - m_ref[0]);
                p[nt][1] = fast_exp2(s[nt][1] - m_ref[0]);
                p[nt][2] = fast_exp2(s[nt][2] - m_ref[1]);
                p[nt][3] = fast_exp2(s[nt][3] - m_ref[1]);
            }
            l_sum[0] += p[0][0] + p[0][1] + p[1][0] + p[1][1];
            l_sum[1] += p[0][2] + p[0][3] + p[1][2] + p[1][3];
            split_pack_bf16(p[0][0], p[0][1], ph[0], pl[0]);
            split_pack_bf16(p[0][2], p[0][3], ph[1], pl[1]);
            split_pack_bf16(p[1][0], p[1][1], ph[2], pl[2]);
            split_pack_bf16(p[1][2], p[1][3], ph[3], pl[3]);
        }
        // O += P V on this warp's output dims
#pragma unroll
        for (int n8 = 0; n8 < kNChunks; n8++) {
            const int nn = hs * kNChunks + n8;
            uint32_t b[4];
            ldmatrix_x4_trans(b[0], b[1], b[2], b[3], sv + swz_row512(pw * 16 + (lm & 1) * 8 + lr, 2 * nn + (lm >> 1)));
            mma_bf16(o[2 * n8], ph[0], ph[1], ph[2], ph[3], b[0], b[1]);
            mma_bf16(o[2 * n8 + 1], ph[0], ph[1], ph[2], ph[3], b[2], b[3]);
            mma_bf16(o[2 * n8], pl[0], pl[1], pl[2], pl[3], b[0], b[1]);
            mma_bf16(o[2 * n8 + 1], pl[0], pl[1], pl[2], pl[3], b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four row-slices through shared memory (the ring is free now) ----
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_sum[r] += __shfl_xor_sync(0xffffffffu, l_sum[r], 1);
        l_sum[r] += __shfl_xor_sync(0xffffffffu, l_sum[r], 2);
    }
    float *s_o = reinterpret_cast<float *>(kv_raw);                 // [4][16][256]
    float *s_ml = reinterpret_cast<float *>(kv_raw + 4 * 16 * kD * 4);  // [4][16][2]
    {
        const int g = lane >> 2, tq = lane & 3;
        if (tq == 0 && hs == 0) {
            s_ml[(pw * 16 + g) * 2 + 0] = m_ref[0];
            s_ml[(pw * 16 + g) * 2 + 1] = l_sum[0];
            s_ml[(pw * 16 + g + 8) * 2 + 0] = m_ref[1];
            s_ml[(pw * 16 + g + 8) * 2 + 1] = l_sum[1];
        }
        float *wo = s_o + (size_t)pw * 16 * kD + hs * (kD / kNS);
#pragma unroll
        for (int i = 0; i < 2 * kNChunks; i++) {
            *reinterpret_cast<float2 *>(wo + g * kD + i * 8 + 2 * tq) = make_float2(o[i][0], o[i][1]);
            *reinterpret_cast<float2 *>(wo + (g + 8) * kD + i * 8 + 2 * tq) = make_float2(o[i][2], o[i][3]);
        }
    }
    __syncthreads();
    // finishes one (token, head) row chunk of 4 dims according to the tail mode
    auto emit = [&](int tk, int head, int d, float4 acc, float M, float lt) {
        if (f.tail == 1) {
            const float inv = lt > 0.f ? 1.0f / lt : 0.f;
            const float *gsrc = q_proj_out ? q_proj_out + ((size_t)tk * H + head) * 2 * kD + kD + d : f.gate + ((size_t)tk * H + head) * kD + d;
            const float4 g = *reinterpret_cast<const float4 *>(gsrc);
            *reinterpret_cast<float4 *>(f.out + ((size_t)tk * H + head) * kD + d) =
                make_float4(acc.x * inv * fast_sigmoid(g.x), acc.y * inv * fast_sigmoid(g.y), acc.z * inv * fast_sigmoid(g.z),
                            acc.w * inv * fast_sigmoid(g.w));
        } else if (f.tail == 2) {
            *reinterpret_cast<float4 *>(f.out + ((size_t)tk * H + head) * kD + d) = acc;
            if (d == 0) {
                f.ml_out[((size_t)tk * H + head) * 2 + 0] = M;
                f.ml_out[((size_t)tk * H + head) * 2 + 1] = lt;
            }
        } else {
            const size_t row = ((((size_t)(f.step & 1) * f.x.nranks + f.x.me) * f.x.cap + tk) * H + head) * (kD + 2);
            for (int r = 0; r < f.x.nranks; r++) {
                float *dst = f.x.peer[r] + row;
                *reinterpret_cast<float2 *>(dst + d) = make_float2(acc.x, acc.y);
                *reinterpret_cast<float2 *>(dst + d + 2) = make_float2(acc.z, acc.w);
                if (d == 0) *reinterpret_cast<float2 *>(dst + kD) = make_float2(M, lt);
            }
        }
    };
    const bool direct = kFused && nsplits == 1;  // this CTA is the only split: finish the rows here
    // A launch that was started as a programmatic dependent of the previous one (another layer's step) has
    // streamed its pages while that launch drained; from here on it writes what later work reads (partials,
    // counters, exchange slots, the output), so every CTA waits for the previous launch to have completed and
    // flushed.  A dependent of a grid that uses launch_dependents has to execute this wait, and with it the
    // launches of one fm_attn_decode_layers call complete in order: whatever follows the last layer in the
    // stream follows all of them.  No effect for an ordinary launch.
    if (kFused) dep_wait();
    for (int r = warp; r < group; r += kDecWarps) {
        float mw[4], M = kNegBig;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            mw[w] = s_ml[(w * 16 + r) * 2];
            M = fmaxf(M, mw[w]);
        }
        float fw[4], lt = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            fw[w] = fast_exp2(mw[w] - M);
            lt += fw[w] * s_ml[(w * 16 + r) * 2 + 1];
        }
        const int head = kvh * group + r;
        const size_t prow = ((size_t)tok * H + head) * nsplits + split;
        float *dst = part_o + prow * kD;
#pragma unroll
        for (int j = 0; j < kD / 128; j++) {
            const int d = (j * 32 + lane) * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float4 v = *reinterpret_cast<const float4 *>(s_o + ((size_t)w * 16 + r) * kD + d);
                acc.x += fw[w] * v.x; acc.y += fw[w] * v.y; acc.z += fw[w] * v.z; acc.w += fw[w] * v.w;
            }
            if (direct)
                emit(tok, head, d, acc, M, lt);
            else
                *reinterpret_cast<float4 *>(dst + d) = acc;
        }
        if (!direct && lane == 0) {
            part_ml[prow * 2 + 0] = M;
            part_ml[prow * 2 + 1] = lt;
        }
    }
    if (!kFused) return;
    if (!direct) {
        // ---- merge of the splits by the last CTA to arrive -------------------------------------------
        // Up to kDecMaxLastCtaSplits splits per (token, KV head): the last CTA of the unit merges them all.
        // More (small batch, long context): the splits form groups of kDecGroup; the last CTA of a group
        // merges the group into one partial per head, the last group to finish merges the groups.  Either
        // way a warp takes whole heads: lane j holds the (max, sum) of part j, the weights travel by
        // shuffle, and the row loads of its heads are in flight together.
        __shared__ int s_last;
        // two heads at a time (with 16 heads per KV head and 8 warps that is the whole share of a warp), so that
        // the loads of both are in flight together; `two` false: the second head is a dummy copy of the first
        struct Merged { float4 a0, a1; float M, lt; };
        auto merge_heads = [&](const float *po0, const float *pml0, const float *po1, const float *pml1, int cnt, Merged &x, Merged &y) {
            const float2 ml0 = lane < cnt ? __ldcg(reinterpret_cast<const float2 *>(pml0) + lane) : make_float2(kNegBig, 0.f);
            const float2 ml1 = lane < cnt ? __ldcg(reinterpret_cast<const float2 *>(pml1) + lane) : make_float2(kNegBig, 0.f);
            x.M = warp_max(ml0.x);
            y.M = warp_max(ml1.x);
            const float w0 = fast_exp2(ml0.x - x.M), w1 = fast_exp2(ml1.x - y.M);
            x.lt = warp_sum(w0 * ml0.y);
            y.lt = warp_sum(w1 * ml1.y);
            x.a0 = x.a1 = y.a0 = y.a1 = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 *s0 = reinterpret_cast<const float4 *>(po0) + lane * 2, *s1 = reinterpret_cast<const float4 *>(po1) + lane * 2;
#pragma unroll 4
            for (int j = 0; j < cnt; j++) {
                const float wa = __shfl_sync(0xffffffffu, w0, j), wb = __shfl_sync(0xffffffffu, w1, j);
                const float4 p0 = __ldcg(s0 + (size_t)j * (kD / 4)), p1 = __ldcg(s0 + (size_t)j * (kD / 4) + 1);
                const float4 q0 = __ldcg(s1 + (size_t)j * (kD / 4)), q1 = __ldcg(s1 + (size_t)j * (kD / 4) + 1);
                x.a0.x += wa * p0.x; x.a0.y += wa * p0.y; x.a0.z += wa * p0.z; x.a0.w += wa * p0.w;
                x.a1.x += wa * p1.x; x.a1.y += wa * p1.y; x.a1.z += wa * p1.z; x.a1.w += wa * p1.w;
                y.a0.x += wb * q0.x; y.a0.y += wb * q0.y; y.a0.z += wb * q0.z; y.a0.w += wb * q0.w;
                y.a1.x += wb * q1.x; y.a1.y += wb * q1.y; y.a1.z += wb * q1.z; y.a1.w += wb * q1.w;
            }
        };
        // arrival at a counter; true for the CTA that completes it (which also resets it)
        auto arrive_last = [&](unsigned int *cnt, int expected) {
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int old = atomicAdd(cnt, 1u);
                s_last = old == (unsigned int)expected - 1;
                if (s_last) *cnt = 0;
            }
            __syncthreads();
            const bool last = s_last != 0;
            if (last) __threadfence();
            return last;
        };
        const int unit = tok * kv.Hkv + kvh;
        if (nsplits <= kDecMaxLastCtaSplits) {
            if (!arrive_last(f.counters + unit, nsplits)) return;
            for (int r = warp; r < group; r += 2 * kDecWarps) {
                const bool two = r + kDecWarps < group;
                const int h0 = kvh * group + r, h1 = two ? h0 + kDecWarps : h0;
                const size_t p0 = ((size_t)tok * H + h0) * nsplits, p1 = ((size_t)tok * H + h1) * nsplits;
                Merged x, y;
                merge_heads(part_o + p0 * kD, part_ml + p0 * 2, part_o + p1 * kD, part_ml + p1 * 2, nsplits, x, y);
                emit(tok, h0, lane * 8, x.a0, x.M, x.lt);
                emit(tok, h0, lane * 8 + 4, x.a1, x.M, x.lt);
                if (two) {
                    emit(tok, h1, lane * 8, y.a0, y.M, y.lt);
                    emit(tok, h1, lane * 8 + 4, y.a1, y.M, y.lt);
                }
            }
        } else {
            const int gi = split / kDecGroup, gfirst = gi * kDecGroup;
            const int gcount = min(kDecGroup, nsplits - gfirst), ngroups = (nsplits + kDecGroup - 1) / kDecGroup;
            if (!arrive_last(f.group_counters + unit * kDecMaxGroups + gi, gcount)) return;
            auto put_group = [&](int head, const Merged &m) {
                const size_t g2 = ((size_t)tok * H + head) * kDecMaxGroups + gi;
                float4 *dst = reinterpret_cast<float4 *>(f.group_o + g2 * kD) + lane * 2;
                dst[0] = m.a0;
                dst[1] = m.a1;
                if (lane == 0) *reinterpret_cast<float2 *>(f.group_ml + g2 * 2) = make_float2(m.M, m.lt);
            };
            for (int r = warp; r < group; r += 2 * kDecWarps) {
                const bool two = r + kDecWarps < group;
                const int h0 = kvh * group + r, h1 = two ? h0 + kDecWarps : h0;
                const size_t p0 = ((size_t)tok * H + h0) * nsplits + gfirst, p1 = ((size_t)tok * H + h1) * nsplits + gfirst;
                Merged x, y;
                merge_heads(part_o + p0 * kD, part_ml + p0 * 2, part_o + p1 * kD, part_ml + p1 * 2, gcount, x, y);
                put_group(h0, x);
                if (two) put_group(h1, y);
            }
            if (!arrive_last(f.counters + unit, ngroups)) return;
            for (int r = warp; r < group; r += 2 * kDecWarps) {
                const bool two = r + kDecWarps < group;
                const int h0 = kvh * group + r, h1 = two ? h0 + kDecWarps : h0;
                const size_t g0 = ((size_t)tok * H + h0) * kDecMaxGroups, g1 = ((size_t)tok * H + h1) * kDecMaxGroups;
                Merged x, y;
                merge_heads(f.group_o + g0 * kD, f.group_ml + g0 * 2, f.group_o + g1 * kD, f.group_ml + g1 * 2, ngroups, x, y);
                emit(tok, h0, lane * 8, x.a0, x.M, x.lt);
                emit(tok, h0, lane * 8 + 4, x.a1, x.M, x.lt);
                if (two) {
                    emit(tok, h1, lane * 8, y.a0, y.M, y.lt);
                    emit(tok, h1, lane * 8 + 4, y.a1, y.M, y.lt);
                }
            }
        }
    }
    if (f.tail == 4) {
        // ---- this CTA has stored the unit's rows into every rank's buffer: publish, wait, merge ----
        __shared__ int s_ok;
        const int nr = f.x.nranks, par = f.step & 1;
        const int nunits = f.x.cap * kv.Hkv, unit = tok * kv.Hkv + kvh;
        if (tid == 0) s_ok = 1;
        __threadfence_system();
        __syncthreads();
        if (tid < nr) {
            uint32_t *theirs = reinterpret_cast<uint32_t *>(f.x.peer[tid] + f.x.unit_flag_offset_floats) + ((size_t)par * nr + f.x.me) * nunits + unit;
            st_release_sys(theirs, f.step);
            const uint32_t *mine_f = reinterpret_cast<const uint32_t *>(f.x.peer[f.x.me] + f.x.unit_flag_offset_floats) + ((size_t)par * nr + tid) * nunits + unit;
            const long long t0 = clock64();
            while ((int32_t)(ld_acquire_sys(mine_f) - f.step) < 0) {
                if (clock64() - t0 > f.x.wait_limit_cycles) {  // rank `tid` never published this unit
                    s_ok = 0;
                    atomicCAS(f.err, 0, (2 << 16) | tid);
                    break;
                }
            }
        }
        __syncthreads();
        const float *mine = f.x.peer[f.x.me];
        for (int r = warp; r < group; r += kDecWarps) {
            const int head = kvh * group + r;
            float *dst = f.out + ((size_t)tok * H + head) * kD + lane * 8;
            if (!s_ok) {
                *reinterpret_cast<float4 *>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(dst + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                continue;
            }
            const size_t row0 = (((size_t)par * nr * f.x.cap + tok) * H + head) * (kD + 2);  // rank 0's row
            const size_t rstride = (size_t)f.x.cap * H * (kD + 2);
            const float2 mlj = lane < nr ? __ldcg(reinterpret_cast<const float2 *>(mine + row0 + lane * rstride + kD)) : make_float2(kNegBig, 0.f);
            const float M = warp_max(mlj.x);
            const float wj = fast_exp2(mlj.x - M);
            const float lt = warp_sum(wj * mlj.y);
            float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < nr; j++) {
                const float w = __shfl_sync(0xffffffffu, wj, j);
                const float2 *src = reinterpret_cast<const float2 *>(mine + row0 + j * rstride + lane * 8);
#pragma unroll
                for (int q2 = 0; q2 < 4; q2++) {
                    const float2 v = __ldcg(src + q2);
                    a[2 * q2] += w * v.x;
                    a[2 * q2 + 1] += w * v.y;
                }
            }
            const float inv = lt > 0.f ? 1.0f / lt : 0.f;
            const float *gsrc = q_proj_out ? q_proj_out + ((size_t)tok * H + head) * 2 * kD + kD + lane * 8 : f.gate + ((size_t)tok * H + head) * kD + lane * 8;
            const float4 g0 = *reinterpret_cast<const float4 *>(gsrc), g1 = *reinterpret_cast<const float4 *>(gsrc + 4);
            *reinterpret_cast<float4 *>(dst) = make_float4(a[0] * inv * fast_sigmoid(g0.x), a[1] * inv * fast_sigmoid(g0.y),
                                                           a[2] * inv * fast_sigmoid(g0.z), a[3] * inv * fast_sigmoid(g0.w));
            *reinterpret_cast<float4 *>(dst + 4) = make_float4(a[4] * inv * fast_sigmoid(g1.x), a[5] * inv * fast_sigmoid(g1.y),
                                                               a[6] * inv * fast_sigmoid(g1.z), a[7] * inv * fast_sigmoid(g1.w));
        }
        return;
    }
    if (f.tail == 3) {
        // this (token, KV head) is in every peer's buffer; the last unit to get here publishes the step
        __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            unsigned int *done = f.counters + gridDim.z * kv.Hkv;
            const unsigned int units = gridDim.y * gridDim.z;
            if (atomicAdd(done, 1u) == units - 1) {
                *done = 0;
                __threadfence_system();
                for (int r = 0; r < f.x.nranks; r++) {
                    uint32_t *flags = reinterpret_cast<uint32_t *>(f.x.peer[r] + f.x.flag_offset_floats);
                    st_release_sys(flags + (f.step & 1) * f.x.nranks + f.x.me, f.step);
                }
            }
        }
    }
}

int launch_attn_decode(const KvView &kv, const RopeParams &rope, const TokSpec &toks, int H,
                       const float *q_proj_out, const float *q, const uint16_t *q_norm_w, float eps,
                       float *part_o, float *part_ml, int nsplits, cudaStream_t st) {
    static unsigned long long configured = 0;  // one bit per device
    if (first_use_on_device(&configured)) {
        if (cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem) != cudaSuccess)
            return -1;
    }
    dim3 grid(nsplits, kv.Hkv, toks.n);
    DecodeFused f = {};
    attn_decode_kernel<false><<<grid, kDecThreads, kDecSmem, st>>>(kv, rope, toks, H, q_proj_out, q, q_norm_w, eps,
                                                                   part_o, part_ml, nsplits, f);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// The whole decode step in one launch (see DecodeFused).
int launch_attn_decode_fused(const KvView &kv, const RopeParams &rope, const TokSpec &toks, int H,
                             const float *q_proj_out, const float *q, const uint16_t *q_norm_w, float eps,
                             float *part_o, float *part_ml, int nsplits, const float *k_new, const float *v_new,
                             const uint16_t *k_norm_w, int tail, const float *gate, float *out, float *ml_out,
                             const XchgView *x, uint32_t step, const DecodeScratch &scr, int *err, bool overlap_prev,
                             cudaStream_t st) {
    static unsigned long long configured = 0;  // one bit per device
    if (first_use_on_device(&configured)) {
        if (cudaFuncSetAttribute(attn_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem) != cudaSuccess)
            return -1;
    }
    if (nsplits > kDecMaxLastCtaSplits && (toks.n > scr.group_tokens || nsplits > kDecGroup * kDecMaxGroups)) return -1;
    dim3 grid(nsplits, kv.Hkv, toks.n);
    DecodeFused f = {};
    f.k_new = k_new; f.v_new = v_new; f.knw = k_norm_w;
    f.tail = tail; f.gate = gate; f.out = out; f.ml_out = ml_out;
    if (x) f.x = *x;
    f.step = step;
    f.counters = scr.counters;
    f.group_counters = scr.group_counters;
    f.group_o = scr.group_o;
    f.group_ml = scr.group_ml;
    f.err = err;
    // overlap_prev: the caller vouches that this launch reads nothing the previous kernel in the
    // stream writes except through the scratch the kernel guards itself (another layer's step).
    // Its CTAs then take SMs as the previous grid's CTAs retire instead of after the grid drains.
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid; lc.blockDim = dim3(kDecThreads); lc.dynamicSmemBytes = kDecSmem; lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = overlap_prev ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&lc, attn_decode_kernel<true>, kv, rope, toks, H, q_proj_out, q, q_norm_w, eps, part_o, part_ml,
                                             nsplits, f);
    return e == cudaSuccess ? 1 : -1;
}

// ---- merge of partial results + sigmoid gate -------------------------------------------------
// grid (H, tokens), block D/4 threads (one float4 each).
// Final mode (out != nullptr && ml_out == nullptr): out = sum_j w_j O_j / sum_j w_j l_j * sigmoid(gate)
// Partial mode (ml_out != nullptr): out = sum_j w_j O_j (relative to the merged maximum), ml_out = (M, l)
__global__ void attn_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml,
                                  int nparts, long long ps_o, long long ps_ml, long long ts_o,
                                  long long ts_ml, long long hs_o, long long hs_ml, int H, int D,
                                  const float *__restrict__ q_proj_out, const float *__restrict__ gate,
                                  float *__restrict__ out, float *__restrict__ ml_out) {
    const int head = blockIdx.x, tok = blockIdx.y, d = threadIdx.x * 4;
    const float *o0 = part_o + tok * ts_o + head * hs_o;
    const float *ml0 = part_ml + tok * ts_ml + head * hs_ml;
    float M = kNegBig;
    for (int j = 0; j < nparts; j++) M = fmaxf(M, ml0[j * ps_ml]);
    float lt = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < nparts; j++) {
        const float w = fast_exp2(ml0[j * ps_ml] - M);
        lt += w * ml0[j * ps_ml + 1];
        const float4 v = *reinterpret_cast<const float4 *>(o0 + j * ps_o + d);
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    float *dst = out + ((size_t)tok * H + head) * D + d;
    if (ml_out != nullptr) {
        *reinterpret_cast<float4 *>(dst) = acc;
        if (threadIdx.x == 0) {
            ml_out[((size_t)tok * H + head) * 2 + 0] = M;
            ml_out[((size_t)tok * H + head) * 2 + 1] = lt;
        }
        return;
    }
    const float inv = lt > 0.f ? 1.0f / lt : 0.f;
    const float *gsrc = q_proj_out ? q_proj_out + ((size_t)tok * H + head) * 2 * D + D + d
                                   : gate + ((size_t)tok * H + head) * D + d;
    const float4 g = *reinterpret_cast<const float4 *>(gsrc);
    float4 r;
    r.x = acc.x * inv * fast_sigmoid(g.x);
    r.y = acc.y * inv * fast_sigmoid(g.y);
    r.z = acc.z * inv * fast_sigmoid(g.z);
    r.w = acc.w * inv * fast_sigmoid(g.w);
    *reinterpret_cast<float4 *>(dst) = r;
}

int launch_attn_merge(const float *part_o, const float *part_ml, int nparts, long long ps_o,
                      long long ps_ml, long long ts_o, long long ts_ml, long long hs_o,
                      long long hs_ml, int ntok, int H, int D, const float *q_proj_out,
                      const float *gate, float *out, float *ml_out, cudaStream_t st) {
    if (ntok <= 0) return 0;
    dim3 grid(H, ntok);
    attn_merge_kernel<<<grid, D / 4, 0, st>>>(part_o, part_ml, nparts, ps_o, ps_ml, ts_o, ts_ml, hs_o,
                                              hs_ml, H, D, q_proj_out, gate, out, ml_out);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

}  // namespace fm

// ---- cross-GPU exchange of partial results over peer memory -----------------------------------
// Each rank of a sequence group owns an exchange buffer that its peers can address (plain peer
// stores over NVLink; no multicast, no collective library call):
//     slots [2 (step parity)][nranks (source)][cap tokens][H][D + 2] floats, then flags [2][nranks].
// attn_merge_push_kernel merges the local split partials of one (token, head) and stores the result
// (un-normalised O, running max, sum) into slot [parity][me] of EVERY rank's buffer; the last CTA
// to finish publishes the step number in every rank's flag [parity][me].  attn_wait_merge_kernel
// waits -- for a bounded time -- until the flags of all sources show the step, then merges the
// nranks partials by log-sum-exp and applies the gate.  The two are separate launches: no CTA waits
// for another CTA of its own GPU, so nothing depends on co-residency.

namespace fm {

// grid (H, tokens), D/4 threads
__global__ void attn_merge_push_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, int nsplits, int H,
                                       XchgView x, uint32_t step, unsigned int *__restrict__ done_counter) {
    constexpr int D = kD;
    const int head = blockIdx.x, tok = blockIdx.y, d = threadIdx.x * 4;
    const float *o0 = part_o + ((size_t)tok * H + head) * nsplits * D;
    const float *ml0 = part_ml + ((size_t)tok * H + head) * nsplits * 2;
    float M = kNegBig;
    for (int j = 0; j < nsplits; j++) M = fmaxf(M, ml0[j * 2]);
    float lt = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < nsplits; j++) {
        const float w = fast_exp2(ml0[j * 2] - M);
        lt += w * ml0[j * 2 + 1];
        const float4 v = *reinterpret_cast<const float4 *>(o0 + (size_t)j * D + d);
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    const int par = step & 1;
    const size_t row = (((size_t)par * x.nranks + x.me) * x.cap + tok) * H + head;
    for (int r = 0; r < x.nranks; r++) {
        float *dst = x.peer[r] + row * (D + 2);
        *reinterpret_cast<float2 *>(dst + d) = make_float2(acc.x, acc.y);  // rows are 8-byte aligned (D + 2 floats)
        *reinterpret_cast<float2 *>(dst + d + 2) = make_float2(acc.z, acc.w);
        if (threadIdx.x == 0) *reinterpret_cast<float2 *>(dst + D) = make_float2(M, lt);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int total = gridDim.x * gridDim.y;
        if (atomicAdd(done_counter, 1u) == total - 1) {
            *done_counter = 0;
            __threadfence_system();
            for (int r = 0; r < x.nranks; r++) {
                uint32_t *flags = reinterpret_cast<uint32_t *>(x.peer[r] + x.flag_offset_floats);
                st_release_sys(flags + par * x.nranks + x.me, step);
            }
        }
    }
}

// grid (H, tokens), D/4 threads
__global__ void attn_wait_merge_kernel(XchgView x, uint32_t step, int H, const float *__restrict__ q_proj_out,
                                       const float *__restrict__ gate, float *__restrict__ out, int *__restrict__ err) {
    constexpr int D = kD;
    __shared__ int s_ok;
    const int head = blockIdx.x, tok = blockIdx.y, d = threadIdx.x * 4;
    const int par = step & 1;
    const float *mine = x.peer[x.me];
    dep_launch_dependents();
    if (threadIdx.x == 0) {
        const uint32_t *flags = reinterpret_cast<const uint32_t *>(mine + x.flag_offset_floats) + par * x.nranks;
        int ok = 1;
        const long long t0 = clock64();
        for (int r = 0; r < x.nranks && ok; r++) {
            while ((int32_t)(ld_acquire_sys(flags + r) - step) < 0) {
                if (clock64() - t0 > x.wait_limit_cycles) {  // a peer never published this step
                    ok = 0;
                    atomicCAS(err, 0, (2 << 16) | r);
                    break;
                }
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    dep_wait();  // launched ahead of the previous kernel's end: its writes are complete from here on
    float *dst = out + ((size_t)tok * H + head) * D + d;
    if (!s_ok) {
        *reinterpret_cast<float4 *>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    float M = kNegBig;
    for (int r = 0; r < x.nranks; r++) {
        const float *row = mine + ((((size_t)par * x.nranks + r) * x.cap + tok) * H + head) * (D + 2);
        M = fmaxf(M, __ldcg(row + D));
    }
    float lt = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < x.nranks; r++) {
        const float *row = mine + ((((size_t)par * x.nranks + r) * x.cap + tok) * H + head) * (D + 2);
        const float w = fast_exp2(__ldcg(row + D) - M);
        lt += w * __ldcg(row + D + 1);
        const float2 a = __ldcg(reinterpret_cast<const float2 *>(row + d)), b = __ldcg(reinterpret_cast<const float2 *>(row + d + 2));
        acc.x += w * a.x; acc.y += w * a.y; acc.z += w * b.x; acc.w += w * b.y;
    }
    const float inv = lt > 0.f ? 1.0f / lt : 0.f;
    const float *gsrc = q_proj_out ? q_proj_out + ((size_t)tok * H + head) * 2 * D + D + d : gate + ((size_t)tok * H + head) * D + d;
    const float4 g = *reinterpret_cast<const float4 *>(gsrc);
    *reinterpret_cast<float4 *>(dst) = make_float4(acc.x * inv * fast_sigmoid(g.x), acc.y * inv * fast_sigmoid(g.y),
                                                   acc.z * inv * fast_sigmoid(g.z), acc.w * inv * fast_sigmoid(g.w));
}

int launch_attn_merge_push(const float *part_o, const float *part_ml, int nsplits, int ntok, int H, const XchgView &x,
                           uint32_t step, unsigned int *done_counter, cudaStream_t st) {
    attn_merge_push_kernel<<<dim3(H, ntok), kD / 4, 0, st>>>(part_o, part_ml, nsplits, H, x, step, done_counter);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}
int launch_attn_wait_merge(const XchgView &x, uint32_t step, int ntok, int H, const float *q_proj_out, const float *gate,
                           float *out, int *err, bool overlap_prev, cudaStream_t st) {
    // overlap_prev: the CTAs may start (and poll the flags) while the kernel that pushes this rank's
    // own rows is still running; they read only what the flags cover
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(H, ntok); lc.blockDim = dim3(kD / 4); lc.dynamicSmemBytes = 0; lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = overlap_prev ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&lc, attn_wait_merge_kernel, x, step, H, q_proj_out, gate, out, err);
    return e == cudaSuccess ? 1 : -1;
}

}  // namespace fm
