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

#include <cuda_fp16.h>

#include "fm_device.cuh"
#include "fm_fp8.cuh"
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
constexpr int kQBytes = 16 * kD * 2;        // 16 heads x 256 16-bit elements
// Warp layout: 4 row-slices of 16 rows per tile x kNS warps per slice.  The warps of a slice split
// the head dim: each computes the partial scores over its 256/kNS dims, the partials are summed
// through shared memory (every warp of the slice then holds the same full scores), and each
// accumulates its own 256/kNS output dims.  More warps per scheduler hide the latency of the
// dependent MMA chains; the accumulator shrinks to 128/kNS registers per thread.
constexpr int kNS = 2;
constexpr int kDecWarps = 4 * kNS;
constexpr int kDecThreads = 32 * kDecWarps;
constexpr int kXchgBytes = 4 * kNS * 32 * 8 * 4;  // partial scores: [slice][split][lane][8] fp32
constexpr int kKSteps = (kD / 16) / kNS;   // k-steps of 16 dims a warp takes in Q K^T
constexpr int kNChunks = (kD / 16) / kNS;  // 16-dim output chunks a warp owns in P V

// Shared-memory ring.  bf16 store: a stage is a K tile and a V tile of 32 KB each, 3 stages.  FP8 store: tiles
// of 16 KB plus the 64 + 64 row scales, 6 stages (the same bytes in flight).
template <bool kFp8>
struct DecRing {
    static constexpr int kTile = kFp8 ? kPage * kD : kPage * kD * 2;
    static constexpr int kStage = kFp8 ? 2 * kTile + 2 * kPage * 4 : 2 * kTile;
    static constexpr int kStages = kFp8 ? 6 : 3;
    static constexpr int kSmem = 2 * kQBytes + kXchgBytes + kStages * kStage;
};
static_assert(DecRing<false>::kSmem <= 227 * 1024 && DecRing<true>::kSmem <= 227 * 1024, "shared memory");
static_assert(DecRing<true>::kStage >= 16 * kD * 4 && DecRing<true>::kStages * DecRing<true>::kStage >= 4 * 16 * kD * 4 + 4 * 16 * 2 * 4,
              "the ring doubles as scratch for q and for the slice merge");

// Rows of 256 B (256 E4M3 bytes) in shared memory, 16-byte chunk c of row r at chunk c ^ (r & 7): the eight row
// addresses of an 8x8 ldmatrix tile hit distinct banks.
__device__ __forceinline__ uint32_t swz_row256(int row, int chunk) {
    return static_cast<uint32_t>(row) * 256u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

template <bool kFp8>
__device__ __forceinline__ void load_tile_async(uint32_t dst, const unsigned char *src, int tid) {
    // 64 rows of 512 B (bf16) or 256 B (E4M3) as 16-byte chunks; consecutive threads take consecutive chunks
    constexpr int kChunksPerRow = kFp8 ? 16 : 32;
#pragma unroll
    for (int i = 0; i < (kPage * kChunksPerRow) / kDecThreads; i++) {
        const int c = tid + i * kDecThreads;
        const int row = c / kChunksPerRow, ch = c % kChunksPerRow;
        cp_async16(dst + (kFp8 ? swz_row256(row, ch) : swz_row512(row, ch)), src + (size_t)c * 16);
    }
}

// D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col)
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
// x = hi + lo with hi = fp16(x), lo = fp16(x - hi): 22 mantissa bits
__device__ __forceinline__ void split_pack_f16(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    const float2 hf = __half22float2(h);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = pack_f16(x0 - hf.x, x1 - hf.y);
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
//     whole sequence-sharded step in this one kernel.  tail = 0: stop at the partials (a merge launch with a
//     CTA per (head, token) follows; used when a sequence is split over the whole machine).
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
    H2oStep h2o;             // H2O store (slot != null): where the new row goes, and where the step's softmax weights are left
};

// kFp8: the store holds E4M3 bytes with one scale per row (fm_fp8.cuh).  The bytes go through the MMAs as fp16
// numbers made by moving bits (value * 2^-8, exact), q as two fp16 terms and the softmax weights as one; the K
// row scale multiplies the score, the V row scale the weight, and the 2^8 comes back in fp32.
template <bool kFused, bool kFp8>
__device__ __forceinline__ void attn_decode_body(const KvView &kv, const RopeParams &rope, const TokSpec &toks, int H,
                                                 const float *__restrict__ q_proj_out, const float *__restrict__ q_in,
                                                 const uint16_t *__restrict__ qnw, float eps, float *__restrict__ part_o,
                                                 float *__restrict__ part_ml, int nsplits, const DecodeFused &f) {
    using Ring = DecRing<kFp8>;
    constexpr int kTileBytes = Ring::kTile, kStageBytes = Ring::kStage, kStages = Ring::kStages;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t s_qhi = smem_u32(smem);
    const uint32_t s_qlo = s_qhi + kQBytes;
    float *s_x = reinterpret_cast<float *>(smem + 2 * kQBytes);
    const uint32_t s_kv = s_qlo + kQBytes + kXchgBytes;  // stage s: K at s_kv + s*kStageBytes, V right after, then the scales
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
    if (kFused && f.h2o.slot != nullptr) row_new = f.h2o.slot[seq];
    const int L = tok_rows(toks, tok);  // rows attended, the new one included (row_new + 1 unless the window wrapped)

    // ---- which page slots this CTA walks ----
    const int gpages = (L + kPage - 1) / kPage;
    const int nslots = gpages > kv.shard_rank ? (gpages - kv.shard_rank + kv.shard_count - 1) / kv.shard_count : 0;
    const int per = (nslots + nsplits - 1) / nsplits;
    const int slot_begin = split * per;
    const int slot_end = min(nslots, slot_begin + per);
    const int ntiles = max(0, slot_end - slot_begin);
    const int *ptab = kv.page_table + (size_t)seq * kv.max_slots;

    // rotation table of this token: one sincos per lane instead of eight per row on a few lanes (the
    // accurate sincosf is some hundred instructions, more beyond |x| ~ 1e5); needs nothing from global memory
    __shared__ float s_rc[64], s_rs[64];
    if (tid < rope.rotary_dim / 2) {
        float sn, cs;
        sincos_reduced(((float)pos / rope.pos_div) * rope.inv_freq[tid], sn, cs);
        s_rc[tid] = cs;
        s_rs[tid] = sn;
    }
    // does this CTA walk the page that takes the step's new row?
    const int page_new = row_new / kPage;
    const int slot_new = page_new / kv.shard_count;
    const bool has_new = kFused && f.k_new != nullptr && page_new % kv.shard_count == kv.shard_rank && slot_new >= slot_begin && slot_new < slot_end;

    // Everything the prologue needs from global memory is requested before anything waits: the page numbers of
    // the first tiles, this warp's two q rows and the norm weight.  (One dependent load after another -- page
    // number, then tile; q row, then the next q row -- used to cost a memory latency each, 3-5 us in all.)
    int first_pages[kStages - 1];
#pragma unroll
    for (int t = 0; t < kStages - 1; t++) first_pages[t] = t < ntiles ? __ldg(ptab + slot_begin + t) : 0;
    float qx[2][8];
    uint4 qw_bits = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = warp + i * kDecWarps;
        if (r < group) {
            const int head = kvh * group + r;
            const float *src = q_proj_out ? q_proj_out + ((size_t)tok * H + head) * 2 * kD : q_in + ((size_t)tok * H + head) * kD;
            const float4 a = __ldg(reinterpret_cast<const float4 *>(src + lane * 8));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(src + lane * 8 + 4));
            qx[i][0] = a.x; qx[i][1] = a.y; qx[i][2] = a.z; qx[i][3] = a.w;
            qx[i][4] = b.x; qx[i][5] = b.y; qx[i][6] = b.z; qx[i][7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) qx[i][j] = 0.f;
        }
    }
    if (qnw != nullptr) qw_bits = __ldg(reinterpret_cast<const uint4 *>(qnw) + lane);
    float new_k = 0.f, new_v = 0.f, new_w = 1.f;  // the new row's element of this thread (own KV head), fetched early too
    if (has_new) {
        new_k = __ldg(f.k_new + ((size_t)tok * kv.Hkv + kvh) * kD + tid);
        new_v = __ldg(f.v_new + ((size_t)tok * kv.Hkv + kvh) * kD + tid);
        if (f.knw != nullptr) new_w = bf16_bits_to_float(__ldg(f.knw + tid));
    }

    auto issue_page = [&](int t, int page) {
        const unsigned char *base = kv_page(kv, page);
        const uint32_t dst = s_kv + (uint32_t)(t % kStages) * kStageBytes;
        load_tile_async<kFp8>(dst, base + kv_tile_offset(kv, 0, kvh), tid);
        load_tile_async<kFp8>(dst + kTileBytes, base + kv_tile_offset(kv, 1, kvh), tid);
        if (kFp8 && tid < 32)  // k_scale[64] | v_scale[64]: 32 chunks of 16 bytes
            cp_async16(dst + 2 * kTileBytes + tid * 16, reinterpret_cast<const unsigned char *>(kv_page_scales(kv, const_cast<unsigned char *>(base), 0)) + tid * 16);
    };
    auto issue = [&](int t) {
        if (t < ntiles) issue_page(t, ptab[slot_begin + t]);
        cp_async_commit();
    };
#pragma unroll
    for (int t = 0; t < kStages - 1; t++) {
        if (t < ntiles) issue_page(t, first_pages[t]);
        cp_async_commit();
    }

    // ---- q: RMS-norm, partial RoPE, scale, split into two 16-bit terms -> shared memory ----
    // the last stage of the ring is free until the first loop iteration: use it as fp32 scratch
    __syncthreads();  // the rotation table is complete
    {
        float *scratch = reinterpret_cast<float *>(kv_raw + (kStages - 1) * kStageBytes);  // [16][256]
        const float qscale = rope.logit_scale * kLog2e;
        const int half = rope.rotary_dim / 2;
        const uint32_t wb[4] = {qw_bits.x, qw_bits.y, qw_bits.z, qw_bits.w};
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = warp + i * kDecWarps;
            float (&x)[8] = qx[i];
            if (r < group && qnw != nullptr) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) ss += x[j] * x[j];
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / kD + eps);
#pragma unroll
                for (int j = 0; j < 8; j++) x[j] = x[j] * inv * bf16_bits_to_float((uint16_t)(wb[j >> 1] >> ((j & 1) * 16)));
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
                        const int ii = d < half ? d : d - half;
                        const float c = s_rc[ii], s = s_rs[ii];
                        x[j] = d < half ? x[j] * c - srow[d + half] * s : srow[d - half] * s + x[j] * c;
                    }
                }
            }
            uint32_t hi[4], lo[4];
            if (!kFp8) {
#pragma unroll
                for (int j = 0; j < 4; j++) split_pack_bf16(x[2 * j] * qscale, x[2 * j + 1] * qscale, hi[j], lo[j]);
                const uint32_t off = swz_row512(r, lane);
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(s_qhi + off), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]));
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(s_qlo + off), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]));
            } else {
                // The K bytes reach the MMA straight from ldmatrix: a thread's register holds dims 4t..4t+3 of a row,
                // where the fp16 fragment wants dims (2t, 2t+1) and (2t+8, 2t+9).  q is stored with the dims of each
                // group of 16 permuted to match -- fragment slot (2t + j) holds dim 4t + j, slot (8 + 2t + j) dim
                // 4t + 2 + j -- so the dot product pairs every K dim with its own q dim.  A lane holds 8 dims = 4
                // pairs: pair 0 and 2 go to the first 16-byte chunk of the group (slots 0..7), pair 1 and 3 to the
                // second (slots 8..15), at word 0/1 for the even lane of the group and 2/3 for the odd one.
#pragma unroll
                for (int j = 0; j < 4; j++) split_pack_f16(x[2 * j] * qscale, x[2 * j + 1] * qscale, hi[j], lo[j]);
                const int grp = lane >> 1, odd = lane & 1;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t off = swz_row512(r, 2 * grp + (j & 1)) + (uint32_t)(2 * odd + (j >> 1)) * 4;
                    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(s_qhi + off), "r"(hi[j]));
                    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(s_qlo + off), "r"(lo[j]));
                }
            }
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
        cp_async_wait<kStages - 2>();
        __syncthreads();  // tile t landed for everyone; everyone is done with tile t-1 (and with q)
        issue(t + kStages - 1);

        const int gpage = (slot_begin + t) * kv.shard_count + kv.shard_rank;
        const uint32_t sk = s_kv + (uint32_t)(t % kStages) * kStageBytes;
        const uint32_t sv = sk + kTileBytes;
        float *s_scales = reinterpret_cast<float *>(kv_raw + (size_t)(t % kStages) * kStageBytes + 2 * kTileBytes);  // FP8: k[64] | v[64]
        if (has_new && gpage == page_new) {
            // this tile holds the step's new row: form it, store it to the page, patch the tile
            const int rn = row_new - gpage * kPage, d = tid;  // 256 threads = 256 dims
            float *red = s_x, *xs = s_x + 32;              // the score-exchange buffer is idle here
            const int half = rope.rotary_dim / 2;
            unsigned char *pg = kv_page(kv, ptab[slot_begin + t]);
            // k of head h: RMS-norm, RoPE (all 256 threads; two barriers inside)
            auto form_k = [&](int h) {
                float x = h == kvh ? new_k : f.k_new[((size_t)tok * kv.Hkv + h) * kD + d];
                if (f.knw != nullptr) {
                    const float ss = warp_sum(x * x);
                    __syncthreads();
                    if (lane == 0) red[warp] = ss;
                    __syncthreads();
                    float tot = 0.f;
#pragma unroll
                    for (int w = 0; w < kDecWarps; w++) tot += red[w];
                    x = x * (1.0f / sqrtf(tot / kD + eps)) * new_w;
                }
                __syncthreads();
                xs[d] = x;
                __syncthreads();
                if (d < rope.rotary_dim) {
                    const int ii = d < half ? d : d - half;
                    const float c = s_rc[ii], sn = s_rs[ii];
                    x = d < half ? x * c - xs[d + half] * sn : xs[d - half] * sn + x * c;
                }
                return x;
            };
            if (!kFp8) {
                const __nv_bfloat16 kb = __float2bfloat16_rn(form_k(kvh));
                const __nv_bfloat16 vb = __float2bfloat16_rn(new_v);
                reinterpret_cast<__nv_bfloat16 *>(pg + kv_tile_offset(kv, 0, kvh))[(size_t)rn * kD + d] = kb;
                reinterpret_cast<__nv_bfloat16 *>(pg + kv_tile_offset(kv, 1, kvh))[(size_t)rn * kD + d] = vb;
                const uint32_t off = swz_row512(rn, d >> 3) + (d & 7) * 2;
                asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(sk + off), "h"(*reinterpret_cast<const unsigned short *>(&kb)) : "memory");
                asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(sv + off), "h"(*reinterpret_cast<const unsigned short *>(&vb)) : "memory");
            } else {
                // the row's scale spans every KV head this context holds (metal_infer/fp8.h:100-108 over kv_dim), so
                // this CTA forms all of them, and encodes and stores its own head
                float kx = 0.f, vx = 0.f, ak = 0.f, av = 0.f;
                for (int h = 0; h < kv.Hkv; h++) {
                    const float x = form_k(h), vv = h == kvh ? new_v : f.v_new[((size_t)tok * kv.Hkv + h) * kD + d];
                    ak = fmaxf(ak, fabsf(x)); av = fmaxf(av, fabsf(vv));
                    if (h == kvh) { kx = x; vx = vv; }
                }
                ak = warp_max(ak); av = warp_max(av);
                __syncthreads();
                if (lane == 0) { red[warp] = ak; red[8 + warp] = av; }
                __syncthreads();
                ak = av = 0.f;
#pragma unroll
                for (int w = 0; w < kDecWarps; w++) { ak = fmaxf(ak, red[w]); av = fmaxf(av, red[8 + w]); }
                const float ksc = ak > 0.f ? ak / 240.0f : 1.0f, vsc = av > 0.f ? av / 240.0f : 1.0f;
                const uint32_t kb = fp8_e4m3_encode_ref(kx, 1.0f / ksc), vb = fp8_e4m3_encode_ref(vx, 1.0f / vsc);
                (pg + kv_tile_offset(kv, 0, kvh))[(size_t)rn * kD + d] = (unsigned char)kb;
                (pg + kv_tile_offset(kv, 1, kvh))[(size_t)rn * kD + d] = (unsigned char)vb;
                const uint32_t off = swz_row256(rn, d >> 4) + (d & 15);
                asm volatile("st.shared.b8 [%0], %1;\n" ::"r"(sk + off), "r"(kb) : "memory");
                asm volatile("st.shared.b8 [%0], %1;\n" ::"r"(sv + off), "r"(vb) : "memory");
                if (tid == 0) {  // every KV head's CTA writes the same two numbers
                    kv_page_scales(kv, pg, 0)[rn] = ksc;
                    kv_page_scales(kv, pg, 1)[rn] = vsc;
                    s_scales[rn] = ksc;
                    s_scales[kPage + rn] = vsc;
                }
            }
            __syncthreads();
        }
        const int p0 = gpage * kPage + pw * 16;  // first row of this slice's 16
        if (p0 >= L) continue;                   // the whole slice skips together

        // partial S = Q K^T over this warp's dims; hi and lo terms in separate accumulators
        float sh[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float sl[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        if (!kFp8) {
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
        } else {
            // one ldmatrix brings rows {0..7, 8..15} x two groups of 16 dims; each register is a whole B fragment
            // once its bytes are widened (dims 4t, 4t+1 | 4t+2, 4t+3: the order q was stored in)
#pragma unroll
            for (int k8 = 0; k8 < kKSteps; k8 += 2) {
                const int kk = hs * kKSteps + k8;
                uint32_t r[4];  // r[0]: rows 0..7, group kk; r[1]: rows 0..7, group kk+1; r[2], r[3]: rows 8..15
                ldmatrix_x4(r[0], r[1], r[2], r[3], sk + swz_row256(pw * 16 + (lm >> 1) * 8 + lr, kk + (lm & 1)));
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const uint32_t b00 = fp8x2_to_f16x2_scaled(r[u], 0x1404), b01 = fp8x2_to_f16x2_scaled(r[u], 0x3424);
                    const uint32_t b10 = fp8x2_to_f16x2_scaled(r[2 + u], 0x1404), b11 = fp8x2_to_f16x2_scaled(r[2 + u], 0x3424);
                    mma_f16(sh[0], qh[k8 + u][0], qh[k8 + u][1], qh[k8 + u][2], qh[k8 + u][3], b00, b01);
                    mma_f16(sh[1], qh[k8 + u][0], qh[k8 + u][1], qh[k8 + u][2], qh[k8 + u][3], b10, b11);
                    mma_f16(sl[0], ql[k8 + u][0], ql[k8 + u][1], ql[k8 + u][2], ql[k8 + u][3], b00, b01);
                    mma_f16(sl[1], ql[k8 + u][0], ql[k8 + u][1], ql[k8 + u][2], ql[k8 + u][3], b10, b11);
                }
            }
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
        float2 vsc[2] = {make_float2(1.f, 1.f), make_float2(1.f, 1.f)};  // V row scales of this thread's 4 rows
        if (kFp8) {
            // row of s[nt][e]: pw*16 + nt*8 + 2*(lane&3) + (e&1)
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const int rr = pw * 16 + nt * 8 + 2 * (lane & 3);
                const float2 ks = *reinterpret_cast<const float2 *>(s_scales + rr);
                vsc[nt] = *reinterpret_cast<const float2 *>(s_scales + kPage + rr);
                s[nt][0] *= ks.x * kFp8HalfScale; s[nt][1] *= ks.y * kFp8HalfScale;
                s[nt][2] *= ks.x * kFp8HalfScale; s[nt][3] *= ks.y * kFp8HalfScale;
            }
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
        // the running maximum lags by up to 2^8 (2^4 with fp16 weights, whose range is smaller)
        const float lag = kFp8 ? 4.f : 8.f;
        const bool grow = (mx[0] > m_ref[0] + lag) || (mx[1] > m_ref[1] + lag);
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
        if (kFused && f.h2o.w != nullptr && hs == 0) {
            // H2O: the un-normalised weights of this slice's 16 rows x 16 heads, and the maximum they refer to; the mass
            // pass turns them into softmax weights once the step's final (max, sum) of every head is known
            const int g = lane >> 2, tq = lane & 3;
            const size_t rstride = (size_t)kv.Hkv * 16;
            float *wr = f.h2o.w + (((size_t)tok * f.h2o.rows_pad + p0) * kv.Hkv + kvh) * 16 + g;
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                float *w0 = wr + (size_t)(nt * 8 + 2 * tq) * rstride;
                w0[0] = p[nt][0]; w0[rstride] = p[nt][1];
                w0[8] = p[nt][2]; w0[rstride + 8] = p[nt][3];
            }
            if (tq == 0) {
                float *mr = f.h2o.mref + ((((size_t)tok * f.h2o.tiles + gpage) * kv.Hkv + kvh) * 4 + pw) * 16;
                mr[g] = m_ref[0];
                mr[g + 8] = m_ref[1];
            }
        }
        if (!kFp8) {
            // weights as two bf16 terms; O += P V on this warp's output dims
            uint32_t ph[4], pl[4];
            split_pack_bf16(p[0][0], p[0][1], ph[0], pl[0]);
            split_pack_bf16(p[0][2], p[0][3], ph[1], pl[1]);
            split_pack_bf16(p[1][0], p[1][1], ph[2], pl[2]);
            split_pack_bf16(p[1][2], p[1][3], ph[3], pl[3]);
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
        } else {
            // weight x V row scale as one fp16 term.  A transposed ldmatrix treats the V bytes as 16-bit units, so a
            // thread gets rows (2t, 2t+1) x dims (2g, 2g+1): bytes 0 and 2 are the B fragment of the group's even
            // dims, bytes 1 and 3 of its odd dims.  Accumulator 2c holds the even dims of 16-dim group c, 2c+1 the odd.
            uint32_t ph[4];
            ph[0] = pack_f16(p[0][0] * vsc[0].x, p[0][1] * vsc[0].y);
            ph[1] = pack_f16(p[0][2] * vsc[0].x, p[0][3] * vsc[0].y);
            ph[2] = pack_f16(p[1][0] * vsc[1].x, p[1][1] * vsc[1].y);
            ph[3] = pack_f16(p[1][2] * vsc[1].x, p[1][3] * vsc[1].y);
#pragma unroll
            for (int n8 = 0; n8 < kNChunks; n8 += 2) {
                const int cc = hs * kNChunks + n8;
                uint32_t r[4];  // r[0]: rows 0..7, group cc; r[1]: rows 8..15, group cc; r[2], r[3]: group cc+1
                ldmatrix_x4_trans(r[0], r[1], r[2], r[3], sv + swz_row256(pw * 16 + (lm & 1) * 8 + lr, cc + (lm >> 1)));
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    mma_f16(o[2 * (n8 + u)], ph[0], ph[1], ph[2], ph[3], fp8x2_to_f16x2_scaled(r[2 * u], 0x2404),
                            fp8x2_to_f16x2_scaled(r[2 * u + 1], 0x2404));
                    mma_f16(o[2 * (n8 + u) + 1], ph[0], ph[1], ph[2], ph[3], fp8x2_to_f16x2_scaled(r[2 * u], 0x3414),
                            fp8x2_to_f16x2_scaled(r[2 * u + 1], 0x3414));
                }
            }
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
        if (!kFp8) {
#pragma unroll
            for (int i = 0; i < 2 * kNChunks; i++) {
                *reinterpret_cast<float2 *>(wo + g * kD + i * 8 + 2 * tq) = make_float2(o[i][0], o[i][1]);
                *reinterpret_cast<float2 *>(wo + (g + 8) * kD + i * 8 + 2 * tq) = make_float2(o[i][2], o[i][3]);
            }
        } else {
            // accumulator 2c: dims 16c + 4tq + {0, 2}, accumulator 2c+1: dims 16c + 4tq + {1, 3}; the 2^8 the
            // widened V bytes lacked comes back here
#pragma unroll
            for (int c = 0; c < kNChunks; c++) {
                *reinterpret_cast<float4 *>(wo + g * kD + c * 16 + 4 * tq) =
                    make_float4(o[2 * c][0] * kFp8HalfScale, o[2 * c + 1][0] * kFp8HalfScale, o[2 * c][1] * kFp8HalfScale, o[2 * c + 1][1] * kFp8HalfScale);
                *reinterpret_cast<float4 *>(wo + (g + 8) * kD + c * 16 + 4 * tq) =
                    make_float4(o[2 * c][2] * kFp8HalfScale, o[2 * c + 1][2] * kFp8HalfScale, o[2 * c][3] * kFp8HalfScale, o[2 * c + 1][3] * kFp8HalfScale);
            }
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
            if (f.ml_out != nullptr && d == 0) {  // the softmax's (max, sum), for the H2O mass accounting
                f.ml_out[((size_t)tk * H + head) * 2 + 0] = M;
                f.ml_out[((size_t)tk * H + head) * 2 + 1] = lt;
            }
        } else if (f.tail == 2) {
            *reinterpret_cast<float4 *>(f.out + ((size_t)tk * H + head) * kD + d) = acc;
            if (d == 0) {
                f.ml_out[((size_t)tk * H + head) * 2 + 0] = M;
                f.ml_out[((size_t)tk * H + head) * 2 + 1] = lt;
            }
        } else {
            const size_t row = ((((size_t)(f.step & (f.x.ring - 1)) * f.x.nranks + f.x.me) * f.x.cap + tk) * H + head) * (kD + 2);
            for (int r = 0; r < f.x.nranks; r++) {
                float *dst = f.x.peer[r] + row;
                *reinterpret_cast<float2 *>(dst + d) = make_float2(acc.x, acc.y);
                *reinterpret_cast<float2 *>(dst + d + 2) = make_float2(acc.z, acc.w);
                if (d == 0) *reinterpret_cast<float2 *>(dst + kD) = make_float2(M, lt);
            }
        }
    };
    const bool direct = kFused && nsplits == 1;  // this CTA is the only split: finish the rows here
    // Nothing written from here on is shared with the launch this one may overlap: partials, counters and outputs
    // are per layer, and the exchange tails write the slot set of their own step (a ring deep enough that a set is
    // only reused after every rank has read it, see fm_exchange_attach).  The wait the overlap owes is at the end
    // of the CTA (attn_decode_kernel).
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
    if (!kFused || f.tail == 0) return;  // tail 0: the partials are all; a merge launch follows
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
        const int nr = f.x.nranks, par = f.step & (f.x.ring - 1);
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
                    st_release_sys(flags + (f.step & (f.x.ring - 1)) * f.x.nranks + f.x.me, f.step);
                }
            }
        }
    }
}

template <bool kFused, bool kFp8>
__global__ void __launch_bounds__(kDecThreads, 1)
attn_decode_kernel(KvView kv, RopeParams rope, TokSpec toks, int H, const float *__restrict__ q_proj_out,
                   const float *__restrict__ q_in, const uint16_t *__restrict__ qnw, float eps,
                   float *__restrict__ part_o, float *__restrict__ part_ml, int nsplits, DecodeFused f) {
    attn_decode_body<kFused, kFp8>(kv, rope, toks, H, q_proj_out, q_in, qnw, eps, part_o, part_ml, nsplits, f);
    // A launch started as a programmatic dependent of the previous one (another layer's step) streamed its pages
    // while that launch drained.  A dependent of a grid that uses launch_dependents has to execute
    // griddepcontrol.wait; every CTA does so here, when its own work is done, so the launches of one
    // fm_attn_decode_layers call complete in order and whatever follows the last layer in the stream follows all
    // of them.  No effect for an ordinary launch.
    if (kFused) dep_wait();
}

// Raises the kernel's dynamic shared-memory limit once per device.
template <bool kFused, bool kFp8>
static bool configure_decode() {
    static unsigned long long configured = 0;  // one bit per device
    if (!first_use_on_device(&configured)) return true;
    return cudaFuncSetAttribute(attn_decode_kernel<kFused, kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecRing<kFp8>::kSmem) == cudaSuccess;
}

int launch_attn_decode(const KvView &kv, const RopeParams &rope, const TokSpec &toks, int H,
                       const float *q_proj_out, const float *q, const uint16_t *q_norm_w, float eps,
                       float *part_o, float *part_ml, int nsplits, cudaStream_t st) {
    if (!(kv.fp8 ? configure_decode<false, true>() : configure_decode<false, false>())) return -1;
    dim3 grid(nsplits, kv.Hkv, toks.n);
    DecodeFused f = {};
    if (kv.fp8)
        attn_decode_kernel<false, true><<<grid, kDecThreads, DecRing<true>::kSmem, st>>>(kv, rope, toks, H, q_proj_out, q, q_norm_w, eps, part_o,
                                                                                           part_ml, nsplits, f);
    else
        attn_decode_kernel<false, false><<<grid, kDecThreads, DecRing<false>::kSmem, st>>>(kv, rope, toks, H, q_proj_out, q, q_norm_w, eps, part_o,
                                                                                             part_ml, nsplits, f);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

// The whole decode step in one launch (see DecodeFused).
int launch_attn_decode_fused(const KvView &kv, const RopeParams &rope, const TokSpec &toks, int H,
                             const float *q_proj_out, const float *q, const uint16_t *q_norm_w, float eps,
                             float *part_o, float *part_ml, int nsplits, const float *k_new, const float *v_new,
                             const uint16_t *k_norm_w, int tail, const float *gate, float *out, float *ml_out,
                             const XchgView *x, uint32_t step, const DecodeScratch &scr, int *err, bool overlap_prev,
                             cudaStream_t st, const H2oStep *h2o) {
    if (!(kv.fp8 ? configure_decode<true, true>() : configure_decode<true, false>())) return -1;
    if (tail != 0 && nsplits > kDecMaxLastCtaSplits && (toks.n > scr.group_tokens || nsplits > kDecGroup * kDecMaxGroups)) return -1;
    if (kv.fp8 && k_new != nullptr && kv.Hkv > 8) return -1;
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
    if (h2o) f.h2o = *h2o;
    // overlap_prev: the caller vouches that this launch reads nothing the previous kernel in the
    // stream writes except through the scratch the kernel guards itself (another layer's step).
    // Its CTAs then take SMs as the previous grid's CTAs retire instead of after the grid drains.
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid; lc.blockDim = dim3(kDecThreads); lc.stream = st;
    lc.dynamicSmemBytes = kv.fp8 ? DecRing<true>::kSmem : DecRing<false>::kSmem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = overlap_prev ? 1 : 0;
    const cudaError_t e = kv.fp8 ? cudaLaunchKernelEx(&lc, attn_decode_kernel<true, true>, kv, rope, toks, H, q_proj_out, q, q_norm_w, eps, part_o,
                                                      part_ml, nsplits, f)
                                 : cudaLaunchKernelEx(&lc, attn_decode_kernel<true, false>, kv, rope, toks, H, q_proj_out, q, q_norm_w, eps, part_o,
                                                      part_ml, nsplits, f);
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

// The same merge for many parts (a sequence split over the whole machine at small batch): one CTA per (head,
// token), 16 warps.  Warp w owns parts w, w+16, ...: a lane holds 8 dims, so a part's row is one coalesced 1 KB
// read per warp, and the rows of up to 8 parts per warp are requested together with the (max, sum) pairs, before
// anything is computed -- the whole merge costs about one trip to L2.  Every warp reads all the pairs (lane j
// holds parts j, j+32, ...) and forms the merged maximum; the sixteen partial sums meet in shared memory.
// Launched as a programmatic dependent of the kernel that writes the parts: its CTAs take SMs as that kernel's
// CTAs retire, fetch the gate row (an input) and wait (griddepcontrol.wait) until the parts are complete.
// Parts of (token, head) are contiguous: part_o [tok][H][nparts][256], part_ml [tok][H][nparts][2].
constexpr int kMergeWarps = 16;
__global__ void __launch_bounds__(32 * kMergeWarps)
attn_merge_wide_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml, int nparts, int H,
                       const float *__restrict__ q_proj_out, const float *__restrict__ gate, float *__restrict__ out,
                       float *__restrict__ ml_out, float *__restrict__ ml_final) {
    __shared__ float4 s_acc[kMergeWarps][64];
    __shared__ float s_w[256];
    const int head = blockIdx.x, tok = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row0 = ((size_t)tok * H + head) * nparts;
    const float2 *ml = reinterpret_cast<const float2 *>(part_ml) + row0;
    const float4 *po = reinterpret_cast<const float4 *>(part_o + row0 * kD) + lane * 2;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ml_out == nullptr && threadIdx.x < 64) {
        const float *gsrc = q_proj_out ? q_proj_out + ((size_t)tok * H + head) * 2 * kD + kD : gate + ((size_t)tok * H + head) * kD;
        g = __ldg(reinterpret_cast<const float4 *>(gsrc) + threadIdx.x);
    }
    dep_wait();
    float2 mlv[8];
    float4 pa[8], pb[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int j = lane + 32 * i;
        mlv[i] = j < nparts ? __ldcg(ml + j) : make_float2(kNegBig, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int j = warp + kMergeWarps * i;
        pa[i] = pb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < nparts) {
            pa[i] = __ldcg(po + (size_t)j * (kD / 4));
            pb[i] = __ldcg(po + (size_t)j * (kD / 4) + 1);
        }
    }
    float M = kNegBig;
#pragma unroll
    for (int i = 0; i < 8; i++) M = fmaxf(M, mlv[i].x);
    M = warp_max(M);
    float lt = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float w = fast_exp2(mlv[i].x - M);
        lt += w * mlv[i].y;
        if (warp == 0) s_w[lane + 32 * i] = w;
    }
    lt = warp_sum(lt);
    __syncthreads();
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int j = warp + kMergeWarps * i;
        const float w = j < nparts ? s_w[j] : 0.f;
        a0.x += w * pa[i].x; a0.y += w * pa[i].y; a0.z += w * pa[i].z; a0.w += w * pa[i].w;
        a1.x += w * pb[i].x; a1.y += w * pb[i].y; a1.z += w * pb[i].z; a1.w += w * pb[i].w;
    }
    for (int j = warp + kMergeWarps * 8; j < nparts; j += kMergeWarps) {  // more than 128 parts
        const float w = s_w[j];
        const float4 p0 = __ldcg(po + (size_t)j * (kD / 4)), p1 = __ldcg(po + (size_t)j * (kD / 4) + 1);
        a0.x += w * p0.x; a0.y += w * p0.y; a0.z += w * p0.z; a0.w += w * p0.w;
        a1.x += w * p1.x; a1.y += w * p1.y; a1.z += w * p1.z; a1.w += w * p1.w;
    }
    s_acc[warp][lane * 2] = a0;
    s_acc[warp][lane * 2 + 1] = a1;
    __syncthreads();
    if (threadIdx.x >= 64) return;
    const int d = threadIdx.x * 4;
    float4 acc = s_acc[0][threadIdx.x];
#pragma unroll
    for (int w = 1; w < kMergeWarps; w++) {
        const float4 v = s_acc[w][threadIdx.x];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float *dst = out + ((size_t)tok * H + head) * kD + d;
    if (ml_out != nullptr) {
        *reinterpret_cast<float4 *>(dst) = acc;
        if (threadIdx.x == 0) {
            ml_out[((size_t)tok * H + head) * 2 + 0] = M;
            ml_out[((size_t)tok * H + head) * 2 + 1] = lt;
        }
        return;
    }
    const float inv = lt > 0.f ? 1.0f / lt : 0.f;
    *reinterpret_cast<float4 *>(dst) = make_float4(acc.x * inv * fast_sigmoid(g.x), acc.y * inv * fast_sigmoid(g.y),
                                                   acc.z * inv * fast_sigmoid(g.z), acc.w * inv * fast_sigmoid(g.w));
    if (ml_final != nullptr && threadIdx.x == 0) {
        ml_final[((size_t)tok * H + head) * 2 + 0] = M;
        ml_final[((size_t)tok * H + head) * 2 + 1] = lt;
    }
}

int launch_attn_merge_wide(const float *part_o, const float *part_ml, int nparts, int ntok, int H, const float *q_proj_out,
                           const float *gate, float *out, float *ml_out, cudaStream_t st, float *ml_final) {
    if (ntok <= 0 || nparts < 1 || nparts > 256) return -1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(H, ntok); lc.blockDim = dim3(32 * kMergeWarps); lc.dynamicSmemBytes = 0; lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, attn_merge_wide_kernel, part_o, part_ml, nparts, H, q_proj_out, gate, out, ml_out, ml_final) == cudaSuccess ? 1 : -1;
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
    const int par = step & (x.ring - 1);
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
    const int par = step & (x.ring - 1);
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
