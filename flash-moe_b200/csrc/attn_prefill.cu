// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Math of the Metal kernels prefill_q_rope_norm_bf16 / prefill_causal_attn
// (metal_infer/shaders.metal:2228-2397; dispatch metal_infer/batched_prefill.h:574-668): q is
// normalised and rotated, token t of the run attends to cache rows [0, row0 + t] (the run's own rows
// are appended by the preparation launch), the result is multiplied by sigmoid(gate).
//
// Organisation
//   attn_prefill_prep_kernel   one launch: q -> RMS-norm, partial RoPE, * (1/sqrt(D)) * log2(e) -> fp16 hi | lo
//                         workspace; the run's k, v rows -> bf16 pages (the append) and fp16 workspace; cached
//                         prefix rows -> fp16 workspace
//   attn_prefill_kernel   one CTA per (128 query tokens, query head):
//       warp 4 (one lane)  TMA producer: q_hi tile once, then K / V tiles of 64 rows into 2-stage rings
//       warp 5 (one lane)  issues tcgen05.mma: S = q_hi K^T + q_lo K^T (M128 N64 K256 each; q_hi from
//                          shared memory, q_lo from tensor memory) into the TMEM score buffer,
//                          O += p_hi V + p_lo V (M128 N256 K64 each, P from tensor memory)
//       warps 0-3          one query row per thread: q_lo row -> TMEM once; per tile tcgen05.ld of the
//                          scores, causal mask, online softmax in the exp2 domain (row-local, no
//                          shuffles), P as fp16 pairs back into TMEM for the next MMA; the accumulator
//                          is rescaled in TMEM only when some row's maximum grew by more than 2^8;
//                          epilogue: O / l * sigmoid(gate) -> fp32 output
//   Precision: q after RoPE and the softmax weights are not representable in 16 bits; a single fp16
//   rounding of either (2^-12) measured 4e-3 against the fp32 reference on short contexts, over the
//   2e-3 bound.  Both therefore enter the MMAs as two fp16 terms (hi + lo) laid side by side along
//   the contraction dimension, the K / V tile being read twice; that doubles the tensor work and is
//   the price of the bound.  K and V are exact (bf16 -> fp16 is lossless inside fp16's range; values
//   beyond +-65504 are clamped).
//   TMEM: 64 columns of scores + 64 of P + 256 of output + 128 of q_lo = 512.
//   Every mbarrier wait is bounded; on expiry the CTA records an error code and winds down.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include "fm_device.cuh"
#include "fm_internal.h"
#include "fm_tc.cuh"

namespace fm {

constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 64;   // kv rows per tile
constexpr int kHD = 256;  // head dim
constexpr int kSlabQ = kBM * 128;  // bytes of one 64-column slab of the q_hi tile
constexpr int kSlabKV = kBN * 128;
constexpr int kQBytesPf = 4 * kSlabQ;    // 64 KB: q_hi
constexpr int kKVBytesPf = 4 * kSlabKV;  // 32 KB per K or V tile
constexpr int kPfSmem = kQBytesPf + 4 * kKVBytesPf + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int kPfThreads = 352;  // 8 softmax warps (two per 32 rows), K producer, MMA issuer, V producer
constexpr int kWarpK = 8, kWarpMma = 9, kWarpV = 10;
// TMEM columns (32-bit each, 128 lanes = the 128 query rows)
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;      // 2 x 64: scores of tile j in buffer j & 1; the tile's softmax weights replace them in
                                   // place (fp16 pairs, the first 32 columns of the buffer)
constexpr uint32_t kColO = 128;    // 256: output accumulator
constexpr uint32_t kColQlo = 384;  // 128: q_lo as fp16 pairs

enum PfBar { BAR_Q = 0, BAR_QLO = 1, BAR_KFULL = 2, BAR_KEMPTY = 4, BAR_VFULL = 6, BAR_VEMPTY = 8, BAR_SFULL = 10,
             BAR_PFULL = 12, BAR_PVDONE = 14, BAR_COUNT = 16 };  // two of each from BAR_KFULL on (ring stage / score buffer)

// Instruction descriptor for kind::f16: fp16 A and B, fp32 accumulate.
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, bool b_mn_major) {
    return (1u << 4)                            // D format fp32
           | (0u << 7) | (0u << 10)             // A, B format fp16
           | (0u << 15)                         // A K-major
           | ((b_mn_major ? 1u : 0u) << 16)     // B major
           | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- operand preparation, one launch, three kinds of CTA (256 threads each) ------------------------
//   blocks [0, n)                q of token t: RMS-norm, partial RoPE, * (1/sqrt(D)) * log2(e) -> fp16
//                                [n][H][hi(256) | lo(256)]; a warp walks heads, a lane holds 8 dims
//   blocks [n, n + n*Hkv)        k, v of token t, KV head h: k RMS-norm + RoPE, then the row goes to its bf16
//                                page (the store proper) and, converted bf16 -> fp16, to the workspace the
//                                attention kernel reads (math of metal_infer/layer_forward.h:574-629)
//   blocks [n + n*Hkv, + row0 - prefix0)   one cached row of the prefix that the workspace does not hold yet:
//                                bf16 page -> fp16 workspace
// K and V are exact in fp16 (bf16 -> fp16 is lossless inside fp16's range; values beyond +-65504 are clamped).
struct PrepParams {
    int n, row0, start_pos, seq, H;
    int prefix0;  // cached rows [prefix0, row0) still have to be converted into the workspace
    const float *q_proj_out, *q_in, *k, *v;
    const uint16_t *qnw, *knw;
    float eps;
    __half *q16, *k16, *v16;
};

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ float clamp_f16(float x) { return fminf(fmaxf(x, -65504.f), 65504.f); }

__global__ void __launch_bounds__(256)
attn_prefill_prep_kernel(KvView kv, RopeParams rope, PrepParams p) {
    __shared__ float s_cos[64], s_sin[64];
    __shared__ float s_x[8][kHD];
    __shared__ float s_red[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int half = rope.rotary_dim / 2;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");  // the attention launch may begin its set-up
    int b = blockIdx.x;
    if (b >= p.n + p.n * kv.Hkv) {
        // ---- prefix row: pages -> fp16 workspace ----
        const int row = p.prefix0 + b - p.n - p.n * kv.Hkv;
        const int page = kv.page_table[(size_t)p.seq * kv.max_slots + row / kv.page_size];
        const int r = row % kv.page_size;
        const unsigned char *pgb = kv_page(kv, page);
        for (int e = tid; e < kv.Hkv * kHD; e += 256) {
            const int kvh = e / kHD, d = e - kvh * kHD;
            const __nv_bfloat16 *kp = reinterpret_cast<const __nv_bfloat16 *>(pgb + kv_tile_offset(kv, 0, kvh)) + (size_t)r * kHD + d;
            const __nv_bfloat16 *vp = reinterpret_cast<const __nv_bfloat16 *>(pgb + kv_tile_offset(kv, 1, kvh)) + (size_t)r * kHD + d;
            p.k16[(size_t)row * kv.Hkv * kHD + e] = __float2half_rn(clamp_f16(__bfloat162float(*kp)));
            p.v16[(size_t)row * kv.Hkv * kHD + e] = __float2half_rn(clamp_f16(__bfloat162float(*vp)));
        }
        return;
    }
    const bool is_q = b < p.n;
    const int t = is_q ? b : (b - p.n) / kv.Hkv;
    if (tid < half) sincos_reduced(((float)(p.start_pos + t) / rope.pos_div) * rope.inv_freq[tid], s_sin[tid], s_cos[tid]);
    __syncthreads();
    if (!is_q) {
        // ---- append: thread d owns dim d of (token t, KV head kvh) ----
        const int kvh = (b - p.n) % kv.Hkv, d = tid, row = p.row0 + t;
        const size_t src = ((size_t)t * kv.Hkv + kvh) * kHD + d;
        float x = p.k[src];
        float *sx = s_x[0];
        if (p.knw != nullptr) {
            const float ss = warp_sum(x * x);
            if (lane == 0) s_red[warp] = ss;
            __syncthreads();
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) tot += s_red[w];
            x = x * (1.0f / sqrtf(tot / kHD + p.eps)) * bf16_bits_to_float(p.knw[d]);
        }
        sx[d] = x;
        __syncthreads();
        if (d < rope.rotary_dim) {
            const int i = d < half ? d : d - half;
            x = d < half ? x * s_cos[i] - sx[d + half] * s_sin[i] : sx[d - half] * s_sin[i] + x * s_cos[i];
        }
        const __nv_bfloat16 kb = __float2bfloat16_rn(x), vb = __float2bfloat16_rn(p.v[src]);
        const int gpage = row / kv.page_size, r = row - gpage * kv.page_size;
        if (gpage % kv.shard_count == kv.shard_rank) {  // on a sequence-sharded store the page's owner keeps the row
            const int page = kv.page_table[(size_t)p.seq * kv.max_slots + gpage / kv.shard_count];
            unsigned char *pg = kv_page(kv, page);
            reinterpret_cast<__nv_bfloat16 *>(pg + kv_tile_offset(kv, 0, kvh))[(size_t)r * kHD + d] = kb;
            reinterpret_cast<__nv_bfloat16 *>(pg + kv_tile_offset(kv, 1, kvh))[(size_t)r * kHD + d] = vb;
        }
        p.k16[((size_t)row * kv.Hkv + kvh) * kHD + d] = __float2half_rn(clamp_f16(__bfloat162float(kb)));
        p.v16[((size_t)row * kv.Hkv + kvh) * kHD + d] = __float2half_rn(clamp_f16(__bfloat162float(vb)));
        return;
    }
    // ---- q of token t ----
    const float qscale = rope.logit_scale * kLog2e;
    float w8[8];
#pragma unroll
    for (int j = 0; j < 8; j++) w8[j] = p.qnw ? bf16_bits_to_float(p.qnw[lane * 8 + j]) : 1.0f;
    for (int h = warp; h < p.H; h += 8) {
        const float *src = p.q_proj_out ? p.q_proj_out + ((size_t)t * p.H + h) * 2 * kHD : p.q_in + ((size_t)t * p.H + h) * kHD;
        const float4 a = __ldg(reinterpret_cast<const float4 *>(src + lane * 8));
        const float4 bq = __ldg(reinterpret_cast<const float4 *>(src + lane * 8 + 4));
        float x[8] = {a.x, a.y, a.z, a.w, bq.x, bq.y, bq.z, bq.w};
        if (p.qnw != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) ss += x[j] * x[j];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / kHD + p.eps);
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = x[j] * inv * w8[j];
        }
        float *sx = s_x[warp];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; j++) sx[lane * 8 + j] = x[j];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int d = lane * 8 + j;
            if (d < rope.rotary_dim) {
                const int i = d < half ? d : d - half;
                x[j] = d < half ? x[j] * s_cos[i] - sx[d + half] * s_sin[i] : sx[d - half] * s_sin[i] + x[j] * s_cos[i];
            }
        }
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float y0 = x[2 * j] * qscale, y1 = x[2 * j + 1] * qscale;
            const __half2 hh = __floats2half2_rn(y0, y1);
            const float2 hf = __half22float2(hh);
            const __half2 ll = __floats2half2_rn(y0 - hf.x, y1 - hf.y);
            hi[j] = *reinterpret_cast<const uint32_t *>(&hh);
            lo[j] = *reinterpret_cast<const uint32_t *>(&ll);
        }
        __half *dst = p.q16 + ((size_t)t * p.H + h) * 2 * kHD + lane * 8;
        *reinterpret_cast<uint4 *>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);        // q_hi
        *reinterpret_cast<uint4 *>(dst + kHD) = make_uint4(lo[0], lo[1], lo[2], lo[3]);  // q_lo
    }
}

// ---- the attention kernel ----------------------------------------------------------------------

struct PfParams {
    int n;         // tokens in the run
    int row0;      // cache rows before the run
    int H, Hkv;
    const __half *q16;        // [n][H][hi(256) | lo(256)]
    const float *q_proj_out;  // gate source: interleaved ...
    const float *gate;        // ... or separate
    float *out;
    int *err;      // device word: 0 ok, else (code << 16 | blockIdx info)
    int two_term_rows;  // query tiles that see fewer cache rows than this keep two fp16 terms for the softmax weights
};

__global__ void __launch_bounds__(kPfThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, PfParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ float s_mx[2][2][kBM];  // row maxima of the two column halves, double-buffered by tile parity
    __shared__ float s_l[2][kBM];      // row sums of the two halves (epilogue)
    // 1024-byte aligned tiles (128-byte swizzle atoms are 1024 bytes)
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t sQ = base;                  // q_hi, 4 slabs
    const uint32_t sK = sQ + kQBytesPf;        // 2 stages
    const uint32_t sV = sK + 2 * kKVBytesPf;   // 2 stages
    const uint32_t sBar = sV + 2 * kKVBytesPf; // BAR_COUNT mbarriers, 8 bytes each
    auto bar = [&](int i) { return sBar + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // heavy tiles first: CTAs are handed out in linear order (x fastest), so x walks the heads and
    // y = 0 is the last (longest) query tile of every head
    const int nqt = gridDim.y;
    const int qt = nqt - 1 - blockIdx.y;
    const int head = blockIdx.x;
    const int kvh = head / (p.H / p.Hkv);
    const int t0 = qt * kBM;
    const int L = p.row0 + p.n;
    const int last_row = min(p.row0 + t0 + kBM - 1, L - 1);  // last cache row any query of this tile sees
    const int ntiles = last_row / kBN + 1;
    // Short query tiles keep a second fp16 term for the softmax weights: with few keys a row's result is a mix of
    // a handful of V rows, and the 2^-11 rounding of a single term shows (2.3e-3 of the result measured, bound
    // 2e-3); over many keys the roundings average out and one term is enough.
    const bool two_p = last_row < p.two_term_rows;

    if (tid == 0) {
        s_abort = 0;
        mbar_init(bar(BAR_Q), 1);
        mbar_init(bar(BAR_QLO), 256);
        for (int s = 0; s < 2; s++) {
            mbar_init(bar(BAR_KFULL + s), 1);
            mbar_init(bar(BAR_KEMPTY + s), 1);
            mbar_init(bar(BAR_VFULL + s), 1);
            mbar_init(bar(BAR_VEMPTY + s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(bar(BAR_SFULL + b), 1);
            mbar_init(bar(BAR_PFULL + b), 256);
            mbar_init(bar(BAR_PVDONE + b), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == kWarpMma) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    volatile int *abortp = &s_abort;
    // Launched as a programmatic dependent of the preparation kernel: everything above overlapped its
    // tail; its outputs (q16, k16, v16) are read from here on.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    if (warp == kWarpK) {
        // ================= TMA producer: q_hi once, then the K tiles =================
        // (K and V have a producer each: the scores run two tiles ahead of the weighted sums, so a K tile is
        // wanted long before the V stage of the same parity is free)
        if (lane == 0) {
            mbar_expect_tx(bar(BAR_Q), kQBytesPf);
            for (int s = 0; s < 4; s++) tma_load_2d(sQ + s * kSlabQ, &map_q, head * 2 * kHD + s * 64, t0, bar(BAR_Q));
            for (int j = 0; j < ntiles; j++) {
                const int b = j & 1, u = j >> 1;
                if (u > 0 && !mbar_wait(bar(BAR_KEMPTY + b), (u - 1) & 1, abortp)) break;
                mbar_expect_tx(bar(BAR_KFULL + b), kKVBytesPf);
                for (int s = 0; s < 4; s++)
                    tma_load_2d(sK + b * kKVBytesPf + s * kSlabKV, &map_k, kvh * kHD + s * 64, j * kBN, bar(BAR_KFULL + b));
            }
        }
    } else if (warp == kWarpV) {
        // ================= TMA producer: the V tiles =================
        if (lane == 0) {
            for (int j = 0; j < ntiles; j++) {
                const int b = j & 1, u = j >> 1;
                if (u > 0 && !mbar_wait(bar(BAR_VEMPTY + b), (u - 1) & 1, abortp)) break;
                mbar_expect_tx(bar(BAR_VFULL + b), kKVBytesPf);
                for (int s = 0; s < 4; s++)
                    tma_load_2d(sV + b * kKVBytesPf + s * kSlabKV, &map_v, kvh * kHD + s * 64, j * kBN, bar(BAR_VFULL + b));
            }
        }
    } else if (warp == kWarpMma) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_f16(kBM, kBN, false);   // S = Q K^T, both K-major
            constexpr uint32_t idesc_o = idesc_f16(kBM, kHD, true);    // O = P V, V is MN-major
            // descriptors differ only in their start-address field (16-byte units): build once, add offsets
            const uint64_t dq0 = smem_desc(sQ, 16, 1024);
            const uint64_t dk0 = smem_desc(sK, 16, 1024);
            const uint64_t dv0 = smem_desc(sV, kSlabKV, 1024);
            auto issue_s = [&](int j) {  // scores of tile j into buffer j & 1, from K stage j & 1
                const uint64_t dk = dk0 + (uint64_t)(((j & 1) * kKVBytesPf) >> 4);
                const uint32_t d_s = tmem + kColS + (uint32_t)(j & 1) * kBN;
#pragma unroll
                for (int ks = 0; ks < kHD / 16; ks++) {  // q_hi from shared memory
                    const uint32_t off_a = (ks >> 2) * kSlabQ + (ks & 3) * 32, off_b = (ks >> 2) * kSlabKV + (ks & 3) * 32;
                    tc_mma_f16(d_s, dq0 + (off_a >> 4), dk + (off_b >> 4), idesc_s, ks > 0);
                }
#pragma unroll
                for (int ks = 0; ks < kHD / 16; ks++) {  // q_lo from tensor memory, same K tile
                    const uint32_t off_b = (ks >> 2) * kSlabKV + (ks & 3) * 32;
                    tc_mma_f16_ta(d_s, tmem + kColQlo + ks * 8, dk + (off_b >> 4), idesc_s, 1);
                }
                tc_commit(bar(BAR_SFULL + (j & 1)));
                tc_commit(bar(BAR_KEMPTY + (j & 1)));
            };
            // The scores run two tiles ahead of the weighted sums: while the softmax threads work on tile j the
            // tensor pipe already computes the scores of tile j + 1 in the other buffer.  The pipe executes in
            // issue order, so the scores of tile j + 2 land in buffer j & 1 only after P_j V_j has read the
            // weights that replaced tile j's scores there.
            bool ok = mbar_wait(bar(BAR_Q), 0, abortp) && mbar_wait(bar(BAR_QLO), 0, abortp) && mbar_wait(bar(BAR_KFULL + 0), 0, abortp);
            if (ok) {
                tc_fence_after();
                issue_s(0);
                if (ntiles > 1) {
                    ok = mbar_wait(bar(BAR_KFULL + 1), 0, abortp);
                    if (ok) {
                        tc_fence_after();
                        issue_s(1);
                    }
                }
            }
            for (int j = 0; ok && j < ntiles; j++) {
                const int b = j & 1, u = j >> 1;
                ok = mbar_wait(bar(BAR_PFULL + b), u & 1, abortp) && mbar_wait(bar(BAR_VFULL + b), u & 1, abortp);
                if (!ok) break;
                tc_fence_after();
                const uint64_t dv = dv0 + (uint64_t)((b * kKVBytesPf) >> 4);
                const int nks = two_p ? 2 * kBN / 16 : kBN / 16;  // the weights of 64 rows: 4 k-steps of 8 columns, per term
                for (int ks = 0; ks < nks; ks++)
                    tc_mma_f16_ta(tmem + kColO, tmem + kColS + (uint32_t)b * kBN + ks * 8, dv + (uint64_t)(((ks & 3) * 2048) >> 4), idesc_o, (j > 0 || ks > 0));
                tc_commit(bar(BAR_PVDONE + b));
                tc_commit(bar(BAR_VEMPTY + b));
                if (j + 2 < ntiles) {
                    ok = mbar_wait(bar(BAR_KFULL + b), ((j + 2) >> 1) & 1, abortp);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(j + 2);
                }
            }
        }
    } else {
        // ================= softmax / correction / epilogue =================
        // Two threads per query row: warps w and w + 4 reach the same 32 TMEM lanes (rows 32 (w & 3) ..), the first
        // takes the left half of every column range, the second the right half.  The pair meets on a 64-thread named
        // barrier for the row maximum; everything else is private to a thread.
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;        // row of the tile = TMEM lane
        const int my_last = p.row0 + t0 + r;      // last cache row this query may see
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pair_bar = 1 + quarter;         // named barrier of the two warps of this quarter
        // q_lo of this row -> tensor memory (two fp16 per column): this thread's 64 of the 128 columns
        {
            const int t = t0 + r;
            const uint4 *src = reinterpret_cast<const uint4 *>(p.q16 + ((size_t)t * p.H + head) * 2 * kHD + kHD) + half * 16;
            uint32_t w0[32], w1[32];
#pragma unroll
            for (int i = 0; i < 8; i++) {  // 16 loads of 16 bytes in flight
                const uint4 v = t < p.n ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
                const uint4 u = t < p.n ? __ldg(src + 8 + i) : make_uint4(0u, 0u, 0u, 0u);
                w0[4 * i] = v.x; w0[4 * i + 1] = v.y; w0[4 * i + 2] = v.z; w0[4 * i + 3] = v.w;
                w1[4 * i] = u.x; w1[4 * i + 1] = u.y; w1[4 * i + 2] = u.z; w1[4 * i + 3] = u.w;
            }
            tc_st32(tmem + lane_base + kColQlo + half * 64, w0);
            tc_st32(tmem + lane_base + kColQlo + half * 64 + 32, w1);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(BAR_QLO));
        }
        float m_ref = kNegBig, l_sum = 0.f;  // l_sum: this thread's columns only; the halves meet in the epilogue
        // ok turns false when a bounded wait gave up (warp-uniform).  A warp in that state touches no tensor memory
        // any more but keeps meeting its partner at the pair's named barrier, once per tile and once in the
        // epilogue, so that neither of the two can be left waiting there.
        bool ok = true;
        for (int j = 0; j < ntiles; j++) {
            const int b = j & 1;
            const uint32_t t_s = tmem + lane_base + kColS + (uint32_t)b * kBN;
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_SFULL + b), (j >> 1) & 1, abortp));
            uint32_t sr[32];
            float mx = kNegBig;
            if (ok) {  // warp-uniform: the tcgen05.ld / st below are warp-collective
                tc_fence_after();
                tc_ld32(t_s + half * 32, sr);
                tc_wait_ld();
                // causal mask and row maximum
                const int col0 = j * kBN + half * 32;
                if (col0 + 31 > p.row0 + t0) {  // the columns reach past the first query's limit
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (col0 + i > my_last) sr[i] = __float_as_uint(kNegBig);
                }
#pragma unroll
                for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(sr[i]));
            }
            s_mx[b][half][r] = mx;
            named_bar_sync(pair_bar, 64);
            mx = fmaxf(mx, s_mx[b][half ^ 1][r]);
            if (!ok) continue;
            const bool grow = mx > m_ref + 8.f;
            const bool any_grow = __any_sync(0xffffffffu, grow);  // the same in both warps of the pair: same values
            if (any_grow) {  // lazy rescale, warp-uniform because tcgen05.ld/st are warp-collective
                // every weighted sum issued so far must have landed before the accumulator is touched
                if (j > 0) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_PVDONE + ((j - 1) & 1)), ((j - 1) >> 1) & 1, abortp));
                    if (!ok) continue;
                    tc_fence_after();
                }
                const float m_new = grow ? mx : m_ref;
                const float corr = fast_exp2(m_ref - m_new);
                m_ref = m_new;
                l_sum *= corr;
                if (j > 0) {
#pragma unroll 1
                    for (int c = half * 128; c < half * 128 + 128; c += 32) {
                        uint32_t o[32];
                        tc_ld32(tmem + lane_base + kColO + c, o);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tc_st32(tmem + lane_base + kColO + c, o);
                    }
                }
            }
            // The weights replace the scores they came from, as fp16 pairs: the first term in columns 0..31 of the
            // buffer, the remainder term -- short query tiles only, see two_p -- in columns 32..63.  The row sum is
            // taken over what the tensor cores will see, so the final division normalises exactly what was
            // accumulated.
            uint32_t ph[16], pl[16];
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const float p0 = fast_exp2(__uint_as_float(sr[2 * i]) - m_ref);
                const float p1 = fast_exp2(__uint_as_float(sr[2 * i + 1]) - m_ref);
                const __half2 hh = __floats2half2_rn(p0, p1);
                const float2 hf = __half22float2(hh);
                ph[i] = *reinterpret_cast<const uint32_t *>(&hh);
                if (two_p) {
                    const __half2 ll = __floats2half2_rn(p0 - hf.x, p1 - hf.y);
                    pl[i] = *reinterpret_cast<const uint32_t *>(&ll);
                    l_sum += p0 + p1;
                } else {
                    l_sum += hf.x + hf.y;
                }
            }
            tc_st16(t_s + half * 16, ph);
            if (two_p) tc_st16(t_s + 32 + half * 16, pl);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(BAR_PFULL + b));
        }
        // epilogue: this thread's half of the row (128 dims).  The first two chunks of the gate row are requested
        // before the wait for the last P V.
        const int t_row = t0 + r;
        const bool live = t_row < p.n;
        const float4 *gp = reinterpret_cast<const float4 *>(
            p.q_proj_out ? p.q_proj_out + ((size_t)(live ? t_row : 0) * p.H + head) * 2 * kHD + kHD
                         : p.gate + ((size_t)(live ? t_row : 0) * p.H + head) * kHD) + half * 32;
        float4 gn[8], gn2[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { gn[i] = __ldg(gp + i); gn2[i] = __ldg(gp + 8 + i); }
        s_l[half][r] = l_sum;
        named_bar_sync(pair_bar, 64);
        l_sum += s_l[half ^ 1][r];
        if (ok && ntiles > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_PVDONE + ((ntiles - 1) & 1)), ((ntiles - 1) >> 1) & 1, abortp));
        if (ok) {
            // All MMAs have completed, so every K / V / q tile in shared memory is dead.  Each thread
            // gates its half row in registers -- the gate row comes straight from global memory through
            // read-only 16-byte loads, two chunks ahead -- and parks the result in shared memory at a
            // pitch of 1040 bytes (conflict-free 128-bit stores, rows still contiguous); every half row then
            // leaves through one 512-byte bulk asynchronous copy.
            tc_fence_after();
            constexpr uint32_t kPitch = 1040;
            const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
                uint32_t o[32];
                tc_ld32(tmem + lane_base + kColO + half * 128 + c, o);
                float4 g[8];
#pragma unroll
                for (int i = 0; i < 8; i++) { g[i] = gn[i]; gn[i] = gn2[i]; }
                if (c + 64 < 128) {  // two chunks ahead
#pragma unroll
                    for (int i = 0; i < 8; i++) gn2[i] = __ldg(gp + ((c + 64) >> 2) + i);
                }
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float y0 = __uint_as_float(o[4 * i]) * inv * fast_sigmoid(g[i].x);
                    const float y1 = __uint_as_float(o[4 * i + 1]) * inv * fast_sigmoid(g[i].y);
                    const float y2 = __uint_as_float(o[4 * i + 2]) * inv * fast_sigmoid(g[i].z);
                    const float y3 = __uint_as_float(o[4 * i + 3]) * inv * fast_sigmoid(g[i].w);
                    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(sQ + r * kPitch + (half * 128 + c + 4 * i) * 4), "f"(y0), "f"(y1),
                                 "f"(y2), "f"(y3)
                                 : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            if (live) {
                float *orow = p.out + ((size_t)t_row * p.H + head) * kHD + half * 128;
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 512;\n" ::"l"(orow), "r"(sQ + r * kPitch + half * 512) : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
            // shared memory must stay valid until the bulk copies have read it
            asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
        }
    }
    // ---- wind down: everyone meets, TMEM goes back ----
    tc_fence_before();
    __syncthreads();
    if (s_abort && tid == 0) atomicCAS(p.err, 0, (1 << 16) | ((blockIdx.y & 0xff) << 8) | (blockIdx.x & 0xff));
    if (warp == kWarpMma) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ---- host --------------------------------------------------------------------------------------
// Query tiles seeing fewer cache rows than this use two fp16 terms for the softmax weights (see two_p).
static int pf_two_term_rows() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("FM_PF_TWO_TERM_ROWS");  // measurement knob
        v = e ? atoi(e) : 1024;
    }
    return v;
}

// 2-D fp16 tensor [rows][cols], box [box_rows][64 cols], 128-byte swizzle, zero fill outside
static bool make_map(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_attn_prefill(const KvView &kv, const RopeParams &rope, int seq, int start_pos, int row0, int prefix0, int n, int H,
                        const float *q_proj_out, const float *q, const float *gate, const float *k, const float *v,
                        const uint16_t *q_norm_w, const uint16_t *k_norm_w, float eps, const PrefillWork &wk, float *out,
                        cudaStream_t st) {
    static unsigned long long configured = 0;  // one bit per device
    if (first_use_on_device(&configured)) {
        if (cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem) != cudaSuccess) return -1;
    }
    const int L = row0 + n;
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, wk.q16, (uint64_t)n, (uint64_t)H * 2 * kHD, kBM) || !make_map(&mk, wk.k16, (uint64_t)L, (uint64_t)kv.Hkv * kHD, kBN) ||
        !make_map(&mv, wk.v16, (uint64_t)L, (uint64_t)kv.Hkv * kHD, kBN))
        return -1;
    PrepParams pp;
    pp.n = n; pp.row0 = row0; pp.start_pos = start_pos; pp.seq = seq; pp.H = H; pp.prefix0 = prefix0;
    pp.q_proj_out = q_proj_out; pp.q_in = q; pp.k = k; pp.v = v; pp.qnw = q_norm_w; pp.knw = k_norm_w; pp.eps = eps;
    pp.q16 = reinterpret_cast<__half *>(wk.q16); pp.k16 = reinterpret_cast<__half *>(wk.k16); pp.v16 = reinterpret_cast<__half *>(wk.v16);
    attn_prefill_prep_kernel<<<n + n * kv.Hkv + (row0 - prefix0), 256, 0, st>>>(kv, rope, pp);
    if (cudaGetLastError() != cudaSuccess) return -1;
    PfParams p;
    p.n = n; p.row0 = row0; p.H = H; p.Hkv = kv.Hkv;
    p.q16 = reinterpret_cast<const __half *>(wk.q16);
    p.q_proj_out = q_proj_out; p.gate = gate; p.out = out; p.err = wk.err;
    p.two_term_rows = pf_two_term_rows();
    // the attention launch overlaps its set-up (barriers, TMEM allocation) with the end of the preparation
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(H, (n + kBM - 1) / kBM); lc.blockDim = dim3(kPfThreads); lc.dynamicSmemBytes = kPfSmem; lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, attn_prefill_kernel, mq, mk, mv, p) == cudaSuccess ? 2 : -1;
}

}  // namespace fm
