// Host-side context and the launcher interface between the C-ABI layer (fm_api.cu) and the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/fm_attn.h"

namespace fm {

constexpr int kMaxList = 64;  // tokens a kernel takes by value in one launch

// Which tokens a launch works on.  mode 0: an explicit list (decode: one token per sequence);
// mode 1: a run of n consecutive tokens of one sequence (prefill).
// A listed token's four numbers sit together (one 16-byte read of the kernel's parameter space).
struct TokEntry {
    int seq, pos, row;
    int nrows;  // cache rows the token attends to (row + 1, or the window once it has wrapped)
};
struct TokSpec {
    int mode;
    int n;
    int seq0, pos0, row0;  // mode 1: token t has pos0 + t, cache row row0 + t
    int pad[3];
    TokEntry e[kMaxList];  // mode 0
    void set(int i, int seq, int pos, int row, int nrows) { e[i].seq = seq; e[i].pos = pos; e[i].row = row; e[i].nrows = nrows; }
};

__host__ __device__ inline void tok_get(const TokSpec &t, int i, int &seq, int &pos, int &row) {
    if (t.mode == 1) {
        seq = t.seq0; pos = t.pos0 + i; row = t.row0 + i;
    } else {
        const TokEntry x = t.e[i];
        seq = x.seq; pos = x.pos; row = x.row;
    }
}

__host__ __device__ inline int tok_rows(const TokSpec &t, int i) { return t.mode == 1 ? t.row0 + i + 1 : t.e[i].nrows; }

// The paged KV store of one layer as a kernel sees it.
// bf16 page:  [2 (K,V)][Hkv][page_size][D] bf16, so one (K or V, head) tile is contiguous.
// FP8 page:   [2 (K,V)][Hkv][page_size][D] E4M3 bytes, then the rows' scales, float k_scale[page_size] and
//             v_scale[page_size] (one scale per position over all KV heads, as KVCache.k_scales / v_scales of
//             metal_infer/layer_forward.h:124-127).
// Row r of a sequence lives in global page r / page_size; a context holds the pages with
// (page % shard_count) == shard_rank, at local slot page / shard_count of its page table.
struct KvView {
    unsigned char *pool;
    size_t page_bytes;
    int fp8;                // 0: bf16 pages, 1: E4M3 pages with per-row scales
    const int *page_table;  // [max_seqs][max_slots] of this layer
    int max_slots;
    int page_size;
    int Hkv;
    int D;
    int shard_rank, shard_count;
};

__host__ __device__ inline size_t kv_page_bytes(int fp8, int Hkv, int page_size, int D) {
    return fp8 ? (size_t)2 * Hkv * page_size * D + (size_t)2 * page_size * sizeof(float)
               : (size_t)2 * Hkv * page_size * D * 2;
}
__host__ __device__ inline unsigned char *kv_page(const KvView &kv, int page) { return kv.pool + (size_t)page * kv.page_bytes; }
// start of the (which = 0 K / 1 V, head) tile inside a page, in bytes
__host__ __device__ inline size_t kv_tile_offset(const KvView &kv, int which, int kvh) {
    return (size_t)(which * kv.Hkv + kvh) * kv.page_size * kv.D * (kv.fp8 ? 1 : 2);
}
// FP8 pages: the page's k_scale[page_size] (which = 0) or v_scale[page_size] (which = 1)
__host__ __device__ inline float *kv_page_scales(const KvView &kv, unsigned char *page_base, int which) {
    return reinterpret_cast<float *>(page_base + (size_t)2 * kv.Hkv * kv.page_size * kv.D) + (size_t)which * kv.page_size;
}

// Exchange buffers of a sequence group as a kernel sees them (see attn_decode.cu).
constexpr int kMaxXchgRanks = 8;
struct XchgView {
    float *peer[kMaxXchgRanks];  // every rank's buffer, addressable from this GPU; peer[me] is the local one
    int nranks, me;
    int cap;                     // token capacity of a slot
    int ring;                    // slot sets, a power of two: exchange step s uses set s & (ring - 1)
    long long flag_offset_floats;       // step flags [ring][nranks]
    long long unit_flag_offset_floats;  // flags per (token, KV head) [ring][nranks][cap * Hkv]
    long long wait_limit_cycles;
};

// H2O bookkeeping of one layer as a kernel sees it (attn_h2o.cu): per sequence, `cap` = budget + 1 physical rows.
struct H2oView {
    float *accum;           // [seqs][cap] accumulated attention mass, by physical row
    int *order;             // [seqs][cap] physical row of the i-th row in cache order
    int *tokpos;            // [seqs][cap] original token index, by physical row
    int *slot;              // [seqs] physical row the next appended token takes
    unsigned int *counter;  // [seqs] arrivals of the mass kernel's CTAs (self-resetting)
    int cap;
};

// What the decode launch of an H2O store needs besides the attention itself: where the step's row goes, and where
// to leave the un-normalised softmax weights of every (row, head) for the mass pass (attn_h2o.cu).
struct H2oStep {
    const int *slot;   // [seqs] physical row the new token takes
    float *w;          // [tokens][rows_pad][Hkv][16] weights exp2(score - mref) of the step's rows
    float *mref;       // [tokens][tiles][Hkv][4][16] the maximum those weights refer to, per 16-row slice of a 64-row tile
    int rows_pad;      // rows per token in `w` (the capacity rounded up to whole tiles)
    int tiles;         // tiles per token in `mref`
};

struct RopeParams {
    float inv_freq[64];  // rotary_dim / 2 entries, computed on the host exactly as the reference does
    int rotary_dim;
    float pos_div;       // linear scaling: position is divided by this
    float logit_scale;   // 1/sqrt(D) * YaRN temperature
};

}  // namespace fm

constexpr int kDecGroup = 16;      // splits per first-level merge group
constexpr int kDecMaxGroups = 16;  // so up to 256 splits per (KV head, sequence)
struct DecodeScratch {
    unsigned int *counters;        // [kMaxList * Hkv + 1]
    unsigned int *group_counters;  // [group_tokens * Hkv * kDecMaxGroups]
    float *group_o, *group_ml;     // [group_tokens][H][kDecMaxGroups][D] and [..][2]
    int group_tokens;              // tokens the two-level merge has room for (it is only needed at small batch)
};

struct FmCtx {
    FmConfig cfg;
    cudaStream_t stream = nullptr;
    int ptr_mode = FM_PTR_DEVICE;
    std::string err;
    int64_t launches = 0;
    int sm_count = 148;

    fm::RopeParams rope;

    // KV store
    unsigned char *pool = nullptr;
    int64_t pool_pages = 0;
    size_t page_bytes = 0;
    int max_slots = 0;      // local page slots per sequence
    int *d_page_table = nullptr;       // [layers][seqs][max_slots]
    std::vector<int> h_page_table;
    std::vector<int> free_pages;
    std::vector<int> page_refs;   // sequences holding each page (0 = free); > 1 after fm_seq_fork
    std::vector<int> kv_len;           // [layers][seqs] global rows

    // GatedDeltaNet state
    float *d_conv_state = nullptr;  // [layers][seqs][ks-1][conv_dim]
    float *d_ssm_state = nullptr;   // [layers][seqs][Hv][dv][dk]
    int conv_dim = 0;
    std::vector<int> gdn_steps;     // [layers][seqs] tokens seen; indexes the conv ring

    // decode attention scratch: split partials
    float *d_part_o = nullptr;   // [batch][H][max_splits][D]
    float *d_part_ml = nullptr;  // [batch][H][max_splits][2]
    int max_splits = 0;
    unsigned int *d_dec_counters = nullptr;  // arrival counters of the fused decode kernel
    DecodeScratch dec_scr = {};              // set 0; layer l uses the pointers advanced by l strides
    size_t part_rows = 0, counter_stride = 0, group_counter_stride = 0, group_rows = 0;

    // prefill scratch: fp16 copies of q (normalised, rotated, scaled) and of the sequence's K, V rows
    void *d_pf_q16 = nullptr;  // [max_batch_tokens][H*D]
    void *d_pf_k16 = nullptr;  // [max_seq_len][Hkv*D]
    void *d_pf_v16 = nullptr;
    // which (layer, sequence) the K / V workspace holds and how many of its rows: a prompt fed in several calls
    // converts each cached row once, not once per call
    int pf_layer = -1, pf_seq = -1, pf_rows = 0;
    int *d_err = nullptr;      // device-side error word written by kernels whose bounded waits expired
    int *h_err = nullptr;      // pinned copy
    void *d_work = nullptr;             // chunked GatedDeltaNet workspace
    size_t work_bytes = 0;

    // H2O eviction: per (layer, sequence) bookkeeping on the device, rows kept on the host
    float *d_h2o_accum = nullptr;
    int *d_h2o_order = nullptr, *d_h2o_tokpos = nullptr, *d_h2o_slot = nullptr;
    unsigned int *d_h2o_counter = nullptr;
    float *d_h2o_ml = nullptr;  // (max, sum) per (token, head) of the step in flight
    int h2o_cap = 0;

    float *d_proj_ssq = nullptr;  // per-token sums of squares of the output projection's epilogue, two sets used alternately
    int proj_parity = 0;

    // cross-GPU exchange of partial results (fm_exchange_attach)
    fm::XchgView xchg = {};
    uint32_t xchg_step = 0;
    unsigned int *d_xchg_counter = nullptr;

    // optional event bracketing of the dominant kernels
    bool prof_on = false;
    // set by fm_attn_decode_layers between layers: the next decode launch may start while the previous
    // layer's kernel drains (different layers touch different pages, inputs and outputs)
    bool overlap_prev = false, overlap_merge = false, overlap_layers = false;
    int overlap_nlayers = 0;
    bool layer_overlap = false;  // fm_set_layer_overlap: consecutive decode calls touch different layers' state
    int last_state_li = -1;      // GatedDeltaNet layer the last decode step updated; -1 after anything else that writes state  // layers of the fm_attn_decode_layers call in progress (valid while overlap_layers)
    std::vector<cudaEvent_t> prof_ev;  // pairs (start, stop)
    size_t prof_used = 0;

    // host-pointer mode staging
    char *h_stage = nullptr;  // pinned
    char *d_stage = nullptr;
    size_t stage_bytes = 0;
    // staging of all layers of one fm_attn_decode_layers call in host-pointer mode (grown on demand)
    char *h_lstage = nullptr, *d_lstage = nullptr;
    size_t lstage_bytes = 0;
    float *d_h2o_w = nullptr, *d_h2o_mref = nullptr, *d_h2o_cand = nullptr;  // the decode launch's weights for the H2O mass pass (H2oStep)
    int h2o_rows_pad = 0, h2o_tiles = 0;
    float *d_gdn_scratch = nullptr;  // per-token records of the streaming GatedDeltaNet step (kMaxList tokens)
    // host-pointer form of the layered decode: copies run on a stream of their own, tied to the launches by events
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_in[3] = {nullptr, nullptr, nullptr}, ev_out[3] = {nullptr, nullptr, nullptr}, ev_idle = nullptr;
};

namespace fm {

// ---- launchers (each returns the number of kernels it queued, or -1 with cudaGetLastError set) ----
int launch_kv_append(const KvView &kv, const RopeParams &rope, const TokSpec &toks, const float *k,
                     const float *v, const uint16_t *k_norm_w, float eps, cudaStream_t st);

int launch_attn_decode(const KvView &kv, const RopeParams &rope, const TokSpec &toks, int H,
                       const float *q_proj_out, const float *q, const uint16_t *q_norm_w, float eps,
                       float *part_o, float *part_ml, int nsplits, cudaStream_t st);

int launch_attn_decode_fused(const KvView &kv, const RopeParams &rope, const TokSpec &toks, int H,
                             const float *q_proj_out, const float *q, const uint16_t *q_norm_w, float eps,
                             float *part_o, float *part_ml, int nsplits, const float *k_new, const float *v_new,
                             const uint16_t *k_norm_w, int tail, const float *gate, float *out, float *ml_out,
                             const XchgView *x, uint32_t step, const DecodeScratch &scr, int *err, bool overlap_prev,
                             cudaStream_t st, const H2oStep *h2o = nullptr);
constexpr int kDecMaxLastCtaSplits = 24;  // more splits per (KV head, sequence): merged in two levels

// merges [nparts] partials per (token, head) laid out with strides, applies the gate
int launch_attn_merge(const float *part_o, const float *part_ml, int nparts, long long part_stride_o,
                      long long part_stride_ml, long long tok_stride_o, long long tok_stride_ml,
                      long long head_stride_o, long long head_stride_ml, int ntok, int H, int D,
                      const float *q_proj_out, const float *gate, float *out, float *ml_out,
                      cudaStream_t st);

// merge of many split partials of (token, head), laid out [tok][H][nparts][..], as a programmatic dependent of the
// launch that writes them
// ml_final (may be null): in final mode, also the merged (max, sum) per (token, head)
int launch_attn_merge_wide(const float *part_o, const float *part_ml, int nparts, int ntok, int H, const float *q_proj_out,
                           const float *gate, float *out, float *ml_out, cudaStream_t st, float *ml_final = nullptr);

int launch_attn_merge_push(const float *part_o, const float *part_ml, int nsplits, int ntok, int H, const XchgView &x,
                           uint32_t step, unsigned int *done_counter, cudaStream_t st);
int launch_attn_wait_merge(const XchgView &x, uint32_t step, int ntok, int H, const float *q_proj_out, const float *gate,
                           float *out, int *err, bool overlap_prev, cudaStream_t st);

// rows [row0, row0 + n) of a sequence to / from fp32 [n][Hkv*D] buffers that start at row0
// `order` (may be null): row i of the export is store row order[i] (an H2O store keeps its rows in place and their cache order aside)
int launch_kv_export(const KvView &kv, int seq, int row0, int n, float *k, float *v, const int *order, cudaStream_t st);
int launch_kv_import(const KvView &kv, int seq, int row0, int n, const float *k, const float *v, cudaStream_t st);
// FP8 store: the stored bytes [n][Hkv*D] and per-row scales [n] themselves
int launch_kv_copy_fp8(const KvView &kv, int seq, int row0, int n, uint8_t *k, uint8_t *v, float *ks, float *vs, bool import,
                       const int *order, cudaStream_t st);

int launch_h2o_mass(const TokSpec &toks, const int *token_index, const H2oView &h, int budget, int sinks, int recent, int H, int Hkv,
                    const float *ml, const H2oStep &step, float *cand, int max_rows, cudaStream_t st);
int launch_h2o_order(const H2oView &h, int seq, int n, cudaStream_t st);  // rebuilds h.order for rows [0, n) of a sequence
int launch_h2o_gather(const H2oView &h, int seq, int n, float *accum_out, int *tokpos_out, cudaStream_t st);
int launch_h2o_init(const H2oView &h, int seq, int n, cudaStream_t st);

// y = W x from 4-bit affine weights, h_mid = residual + y, h_post = rms-norm(h_mid) * w (out_proj.cu); n <= 8 tokens,
// ssq: two sets of 8 floats (zero at creation) used alternately, *parity the set of this call.  h_post may be null.
int launch_out_proj_q4(const uint32_t *w, const uint16_t *scales, const uint16_t *biases, int out_dim, int in_dim, int n, const float *x,
                       const float *residual, const uint16_t *norm_w, float eps, float *h_mid, float *h_post, float *ssq, int *parity,
                       cudaStream_t st);

struct PrefillWork {
    void *q16, *k16, *v16;
    int *err;
};
// prefix0: the fp16 workspace already holds cached rows [0, prefix0) of this (layer, sequence)
int launch_attn_prefill(const KvView &kv, const RopeParams &rope, int seq, int start_pos, int row0, int prefix0, int n, int H,
                        const float *q_proj_out, const float *q, const float *gate, const float *k, const float *v,
                        const uint16_t *q_norm_w, const uint16_t *k_norm_w, float eps, const PrefillWork &wk, float *out,
                        cudaStream_t st);

struct GdnDims {
    int Hv, Hk, dk, dv, ks, conv_dim;
    float eps;
};
int launch_gdn_decode(const GdnDims &g, const TokSpec &toks, float *conv_state, float *ssm_state,
                      long long conv_seq_stride, long long ssm_seq_stride, const float *qkv,
                      const float *z, const float *beta, const float *alpha, const uint16_t *conv_w,
                      const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, float *out,
                      bool overlap_prev, cudaStream_t st);
// The same step as a prep launch + a persistent launch that streams the states (for many (head, sequence) pairs);
// `scratch` holds gdn_decode_scratch_bytes(g, toks.n) bytes, z must be 16-byte aligned.  Returns the launches made.
size_t gdn_decode_scratch_bytes(const GdnDims &g, int tokens);
int launch_gdn_decode_stream(const GdnDims &g, const TokSpec &toks, float *conv_state, float *ssm_state, long long conv_seq_stride,
                             long long ssm_seq_stride, const float *qkv, const float *z, const float *beta, const float *alpha,
                             const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias, const uint16_t *norm_w, float *out,
                             float *scratch, int sm_count, int *err, cudaStream_t st);
int launch_gdn_prefill(const GdnDims &g, int n, int chunk, int step0, float *conv_state, float *ssm_state,
                       const float *qkv, const float *z, const float *beta, const float *alpha,
                       const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                       const uint16_t *norm_w, float *out, void *work, size_t work_bytes, int *err,
                       cudaStream_t st);
size_t gdn_prefill_work_bytes(const GdnDims &g, int max_tokens, int chunk);

// True the first time it is called for the current device with a given per-call-site flag word: function
// attributes (dynamic shared memory limits) are per device, and one process may hold contexts on several.
inline bool first_use_on_device(unsigned long long *done_mask) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    const unsigned long long bit = 1ull << dev;
    if (*done_mask & bit) return false;
    *done_mask |= bit;
    return true;
}

}  // namespace fm
