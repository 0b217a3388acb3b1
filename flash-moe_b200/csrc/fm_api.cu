// C-ABI layer: context, paged-KV page allocator, pointer-mode staging, argument checks, and the
// host-side sequencing of the kernels for each entry point of include/fm_attn.h.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <new>

#include <cstdlib>

#include "fm_internal.h"

using namespace fm;

static std::string g_create_error;

static fm_status fail(FmCtx *ctx, fm_status st, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->err = buf; else g_create_error = buf;
    return st;
}

#define FM_CUDA(ctx, call)                                                                          \
    do {                                                                                            \
        cudaError_t e__ = (call);                                                                   \
        if (e__ != cudaSuccess)                                                                     \
            return fail(ctx, FM_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__));         \
    } while (0)

static fm_status launched(FmCtx *ctx, int n, const char *what) {
    if (n < 0) return fail(ctx, FM_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(cudaGetLastError()));
    ctx->launches += n;
    return FM_OK;
}

extern "C" void fm_default_config(FmConfig *c) {
    memset(c, 0, sizeof *c);
    c->num_attn_heads = 32; c->num_kv_heads = 2; c->head_dim = 256; c->rotary_dim = 64;
    c->rope_theta = 1e7f; c->rms_norm_eps = 1e-6f;
    c->rope_scaling_mode = 0; c->rope_scale_factor = 1.0f; c->rope_orig_max_pos = 262144;
    c->num_full_layers = 15;
    c->linear_num_v_heads = 64; c->linear_num_k_heads = 16; c->linear_key_dim = 128;
    c->linear_value_dim = 128; c->conv_kernel_size = 4; c->num_linear_layers = 45;
    c->max_seqs = 1; c->max_seq_len = 8192; c->page_size = 64; c->kv_pool_pages = 0;
    c->max_batch_tokens = 64;
    c->seq_shard_rank = 0; c->seq_shard_count = 1; c->device = 0;
    c->kv_dtype = FM_KV_BF16;
    c->h2o_budget = 0; c->h2o_num_sinks = 4;
}

// RoPE frequency of pair i under the scaling modes of metal_infer/layer_forward.h:22-63, evaluated
// on the host in fp32 with the same expressions so that device angles equal the CPU path's.
static float rope_inv_freq(const FmConfig &c, int i) {
    const float base = c.rope_theta;
    const int rot = c.rotary_dim;
    const float s = c.rope_scale_factor;
    const float expo = (float)(2 * i) / rot;
    if (c.rope_scaling_mode == 0 || s <= 1.0f || c.rope_scaling_mode == 1) return 1.0f / powf(base, expo);
    const float base_ntk = base * powf(s, (float)rot / (rot - 2));
    if (c.rope_scaling_mode == 2) return 1.0f / powf(base_ntk, expo);
    const float f_orig = 1.0f / powf(base, expo), f_ntk = 1.0f / powf(base_ntk, expo);
    const float wavelength = 2.0f * M_PI / f_orig;
    const float lo = (float)c.rope_orig_max_pos, hi = lo / 32.0f;
    if (wavelength < hi) return f_orig;
    if (wavelength > lo) return f_ntk;
    const float ramp = (wavelength - hi) / (lo - hi);
    return f_orig * (1.0f - ramp) + f_ntk * ramp;
}

static size_t stage_need(const FmConfig &c) {
    // largest set of host tensors one call moves: prefill q_proj_out + k + v + out, or the
    // GatedDeltaNet inputs + output
    const size_t n = (size_t)c.max_batch_tokens;
    const size_t attn = n * ((size_t)c.num_attn_heads * c.head_dim * 3 + (size_t)c.num_kv_heads * c.head_dim * 2) * 4;
    const size_t conv_dim = 2 * (size_t)c.linear_num_k_heads * c.linear_key_dim + (size_t)c.linear_num_v_heads * c.linear_value_dim;
    const size_t gdn = n * (conv_dim + 2 * (size_t)c.linear_num_v_heads * c.linear_value_dim + 2 * (size_t)c.linear_num_v_heads) * 4;
    return std::max(attn, gdn) + (1 << 20);
}

extern "C" fm_status fm_create(const FmConfig *cfg, FmCtx **out) {
    if (!cfg || !out) return fail(nullptr, FM_ERR_INVALID, "fm_create: null argument");
    *out = nullptr;
    const FmConfig &c = *cfg;
    const bool has_attn = c.num_full_layers > 0, has_gdn = c.num_linear_layers > 0;
    if (c.max_seqs < 1 || c.max_batch_tokens < 1 || c.seq_shard_count < 1 || c.seq_shard_rank < 0 ||
        c.seq_shard_rank >= c.seq_shard_count)
        return fail(nullptr, FM_ERR_INVALID, "fm_create: bad max_seqs / max_batch_tokens / sequence sharding");
    if (has_attn) {
        if (c.head_dim != 256) return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: head_dim %d (kernels are built for 256)", c.head_dim);
        if (c.page_size != 64) return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: page_size %d (kernels are built for 64)", c.page_size);
        if (c.num_kv_heads < 1 || c.num_attn_heads % c.num_kv_heads != 0 || c.num_attn_heads / c.num_kv_heads > 16)
            return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: %d query heads per KV head (1..16 supported)",
                        c.num_kv_heads ? c.num_attn_heads / c.num_kv_heads : 0);
        if (c.rotary_dim < 0 || c.rotary_dim > 128 || c.rotary_dim % 2 != 0 || c.rotary_dim > c.head_dim)
            return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: rotary_dim %d (even, <= 128)", c.rotary_dim);
        if (c.max_seq_len < 1) return fail(nullptr, FM_ERR_INVALID, "fm_create: max_seq_len %d", c.max_seq_len);
        if (c.sliding_window < 0 || c.sliding_window > c.max_seq_len)
            return fail(nullptr, FM_ERR_INVALID, "fm_create: sliding_window %d (0, or 1..max_seq_len)", c.sliding_window);
        if (c.kv_dtype != FM_KV_BF16 && c.kv_dtype != FM_KV_FP8_E4M3)
            return fail(nullptr, FM_ERR_INVALID, "fm_create: kv_dtype %d (FM_KV_BF16 or FM_KV_FP8_E4M3)", c.kv_dtype);
        if (c.h2o_budget < 0 || c.h2o_num_sinks < 0)
            return fail(nullptr, FM_ERR_INVALID, "fm_create: h2o_budget %d / h2o_num_sinks %d", c.h2o_budget, c.h2o_num_sinks);
        if (c.h2o_budget > 0 && c.seq_shard_count != 1)
            return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: H2O eviction needs the whole sequence on one context (seq_shard_count=1)");
        if (c.h2o_budget > 0 && c.num_kv_heads > 8)
            return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: H2O eviction takes at most 8 KV heads per context (%d)", c.num_kv_heads);
        if (c.kv_dtype == FM_KV_FP8_E4M3 && c.num_kv_heads > 8)
            return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: an FP8 store takes at most 8 KV heads per context (%d)", c.num_kv_heads);
    }
    if (has_gdn) {
        if (c.linear_key_dim != 128 || c.linear_value_dim != 128 || c.conv_kernel_size != 4)
            return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: GatedDeltaNet dims %dx%d conv %d (built for 128x128, conv 4)",
                        c.linear_key_dim, c.linear_value_dim, c.conv_kernel_size);
        if (c.linear_num_k_heads < 1 || c.linear_num_v_heads % c.linear_num_k_heads != 0)
            return fail(nullptr, FM_ERR_INVALID, "fm_create: v heads must be a multiple of k heads");
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        return fail(nullptr, FM_ERR_CUDA, "fm_create: no CUDA device (this library has no CPU path)");
    if (c.device < 0 || c.device >= ndev) return fail(nullptr, FM_ERR_INVALID, "fm_create: device %d of %d", c.device, ndev);

    FmCtx *ctx = new (std::nothrow) FmCtx();
    if (!ctx) return fail(nullptr, FM_ERR_NOMEM, "fm_create: out of host memory");
    ctx->cfg = c;
    if (c.h2o_budget > 0) ctx->cfg.sliding_window = 0;  // H2O replaces the window when both are set (layer_forward.h:148-152)
#define CREATE_CUDA(call)                                                                               \
    do {                                                                                                \
        cudaError_t e__ = (call);                                                                       \
        if (e__ != cudaSuccess) {                                                                       \
            fm_status st__ = fail(nullptr, e__ == cudaErrorMemoryAllocation ? FM_ERR_NOMEM : FM_ERR_CUDA, \
                                  "fm_create: %s failed: %s", #call, cudaGetErrorString(e__));          \
            fm_destroy(ctx);                                                                            \
            return st__;                                                                                \
        }                                                                                               \
    } while (0)
    CREATE_CUDA(cudaSetDevice(c.device));
    cudaDeviceProp prop;
    CREATE_CUDA(cudaGetDeviceProperties(&prop, c.device));
    ctx->sm_count = prop.multiProcessorCount;
    if (prop.major < 10) {
        fm_destroy(ctx);
        return fail(nullptr, FM_ERR_UNSUPPORTED, "fm_create: device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor);
    }

    if (has_attn) {
        ctx->rope.rotary_dim = c.rotary_dim;
        for (int i = 0; i < c.rotary_dim / 2; i++) ctx->rope.inv_freq[i] = rope_inv_freq(c, i);
        ctx->rope.pos_div = (c.rope_scaling_mode == 1 && c.rope_scale_factor > 1.0f) ? c.rope_scale_factor : 1.0f;
        float yarn = 1.0f;
        if (c.rope_scaling_mode == 3 && c.rope_scale_factor > 1.0f) yarn = sqrtf(0.1f * logf(c.rope_scale_factor) + 1.0f);
        ctx->rope.logit_scale = (1.0f / sqrtf((float)c.head_dim)) * yarn;

        // a sliding window or an H2O budget bounds the rows a sequence can hold, whatever max_seq_len says
        const int max_rows = c.h2o_budget > 0 ? std::min(c.max_seq_len, c.h2o_budget + 1)
                           : c.sliding_window > 0 ? std::min(c.max_seq_len, c.sliding_window) : c.max_seq_len;
        const int gpages = (max_rows + c.page_size - 1) / c.page_size;
        ctx->max_slots = (gpages + c.seq_shard_count - 1) / c.seq_shard_count;
        ctx->page_bytes = kv_page_bytes(c.kv_dtype == FM_KV_FP8_E4M3, c.num_kv_heads, c.page_size, c.head_dim);
        ctx->pool_pages = c.kv_pool_pages > 0 ? c.kv_pool_pages
                                              : (int64_t)ctx->max_slots * c.max_seqs * c.num_full_layers;
        CREATE_CUDA(cudaMalloc(&ctx->pool, (size_t)ctx->pool_pages * ctx->page_bytes));
        // zero so that rows past a sequence's end hold finite values (they meet zero weights)
        CREATE_CUDA(cudaMemset(ctx->pool, 0, (size_t)ctx->pool_pages * ctx->page_bytes));
        const size_t nent = (size_t)c.num_full_layers * c.max_seqs * ctx->max_slots;
        ctx->h_page_table.assign(nent, -1);
        CREATE_CUDA(cudaMalloc(&ctx->d_page_table, nent * sizeof(int)));
        CREATE_CUDA(cudaMemset(ctx->d_page_table, 0, nent * sizeof(int)));
        ctx->free_pages.resize((size_t)ctx->pool_pages);
        for (int64_t i = 0; i < ctx->pool_pages; i++) ctx->free_pages[(size_t)i] = (int)(ctx->pool_pages - 1 - i);
        ctx->page_refs.assign((size_t)ctx->pool_pages, 0);
        ctx->kv_len.assign((size_t)c.num_full_layers * c.max_seqs, 0);

        // Split partials: at most ~2 CTAs per SM plus one per (KV head, sequence), 16 head rows each.  Every layer
        // has its own set of partials and arrival counters, so the launches of consecutive layers never share
        // scratch and need no ordering among themselves (fm_attn_decode_layers overlaps them).
        ctx->max_splits = std::max(1, ctx->sm_count);
        const size_t nsets = (size_t)c.num_full_layers;
        const size_t rows = ((size_t)2 * ctx->sm_count + (size_t)c.num_kv_heads * c.max_batch_tokens) * 16 + 64;
        ctx->part_rows = rows;
        ctx->counter_stride = (size_t)kMaxList * c.num_kv_heads + 1;
        CREATE_CUDA(cudaMalloc(&ctx->d_part_o, nsets * rows * c.head_dim * sizeof(float)));
        CREATE_CUDA(cudaMalloc(&ctx->d_part_ml, nsets * rows * 2 * sizeof(float)));
        CREATE_CUDA(cudaMalloc(&ctx->d_dec_counters, nsets * ctx->counter_stride * sizeof(unsigned int)));
        CREATE_CUDA(cudaMemset(ctx->d_dec_counters, 0, nsets * ctx->counter_stride * sizeof(unsigned int)));
        // second-level scratch of the split merge, needed only when few sequences are split many ways
        DecodeScratch &ds = ctx->dec_scr;
        ds.counters = ctx->d_dec_counters;
        ds.group_tokens = 8;
        const size_t gc = (size_t)ds.group_tokens * c.num_kv_heads * kDecMaxGroups;
        const size_t grows = (size_t)ds.group_tokens * c.num_attn_heads * kDecMaxGroups;
        ctx->group_counter_stride = gc;
        ctx->group_rows = grows;
        CREATE_CUDA(cudaMalloc(&ds.group_counters, nsets * gc * sizeof(unsigned int)));
        CREATE_CUDA(cudaMemset(ds.group_counters, 0, nsets * gc * sizeof(unsigned int)));
        CREATE_CUDA(cudaMalloc(&ds.group_o, nsets * grows * c.head_dim * sizeof(float)));
        CREATE_CUDA(cudaMalloc(&ds.group_ml, nsets * grows * 2 * sizeof(float)));
        if (c.h2o_budget > 0) {
            ctx->h2o_cap = c.h2o_budget + 1;
            const size_t ne = (size_t)c.num_full_layers * c.max_seqs * ctx->h2o_cap, ns = (size_t)c.num_full_layers * c.max_seqs;
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_accum, ne * sizeof(float)));
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_order, ne * sizeof(int)));
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_tokpos, ne * sizeof(int)));
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_slot, ns * sizeof(int)));
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_counter, ns * sizeof(unsigned int)));
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_ml, (size_t)kMaxList * c.num_attn_heads * 2 * sizeof(float)));
            // the decode launch's per-(row, head) weights of one step, consumed by the mass pass right after it
            const size_t ntok = (size_t)std::min(kMaxList, std::max(1, c.max_batch_tokens));
            ctx->h2o_tiles = (ctx->h2o_cap + c.page_size - 1) / c.page_size;
            ctx->h2o_rows_pad = ctx->h2o_tiles * c.page_size;
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_w, ntok * ctx->h2o_rows_pad * c.num_kv_heads * 16 * sizeof(float)));
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_mref, ntok * ctx->h2o_tiles * c.num_kv_heads * 64 * sizeof(float)));
            CREATE_CUDA(cudaMalloc(&ctx->d_h2o_cand, ntok * ctx->h2o_tiles * 4 * sizeof(float)));
            CREATE_CUDA(cudaMemset(ctx->d_h2o_accum, 0, ne * sizeof(float)));
            CREATE_CUDA(cudaMemset(ctx->d_h2o_order, 0, ne * sizeof(int)));
            CREATE_CUDA(cudaMemset(ctx->d_h2o_tokpos, 0, ne * sizeof(int)));
            CREATE_CUDA(cudaMemset(ctx->d_h2o_slot, 0, ns * sizeof(int)));
            CREATE_CUDA(cudaMemset(ctx->d_h2o_counter, 0, ns * sizeof(unsigned int)));
        }
        {
            CREATE_CUDA(cudaMalloc(&ctx->d_pf_q16, (size_t)c.max_batch_tokens * c.num_attn_heads * c.head_dim * 2 * 2));  // hi | lo
            CREATE_CUDA(cudaMalloc(&ctx->d_pf_k16, (size_t)c.max_seq_len * c.num_kv_heads * c.head_dim * 2));
            CREATE_CUDA(cudaMalloc(&ctx->d_pf_v16, (size_t)c.max_seq_len * c.num_kv_heads * c.head_dim * 2));
        }
    }
    if (has_gdn) {
        ctx->conv_dim = 2 * c.linear_num_k_heads * c.linear_key_dim + c.linear_num_v_heads * c.linear_value_dim;
        // conv history kept as a ring of ks rows (see gdn_decode.cu) + the token count that indexes it
        const size_t conv_n = (size_t)c.num_linear_layers * c.max_seqs * c.conv_kernel_size * ctx->conv_dim;
        const size_t ssm_n = (size_t)c.num_linear_layers * c.max_seqs * c.linear_num_v_heads * c.linear_value_dim * c.linear_key_dim;
        CREATE_CUDA(cudaMalloc(&ctx->d_conv_state, conv_n * sizeof(float)));
        CREATE_CUDA(cudaMalloc(&ctx->d_ssm_state, ssm_n * sizeof(float)));
        CREATE_CUDA(cudaMemset(ctx->d_conv_state, 0, conv_n * sizeof(float)));
        CREATE_CUDA(cudaMemset(ctx->d_ssm_state, 0, ssm_n * sizeof(float)));
        ctx->gdn_steps.assign((size_t)c.num_linear_layers * c.max_seqs, 0);
        GdnDims g{c.linear_num_v_heads, c.linear_num_k_heads, c.linear_key_dim, c.linear_value_dim, c.conv_kernel_size, ctx->conv_dim, c.rms_norm_eps};
        ctx->work_bytes = gdn_prefill_work_bytes(g, c.max_batch_tokens, 64);
        if (ctx->work_bytes) CREATE_CUDA(cudaMalloc(&ctx->d_work, ctx->work_bytes));
    }
    if (c.num_linear_layers > 0 && c.linear_key_dim == 128 && c.linear_value_dim == 128)
        CREATE_CUDA(cudaMalloc(&ctx->d_gdn_scratch, gdn_decode_scratch_bytes(GdnDims{c.linear_num_v_heads, c.linear_num_k_heads, 128, 128, 0, 0, 0.f}, kMaxList)));
    CREATE_CUDA(cudaMalloc(&ctx->d_proj_ssq, 16 * sizeof(float)));
    CREATE_CUDA(cudaMemset(ctx->d_proj_ssq, 0, 16 * sizeof(float)));
    CREATE_CUDA(cudaMalloc(&ctx->d_err, sizeof(int)));
    CREATE_CUDA(cudaMemset(ctx->d_err, 0, sizeof(int)));
    CREATE_CUDA(cudaMallocHost(&ctx->h_err, sizeof(int)));
    *ctx->h_err = 0;
    ctx->stage_bytes = stage_need(c);
    CREATE_CUDA(cudaMallocHost(&ctx->h_stage, ctx->stage_bytes));
    CREATE_CUDA(cudaMalloc(&ctx->d_stage, ctx->stage_bytes));
    CREATE_CUDA(cudaDeviceSynchronize());
#undef CREATE_CUDA
    *out = ctx;
    return FM_OK;
}

extern "C" void fm_destroy(FmCtx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->cfg.device);
    cudaDeviceSynchronize();
    cudaFree(ctx->pool); cudaFree(ctx->d_page_table); cudaFree(ctx->d_conv_state); cudaFree(ctx->d_ssm_state);
    cudaFree(ctx->dec_scr.group_counters); cudaFree(ctx->dec_scr.group_o); cudaFree(ctx->dec_scr.group_ml);
    cudaFree(ctx->d_part_o); cudaFree(ctx->d_part_ml); cudaFree(ctx->d_dec_counters); cudaFree(ctx->d_xchg_counter); cudaFree(ctx->d_pf_q16); cudaFree(ctx->d_pf_k16); cudaFree(ctx->d_pf_v16); cudaFree(ctx->d_err);
    if (ctx->h_err) cudaFreeHost(ctx->h_err); cudaFree(ctx->d_work);
    cudaFree(ctx->d_h2o_accum); cudaFree(ctx->d_h2o_order); cudaFree(ctx->d_h2o_tokpos); cudaFree(ctx->d_h2o_slot);
    cudaFree(ctx->d_h2o_counter); cudaFree(ctx->d_h2o_ml); cudaFree(ctx->d_h2o_w); cudaFree(ctx->d_h2o_mref); cudaFree(ctx->d_h2o_cand);
    cudaFree(ctx->d_proj_ssq);
    cudaFree(ctx->d_gdn_scratch);
    cudaFree(ctx->d_stage);
    cudaFree(ctx->d_lstage);
    if (ctx->h_lstage) cudaFreeHost(ctx->h_lstage);
    for (int i = 0; i < 3; i++) {
        if (ctx->ev_in[i]) cudaEventDestroy(ctx->ev_in[i]);
        if (ctx->ev_out[i]) cudaEventDestroy(ctx->ev_out[i]);
    }
    if (ctx->ev_idle) cudaEventDestroy(ctx->ev_idle);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
    for (cudaEvent_t e : ctx->prof_ev) cudaEventDestroy(e);
    if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
    delete ctx;
}

extern "C" const char *fm_last_error(const FmCtx *ctx) { return ctx ? ctx->err.c_str() : g_create_error.c_str(); }

extern "C" fm_status fm_set_stream(FmCtx *ctx, void *s) {
    if (!ctx) return FM_ERR_INVALID;
    ctx->stream = (cudaStream_t)s;
    return FM_OK;
}
extern "C" fm_status fm_set_pointer_mode(FmCtx *ctx, int mode) {
    if (!ctx) return FM_ERR_INVALID;
    if (mode != FM_PTR_DEVICE && mode != FM_PTR_HOST) return fail(ctx, FM_ERR_INVALID, "fm_set_pointer_mode: mode %d", mode);
    ctx->ptr_mode = mode;
    return FM_OK;
}
// A kernel whose bounded device-side wait expired leaves a code in the error word.
static fm_status check_device_error(FmCtx *ctx) {
    if (*ctx->h_err == 0) return FM_OK;
    const int code = *ctx->h_err;
    *ctx->h_err = 0;
    cudaMemsetAsync(ctx->d_err, 0, sizeof(int), ctx->stream);
    return fail(ctx, FM_ERR_TIMEOUT, "a device-side wait expired (code 0x%x); the results of that call are invalid", code);
}

// The error word comes to the host only where the host waits anyway (a copy per call would sit
// between consecutive launches of a device-pointer caller).
extern "C" fm_status fm_synchronize(FmCtx *ctx) {
    if (!ctx) return FM_ERR_INVALID;
    FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return check_device_error(ctx);
}
extern "C" fm_status fm_set_layer_overlap(FmCtx *ctx, int on) {
    if (!ctx) return FM_ERR_INVALID;
    ctx->layer_overlap = on != 0;
    return FM_OK;
}
extern "C" int64_t fm_launch_count(const FmCtx *ctx) { return ctx ? ctx->launches : 0; }

// ---- event bracketing of the dominant kernels --------------------------------------------------
struct ProfScope {
    FmCtx *ctx;
    cudaEvent_t stop = nullptr;
    explicit ProfScope(FmCtx *c) : ctx(c) {
        if (!c->prof_on) return;
        if (c->prof_used + 2 > c->prof_ev.size()) {
            cudaEvent_t a, b;
            if (c->prof_ev.size() >= 1 << 16 || cudaEventCreate(&a) != cudaSuccess) return;
            if (cudaEventCreate(&b) != cudaSuccess) { cudaEventDestroy(a); return; }
            c->prof_ev.push_back(a);
            c->prof_ev.push_back(b);
        }
        cudaEventRecord(c->prof_ev[c->prof_used], c->stream);
        stop = c->prof_ev[c->prof_used + 1];
        c->prof_used += 2;
    }
    ~ProfScope() {
        if (stop) cudaEventRecord(stop, ctx->stream);
    }
};

extern "C" fm_status fm_profile_enable(FmCtx *ctx, int on) {
    if (!ctx) return FM_ERR_INVALID;
    ctx->prof_on = on != 0;
    return FM_OK;
}

extern "C" fm_status fm_profile_read(FmCtx *ctx, int *launches, double *total_ms) {
    if (!ctx || !launches || !total_ms) return FM_ERR_INVALID;
    FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    double tot = 0.0;
    for (size_t i = 0; i + 1 < ctx->prof_used; i += 2) {
        float ms = 0.f;
        FM_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->prof_ev[i], ctx->prof_ev[i + 1]));
        tot += ms;
    }
    *launches = (int)(ctx->prof_used / 2);
    *total_ms = tot;
    ctx->prof_used = 0;
    return FM_OK;
}

// ---- KV bookkeeping ---------------------------------------------------------------------------
static inline size_t lidx(const FmCtx *ctx, int layer, int seq) { return (size_t)layer * ctx->cfg.max_seqs + seq; }

static KvView kv_view(const FmCtx *ctx, int fa_idx) {
    KvView v;
    v.pool = ctx->pool;
    v.page_bytes = ctx->page_bytes;
    v.fp8 = ctx->cfg.kv_dtype == FM_KV_FP8_E4M3;
    v.page_table = ctx->d_page_table + (size_t)fa_idx * ctx->cfg.max_seqs * ctx->max_slots;
    v.max_slots = ctx->max_slots;
    v.page_size = ctx->cfg.page_size;
    v.Hkv = ctx->cfg.num_kv_heads;
    v.D = ctx->cfg.head_dim;
    v.shard_rank = ctx->cfg.seq_shard_rank;
    v.shard_count = ctx->cfg.seq_shard_count;
    return v;
}

// Makes sure the locally-held pages covering rows [0, new_len) of (layer, seq) exist.
// Pages are reference-counted: a forked sequence shares the full pages of its source.
static inline int take_page(FmCtx *ctx) {
    const int p = ctx->free_pages.back();
    ctx->free_pages.pop_back();
    ctx->page_refs[(size_t)p] = 1;
    return p;
}
static inline void release_page(FmCtx *ctx, int p) {
    if (--ctx->page_refs[(size_t)p] == 0) ctx->free_pages.push_back(p);
}

// Rows of the store a sequence occupies after `count` tokens, and the row token number `count` goes to.
// (H2O: `count` tokens occupy min(count, budget + 1) rows while the step that appended the last one runs and
// min(count, budget) once it has evicted -- rows_kept; the row a token goes to is decided on the device.)
static inline int rows_held(const FmConfig &c, int count) {
    if (c.h2o_budget > 0) return std::min(count, c.h2o_budget + 1);
    return c.sliding_window > 0 ? std::min(count, c.sliding_window) : count;
}
static inline int rows_kept(const FmConfig &c, int count) { return c.h2o_budget > 0 ? std::min(count, c.h2o_budget) : rows_held(c, count); }
static inline int row_of(const FmConfig &c, int count) {
    if (c.h2o_budget > 0) return std::min(count, c.h2o_budget);
    return c.sliding_window > 0 ? count % c.sliding_window : count;
}
static H2oView h2o_view(const FmCtx *ctx, int fa_idx) {
    H2oView h;
    const size_t s = (size_t)fa_idx * ctx->cfg.max_seqs;
    h.cap = ctx->h2o_cap;
    h.accum = ctx->d_h2o_accum + s * h.cap;
    h.order = ctx->d_h2o_order + s * h.cap;
    h.tokpos = ctx->d_h2o_tokpos + s * h.cap;
    h.slot = ctx->d_h2o_slot + s;
    h.counter = ctx->d_h2o_counter + s;
    return h;
}

static fm_status ensure_pages(FmCtx *ctx, int fa_idx, int seq, int new_len) {
    const FmConfig &c = ctx->cfg;
    if (c.sliding_window == 0 && c.h2o_budget == 0 && new_len > c.max_seq_len)
        return fail(ctx, FM_ERR_CAPACITY, "KV cache overflow (pos=%d >= cap=%d)", new_len - 1, c.max_seq_len);
    new_len = rows_held(c, new_len);
    const int gpages = (new_len + c.page_size - 1) / c.page_size;
    const int nslots = gpages > c.seq_shard_rank ? (gpages - c.seq_shard_rank + c.seq_shard_count - 1) / c.seq_shard_count : 0;
    int *tab = &ctx->h_page_table[((size_t)fa_idx * c.max_seqs + seq) * ctx->max_slots];
    int first_new = -1, need = 0;
    for (int s = 0; s < nslots; s++)
        if (tab[s] < 0) { if (first_new < 0) first_new = s; need++; }
    if (need == 0) return FM_OK;
    if ((size_t)need > ctx->free_pages.size())
        return fail(ctx, FM_ERR_CAPACITY, "KV page pool exhausted (%d more pages needed, %zu free)", need, ctx->free_pages.size());
    for (int s = first_new; s < nslots; s++)
        if (tab[s] < 0) tab[s] = take_page(ctx);
    int *dtab = ctx->d_page_table + ((size_t)fa_idx * c.max_seqs + seq) * ctx->max_slots;
    // pageable-source copies are staged by the runtime before the call returns, so `tab` may change later
    FM_CUDA(ctx, cudaMemcpyAsync(dtab + first_new, tab + first_new, (size_t)(nslots - first_new) * sizeof(int),
                                 cudaMemcpyHostToDevice, ctx->stream));
    return FM_OK;
}

extern "C" int fm_kv_len(const FmCtx *ctx, int fa_idx, int seq) {
    if (!ctx || fa_idx < 0 || fa_idx >= ctx->cfg.num_full_layers || seq < 0 || seq >= ctx->cfg.max_seqs) return -1;
    return ctx->kv_len[lidx(ctx, fa_idx, seq)];
}

extern "C" fm_status fm_reset(FmCtx *ctx, int seq) {
    if (!ctx) return FM_ERR_INVALID;
    ctx->last_state_li = -1;  // the next GatedDeltaNet step is not launched under this call's tail
    const FmConfig &c = ctx->cfg;
    if (seq < -1 || seq >= c.max_seqs) return fail(ctx, FM_ERR_INVALID, "fm_reset: seq %d", seq);
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const int s0 = seq < 0 ? 0 : seq, s1 = seq < 0 ? c.max_seqs : seq + 1;
    ctx->pf_layer = -1;  // the prefill workspace may hold rows of a sequence that is going away
    for (int l = 0; l < c.num_full_layers; l++)
        for (int s = s0; s < s1; s++) {
            int *tab = &ctx->h_page_table[((size_t)l * c.max_seqs + s) * ctx->max_slots];
            for (int i = 0; i < ctx->max_slots; i++)
                if (tab[i] >= 0) { release_page(ctx, tab[i]); tab[i] = -1; }
            ctx->kv_len[lidx(ctx, l, s)] = 0;
            if (c.h2o_budget > 0) {
                fm_status st = launched(ctx, launch_h2o_init(h2o_view(ctx, l), s, 0, ctx->stream), "h2o_init");
                if (st) return st;
            }
        }
    for (int l = 0; l < c.num_linear_layers; l++)
        for (int s = s0; s < s1; s++) {
            const size_t cn = (size_t)c.conv_kernel_size * ctx->conv_dim;
            const size_t sn = (size_t)c.linear_num_v_heads * c.linear_value_dim * c.linear_key_dim;
            FM_CUDA(ctx, cudaMemsetAsync(ctx->d_conv_state + lidx(ctx, l, s) * cn, 0, cn * sizeof(float), ctx->stream));
            FM_CUDA(ctx, cudaMemsetAsync(ctx->d_ssm_state + lidx(ctx, l, s) * sn, 0, sn * sizeof(float), ctx->stream));
            ctx->gdn_steps[lidx(ctx, l, s)] = 0;
        }
    return FM_OK;
}

extern "C" int64_t fm_kv_free_pages(const FmCtx *ctx) { return ctx ? (int64_t)ctx->free_pages.size() : -1; }

// dst becomes a copy of src without copying what cannot change: the full pages of src are shared by
// reference (appends never touch a full page), the partly filled last page and the recurrent state are
// copied.  Work is ordered on the context's stream.
extern "C" fm_status fm_seq_fork(FmCtx *ctx, int src, int dst) {
    if (!ctx) return FM_ERR_INVALID;
    const FmConfig &c = ctx->cfg;
    if (src < 0 || src >= c.max_seqs || dst < 0 || dst >= c.max_seqs || src == dst)
        return fail(ctx, FM_ERR_INVALID, "fm_seq_fork: sequences %d -> %d of %d", src, dst, c.max_seqs);
    if ((c.sliding_window > 0 || c.h2o_budget > 0) && c.num_full_layers > 0)
        return fail(ctx, FM_ERR_UNSUPPORTED, "fm_seq_fork: pages of a sliding-window or H2O store are rewritten in place and cannot be shared");
    // pages to copy: one per layer whose last local page is partly filled.  The demand is checked before dst is
    // touched (an error changes no state); the pages dst alone holds come back to the pool when it is reset.
    size_t need = 0, reclaim = 0;
    for (int l = 0; l < c.num_full_layers; l++) {
        const int len = ctx->kv_len[lidx(ctx, l, src)];
        const int gp = len / c.page_size;  // the partly filled global page, if any
        if (len % c.page_size != 0 && gp % c.seq_shard_count == c.seq_shard_rank) need++;
        const int *dtab = &ctx->h_page_table[((size_t)l * c.max_seqs + dst) * ctx->max_slots];
        for (int s = 0; s < ctx->max_slots; s++)
            if (dtab[s] >= 0 && ctx->page_refs[(size_t)dtab[s]] == 1) reclaim++;
    }
    if (need > ctx->free_pages.size() + reclaim)
        return fail(ctx, FM_ERR_CAPACITY, "KV page pool exhausted (%zu more pages needed, %zu free)", need, ctx->free_pages.size() + reclaim);
    fm_status st = fm_reset(ctx, dst);
    if (st) return st;
    const size_t page_bytes = ctx->page_bytes;
    for (int l = 0; l < c.num_full_layers; l++) {
        const int len = ctx->kv_len[lidx(ctx, l, src)];
        int *stab = &ctx->h_page_table[((size_t)l * c.max_seqs + src) * ctx->max_slots];
        int *dtab = &ctx->h_page_table[((size_t)l * c.max_seqs + dst) * ctx->max_slots];
        for (int s = 0; s < ctx->max_slots; s++) {
            if (stab[s] < 0) continue;
            const int gp = s * c.seq_shard_count + c.seq_shard_rank;
            if ((gp + 1) * c.page_size <= len) {
                dtab[s] = stab[s];
                ctx->page_refs[(size_t)stab[s]]++;
            } else if (gp * c.page_size < len) {
                dtab[s] = take_page(ctx);
                FM_CUDA(ctx, cudaMemcpyAsync(ctx->pool + (size_t)dtab[s] * page_bytes, ctx->pool + (size_t)stab[s] * page_bytes,
                                             page_bytes, cudaMemcpyDeviceToDevice, ctx->stream));
            }
        }
        FM_CUDA(ctx, cudaMemcpyAsync(ctx->d_page_table + ((size_t)l * c.max_seqs + dst) * ctx->max_slots, dtab,
                                     (size_t)ctx->max_slots * sizeof(int), cudaMemcpyHostToDevice, ctx->stream));
        ctx->kv_len[lidx(ctx, l, dst)] = len;
    }
    const size_t cn = (size_t)c.conv_kernel_size * ctx->conv_dim;
    const size_t sn = (size_t)c.linear_num_v_heads * c.linear_value_dim * c.linear_key_dim;
    for (int l = 0; l < c.num_linear_layers; l++) {
        FM_CUDA(ctx, cudaMemcpyAsync(ctx->d_conv_state + lidx(ctx, l, dst) * cn, ctx->d_conv_state + lidx(ctx, l, src) * cn,
                                     cn * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        FM_CUDA(ctx, cudaMemcpyAsync(ctx->d_ssm_state + lidx(ctx, l, dst) * sn, ctx->d_ssm_state + lidx(ctx, l, src) * sn,
                                     sn * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        ctx->gdn_steps[lidx(ctx, l, dst)] = ctx->gdn_steps[lidx(ctx, l, src)];
    }
    return FM_OK;
}

// ---- pointer-mode staging ---------------------------------------------------------------------
// In host-pointer mode inputs are packed into the pinned buffer, moved with one copy, and the
// kernels read the device twin; outputs come back the same way.
struct Stager {
    FmCtx *ctx;
    size_t off = 0;
    size_t in_end = 0;
    bool host;
    explicit Stager(FmCtx *c) : ctx(c), host(c->ptr_mode == FM_PTR_HOST) {}
    template <typename T>
    const T *in(const T *p, size_t count, bool *ok) {
        if (!host || p == nullptr) return p;
        const size_t bytes = (count * sizeof(T) + 255) & ~(size_t)255;
        if (off + bytes > ctx->stage_bytes) { *ok = false; return nullptr; }
        memcpy(ctx->h_stage + off, p, count * sizeof(T));
        const T *d = reinterpret_cast<const T *>(ctx->d_stage + off);
        off += bytes;
        in_end = off;
        return d;
    }
    cudaError_t push() {
        if (!host || in_end == 0) return cudaSuccess;
        return cudaMemcpyAsync(ctx->d_stage, ctx->h_stage, in_end, cudaMemcpyHostToDevice, ctx->stream);
    }
    template <typename T>
    T *out(T *p, size_t count, bool *ok, size_t *where) {
        if (!host || p == nullptr) return p;
        const size_t bytes = (count * sizeof(T) + 255) & ~(size_t)255;
        if (off + bytes > ctx->stage_bytes) { *ok = false; return nullptr; }
        *where = off;
        T *d = reinterpret_cast<T *>(ctx->d_stage + off);
        off += bytes;
        return d;
    }
    // device -> pinned -> caller; blocks until the data is in the caller's buffer
    template <typename T>
    cudaError_t pull(T *host_dst, size_t where, size_t count) {
        if (!host || host_dst == nullptr) return cudaSuccess;
        cudaError_t e = cudaMemcpyAsync(ctx->h_stage + where, ctx->d_stage + where, count * sizeof(T),
                                        cudaMemcpyDeviceToHost, ctx->stream);
        if (e != cudaSuccess) return e;
        e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return e;
        memcpy(host_dst, ctx->h_stage + where, count * sizeof(T));
        return cudaSuccess;
    }
};

// ---- token lists ------------------------------------------------------------------------------
static fm_status check_layer_seq(FmCtx *ctx, const char *fn, int layer, int nlayers, const int *seq, int n) {
    if (layer < 0 || layer >= nlayers) return fail(ctx, FM_ERR_INVALID, "%s: layer index %d of %d", fn, layer, nlayers);
    if (n < 0 || n > ctx->cfg.max_batch_tokens) return fail(ctx, FM_ERR_INVALID, "%s: n=%d exceeds max_batch_tokens=%d", fn, n, ctx->cfg.max_batch_tokens);
    for (int i = 0; i < n; i++)
        if (seq[i] < 0 || seq[i] >= ctx->cfg.max_seqs) return fail(ctx, FM_ERR_INVALID, "%s: seq[%d]=%d of %d", fn, i, seq[i], ctx->cfg.max_seqs);
    return FM_OK;
}

// Appends tokens [i0, i1) of an explicit list (bookkeeping already validated); k, v device pointers.
static fm_status append_list(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, const int *rows, int n,
                             const float *k, const float *v, const uint16_t *knw) {
    const KvView kv = kv_view(ctx, fa_idx);
    const size_t kv_dim = (size_t)ctx->cfg.num_kv_heads * ctx->cfg.head_dim;
    for (int i0 = 0; i0 < n; i0 += kMaxList) {
        TokSpec t;
        t.mode = 0;
        t.n = std::min(kMaxList, n - i0);
        for (int i = 0; i < t.n; i++) t.set(i, seq[i0 + i], pos[i0 + i], rows[i0 + i], rows[i0 + i] + 1);
        fm_status st = launched(ctx, launch_kv_append(kv, ctx->rope, t, k + i0 * kv_dim, v + i0 * kv_dim, knw, ctx->cfg.rms_norm_eps, ctx->stream), "kv_append");
        if (st) return st;
    }
    return FM_OK;
}

// Reserves rows for n tokens (token i goes to sequence seq[i]); fills rows[]. All-or-nothing.
// With a sliding window the row is the token count modulo the window and nothing ever overflows.
static fm_status reserve_rows(FmCtx *ctx, int fa_idx, const int *seq, int n, std::vector<int> &rows, std::vector<int> *nrows = nullptr) {
    const FmConfig &c = ctx->cfg;
    rows.resize(n);
    if (nrows) nrows->resize(n);
    std::vector<int> add(c.max_seqs, 0);
    for (int i = 0; i < n; i++) {
        const int count = ctx->kv_len[lidx(ctx, fa_idx, seq[i])] + add[seq[i]];
        add[seq[i]]++;
        if (c.sliding_window == 0 && c.h2o_budget == 0 && count >= c.max_seq_len)
            return fail(ctx, FM_ERR_CAPACITY, "KV cache overflow (pos=%d >= cap=%d)", count, c.max_seq_len);
        rows[i] = row_of(c, count);
        if (nrows) (*nrows)[i] = rows_held(c, count + 1);
    }
    // page demand check before touching anything
    size_t need = 0;
    for (int s = 0; s < c.max_seqs; s++) {
        if (!add[s]) continue;
        const int new_len = rows_held(c, ctx->kv_len[lidx(ctx, fa_idx, s)] + add[s]);
        const int gpages = (new_len + c.page_size - 1) / c.page_size;
        const int nslots = gpages > c.seq_shard_rank ? (gpages - c.seq_shard_rank + c.seq_shard_count - 1) / c.seq_shard_count : 0;
        const int *tab = &ctx->h_page_table[((size_t)fa_idx * c.max_seqs + s) * ctx->max_slots];
        for (int j = 0; j < nslots; j++) need += tab[j] < 0;
    }
    if (need > ctx->free_pages.size())
        return fail(ctx, FM_ERR_CAPACITY, "KV page pool exhausted (%zu more pages needed, %zu free)", need, ctx->free_pages.size());
    for (int s = 0; s < c.max_seqs; s++) {
        if (!add[s]) continue;
        fm_status st = ensure_pages(ctx, fa_idx, s, ctx->kv_len[lidx(ctx, fa_idx, s)] + add[s]);
        if (st) return st;
    }
    for (int s = 0; s < c.max_seqs; s++) ctx->kv_len[lidx(ctx, fa_idx, s)] += add[s];
    return FM_OK;
}

extern "C" fm_status fm_kv_append_rope(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int n,
                                       const float *k, const float *v, const uint16_t *k_norm_w) {
    if (!ctx) return FM_ERR_INVALID;
    if (!seq || !pos || !k || !v) return fail(ctx, FM_ERR_INVALID, "fm_kv_append_rope: null argument");
    fm_status st = check_layer_seq(ctx, "fm_kv_append_rope", fa_idx, ctx->cfg.num_full_layers, seq, n);
    if (st) return st;
    if (n == 0) return FM_OK;
    if (ctx->cfg.h2o_budget > 0)
        return fail(ctx, FM_ERR_UNSUPPORTED, "fm_kv_append_rope: with H2O eviction a row is appended by the decode step that attends to it");
    FM_CUDA(ctx, cudaSetDevice(ctx->cfg.device));
    const size_t kv_dim = (size_t)ctx->cfg.num_kv_heads * ctx->cfg.head_dim;
    Stager sg(ctx);
    bool ok = true;
    const float *dk = sg.in(k, n * kv_dim, &ok), *dv = sg.in(v, n * kv_dim, &ok);
    const uint16_t *dw = sg.in(k_norm_w, (size_t)ctx->cfg.head_dim, &ok);
    if (!ok) return fail(ctx, FM_ERR_INVALID, "fm_kv_append_rope: staging buffer too small");
    std::vector<int> rows;
    st = reserve_rows(ctx, fa_idx, seq, n, rows);
    if (st) return st;
    FM_CUDA(ctx, sg.push());
    st = append_list(ctx, fa_idx, seq, pos, rows.data(), n, dk, dv, dw);
    if (st) return st;
    if (sg.host) FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return FM_OK;
}

// Splits per (KV head, sequence): one CTA per SM is resident (shared memory), so the grid should be
// as close to the SM count as possible without exceeding it -- a few CTAs over would run as a
// second, nearly empty wave.
static int pick_splits(const FmCtx *ctx, int batch, int max_len, bool exchange = false) {
    const FmConfig &c = ctx->cfg;
    const int units = c.num_kv_heads * batch;
    int want = std::max(1, ctx->sm_count / units);
    const int gpages = (max_len + c.page_size - 1) / c.page_size;
    const int slots = (gpages + c.seq_shard_count - 1) / c.seq_shard_count;
    want = std::min(want, std::max(1, slots));
    if (ctx->overlap_layers) {
        // Launches of consecutive layers overlap.  When a full-width launch would be short (under ~64 tiles
        // per CTA) its start-up and merge tail are a large share of it and, holding every SM, it keeps the
        // next layer from starting: a quarter of the width with at least 8 tiles per CTA lets about four
        // layers stream side by side, each hiding the others' prologues and tails (batch 1: 17.6 -> 5.1 us
        // per layer at 4K, 48.9 -> 40.9 at 128K).  Long launches keep the full width.
        // With the peer exchange in the tail the launches complete in order, and a narrow launch whose CTAs
        // have to wait for their turn holds its SMs meanwhile: measured at batch 8 x 128K, full width is better
        // at 57 tiles per CTA (4 GPUs: 91 vs 101 us per layer), a quarter at 29 (8 GPUs: 56 vs 64).
        const int tiles_full = (slots + want - 1) / want;
        if (tiles_full < (exchange ? 40 : 64)) {
            const int full = want;
            want = std::max(1, std::min(want / 4, (slots + 7) / 8));
            // The CTAs of the call's layers fill the SMs in waves; a width whose CTA count over all layers just
            // misses a whole number of waves pays for a nearly empty one (8 GPUs, batch 8 x 128K: 15 layers x 32 CTAs
            // = 3.2 waves of 129 tiles cost 4; 48 CTAs per layer = 4.9 waves of 86 tiles cost 5: 55 -> 47 us per
            // layer expected).  Cost of a width: waves x (tiles per CTA + a CTA's fixed cost, about 6 tiles' time);
            // the quarter width stays unless another one is clearly cheaper.
            if (ctx->overlap_nlayers > 1 && batch >= 4) {
                auto cost = [&](int w) {
                    const long long ctas = (long long)ctx->overlap_nlayers * units * w;
                    const long long waves = (ctas + ctx->sm_count - 1) / ctx->sm_count;
                    return waves * ((slots + w - 1) / w + 6);
                };
                int best = want;
                for (int w = want + 1; w <= full; w++)
                    if ((slots + w - 1) / w >= 8 && cost(w) * 100 < cost(best) * 95) best = w;
                want = best;
            }
        }
    }
    want = std::min(want, kDecGroup * kDecMaxGroups);
    if (batch > ctx->dec_scr.group_tokens) want = std::min(want, kDecMaxLastCtaSplits);  // no second-level scratch for that many tokens
    return std::max(1, std::min(want, ctx->max_splits));
}

static inline bool sg_host(const FmCtx *ctx) { return ctx->ptr_mode == FM_PTR_HOST; }

// Scratch set of one full-attention layer.
struct LayerScratch {
    float *part_o, *part_ml;
    DecodeScratch scr;
};
static LayerScratch layer_scratch(const FmCtx *ctx, int fa_idx) {
    LayerScratch ls;
    const size_t s = (size_t)fa_idx, D = (size_t)ctx->cfg.head_dim;
    ls.part_o = ctx->d_part_o + s * ctx->part_rows * D;
    ls.part_ml = ctx->d_part_ml + s * ctx->part_rows * 2;
    ls.scr = ctx->dec_scr;
    ls.scr.counters += s * ctx->counter_stride;
    ls.scr.group_counters += s * ctx->group_counter_stride;
    ls.scr.group_o += s * ctx->group_rows * D;
    ls.scr.group_ml += s * ctx->group_rows * 2;
    return ls;
}

// Shared body of fm_attn_decode / fm_attn_decode_partial (device pointers).
static fm_status decode_core(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                             const float *q_proj_out, const float *q, const float *gate, const float *k,
                             const float *v, const uint16_t *qnw, const uint16_t *knw, float *out,
                             float *o_part, float *ml_part) {
    const FmConfig &c = ctx->cfg;
    const int H = c.num_attn_heads, D = c.head_dim;
    const bool h2o = c.h2o_budget > 0;
    if (h2o && (k == nullptr || out == nullptr))
        return fail(ctx, FM_ERR_UNSUPPORTED, "fm_attn_decode: with H2O eviction a step appends its row and produces the final output");
    std::vector<int> rows(batch), nrows(batch), tok_index(batch);
    for (int i = 0; i < batch; i++) tok_index[i] = ctx->kv_len[lidx(ctx, fa_idx, seq[i])];  // tokens seen before this one
    if (k != nullptr) {
        fm_status st = reserve_rows(ctx, fa_idx, seq, batch, rows, &nrows);  // pages and lengths; the kernel writes the rows
        if (st) return st;
    } else {
        for (int i = 0; i < batch; i++) {
            const int count = ctx->kv_len[lidx(ctx, fa_idx, seq[i])];
            if (count < 1) return fail(ctx, FM_ERR_INVALID, "fm_attn_decode: sequence %d is empty and no k/v given", seq[i]);
            rows[i] = row_of(c, count - 1);
            nrows[i] = rows_held(c, count);
        }
    }
    const KvView kv = kv_view(ctx, fa_idx);
    const size_t kvd = (size_t)c.num_kv_heads * D;
    for (int i0 = 0; i0 < batch; i0 += kMaxList) {
        TokSpec t;
        t.mode = 0;
        t.n = std::min(kMaxList, batch - i0);
        int max_len = 1;
        for (int i = 0; i < t.n; i++) {
            t.set(i, seq[i0 + i], pos[i0 + i], rows[i0 + i], nrows[i0 + i]);
            max_len = std::max(max_len, nrows[i0 + i]);
        }
        const int ns = pick_splits(ctx, t.n, max_len);
        const float *qp = q_proj_out ? q_proj_out + (size_t)i0 * H * 2 * D : nullptr;
        const float *qq = q ? q + (size_t)i0 * H * D : nullptr;
        const float *gp = gate ? gate + (size_t)i0 * H * D : nullptr;
        float *op = (out ? out : o_part) + (size_t)i0 * H * D;
        float *mlp = ml_part ? ml_part + (size_t)i0 * H * 2 : nullptr;
        // One launch: append of the new rows, split-KV attention, merge of the splits, gate.  When a sequence is split
        // over the whole machine (small batch) one CTA cannot merge all the parts quickly -- it would pull more than
        // a megabyte through a single SM -- so the launch stops at the parts (tail 0) and a merge launch with a CTA
        // per (head, token) follows as its programmatic dependent.
        ProfScope prof(ctx);
        const LayerScratch ls = layer_scratch(ctx, fa_idx);
        const bool wide = ns > kDecMaxLastCtaSplits;
        const H2oView hv = h2o ? h2o_view(ctx, fa_idx) : H2oView{};
        const H2oStep hstep = {hv.slot, ctx->d_h2o_w, ctx->d_h2o_mref, ctx->h2o_rows_pad, ctx->h2o_tiles};
        fm_status st = launched(ctx, launch_attn_decode_fused(kv, ctx->rope, t, H, qp, qq, qnw, c.rms_norm_eps, ls.part_o, ls.part_ml, ns,
                                                              k ? k + i0 * kvd : nullptr, v ? v + i0 * kvd : nullptr, knw, wide ? 0 : (out ? 1 : 2),
                                                              gp, op, h2o ? ctx->d_h2o_ml : mlp, nullptr, 0, ls.scr, ctx->d_err,
                                                              ctx->overlap_prev && i0 == 0 && !sg_host(ctx), ctx->stream, h2o ? &hstep : nullptr),
                                "attn_decode");
        if (st) return st;
        if (wide) {
            st = launched(ctx, launch_attn_merge_wide(ls.part_o, ls.part_ml, ns, t.n, H, qp, gp, op, mlp, ctx->stream, h2o ? ctx->d_h2o_ml : nullptr),
                          "attn_merge");
            if (st) return st;
        }
        if (h2o) {
            // the step's attention mass per cache row, and the eviction if the budget is exceeded (attn_h2o.cu)
            const int recent = (c.h2o_budget - c.h2o_num_sinks) / 4;  // kv_cache_new(), metal_infer/layer_forward.h:203
            st = launched(ctx, launch_h2o_mass(t, tok_index.data() + i0, hv, c.h2o_budget, c.h2o_num_sinks, recent, H, c.num_kv_heads, ctx->d_h2o_ml,
                                               hstep, ctx->d_h2o_cand, max_len, ctx->stream), "h2o_mass");
            if (st) return st;
        }
    }
    return FM_OK;
}

static fm_status decode_entry(FmCtx *ctx, const char *fn, int fa_idx, const int *seq, const int *pos, int batch,
                              const float *q_proj_out, const float *q, const float *gate, const float *k,
                              const float *v, const uint16_t *qnw, const uint16_t *knw, float *out, float *o_part,
                              float *ml_part) {
    if (!ctx) return FM_ERR_INVALID;
    const bool partial = o_part != nullptr;
    if (!seq || !pos || (!partial && !out) || (partial && !ml_part)) return fail(ctx, FM_ERR_INVALID, "%s: null argument", fn);
    if (!q_proj_out && (!q || (!partial && !gate))) return fail(ctx, FM_ERR_INVALID, "%s: give q_proj_out, or q and gate", fn);
    if ((k == nullptr) != (v == nullptr)) return fail(ctx, FM_ERR_INVALID, "%s: k and v go together", fn);
    fm_status st = check_layer_seq(ctx, fn, fa_idx, ctx->cfg.num_full_layers, seq, batch);
    if (st) return st;
    if (batch == 0) return FM_OK;
    for (int i = 0; i < batch; i++)
        for (int j = 0; j < i; j++)
            if (seq[i] == seq[j]) return fail(ctx, FM_ERR_INVALID, "%s: sequence %d appears twice in one step", fn, seq[i]);
    FM_CUDA(ctx, cudaSetDevice(ctx->cfg.device));
    const FmConfig &c = ctx->cfg;
    const size_t qd = (size_t)c.num_attn_heads * c.head_dim, kvd = (size_t)c.num_kv_heads * c.head_dim;
    Stager sg(ctx);
    bool ok = true;
    const float *d_qp = sg.in(q_proj_out, batch * qd * 2, &ok);
    const float *d_q = sg.in(q_proj_out ? nullptr : q, batch * qd, &ok);
    const float *d_g = sg.in(q_proj_out ? nullptr : gate, batch * qd, &ok);
    const float *d_k = sg.in(k, batch * kvd, &ok), *d_v = sg.in(v, batch * kvd, &ok);
    const uint16_t *d_qn = sg.in(qnw, (size_t)c.head_dim, &ok), *d_kn = sg.in(knw, (size_t)c.head_dim, &ok);
    size_t w_out = 0, w_ml = 0;
    float *d_out = sg.out(partial ? o_part : out, batch * qd, &ok, &w_out);
    float *d_ml = sg.out(ml_part, batch * (size_t)c.num_attn_heads * 2, &ok, &w_ml);
    if (!ok) return fail(ctx, FM_ERR_INVALID, "%s: staging buffer too small", fn);
    FM_CUDA(ctx, sg.push());
    st = decode_core(ctx, fa_idx, seq, pos, batch, d_qp, d_q, d_g, d_k, d_v, d_qn, d_kn, partial ? nullptr : d_out,
                     partial ? d_out : nullptr, d_ml);
    if (st) return st;
    if (sg.host) {
        if (partial) FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_stage + w_ml, ctx->d_stage + w_ml, batch * (size_t)c.num_attn_heads * 2 * 4, cudaMemcpyDeviceToHost, ctx->stream));
        FM_CUDA(ctx, sg.pull(partial ? o_part : out, w_out, batch * qd));
        if (partial) memcpy(ml_part, ctx->h_stage + w_ml, batch * (size_t)c.num_attn_heads * 2 * 4);
    }
    return FM_OK;
}

extern "C" fm_status fm_attn_decode(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                                    const float *q_proj_out, const float *q, const float *gate, const float *k,
                                    const float *v, const uint16_t *q_norm_w, const uint16_t *k_norm_w, float *out) {
    return decode_entry(ctx, "fm_attn_decode", fa_idx, seq, pos, batch, q_proj_out, q, gate, k, v, q_norm_w, k_norm_w, out, nullptr, nullptr);
}

extern "C" fm_status fm_attn_decode_partial(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                                            const float *q_proj_out, const float *q, const float *k, const float *v,
                                            const uint16_t *q_norm_w, const uint16_t *k_norm_w, float *o_part,
                                            float *ml_part) {
    if (ctx && !o_part) return fail(ctx, FM_ERR_INVALID, "fm_attn_decode_partial: null argument");
    return decode_entry(ctx, "fm_attn_decode_partial", fa_idx, seq, pos, batch, q_proj_out, q, nullptr, k, v, q_norm_w, k_norm_w, nullptr, o_part, ml_part);
}

extern "C" fm_status fm_attn_merge_gate(FmCtx *ctx, int nparts, const float *o_parts, const float *ml_parts,
                                        const float *q_proj_out, const float *gate, int batch, float *out) {
    if (!ctx) return FM_ERR_INVALID;
    if (!o_parts || !ml_parts || !out || (!q_proj_out && !gate) || nparts < 1) return fail(ctx, FM_ERR_INVALID, "fm_attn_merge_gate: bad argument");
    if (batch < 0 || (size_t)batch * nparts > (size_t)ctx->cfg.max_batch_tokens * 64) return fail(ctx, FM_ERR_INVALID, "fm_attn_merge_gate: batch %d", batch);
    if (batch == 0) return FM_OK;
    FM_CUDA(ctx, cudaSetDevice(ctx->cfg.device));
    const FmConfig &c = ctx->cfg;
    const int H = c.num_attn_heads, D = c.head_dim;
    const size_t qd = (size_t)H * D;
    Stager sg(ctx);
    bool ok = true;
    const float *d_o = sg.in(o_parts, (size_t)nparts * batch * qd, &ok);
    const float *d_ml = sg.in(ml_parts, (size_t)nparts * batch * H * 2, &ok);
    const float *d_qp = sg.in(q_proj_out, batch * qd * 2, &ok);
    const float *d_g = sg.in(q_proj_out ? nullptr : gate, batch * qd, &ok);
    size_t w_out = 0;
    float *d_out = sg.out(out, batch * qd, &ok, &w_out);
    if (!ok) return fail(ctx, FM_ERR_INVALID, "fm_attn_merge_gate: staging buffer too small");
    FM_CUDA(ctx, sg.push());
    fm_status st = launched(ctx, launch_attn_merge(d_o, d_ml, nparts, (long long)batch * qd, (long long)batch * H * 2, (long long)qd,
                                                   (long long)H * 2, D, 2, batch, H, D, d_qp, d_g, d_out, nullptr, ctx->stream), "attn_merge");
    if (st) return st;
    FM_CUDA(ctx, sg.pull(out, w_out, batch * qd));
    return FM_OK;
}

extern "C" fm_status fm_attn_prefill(FmCtx *ctx, int fa_idx, int seq, int start_pos, int n, const float *q_proj_out,
                                     const float *q, const float *gate, const float *k, const float *v,
                                     const uint16_t *q_norm_w, const uint16_t *k_norm_w, float *out) {
    if (!ctx) return FM_ERR_INVALID;
    if (!k || !v || !out || (!q_proj_out && (!q || !gate))) return fail(ctx, FM_ERR_INVALID, "fm_attn_prefill: null argument");
    const FmConfig &c = ctx->cfg;
    if (fa_idx < 0 || fa_idx >= c.num_full_layers || seq < 0 || seq >= c.max_seqs) return fail(ctx, FM_ERR_INVALID, "fm_attn_prefill: layer %d / seq %d", fa_idx, seq);
    if (n < 0 || n > c.max_batch_tokens) return fail(ctx, FM_ERR_INVALID, "fm_attn_prefill: n=%d exceeds max_batch_tokens=%d", n, c.max_batch_tokens);
    if (c.kv_dtype != FM_KV_BF16) return fail(ctx, FM_ERR_UNSUPPORTED, "fm_attn_prefill: the store is FP8; feed the prompt through fm_attn_decode");
    if (c.h2o_budget > 0) return fail(ctx, FM_ERR_UNSUPPORTED, "fm_attn_prefill: H2O eviction works per decode step; feed the prompt through fm_attn_decode");
    if (n == 0) return FM_OK;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const size_t qd = (size_t)c.num_attn_heads * c.head_dim, kvd = (size_t)c.num_kv_heads * c.head_dim;
    Stager sg(ctx);
    bool ok = true;
    const float *d_qp = sg.in(q_proj_out, n * qd * 2, &ok);
    const float *d_q = sg.in(q_proj_out ? nullptr : q, n * qd, &ok);
    const float *d_g = sg.in(q_proj_out ? nullptr : gate, n * qd, &ok);
    const float *d_k = sg.in(k, n * kvd, &ok), *d_v = sg.in(v, n * kvd, &ok);
    const uint16_t *d_qn = sg.in(q_norm_w, (size_t)c.head_dim, &ok), *d_kn = sg.in(k_norm_w, (size_t)c.head_dim, &ok);
    size_t w_out = 0;
    float *d_out = sg.out(out, n * qd, &ok, &w_out);
    if (!ok) return fail(ctx, FM_ERR_INVALID, "fm_attn_prefill: staging buffer too small");
    const int row0 = ctx->kv_len[lidx(ctx, fa_idx, seq)];
    // Sequence-sharded store: every rank of the sequence group is given the run's k and v (they belong to its KV-head
    // group), keeps the rows of the pages it owns and attends over the whole sequence out of its operand workspace,
    // which holds every row that came through fm_attn_prefill.  Rows that came another way (decode steps, imports)
    // sit on their owners only and are not in the workspace.
    if (c.seq_shard_count != 1 && row0 > 0 && !(ctx->pf_layer == fa_idx && ctx->pf_seq == seq && ctx->pf_rows == row0))
        return fail(ctx, FM_ERR_UNSUPPORTED, "fm_attn_prefill: on a sequence-sharded store a prompt has to go through consecutive "
                    "fm_attn_prefill calls of one (layer, sequence), from its first token (%d rows are cached, %d of them in reach)", row0,
                    ctx->pf_layer == fa_idx && ctx->pf_seq == seq ? ctx->pf_rows : 0);
    if (c.sliding_window > 0 && row0 + n > c.sliding_window)
        return fail(ctx, FM_ERR_UNSUPPORTED, "fm_attn_prefill: the run would wrap the sliding window (%d + %d > %d); feed it through fm_attn_decode", row0, n, c.sliding_window);
    if (row0 + n > c.max_seq_len) return fail(ctx, FM_ERR_CAPACITY, "KV cache overflow (pos=%d >= cap=%d)", row0 + n - 1, c.max_seq_len);
    fm_status st = ensure_pages(ctx, fa_idx, seq, row0 + n);
    if (st) return st;
    ctx->kv_len[lidx(ctx, fa_idx, seq)] = row0 + n;
    FM_CUDA(ctx, sg.push());
    const KvView kv = kv_view(ctx, fa_idx);
    {
        // two launches: operand preparation (which is also the append), then the attention kernel
        ProfScope prof(ctx);
        const PrefillWork wk{ctx->d_pf_q16, ctx->d_pf_k16, ctx->d_pf_v16, ctx->d_err};
        const int prefix0 = (ctx->pf_layer == fa_idx && ctx->pf_seq == seq && ctx->pf_rows <= row0) ? ctx->pf_rows : 0;
        ctx->pf_layer = -1;
        st = launched(ctx, launch_attn_prefill(kv, ctx->rope, seq, start_pos, row0, prefix0, n, c.num_attn_heads, d_qp, d_q, d_g, d_k, d_v, d_qn,
                                               d_kn, c.rms_norm_eps, wk, d_out, ctx->stream), "attn_prefill");
        if (st == FM_OK) { ctx->pf_layer = fa_idx; ctx->pf_seq = seq; ctx->pf_rows = row0 + n; }
    }
    if (st) return st;
    if (sg.host) FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    FM_CUDA(ctx, sg.pull(out, w_out, n * qd));
    if (sg.host) return check_device_error(ctx);
    return FM_OK;
}

// ---- output projection + residual + post-attention norm ---------------------------------------
extern "C" fm_status fm_proj_upload(FmCtx *ctx, const FmProjWeights *h, FmProjWeights *d) {
    if (!ctx) return FM_ERR_INVALID;
    if (!h || !d || !h->w || !h->scales || !h->biases) return fail(ctx, FM_ERR_INVALID, "fm_proj_upload: null argument");
    if (h->format != FM_W_Q4_AFFINE || h->group_size != 64 || h->out_dim < 1 || h->in_dim < 64 || h->in_dim % 64)
        return fail(ctx, FM_ERR_UNSUPPORTED, "fm_proj_upload: format %d, group size %d, %d x %d", h->format, h->group_size, h->out_dim, h->in_dim);
    FM_CUDA(ctx, cudaSetDevice(ctx->cfg.device));
    const size_t wb = (size_t)h->out_dim * (h->in_dim / 8) * 4, sb = (size_t)h->out_dim * (h->in_dim / 64) * 2;
    char *buf = nullptr;
    const size_t o_s = (wb + 255) & ~(size_t)255, o_b = o_s + ((sb + 255) & ~(size_t)255);
    cudaError_t e = cudaMalloc(&buf, o_b + sb);
    if (e != cudaSuccess) return fail(ctx, FM_ERR_NOMEM, "fm_proj_upload: %s", cudaGetErrorString(e));
    if ((e = cudaMemcpyAsync(buf, h->w, wb, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess ||
        (e = cudaMemcpyAsync(buf + o_s, h->scales, sb, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess ||
        (e = cudaMemcpyAsync(buf + o_b, h->biases, sb, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess ||
        (e = cudaStreamSynchronize(ctx->stream)) != cudaSuccess) {
        cudaFree(buf);
        return fail(ctx, FM_ERR_CUDA, "fm_proj_upload: %s", cudaGetErrorString(e));
    }
    *d = *h;
    d->w = reinterpret_cast<const uint32_t *>(buf);
    d->scales = reinterpret_cast<const uint16_t *>(buf + o_s);
    d->biases = reinterpret_cast<const uint16_t *>(buf + o_b);
    return FM_OK;
}

extern "C" void fm_proj_free(FmCtx *ctx, FmProjWeights *d) {
    if (!ctx || !d || !d->w) return;
    cudaSetDevice(ctx->cfg.device);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(const_cast<uint32_t *>(d->w));  // one allocation holds all three arrays
    d->w = nullptr; d->scales = d->biases = nullptr;
}

extern "C" fm_status fm_out_proj_norm(FmCtx *ctx, const FmProjWeights *w, int n, const float *x, const float *residual,
                                      const uint16_t *norm_w, float *h_mid, float *h_post) {
    if (!ctx) return FM_ERR_INVALID;
    if (!w || !w->w || !w->scales || !w->biases || !x || !h_mid || n < 0) return fail(ctx, FM_ERR_INVALID, "fm_out_proj_norm: null argument");
    if (w->format != FM_W_Q4_AFFINE || w->group_size != 64 || w->in_dim % 512 || w->out_dim < 1 || w->in_dim < 512 || w->in_dim > 24576 || w->out_dim % 4)
        return fail(ctx, FM_ERR_UNSUPPORTED, "fm_out_proj_norm: format %d, group size %d, %d x %d (in a multiple of 512 up to 24576, out of 4)",
                    w->format, w->group_size, w->out_dim, w->in_dim);
    if (n == 0) return FM_OK;
    FM_CUDA(ctx, cudaSetDevice(ctx->cfg.device));
    const size_t in = (size_t)w->in_dim, out = (size_t)w->out_dim;
    for (int t0 = 0; t0 < n; t0 += 8) {  // 8 tokens ride along one pass over the weights
        const int m = std::min(8, n - t0);
        Stager sg(ctx);
        bool ok = true;
        const float *d_x = sg.in(x + t0 * in, m * in, &ok);
        const float *d_r = sg.in(residual ? residual + t0 * out : nullptr, m * out, &ok);
        const uint16_t *d_w = sg.in(norm_w, out, &ok);
        size_t w_mid = 0, w_post = 0;
        float *d_mid = sg.out(h_mid + t0 * out, m * out, &ok, &w_mid);
        float *d_post = sg.out(h_post ? h_post + t0 * out : nullptr, m * out, &ok, &w_post);
        if (!ok) return fail(ctx, FM_ERR_INVALID, "fm_out_proj_norm: staging buffer too small (raise max_batch_tokens)");
        FM_CUDA(ctx, sg.push());
        fm_status st = launched(ctx, launch_out_proj_q4(w->w, w->scales, w->biases, w->out_dim, w->in_dim, m, d_x, d_r, d_w, ctx->cfg.rms_norm_eps,
                                                        d_mid, d_post, ctx->d_proj_ssq, &ctx->proj_parity, ctx->stream), "out_proj");
        if (st) return st;
        if (sg.host && h_post) FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_stage + w_post, ctx->d_stage + w_post, m * out * 4, cudaMemcpyDeviceToHost, ctx->stream));
        FM_CUDA(ctx, sg.pull(h_mid + t0 * out, w_mid, m * out));
        if (sg.host && h_post) memcpy(h_post + t0 * out, ctx->h_stage + w_post, m * out * 4);
    }
    return FM_OK;
}

// ---- GatedDeltaNet ----------------------------------------------------------------------------
static GdnDims gdn_dims(const FmCtx *ctx) {
    const FmConfig &c = ctx->cfg;
    return GdnDims{c.linear_num_v_heads, c.linear_num_k_heads, c.linear_key_dim, c.linear_value_dim, c.conv_kernel_size, ctx->conv_dim, c.rms_norm_eps};
}

// (head, sequence) pairs per launch from which the GatedDeltaNet step takes its persistent form; FM_GDN_STREAM_MIN_PAIRS
// overrides it (a very large value keeps the cluster kernel everywhere)
static int gdn_stream_min_pairs() {
    static const int v = [] {
        const char *e = getenv("FM_GDN_STREAM_MIN_PAIRS");
        return e && *e ? atoi(e) : 512;
    }();
    return v;
}

extern "C" fm_status fm_gdn_decode(FmCtx *ctx, int li, const int *seq, int batch, const float *qkv, const float *z,
                                   const float *beta, const float *alpha, const uint16_t *conv_w, const float *A_log,
                                   const uint16_t *dt_bias, const uint16_t *norm_w, float *out) {
    if (!ctx) return FM_ERR_INVALID;
    if (!seq || !qkv || !z || !beta || !alpha || !out) return fail(ctx, FM_ERR_INVALID, "fm_gdn_decode: null argument");
    fm_status st = check_layer_seq(ctx, "fm_gdn_decode", li, ctx->cfg.num_linear_layers, seq, batch);
    if (st) return st;
    if (batch == 0) return FM_OK;
    for (int i = 0; i < batch; i++)
        for (int j = 0; j < i; j++)
            if (seq[i] == seq[j]) return fail(ctx, FM_ERR_INVALID, "fm_gdn_decode: sequence %d appears twice in one step", seq[i]);
    const FmConfig &c = ctx->cfg;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const size_t vd = (size_t)c.linear_num_v_heads * c.linear_value_dim, hv = (size_t)c.linear_num_v_heads;
    Stager sg(ctx);
    bool ok = true;
    const float *d_qkv = sg.in(qkv, (size_t)batch * ctx->conv_dim, &ok), *d_z = sg.in(z, batch * vd, &ok);
    const float *d_b = sg.in(beta, batch * hv, &ok), *d_a = sg.in(alpha, batch * hv, &ok);
    const uint16_t *d_cw = sg.in(conv_w, (size_t)ctx->conv_dim * c.conv_kernel_size, &ok);
    const float *d_al = sg.in(A_log, hv, &ok);
    const uint16_t *d_db = sg.in(dt_bias, hv, &ok), *d_nw = sg.in(norm_w, (size_t)c.linear_value_dim, &ok);
    size_t w_out = 0;
    float *d_out = sg.out(out, batch * vd, &ok, &w_out);
    if (!ok) return fail(ctx, FM_ERR_INVALID, "fm_gdn_decode: staging buffer too small");
    FM_CUDA(ctx, sg.push());
    const size_t cn = (size_t)c.conv_kernel_size * ctx->conv_dim, sn = vd * c.linear_key_dim;
    const GdnDims g = gdn_dims(ctx);
    for (int i0 = 0; i0 < batch; i0 += kMaxList) {
        TokSpec t;
        t.mode = 0;
        t.n = std::min(kMaxList, batch - i0);
        for (int i = 0; i < t.n; i++) {
            t.set(i, seq[i0 + i], ctx->gdn_steps[lidx(ctx, li, seq[i0 + i])], 0, 0);
        }
        ProfScope prof(ctx);
        float *conv_l = ctx->d_conv_state + (size_t)li * c.max_seqs * cn, *ssm_l = ctx->d_ssm_state + (size_t)li * c.max_seqs * sn;
        // several (head, sequence) pairs per SM: the persistent form that streams the states; else one CTA cluster per pair
        const bool stream = ctx->d_gdn_scratch != nullptr && g.Hv * t.n >= gdn_stream_min_pairs() && ((uintptr_t)(d_z + i0 * vd) & 15) == 0;
        if (stream)
            st = launched(ctx, launch_gdn_decode_stream(g, t, conv_l, ssm_l, (long long)cn, (long long)sn, d_qkv + (size_t)i0 * ctx->conv_dim,
                                                        d_z + i0 * vd, d_b + i0 * hv, d_a + i0 * hv, d_cw, d_al, d_db, d_nw, d_out + i0 * vd,
                                                        ctx->d_gdn_scratch, ctx->sm_count, ctx->d_err, ctx->stream), "gdn_decode_stream");
        else
            st = launched(ctx, launch_gdn_decode(g, t, conv_l, ssm_l, (long long)cn, (long long)sn, d_qkv + (size_t)i0 * ctx->conv_dim, d_z + i0 * vd,
                                                 d_b + i0 * hv, d_a + i0 * hv, d_cw, d_al, d_db, d_nw, d_out + i0 * vd,
                                                 // not behind a step of the same layer, nor behind a prefill, import or reset
                                                 ctx->layer_overlap && !sg.host && ctx->last_state_li >= 0 && ctx->last_state_li != li,
                                                 ctx->stream), "gdn_decode");
        if (st) return st;
        for (int i = 0; i < t.n; i++) ctx->gdn_steps[lidx(ctx, li, seq[i0 + i])]++;  // only once the step is queued
        ctx->last_state_li = li;
    }
    if (sg.host) FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    FM_CUDA(ctx, sg.pull(out, w_out, batch * vd));
    if (sg.host) return check_device_error(ctx);
    return FM_OK;
}

extern "C" fm_status fm_gdn_prefill(FmCtx *ctx, int li, int seq, int n, int chunk, const float *qkv, const float *z,
                                    const float *beta, const float *alpha, const uint16_t *conv_w, const float *A_log,
                                    const uint16_t *dt_bias, const uint16_t *norm_w, float *out) {
    if (!ctx) return FM_ERR_INVALID;
    ctx->last_state_li = -1;  // the next GatedDeltaNet step is not launched under this call's tail
    if (!qkv || !z || !beta || !alpha || !out) return fail(ctx, FM_ERR_INVALID, "fm_gdn_prefill: null argument");
    const FmConfig &c = ctx->cfg;
    if (li < 0 || li >= c.num_linear_layers || seq < 0 || seq >= c.max_seqs) return fail(ctx, FM_ERR_INVALID, "fm_gdn_prefill: layer %d / seq %d", li, seq);
    if (n < 0 || n > c.max_batch_tokens) return fail(ctx, FM_ERR_INVALID, "fm_gdn_prefill: n=%d exceeds max_batch_tokens=%d", n, c.max_batch_tokens);
    if (chunk == 0) chunk = 64;
    if (chunk != 64) return fail(ctx, FM_ERR_UNSUPPORTED, "fm_gdn_prefill: chunk %d (built for 64)", chunk);
    if (n == 0) return FM_OK;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const size_t vd = (size_t)c.linear_num_v_heads * c.linear_value_dim, hv = (size_t)c.linear_num_v_heads;
    Stager sg(ctx);
    bool ok = true;
    const float *d_qkv = sg.in(qkv, (size_t)n * ctx->conv_dim, &ok), *d_z = sg.in(z, n * vd, &ok);
    const float *d_b = sg.in(beta, n * hv, &ok), *d_a = sg.in(alpha, n * hv, &ok);
    const uint16_t *d_cw = sg.in(conv_w, (size_t)ctx->conv_dim * c.conv_kernel_size, &ok);
    const float *d_al = sg.in(A_log, hv, &ok);
    const uint16_t *d_db = sg.in(dt_bias, hv, &ok), *d_nw = sg.in(norm_w, (size_t)c.linear_value_dim, &ok);
    size_t w_out = 0;
    float *d_out = sg.out(out, n * vd, &ok, &w_out);
    if (!ok) return fail(ctx, FM_ERR_INVALID, "fm_gdn_prefill: staging buffer too small");
    FM_CUDA(ctx, sg.push());
    const size_t cn = (size_t)c.conv_kernel_size * ctx->conv_dim, sn = vd * c.linear_key_dim;
    GdnDims g = gdn_dims(ctx);
    const int step0 = ctx->gdn_steps[lidx(ctx, li, seq)];
    fm_status st;
    {
        ProfScope prof(ctx);
        st = launched(ctx, launch_gdn_prefill(g, n, chunk, step0, ctx->d_conv_state + lidx(ctx, li, seq) * cn, ctx->d_ssm_state + lidx(ctx, li, seq) * sn,
                                                    d_qkv, d_z, d_b, d_a, d_cw, d_al, d_db, d_nw, d_out, ctx->d_work, ctx->work_bytes, ctx->d_err, ctx->stream), "gdn_prefill");
    }
    if (st) return st;
    ctx->gdn_steps[lidx(ctx, li, seq)] = step0 + n;
    FM_CUDA(ctx, sg.pull(out, w_out, n * vd));
    return FM_OK;
}

// ---- snapshot / restore -----------------------------------------------------------------------
// Host-pointer mode moves the rows through the context's own staging pair in chunks (no allocation per call:
// the reference takes and restores this snapshot per request, metal_infer/generate.h:897-939).
template <typename Row>  // Row(row0, n, d_k, d_v, d_ks, d_vs, h_k, h_v, h_ks, h_vs, to_device) handles one chunk
static fm_status staged_rows(FmCtx *ctx, int len, size_t row_bytes_each, bool with_scales, Row chunk_fn) {
    // staging layout per chunk of n rows: k | v | k_scales | v_scales
    const size_t per_row = 2 * row_bytes_each + (with_scales ? 8 : 0);
    const int chunk = (int)std::min<size_t>((size_t)len, std::max<size_t>(1, (ctx->stage_bytes - 1024) / per_row));
    for (int row0 = 0; row0 < len; row0 += chunk) {
        const int n = std::min(chunk, len - row0);
        const size_t o_v = ((size_t)n * row_bytes_each + 255) & ~(size_t)255, o_ks = 2 * o_v, o_vs = o_ks + (((size_t)n * 4 + 255) & ~(size_t)255);
        const fm_status st = chunk_fn(row0, n, o_v, o_ks, o_vs);
        if (st) return st;
    }
    return FM_OK;
}

static fm_status kv_export_check(FmCtx *ctx, const char *fn, int fa_idx, int seq, bool ptrs_ok, int max_rows, int *len_out, int *len) {
    const FmConfig &c = ctx->cfg;
    if (fa_idx < 0 || fa_idx >= c.num_full_layers || seq < 0 || seq >= c.max_seqs || !ptrs_ok)
        return fail(ctx, FM_ERR_INVALID, "%s: bad argument", fn);
    *len = rows_kept(c, ctx->kv_len[lidx(ctx, fa_idx, seq)]);  // rows in store order (a wrapped window is not unrolled)
    if (len_out) *len_out = *len;
    if (*len > max_rows) return fail(ctx, FM_ERR_INVALID, "%s: %d rows held, room for %d", fn, *len, max_rows);
    return FM_OK;
}

// The cache order of an H2O store is rebuilt from the token positions when something is exported (attn_h2o.cu).
static fm_status h2o_refresh_order(FmCtx *ctx, int fa_idx, int seq) {
    if (ctx->cfg.h2o_budget <= 0) return FM_OK;
    return launched(ctx, launch_h2o_order(h2o_view(ctx, fa_idx), seq, rows_held(ctx->cfg, ctx->kv_len[lidx(ctx, fa_idx, seq)]), ctx->stream),
                    "h2o_order");
}

extern "C" fm_status fm_kv_export(FmCtx *ctx, int fa_idx, int seq, float *k, float *v, int max_rows, int *len_out) {
    if (!ctx) return FM_ERR_INVALID;
    const FmConfig &c = ctx->cfg;
    int len = 0;
    fm_status st = kv_export_check(ctx, "fm_kv_export", fa_idx, seq, k && v, max_rows, len_out, &len);
    if (st || len == 0) return st;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const size_t kvd = (size_t)c.num_kv_heads * c.head_dim;
    const KvView kv = kv_view(ctx, fa_idx);
    const int *order = c.h2o_budget > 0 ? h2o_view(ctx, fa_idx).order + (size_t)seq * ctx->h2o_cap : nullptr;  // cache order of an H2O store
    if ((st = h2o_refresh_order(ctx, fa_idx, seq)) != FM_OK) return st;
    if (ctx->ptr_mode == FM_PTR_DEVICE)
        return launched(ctx, launch_kv_export(kv, seq, 0, len, k, v, order, ctx->stream), "kv_export");
    return staged_rows(ctx, len, kvd * 4, false, [&](int row0, int n, size_t o_v, size_t, size_t) -> fm_status {
        float *dk = reinterpret_cast<float *>(ctx->d_stage), *dv = reinterpret_cast<float *>(ctx->d_stage + o_v);
        // rows another shard holds are left alone in the caller's arrays: start from what is there
        memcpy(ctx->h_stage, k + (size_t)row0 * kvd, (size_t)n * kvd * 4);
        memcpy(ctx->h_stage + o_v, v + (size_t)row0 * kvd, (size_t)n * kvd * 4);
        FM_CUDA(ctx, cudaMemcpyAsync(ctx->d_stage, ctx->h_stage, o_v + (size_t)n * kvd * 4, cudaMemcpyHostToDevice, ctx->stream));
        const fm_status s2 = launched(ctx, launch_kv_export(kv, seq, row0, n, dk, dv, order, ctx->stream), "kv_export");
        if (s2) return s2;
        FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_stage, ctx->d_stage, o_v + (size_t)n * kvd * 4, cudaMemcpyDeviceToHost, ctx->stream));
        FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        memcpy(k + (size_t)row0 * kvd, ctx->h_stage, (size_t)n * kvd * 4);
        memcpy(v + (size_t)row0 * kvd, ctx->h_stage + o_v, (size_t)n * kvd * 4);
        return FM_OK;
    });
}

// Drops the sequence's pages of one layer (some may be shared with a fork and must not be overwritten) and takes
// fresh ones for `len` rows -- after checking that the pool, with the pages this sequence alone holds, covers the
// demand, so that an error changes nothing.
static fm_status kv_import_prepare(FmCtx *ctx, const char *fn, int fa_idx, int seq, bool ptrs_ok, int len) {
    const FmConfig &c = ctx->cfg;
    if (fa_idx < 0 || fa_idx >= c.num_full_layers || seq < 0 || seq >= c.max_seqs || len < 0 || (len > 0 && !ptrs_ok))
        return fail(ctx, FM_ERR_INVALID, "%s: bad argument", fn);
    if (len > c.max_seq_len) return fail(ctx, FM_ERR_CAPACITY, "KV cache overflow (pos=%d >= cap=%d)", len - 1, c.max_seq_len);
    if (c.sliding_window > 0 && len > c.sliding_window)
        return fail(ctx, FM_ERR_INVALID, "%s: %d rows do not fit the sliding window of %d", fn, len, c.sliding_window);
    if (c.h2o_budget > 0 && len > c.h2o_budget)
        return fail(ctx, FM_ERR_INVALID, "%s: %d rows exceed the H2O budget of %d", fn, len, c.h2o_budget);
    FM_CUDA(ctx, cudaSetDevice(c.device));
    ctx->pf_layer = -1;
    int *tab = &ctx->h_page_table[((size_t)fa_idx * c.max_seqs + seq) * ctx->max_slots];
    size_t reclaim = 0;
    for (int i = 0; i < ctx->max_slots; i++)
        if (tab[i] >= 0 && ctx->page_refs[(size_t)tab[i]] == 1) reclaim++;
    const int gpages = (rows_held(c, len) + c.page_size - 1) / c.page_size;
    const size_t need = gpages > c.seq_shard_rank ? (size_t)(gpages - c.seq_shard_rank + c.seq_shard_count - 1) / c.seq_shard_count : 0;
    if (need > ctx->free_pages.size() + reclaim)
        return fail(ctx, FM_ERR_CAPACITY, "KV page pool exhausted (%zu pages needed, %zu free)", need, ctx->free_pages.size() + reclaim);
    for (int i = 0; i < ctx->max_slots; i++)
        if (tab[i] >= 0) { release_page(ctx, tab[i]); tab[i] = -1; }
    fm_status st = ensure_pages(ctx, fa_idx, seq, len);
    if (st) return st;
    ctx->kv_len[lidx(ctx, fa_idx, seq)] = len;
    if (c.h2o_budget > 0) {  // imported rows start in their own order, with no mass yet
        st = launched(ctx, launch_h2o_init(h2o_view(ctx, fa_idx), seq, len, ctx->stream), "h2o_init");
        if (st) return st;
    }
    return FM_OK;
}

extern "C" fm_status fm_kv_import(FmCtx *ctx, int fa_idx, int seq, const float *k, const float *v, int len) {
    if (!ctx) return FM_ERR_INVALID;
    const FmConfig &c = ctx->cfg;
    fm_status st = kv_import_prepare(ctx, "fm_kv_import", fa_idx, seq, k && v, len);
    if (st || len == 0) return st;
    const size_t kvd = (size_t)c.num_kv_heads * c.head_dim;
    const KvView kv = kv_view(ctx, fa_idx);
    if (ctx->ptr_mode == FM_PTR_DEVICE)
        return launched(ctx, launch_kv_import(kv, seq, 0, len, k, v, ctx->stream), "kv_import");
    return staged_rows(ctx, len, kvd * 4, false, [&](int row0, int n, size_t o_v, size_t, size_t) -> fm_status {
        memcpy(ctx->h_stage, k + (size_t)row0 * kvd, (size_t)n * kvd * 4);
        memcpy(ctx->h_stage + o_v, v + (size_t)row0 * kvd, (size_t)n * kvd * 4);
        FM_CUDA(ctx, cudaMemcpyAsync(ctx->d_stage, ctx->h_stage, o_v + (size_t)n * kvd * 4, cudaMemcpyHostToDevice, ctx->stream));
        const fm_status s2 = launched(ctx, launch_kv_import(kv, seq, row0, n, reinterpret_cast<const float *>(ctx->d_stage),
                                                            reinterpret_cast<const float *>(ctx->d_stage + o_v), ctx->stream), "kv_import");
        if (s2) return s2;
        FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the staging pair is reused by the next chunk
        return FM_OK;
    });
}

extern "C" fm_status fm_kv_export_fp8(FmCtx *ctx, int fa_idx, int seq, uint8_t *k8, uint8_t *v8, float *k_scales, float *v_scales,
                                      int max_rows, int *len_out) {
    if (!ctx) return FM_ERR_INVALID;
    const FmConfig &c = ctx->cfg;
    if (c.kv_dtype != FM_KV_FP8_E4M3) return fail(ctx, FM_ERR_INVALID, "fm_kv_export_fp8: the store is not FP8");
    int len = 0;
    fm_status st = kv_export_check(ctx, "fm_kv_export_fp8", fa_idx, seq, k8 && v8 && k_scales && v_scales, max_rows, len_out, &len);
    if (st || len == 0) return st;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const size_t kvd = (size_t)c.num_kv_heads * c.head_dim;
    const KvView kv = kv_view(ctx, fa_idx);
    const int *order = c.h2o_budget > 0 ? h2o_view(ctx, fa_idx).order + (size_t)seq * ctx->h2o_cap : nullptr;
    if ((st = h2o_refresh_order(ctx, fa_idx, seq)) != FM_OK) return st;
    if (ctx->ptr_mode == FM_PTR_DEVICE)
        return launched(ctx, launch_kv_copy_fp8(kv, seq, 0, len, k8, v8, k_scales, v_scales, false, order, ctx->stream), "kv_export_fp8");
    return staged_rows(ctx, len, kvd, true, [&](int row0, int n, size_t o_v, size_t o_ks, size_t o_vs) -> fm_status {
        char *hs = ctx->h_stage, *ds = ctx->d_stage;
        memcpy(hs, k8 + (size_t)row0 * kvd, (size_t)n * kvd);
        memcpy(hs + o_v, v8 + (size_t)row0 * kvd, (size_t)n * kvd);
        memcpy(hs + o_ks, k_scales + row0, (size_t)n * 4);
        memcpy(hs + o_vs, v_scales + row0, (size_t)n * 4);
        FM_CUDA(ctx, cudaMemcpyAsync(ds, hs, o_vs + (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
        const fm_status s2 = launched(ctx, launch_kv_copy_fp8(kv, seq, row0, n, reinterpret_cast<uint8_t *>(ds), reinterpret_cast<uint8_t *>(ds + o_v),
                                                              reinterpret_cast<float *>(ds + o_ks), reinterpret_cast<float *>(ds + o_vs), false,
                                                              order, ctx->stream), "kv_export_fp8");
        if (s2) return s2;
        FM_CUDA(ctx, cudaMemcpyAsync(hs, ds, o_vs + (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        memcpy(k8 + (size_t)row0 * kvd, hs, (size_t)n * kvd);
        memcpy(v8 + (size_t)row0 * kvd, hs + o_v, (size_t)n * kvd);
        memcpy(k_scales + row0, hs + o_ks, (size_t)n * 4);
        memcpy(v_scales + row0, hs + o_vs, (size_t)n * 4);
        return FM_OK;
    });
}

extern "C" fm_status fm_kv_import_fp8(FmCtx *ctx, int fa_idx, int seq, const uint8_t *k8, const uint8_t *v8, const float *k_scales,
                                      const float *v_scales, int len) {
    if (!ctx) return FM_ERR_INVALID;
    const FmConfig &c = ctx->cfg;
    if (c.kv_dtype != FM_KV_FP8_E4M3) return fail(ctx, FM_ERR_INVALID, "fm_kv_import_fp8: the store is not FP8");
    fm_status st = kv_import_prepare(ctx, "fm_kv_import_fp8", fa_idx, seq, k8 && v8 && k_scales && v_scales, len);
    if (st || len == 0) return st;
    const size_t kvd = (size_t)c.num_kv_heads * c.head_dim;
    const KvView kv = kv_view(ctx, fa_idx);
    if (ctx->ptr_mode == FM_PTR_DEVICE)
        return launched(ctx, launch_kv_copy_fp8(kv, seq, 0, len, const_cast<uint8_t *>(k8), const_cast<uint8_t *>(v8), const_cast<float *>(k_scales),
                                                const_cast<float *>(v_scales), true, nullptr, ctx->stream), "kv_import_fp8");
    return staged_rows(ctx, len, kvd, true, [&](int row0, int n, size_t o_v, size_t o_ks, size_t o_vs) -> fm_status {
        char *hs = ctx->h_stage, *ds = ctx->d_stage;
        memcpy(hs, k8 + (size_t)row0 * kvd, (size_t)n * kvd);
        memcpy(hs + o_v, v8 + (size_t)row0 * kvd, (size_t)n * kvd);
        memcpy(hs + o_ks, k_scales + row0, (size_t)n * 4);
        memcpy(hs + o_vs, v_scales + row0, (size_t)n * 4);
        FM_CUDA(ctx, cudaMemcpyAsync(ds, hs, o_vs + (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
        const fm_status s2 = launched(ctx, launch_kv_copy_fp8(kv, seq, row0, n, reinterpret_cast<uint8_t *>(ds), reinterpret_cast<uint8_t *>(ds + o_v),
                                                              reinterpret_cast<float *>(ds + o_ks), reinterpret_cast<float *>(ds + o_vs), true,
                                                              nullptr, ctx->stream), "kv_import_fp8");
        if (s2) return s2;
        FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return FM_OK;
    });
}

extern "C" fm_status fm_h2o_export(FmCtx *ctx, int fa_idx, int seq, float *accum, int *token_positions, int max_rows, int *n_out) {
    if (!ctx) return FM_ERR_INVALID;
    const FmConfig &c = ctx->cfg;
    if (c.h2o_budget <= 0) return fail(ctx, FM_ERR_INVALID, "fm_h2o_export: H2O eviction is off");
    if (fa_idx < 0 || fa_idx >= c.num_full_layers || seq < 0 || seq >= c.max_seqs) return fail(ctx, FM_ERR_INVALID, "fm_h2o_export: bad argument");
    const int n = rows_kept(c, ctx->kv_len[lidx(ctx, fa_idx, seq)]);
    if (n_out) *n_out = n;
    if (n > max_rows) return fail(ctx, FM_ERR_INVALID, "fm_h2o_export: %d rows kept, room for %d", n, max_rows);
    if (n == 0) return FM_OK;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const H2oView h = h2o_view(ctx, fa_idx);
    {
        const fm_status so = h2o_refresh_order(ctx, fa_idx, seq);
        if (so) return so;
    }
    if (ctx->ptr_mode == FM_PTR_DEVICE) return launched(ctx, launch_h2o_gather(h, seq, n, accum, token_positions, ctx->stream), "h2o_gather");
    if ((size_t)n * 8 + 512 > ctx->stage_bytes) return fail(ctx, FM_ERR_INVALID, "fm_h2o_export: staging buffer too small");
    float *da = reinterpret_cast<float *>(ctx->d_stage);
    int *dt = reinterpret_cast<int *>(ctx->d_stage + (((size_t)n * 4 + 255) & ~(size_t)255));
    const fm_status st = launched(ctx, launch_h2o_gather(h, seq, n, da, dt, ctx->stream), "h2o_gather");
    if (st) return st;
    if (accum) FM_CUDA(ctx, cudaMemcpyAsync(accum, da, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (token_positions) FM_CUDA(ctx, cudaMemcpyAsync(token_positions, dt, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return FM_OK;
}

// conv history: the reference keeps [(ks-1)][conv_dim], oldest first; the device keeps a ring of ks
// rows indexed by token count.  Export / import translate between the two.
extern "C" fm_status fm_state_export(FmCtx *ctx, int li, int seq, float *conv, float *ssm) {
    if (!ctx) return FM_ERR_INVALID;
    const FmConfig &c = ctx->cfg;
    if (li < 0 || li >= c.num_linear_layers || seq < 0 || seq >= c.max_seqs) return fail(ctx, FM_ERR_INVALID, "fm_state_export: bad argument");
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const cudaMemcpyKind kind = ctx->ptr_mode == FM_PTR_HOST ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    const size_t cd = (size_t)ctx->conv_dim, ks = (size_t)c.conv_kernel_size;
    const size_t sn = (size_t)c.linear_num_v_heads * c.linear_value_dim * c.linear_key_dim;
    const int step = ctx->gdn_steps[lidx(ctx, li, seq)];
    if (conv) {
        const float *ring = ctx->d_conv_state + lidx(ctx, li, seq) * ks * cd;
        for (int j = 0; j < (int)ks - 1; j++) {
            const int tokidx = step - ((int)ks - 1) + j;
            if (tokidx >= 0)
                FM_CUDA(ctx, cudaMemcpyAsync(conv + j * cd, ring + (size_t)(tokidx % (int)ks) * cd, cd * sizeof(float), kind, ctx->stream));
            else if (ctx->ptr_mode == FM_PTR_HOST)
                memset(conv + j * cd, 0, cd * sizeof(float));
            else
                FM_CUDA(ctx, cudaMemsetAsync(conv + j * cd, 0, cd * sizeof(float), ctx->stream));
        }
    }
    if (ssm) FM_CUDA(ctx, cudaMemcpyAsync(ssm, ctx->d_ssm_state + lidx(ctx, li, seq) * sn, sn * sizeof(float), kind, ctx->stream));
    if (ctx->ptr_mode == FM_PTR_HOST) FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return FM_OK;
}

extern "C" fm_status fm_state_import(FmCtx *ctx, int li, int seq, const float *conv, const float *ssm) {
    if (!ctx) return FM_ERR_INVALID;
    ctx->last_state_li = -1;  // the next GatedDeltaNet step is not launched under this call's tail
    const FmConfig &c = ctx->cfg;
    if (li < 0 || li >= c.num_linear_layers || seq < 0 || seq >= c.max_seqs) return fail(ctx, FM_ERR_INVALID, "fm_state_import: bad argument");
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const cudaMemcpyKind kind = ctx->ptr_mode == FM_PTR_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    const size_t cd = (size_t)ctx->conv_dim, ks = (size_t)c.conv_kernel_size;
    const size_t sn = (size_t)c.linear_num_v_heads * c.linear_value_dim * c.linear_key_dim;
    if (conv) {
        // restart the ring: history rows become tokens 0..ks-2, the next token is number ks-1
        float *ring = ctx->d_conv_state + lidx(ctx, li, seq) * ks * cd;
        FM_CUDA(ctx, cudaMemcpyAsync(ring, conv, (ks - 1) * cd * sizeof(float), kind, ctx->stream));
        ctx->gdn_steps[lidx(ctx, li, seq)] = (int)ks - 1;
    }
    if (ssm) FM_CUDA(ctx, cudaMemcpyAsync(ctx->d_ssm_state + lidx(ctx, li, seq) * sn, ssm, sn * sizeof(float), kind, ctx->stream));
    if (ctx->ptr_mode == FM_PTR_HOST) FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return FM_OK;
}

// ---- cross-GPU exchange of decode partials over peer memory ------------------------------------
static int xchg_cap(const FmCtx *ctx) { return std::min(ctx->cfg.max_batch_tokens, kMaxList); }
// Slot sets of the exchange: step s uses set s & (ring - 1).  Within one fm_attn_decode_layers call up to
// num_full_layers launches are in flight at once (each a programmatic dependent of the one before, all complete in
// order, the first one behind everything earlier in the stream), and nothing orders a launch's push behind the
// earlier launches' reads.  A rank that pushes step s has completed every call before the current one, i.e. every
// step <= s - n (n = num_full_layers); completing a step means every peer has pushed it, and a peer that has pushed
// step x has itself completed every step <= x - n, reads included.  So when step s is pushed, every rank has read all
// steps <= s - 2n: a ring of at least 2n sets is never overwritten while in use.
static int xchg_ring(const FmCtx *ctx) {
    int r = 2;
    while (r < 2 * ctx->cfg.num_full_layers) r <<= 1;
    return r;
}
static size_t xchg_slot_floats(const FmCtx *ctx, int nranks) {
    return (size_t)xchg_ring(ctx) * nranks * xchg_cap(ctx) * ctx->cfg.num_attn_heads * (ctx->cfg.head_dim + 2);
}
static size_t xchg_step_flag_bytes(const FmCtx *ctx, int nranks) { return ((size_t)xchg_ring(ctx) * nranks * 4 + 255) & ~(size_t)255; }

extern "C" size_t fm_exchange_bytes(const FmCtx *ctx, int nranks) {
    if (!ctx || nranks < 1 || nranks > kMaxXchgRanks) return 0;
    const size_t slots = (xchg_slot_floats(ctx, nranks) * sizeof(float) + 255) & ~(size_t)255;
    // after the slots: step flags [ring][nranks], then flags per (token, KV head) [ring][nranks][cap * Hkv], 32 bits each
    const size_t unit_flags = ((size_t)xchg_ring(ctx) * nranks * xchg_cap(ctx) * ctx->cfg.num_kv_heads * 4 + 255) & ~(size_t)255;
    return slots + xchg_step_flag_bytes(ctx, nranks) + unit_flags;
}

extern "C" fm_status fm_exchange_attach(FmCtx *ctx, int nranks, int my_index, void *const *peer_bufs) {
    if (!ctx) return FM_ERR_INVALID;
    if (nranks < 1 || nranks > kMaxXchgRanks || my_index < 0 || my_index >= nranks || !peer_bufs)
        return fail(ctx, FM_ERR_INVALID, "fm_exchange_attach: %d ranks (1..%d), index %d", nranks, kMaxXchgRanks, my_index);
    if (ctx->cfg.num_full_layers <= 0) return fail(ctx, FM_ERR_INVALID, "fm_exchange_attach: context holds no full-attention layers");
    for (int r = 0; r < nranks; r++)
        if (!peer_bufs[r]) return fail(ctx, FM_ERR_INVALID, "fm_exchange_attach: peer buffer %d is null", r);
    FM_CUDA(ctx, cudaSetDevice(ctx->cfg.device));
    if (!ctx->d_xchg_counter) {
        FM_CUDA(ctx, cudaMalloc(&ctx->d_xchg_counter, sizeof(unsigned int)));
        FM_CUDA(ctx, cudaMemset(ctx->d_xchg_counter, 0, sizeof(unsigned int)));
    }
    XchgView &x = ctx->xchg;
    for (int r = 0; r < nranks; r++) x.peer[r] = static_cast<float *>(peer_bufs[r]);
    x.nranks = nranks;
    x.me = my_index;
    x.cap = xchg_cap(ctx);
    x.ring = xchg_ring(ctx);
    x.flag_offset_floats = (long long)(((xchg_slot_floats(ctx, nranks) * sizeof(float) + 255) & ~(size_t)255) / sizeof(float));
    x.unit_flag_offset_floats = x.flag_offset_floats + (long long)(xchg_step_flag_bytes(ctx, nranks) / sizeof(float));
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->cfg.device);
    x.wait_limit_cycles = (long long)(khz > 0 ? khz : 1900000) * 500;  // about half a second of SM clock
    ctx->xchg_step = 0;
    // the local buffer starts zeroed: flags hold step 0, the first exchange is step 1
    FM_CUDA(ctx, cudaMemsetAsync(x.peer[my_index], 0, fm_exchange_bytes(ctx, nranks), ctx->stream));
    FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return FM_OK;
}

// Shared body of the exchange step.  out == nullptr: push only (the rows go to the peers, the step is
// published; fm_attn_decode_exchange_merge finishes).  out != nullptr: the whole step in the decode
// launch where the split count allows (*finished = true), else push only.
static fm_status xchg_push(FmCtx *ctx, const char *fn, int fa_idx, const int *seq, const int *pos, int batch,
                           const float *q_proj_out, const float *q, const float *k, const float *v,
                           const uint16_t *q_norm_w, const uint16_t *k_norm_w, const float *gate, float *out, bool *finished) {
    if (!ctx) return FM_ERR_INVALID;
    *finished = false;
    if (ctx->xchg.nranks < 1) return fail(ctx, FM_ERR_INVALID, "%s: call fm_exchange_attach first", fn);
    if (ctx->cfg.h2o_budget > 0) return fail(ctx, FM_ERR_UNSUPPORTED, "%s: not with H2O eviction", fn);
    if (!seq || !pos || (!q_proj_out && !q)) return fail(ctx, FM_ERR_INVALID, "%s: null argument", fn);
    if ((k == nullptr) != (v == nullptr)) return fail(ctx, FM_ERR_INVALID, "%s: k and v go together", fn);
    fm_status st = check_layer_seq(ctx, fn, fa_idx, ctx->cfg.num_full_layers, seq, batch);
    if (st) return st;
    if (batch < 1 || batch > ctx->xchg.cap) return fail(ctx, FM_ERR_INVALID, "%s: batch %d (1..%d)", fn, batch, ctx->xchg.cap);
    for (int i = 0; i < batch; i++)
        for (int j = 0; j < i; j++)
            if (seq[i] == seq[j]) return fail(ctx, FM_ERR_INVALID, "%s: sequence %d appears twice in one step", fn, seq[i]);
    const FmConfig &c = ctx->cfg;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const int H = c.num_attn_heads, D = c.head_dim;
    const size_t qd = (size_t)H * D, kvd = (size_t)c.num_kv_heads * D;
    Stager sg(ctx);
    bool ok = true;
    const float *d_qp = sg.in(q_proj_out, batch * qd * 2, &ok);
    const float *d_q = sg.in(q_proj_out ? nullptr : q, batch * qd, &ok);
    const float *d_k = sg.in(k, batch * kvd, &ok), *d_v = sg.in(v, batch * kvd, &ok);
    const uint16_t *d_qn = sg.in(q_norm_w, (size_t)D, &ok), *d_kn = sg.in(k_norm_w, (size_t)D, &ok);
    std::vector<int> rows(batch), nrows(batch);
    int max_len = 1;
    for (int i = 0; i < batch; i++) max_len = std::max(max_len, rows_held(c, ctx->kv_len[lidx(ctx, fa_idx, seq[i])] + (k ? 1 : 0)));
    const int ns = pick_splits(ctx, batch, max_len, /*exchange=*/true);
    const bool whole = out != nullptr;
    const float *d_g = whole ? sg.in(q_proj_out ? nullptr : gate, batch * qd, &ok) : nullptr;
    size_t w_out = 0;
    float *d_out = whole ? sg.out(out, batch * qd, &ok, &w_out) : nullptr;
    if (!ok) return fail(ctx, FM_ERR_INVALID, "%s: staging buffer too small", fn);
    if (k != nullptr) {
        st = reserve_rows(ctx, fa_idx, seq, batch, rows, &nrows);
        if (st) return st;
    } else {
        for (int i = 0; i < batch; i++) {
            const int count = ctx->kv_len[lidx(ctx, fa_idx, seq[i])];
            if (count < 1) return fail(ctx, FM_ERR_INVALID, "%s: sequence %d is empty and no k/v given", fn, seq[i]);
            rows[i] = row_of(c, count - 1);
            nrows[i] = rows_held(c, count);
        }
    }
    FM_CUDA(ctx, sg.push());
    TokSpec t;
    t.mode = 0;
    t.n = batch;
    for (int i = 0; i < batch; i++) t.set(i, seq[i], pos[i], rows[i], nrows[i]);
    ctx->xchg_step++;
    {
        // one launch: append, split-KV attention, merge of the splits, rows into every peer's buffer; then either the
        // step is published for the separate merge, or the peers' rows are awaited, merged and gated right there
        ProfScope prof(ctx);
        const LayerScratch ls = layer_scratch(ctx, fa_idx);
        st = launched(ctx, launch_attn_decode_fused(kv_view(ctx, fa_idx), ctx->rope, t, H, d_qp, d_q, d_qn, c.rms_norm_eps, ls.part_o,
                                                    ls.part_ml, ns, d_k, d_v, d_kn, whole ? 4 : 3, d_g, d_out, nullptr, &ctx->xchg,
                                                    ctx->xchg_step, ls.scr, ctx->d_err, ctx->overlap_prev && !sg.host,
                                                    ctx->stream),
                      "attn_decode");
    }
    if (st) return st;
    *finished = whole;
    if (whole) {
        if (sg.host) FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
        FM_CUDA(ctx, sg.pull(out, w_out, batch * qd));
        if (sg.host) return check_device_error(ctx);
        return FM_OK;
    }
    if (sg.host) FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the staged inputs may be reused by the next call
    return FM_OK;
}

extern "C" fm_status fm_attn_decode_exchange_push(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                                                  const float *q_proj_out, const float *q, const float *k, const float *v,
                                                  const uint16_t *q_norm_w, const uint16_t *k_norm_w) {
    bool finished;
    return xchg_push(ctx, "fm_attn_decode_exchange_push", fa_idx, seq, pos, batch, q_proj_out, q, k, v, q_norm_w, k_norm_w, nullptr, nullptr,
                     &finished);
}

extern "C" fm_status fm_attn_decode_exchange_merge(FmCtx *ctx, int batch, const float *q_proj_out, const float *gate, float *out) {
    if (!ctx) return FM_ERR_INVALID;
    const char *fn = "fm_attn_decode_exchange_merge";
    if (ctx->xchg.nranks < 1 || ctx->xchg_step == 0) return fail(ctx, FM_ERR_INVALID, "%s: nothing was pushed", fn);
    if (!out || (!q_proj_out && !gate)) return fail(ctx, FM_ERR_INVALID, "%s: null argument", fn);
    if (batch < 1 || batch > ctx->xchg.cap) return fail(ctx, FM_ERR_INVALID, "%s: batch %d (1..%d)", fn, batch, ctx->xchg.cap);
    const FmConfig &c = ctx->cfg;
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const size_t qd = (size_t)c.num_attn_heads * c.head_dim;
    Stager sg(ctx);
    bool ok = true;
    const float *d_qp = sg.in(q_proj_out, batch * qd * 2, &ok);
    const float *d_g = sg.in(q_proj_out ? nullptr : gate, batch * qd, &ok);
    size_t w_out = 0;
    float *d_out = sg.out(out, batch * qd, &ok, &w_out);
    if (!ok) return fail(ctx, FM_ERR_INVALID, "%s: staging buffer too small", fn);
    FM_CUDA(ctx, sg.push());
    fm_status st = launched(ctx, launch_attn_wait_merge(ctx->xchg, ctx->xchg_step, batch, c.num_attn_heads, d_qp, d_g, d_out, ctx->d_err,
                                                        ctx->overlap_merge && !sg.host, ctx->stream), "attn_wait_merge");
    if (st) return st;
    if (sg.host) FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    FM_CUDA(ctx, sg.pull(out, w_out, batch * qd));
    if (sg.host) return check_device_error(ctx);
    return FM_OK;
}

extern "C" fm_status fm_attn_decode_exchange(FmCtx *ctx, int fa_idx, const int *seq, const int *pos, int batch,
                                             const float *q_proj_out, const float *q, const float *gate, const float *k,
                                             const float *v, const uint16_t *q_norm_w, const uint16_t *k_norm_w, float *out) {
    if (ctx && (!out || (!q_proj_out && !gate))) return fail(ctx, FM_ERR_INVALID, "fm_attn_decode_exchange: null argument");
    bool finished = false;
    fm_status st = xchg_push(ctx, "fm_attn_decode_exchange", fa_idx, seq, pos, batch, q_proj_out, q, k, v, q_norm_w, k_norm_w, gate, out,
                             &finished);
    if (st || finished) return st;
    return fm_attn_decode_exchange_merge(ctx, batch, q_proj_out, gate, out);
}

// ---- one token through several full-attention layers -------------------------------------------
static bool is_pinned(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeHost;
}

// Host-pointer form.  The layers' inputs go to the device in two groups (the first three layers | the rest) on a copy
// stream, each group's launches waiting for its event only, so that all but the first small copy run under the first
// layers' kernels; the outputs come back in two as well (all but the last layer | the last), so that only the last
// layer's rows are copied after the last kernel.  Every cut costs the overlap between two layers' launches, hence so
// few; the launches of a run between two cuts pick their width for that run's number of layers (pick_splits).  Page-locked caller buffers are copied directly;
// pageable ones pass through the context's own page-locked staging area.
static fm_status decode_layers_host(FmCtx *ctx, int first_layer, int n_layers, const int *seq, const int *pos, int batch,
                                    const float *q_proj_out, size_t sq, const float *k, const float *v, size_t skv,
                                    const uint16_t *qnw, const uint16_t *knw, float *out, size_t so, int exchange) {
    const FmConfig &c = ctx->cfg;
    if (batch < 0 || batch > c.max_batch_tokens) return fail(ctx, FM_ERR_INVALID, "fm_attn_decode_layers: batch %d", batch);
    FM_CUDA(ctx, cudaSetDevice(c.device));
    const size_t qf = (size_t)batch * c.num_attn_heads * 2 * c.head_dim, kvf = (size_t)batch * c.num_kv_heads * c.head_dim;
    const size_t of = (size_t)batch * c.num_attn_heads * c.head_dim, nl = (size_t)n_layers;
    auto up = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t o_w = 0, o_q = 1024, o_k = o_q + up(nl * qf * 4), o_v = o_k + up(nl * kvf * 4), o_out = o_v + up(nl * kvf * 4);
    const size_t need = o_out + up(nl * of * 4);
    if (need > ctx->lstage_bytes) {
        FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(ctx->d_lstage);
        if (ctx->h_lstage) cudaFreeHost(ctx->h_lstage);
        ctx->d_lstage = ctx->h_lstage = nullptr;
        ctx->lstage_bytes = 0;
        FM_CUDA(ctx, cudaMallocHost(&ctx->h_lstage, need));
        FM_CUDA(ctx, cudaMalloc(&ctx->d_lstage, need));
        ctx->lstage_bytes = need;
    }
    if (ctx->copy_stream == nullptr) {
        FM_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
        for (int i = 0; i < 3; i++) {
            FM_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming));
            FM_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_out[i], cudaEventDisableTiming));
        }
        FM_CUDA(ctx, cudaEventCreateWithFlags(&ctx->ev_idle, cudaEventDisableTiming));
    }
    cudaStream_t cs = ctx->copy_stream;
    char *hs = ctx->h_lstage, *ds = ctx->d_lstage;
    // whatever the caller queued on the context's stream before this call (it may still read the staging area)
    FM_CUDA(ctx, cudaEventRecord(ctx->ev_idle, ctx->stream));
    FM_CUDA(ctx, cudaStreamWaitEvent(cs, ctx->ev_idle, 0));
    // host -> device of layers [a, b): blocks of `block` floats, `stride` floats apart at the source
    auto send = [&](const float *src, size_t stride, size_t block, size_t off, size_t a, size_t b) -> cudaError_t {
        if (src == nullptr || block == 0 || b <= a) return cudaSuccess;
        if (is_pinned(src))
            return cudaMemcpy2DAsync(ds + off + a * block * 4, block * 4, src + a * stride, stride * 4, block * 4, b - a, cudaMemcpyHostToDevice, cs);
        for (size_t l = a; l < b; l++) memcpy(hs + off + l * block * 4, src + l * stride, block * 4);
        return cudaMemcpyAsync(ds + off + a * block * 4, hs + off + a * block * 4, (b - a) * block * 4, cudaMemcpyHostToDevice, cs);
    };
    if (qnw) memcpy(hs + o_w, qnw, (size_t)c.head_dim * 2);
    if (knw) memcpy(hs + o_w + 512, knw, (size_t)c.head_dim * 2);
    if (qnw || knw) FM_CUDA(ctx, cudaMemcpyAsync(ds + o_w, hs + o_w, 1024, cudaMemcpyHostToDevice, cs));
    const size_t first = 3;  // layers whose inputs go first: their kernels cover the copy of the rest
    const size_t in_end[3] = {std::min(first, nl), std::min(first, nl), nl};
    const size_t out_end[3] = {0, nl > 1 ? nl - 1 : 0, nl};
    for (int g = 0; g < 3; g++) {
        const size_t a = g ? in_end[g - 1] : 0, b = in_end[g];
        if (b <= a) continue;
        FM_CUDA(ctx, send(q_proj_out, sq, qf, o_q, a, b));
        FM_CUDA(ctx, send(k, skv, kvf, o_k, a, b));
        FM_CUDA(ctx, send(v, skv, kvf, o_v, a, b));
        FM_CUDA(ctx, cudaEventRecord(ctx->ev_in[g], cs));
    }
    const bool direct = is_pinned(out);
    // the launches, cut where an input group starts or an output group ends
    ctx->ptr_mode = FM_PTR_DEVICE;
    fm_status st = FM_OK;
    size_t at = 0;
    while (at < nl && st == FM_OK) {
        size_t stop = nl;
        for (int g = 0; g < 3; g++) {
            if (in_end[g] > at) stop = std::min(stop, in_end[g]);
            if (out_end[g] > at) stop = std::min(stop, out_end[g]);
        }
        cudaError_t e = cudaSuccess;
        for (int g = 0; g < 3; g++)
            if ((g ? in_end[g - 1] : 0) == at && in_end[g] > at) e = cudaStreamWaitEvent(ctx->stream, ctx->ev_in[g], 0);
        if (e != cudaSuccess) { st = fail(ctx, FM_ERR_CUDA, "fm_attn_decode_layers: %s", cudaGetErrorString(e)); break; }
        st = fm_attn_decode_layers(ctx, first_layer + (int)at, (int)(stop - at), seq, pos, batch, reinterpret_cast<const float *>(ds + o_q) + at * qf, qf,
                                   k ? reinterpret_cast<const float *>(ds + o_k) + at * kvf : nullptr,
                                   v ? reinterpret_cast<const float *>(ds + o_v) + at * kvf : nullptr, kvf,
                                   qnw ? reinterpret_cast<const uint16_t *>(ds + o_w) : nullptr,
                                   knw ? reinterpret_cast<const uint16_t *>(ds + o_w + 512) : nullptr,
                                   reinterpret_cast<float *>(ds + o_out) + at * of, of, exchange);
        if (st) break;
        for (int g = 0; g < 3 && e == cudaSuccess; g++) {
            const size_t a = g ? out_end[g - 1] : 0, b = out_end[g];
            if (b != stop || b <= a) continue;
            e = cudaEventRecord(ctx->ev_out[g], ctx->stream);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, ctx->ev_out[g], 0);
            if (e != cudaSuccess) break;
            if (direct)
                e = cudaMemcpy2DAsync(out + a * so, so * 4, ds + o_out + a * of * 4, of * 4, of * 4, b - a, cudaMemcpyDeviceToHost, cs);
            else
                e = cudaMemcpyAsync(hs + o_out + a * of * 4, ds + o_out + a * of * 4, (b - a) * of * 4, cudaMemcpyDeviceToHost, cs);
        }
        if (e != cudaSuccess) { st = fail(ctx, FM_ERR_CUDA, "fm_attn_decode_layers: %s", cudaGetErrorString(e)); break; }
        at = stop;
    }
    ctx->ptr_mode = FM_PTR_HOST;
    if (st) {  // leave nothing in flight that touches the caller's buffers
        cudaStreamSynchronize(cs);
        cudaStreamSynchronize(ctx->stream);
        return st;
    }
    FM_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    FM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    FM_CUDA(ctx, cudaStreamSynchronize(cs));
    if (!direct)
        for (size_t l = 0; l < nl; l++) memcpy(out + l * so, hs + o_out + l * of * 4, of * 4);
    return check_device_error(ctx);
}

extern "C" fm_status fm_attn_decode_layers(FmCtx *ctx, int first_layer, int n_layers, const int *seq, const int *pos, int batch,
                                           const float *q_proj_out, size_t layer_stride_q, const float *k, const float *v,
                                           size_t layer_stride_kv, const uint16_t *q_norm_w, const uint16_t *k_norm_w, float *out,
                                           size_t layer_stride_out, int exchange) {
    if (!ctx) return FM_ERR_INVALID;
    if (!q_proj_out || !out || n_layers < 0) return fail(ctx, FM_ERR_INVALID, "fm_attn_decode_layers: bad argument");
    if ((k == nullptr) != (v == nullptr)) return fail(ctx, FM_ERR_INVALID, "fm_attn_decode_layers: k and v go together");
    if (ctx->ptr_mode == FM_PTR_HOST && n_layers > 0 && batch > 0)
        return decode_layers_host(ctx, first_layer, n_layers, seq, pos, batch, q_proj_out, layer_stride_q, k, v, layer_stride_kv, q_norm_w,
                                  k_norm_w, out, layer_stride_out, exchange);
    // Between layers nothing is shared but the library's own scratch, which the kernels guard: a
    // layer's launch may overlap the end of the previous one.  Not while launches are bracketed by
    // timing events, and not in host-pointer mode (copies sit between the launches anyway).
    struct Overlap {
        FmCtx *c;
        ~Overlap() { c->overlap_prev = c->overlap_merge = c->overlap_layers = false; }
    } guard{ctx};
    // (layers whose outputs would alias are kept in full stream order)
    const bool distinct = layer_stride_out >= (size_t)std::max(batch, 0) * ctx->cfg.num_attn_heads * ctx->cfg.head_dim;
    ctx->overlap_layers = !ctx->prof_on && n_layers > 1 && distinct;
    ctx->overlap_nlayers = n_layers;
    for (int l = 0; l < n_layers; l++) {
        ctx->overlap_prev = l > 0 && ctx->overlap_layers;
        ctx->overlap_merge = !ctx->prof_on;
        const float *qp = q_proj_out + (size_t)l * layer_stride_q;
        const float *kk = k ? k + (size_t)l * layer_stride_kv : nullptr, *vv = v ? v + (size_t)l * layer_stride_kv : nullptr;
        float *oo = out + (size_t)l * layer_stride_out;
        const fm_status st = exchange ? fm_attn_decode_exchange(ctx, first_layer + l, seq, pos, batch, qp, nullptr, nullptr, kk, vv, q_norm_w, k_norm_w, oo)
                                      : fm_attn_decode(ctx, first_layer + l, seq, pos, batch, qp, nullptr, nullptr, kk, vv, q_norm_w, k_norm_w, oo);
        if (st) return st;
    }
    return FM_OK;
}
