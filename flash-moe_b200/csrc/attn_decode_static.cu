// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: a plugin that runs inside another
// engine's memory plan (every byte of HBM already handed to that engine's arena), a real-time
// serving loop that forbids allocator calls after start-up, or code that lives under a tool which
// intercepts allocation.  Such callers also cannot use fm_create, which allocates the page pool and
// the scratch for the split-KV partial results.  fm_attn_decode_static gives them the decode step
// anyway: they own the KV pages, the page table, the inputs and the output; the only memory the
// kernels need beyond that -- the per-split partial results that the merge kernel reads back -- is
// the fixed array below, which is part of the library image and lives on every GPU that loads the
// library until the process exits.
#include <math.h>
#include <stdio.h>

#include <algorithm>

#include "fm_internal.h"

namespace {

// Partial-result rows (one per token x query head x split).  Each row is 256 floats of
// un-normalised output; its (max, sum) pair lives in the second part of the array.
constexpr int kStaticRows = 8192;
constexpr int kRowFloats = 256;
constexpr size_t kStaticFloats = (size_t)kStaticRows * (kRowFloats + 2);

// 8.45 MB per GPU.  Host code must not use this name as a pointer: on the host it is only a
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_decode_scratch[kStaticFloats];

constexpr int kMaxDevices = 64;
float *g_scratch_addr[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

void set_err(char *err, size_t cap, const char *fmt, int a = 0, int b = 0, int c = 0) {
    if (err && cap) snprintf(err, cap, fmt, a, b, c);
}

}  // namespace

extern "C" fm_status fm_attn_decode_static(const FmStaticDecodeArgs *a, char *err, size_t err_cap) {
    using namespace fm;
    if (err && err_cap) err[0] = 0;
    if (!a || !a->kv_pages || !a->page_table || !a->kv_len || !a->pos || !a->out ||
        (!a->q_proj_out && (!a->q || !a->gate))) {
        set_err(err, err_cap, "fm_attn_decode_static: null argument");
        return FM_ERR_INVALID;
    }
    if (a->batch < 1 || a->batch > kMaxList) {
        set_err(err, err_cap, "fm_attn_decode_static: batch %d (1..%d)", a->batch, kMaxList);
        return FM_ERR_INVALID;
    }
    if (a->num_attn_heads < 1 || a->max_pages_per_seq < 1 || (a->rotary_dim > 0 && !(a->rope_theta > 0.f))) {
        set_err(err, err_cap, "fm_attn_decode_static: %d query heads, %d pages per sequence, or rope_theta <= 0", a->num_attn_heads,
                a->max_pages_per_seq);
        return FM_ERR_INVALID;
    }
    if (a->num_kv_heads < 1 || a->num_attn_heads % a->num_kv_heads != 0 || a->num_attn_heads / a->num_kv_heads > 16 ||
        a->rotary_dim < 0 || a->rotary_dim > 128 || (a->rotary_dim & 1)) {
        set_err(err, err_cap, "fm_attn_decode_static: %d query / %d KV heads, rotary %d not supported", a->num_attn_heads,
                a->num_kv_heads, a->rotary_dim);
        return FM_ERR_UNSUPPORTED;
    }
    // the smallest use of the scratch is one split per (token, head)
    if ((long long)a->batch * a->num_attn_heads > kStaticRows) {
        set_err(err, err_cap, "fm_attn_decode_static: batch x heads = %d exceeds the fixed scratch of %d partial rows",
                a->batch * a->num_attn_heads, kStaticRows);
        return FM_ERR_CAPACITY;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_err(err, err_cap, "fm_attn_decode_static: no current CUDA device");
        return FM_ERR_CUDA;
    }
    // One-time set-up per device, with that device current: resolve the device address of the
    // scratch array and read the SM count.  (Do the first call on a device outside stream capture.)
    if (g_scratch_addr[dev] == nullptr) {
        float *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_decode_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_err(err, err_cap, "fm_attn_decode_static: cudaGetSymbolAddress failed (%d)", (int)e);
            return FM_ERR_CUDA;
        }
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms < 1) {
            set_err(err, err_cap, "fm_attn_decode_static: cannot read the SM count (%d)", (int)e);
            return FM_ERR_CUDA;
        }
        g_sm_count[dev] = sms;
        g_scratch_addr[dev] = p;
    }
    float *part_o = g_scratch_addr[dev];
    float *part_ml = part_o + (size_t)kStaticRows * kRowFloats;

    RopeParams rope;
    rope.rotary_dim = a->rotary_dim;
    for (int i = 0; i < a->rotary_dim / 2; i++)
        rope.inv_freq[i] = 1.0f / powf(a->rope_theta, (float)(2 * i) / a->rotary_dim);
    rope.pos_div = 1.0f;
    rope.logit_scale = 1.0f / sqrtf(256.0f);

    KvView kv;
    kv.pool = reinterpret_cast<unsigned char *>(const_cast<void *>(a->kv_pages));
    kv.page_bytes = fm::kv_page_bytes(0, a->num_kv_heads, 64, 256);
    kv.fp8 = 0;
    kv.page_table = a->page_table;
    kv.max_slots = a->max_pages_per_seq;
    kv.page_size = 64;
    kv.Hkv = a->num_kv_heads;
    kv.D = 256;
    kv.shard_rank = 0;
    kv.shard_count = 1;

    TokSpec t;
    t.mode = 0;
    t.n = a->batch;
    int max_len = 1;
    for (int i = 0; i < a->batch; i++) {
        if (a->kv_len[i] < 1 || (a->kv_len[i] + 63) / 64 > a->max_pages_per_seq) {
            set_err(err, err_cap, "fm_attn_decode_static: kv_len[%d] = %d outside the page table (%d pages)", i, a->kv_len[i],
                    a->max_pages_per_seq);
            return FM_ERR_INVALID;
        }
        t.set(i, i, a->pos[i], a->kv_len[i] - 1, a->kv_len[i]);
        max_len = std::max(max_len, a->kv_len[i]);
    }
    // splits: fill the SMs, stay within the pages available and within the fixed scratch
    int ns = std::max(1, g_sm_count[dev] / (a->num_kv_heads * a->batch));
    ns = std::min(ns, (max_len + 63) / 64);
    ns = std::min(ns, kStaticRows / (a->batch * a->num_attn_heads));
    ns = std::max(ns, 1);

    const int H = a->num_attn_heads, D = 256;
    cudaStream_t st = (cudaStream_t)a->stream;
    if (launch_attn_decode(kv, rope, t, H, a->q_proj_out, a->q, a->q_norm_w, a->rms_norm_eps, part_o, part_ml, ns, st) < 0 ||
        launch_attn_merge(part_o, part_ml, ns, D, 2, (long long)H * ns * D, (long long)H * ns * 2, (long long)ns * D,
                          (long long)ns * 2, t.n, H, D, a->q_proj_out, a->gate, a->out, nullptr, st) < 0) {
        set_err(err, err_cap, "fm_attn_decode_static: kernel launch failed");
        return FM_ERR_CUDA;
    }
    return FM_OK;
}
