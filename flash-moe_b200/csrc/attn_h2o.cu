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
// The decode launch of a step leaves, for every row it streams, the un-normalised softmax weights exp2(score - mref)
// of the 16 query heads of each KV head (128 bytes per row next to the 1 KB of K and V it reads) and the running
// maximum mref they refer to, per 16-row slice.  After it, h2o_mass_kernel
//   * scales them by exp2(mref - max) / sum with the step's final (max, sum) of every head, which the decode launch
//     also leaves, and adds the sum over the heads to the row's accumulated mass (a pass over 128 bytes per row:
//     recomputing q . K in a second pass over the K rows measured 940 us per layer at 8 x 32768 rows, ten times the
//     decode launch itself);
//   * every CTA also proposes the lightest unprotected row of its tile; the last CTA to finish records the new row's
//     token position and, if the rows now exceed the budget, picks the lightest proposal (ties: the later row, which is
//     what the reference's strict `>` selection of the rows to KEEP leaves out) and publishes its physical row as the
//     next free slot.  Cache order is chronological and one row goes per step, so "cache index in [sinks, n - recent)"
//     is the same as "token position in [sinks, t_new - recent]": no pass over the cache order is needed, and `order`
//     itself is only rebuilt (by ranking the token positions, h2o_order_kernel) when something is exported.
// Nothing comes back to the host: the row count per step is a function of the token count alone.
#include "fm_device.cuh"
#include "fm_fp8.cuh"
#include "fm_internal.h"

namespace fm {

constexpr int kH2oRowsPerCta = 64;  // one tile of the decode kernel
constexpr int kH2oThreads = 256;

struct H2oParams {
    H2oView h;           // this layer's arrays, indexed [seq][cap]
    int budget, sinks, recent;
    int H, Hkv;
    const float *ml;     // [tokens][H][2] (max in log2 units, sum) from the decode launch
    H2oStep step;        // the weights and their reference maxima, as the decode launch left them
    float4 *cand;        // [tokens][tiles] lightest unprotected row of each tile: (mass, token position, physical row, -)
    int token_index[kMaxList];  // how many tokens the sequence had seen before this one (KVCache.len at the append)
};

// grid (tiles of 64 rows, tokens), 256 threads: four threads per row, each a quarter of the row's Hkv x 16 weights
__global__ void __launch_bounds__(kH2oThreads)
h2o_mass_kernel(TokSpec toks, H2oParams p) {
    __shared__ float s_f[8 * 4 * 16];  // per (KV head, 16-row slice, head): exp2(mref - max) / sum
    __shared__ int s_last;
    __shared__ float s_val[kH2oThreads / 32];
    __shared__ int s_idx[kH2oThreads / 32], s_tp[kH2oThreads / 32];
    const int tok = blockIdx.y, tile = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int seq, pos, row_unused;
    tok_get(toks, tok, seq, pos, row_unused);
    const int n = tok_rows(toks, tok);  // rows attended this step, the new one included
    const int cap = p.h.cap;
    const int row_new = p.h.slot[seq];
    float *accum = p.h.accum + (size_t)seq * cap;
    int *tokpos = p.h.tokpos + (size_t)seq * cap;
    const int group = p.H / p.Hkv, nw = p.Hkv * 16;

    for (int i = tid; i < p.Hkv * 64; i += kH2oThreads) {
        const int kvh = i >> 6, h16 = i & 15;
        float fct = 0.f;
        if (h16 < group) {
            const float2 ml = *reinterpret_cast<const float2 *>(p.ml + ((size_t)tok * p.H + kvh * group + h16) * 2);
            const float mr = p.step.mref[(((size_t)tok * p.step.tiles + tile) * p.Hkv) * 64 + i];
            fct = ml.y > 0.f ? fast_exp2(mr - ml.x) / ml.y : 0.f;
        }
        s_f[i] = fct;
    }
    __syncthreads();
    // protection by token position (see the file header)
    int sinks = min(p.sinks, p.budget), recent = p.recent;
    if (sinks + recent > p.budget) recent = p.budget - sinks;
    const int t_new = p.token_index[tok], tp_hi = t_new - recent;
    float best = 3.0e38f;
    int bt = -1, br = -1;  // token position and physical row of the lightest so far; the later one among equals
    {
        const int r = tile * kH2oRowsPerCta + (tid >> 2), part = tid & 3;  // this thread's row and quarter
        float mass = 0.f;
        if (r < n) {
            const float *w = p.step.w + ((size_t)tok * p.step.rows_pad + r) * nw;
            const int slice = (tid >> 2) >> 4;
            for (int e = part * 4; e < nw; e += 16) {  // float4 number e/4 of the row; the quarters interleave
                const float4 v = *reinterpret_cast<const float4 *>(w + e);
                const float *fc = s_f + ((e >> 4) * 4 + slice) * 16 + (e & 15);
                mass += v.x * fc[0] + v.y * fc[1] + v.z * fc[2] + v.w * fc[3];
            }
        }
        mass += __shfl_xor_sync(0xffffffffu, mass, 1);
        mass += __shfl_xor_sync(0xffffffffu, mass, 2);
        if (r < n && part == 0) {
            const float a = (r == row_new ? 0.f : accum[r]) + mass;  // the new row starts from zero (layer_forward.h:621)
            accum[r] = a;
            const int tp = r == row_new ? t_new : tokpos[r];
            if (r == row_new) tokpos[r] = t_new;
            if (tp >= sinks && tp <= tp_hi) { best = a; bt = tp; br = r; }
        }
    }
    auto better = [](float oa, int ot, float a, int t) { return ot >= 0 && (t < 0 || oa < a || (oa == a && ot > t)); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int ot = __shfl_xor_sync(0xffffffffu, bt, o), orow = __shfl_xor_sync(0xffffffffu, br, o);
        if (better(ob, ot, best, bt)) { best = ob; bt = ot; br = orow; }
    }
    if (lane == 0) { s_val[warp] = best; s_tp[warp] = bt; s_idx[warp] = br; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kH2oThreads / 32; w++)
            if (better(s_val[w], s_tp[w], s_val[0], s_tp[0])) { s_val[0] = s_val[w]; s_tp[0] = s_tp[w]; s_idx[0] = s_idx[w]; }
        p.cand[(size_t)tok * gridDim.x + tile] = make_float4(s_val[0], __int_as_float(s_tp[0]), __int_as_float(s_idx[0]), 0.f);
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
    int next_slot = n;  // no eviction: the next row extends the dense range
    if (n > p.budget) {
        // cache rows [sinks, n - recent) may go; the lightest goes, the later one among equals
        const int ev0 = sinks, ev1 = n - recent;
        const int heavy = p.budget - sinks - recent;
        if (ev1 - ev0 > 0 && heavy < ev1 - ev0) {
            best = 3.0e38f; bt = -1; br = -1;
            for (int i = tid; i < (int)gridDim.x; i += kH2oThreads) {
                const float4 c = __ldcg(p.cand + (size_t)tok * gridDim.x + i);
                if (better(c.x, __float_as_int(c.y), best, bt)) { best = c.x; bt = __float_as_int(c.y); br = __float_as_int(c.z); }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int ot = __shfl_xor_sync(0xffffffffu, bt, o), orow = __shfl_xor_sync(0xffffffffu, br, o);
                if (better(ob, ot, best, bt)) { best = ob; bt = ot; br = orow; }
            }
            __syncthreads();
            if (lane == 0) { s_val[warp] = best; s_tp[warp] = bt; s_idx[warp] = br; }
            __syncthreads();
            if (tid == 0) {
                for (int w = 1; w < kH2oThreads / 32; w++)
                    if (better(s_val[w], s_tp[w], s_val[0], s_tp[0])) { s_val[0] = s_val[w]; s_tp[0] = s_tp[w]; s_idx[0] = s_idx[w]; }
                if (s_idx[0] >= 0) {
                    next_slot = s_idx[0];
                    tokpos[next_slot] = 0x7fffffff;  // a free row ranks after every live one (h2o_order_kernel)
                }
            }
        }
    }
    if (tid == 0) p.h.slot[seq] = next_slot;
}

// Cache order from the token positions: order[rank of row r] = r for the physical rows r < n, rank = how many rows
// are older.  grid (ceil(n / 256)), 256 threads.  Only exports need it.
__global__ void __launch_bounds__(256)
h2o_order_kernel(H2oView h, int seq, int n) {
    __shared__ int s_tp2[256];
    const int r = blockIdx.x * 256 + threadIdx.x;
    const int *tokpos = h.tokpos + (size_t)seq * h.cap;
    const int mine = r < n ? tokpos[r] : 0;
    int rank = 0;
    for (int base = 0; base < n; base += 256) {
        __syncthreads();
        s_tp2[threadIdx.x] = base + (int)threadIdx.x < n ? tokpos[base + threadIdx.x] : 0x7fffffff;
        __syncthreads();
        const int m = min(256, n - base);
        for (int j = 0; j < m; j++) rank += (s_tp2[j] < mine) || (s_tp2[j] == mine && base + j < r);
    }
    if (r < n) h.order[(size_t)seq * h.cap + rank] = r;
}

int launch_h2o_order(const H2oView &h, int seq, int n, cudaStream_t st) {
    if (n <= 0) return 0;
    h2o_order_kernel<<<(n + 255) / 256, 256, 0, st>>>(h, seq, n);
    return cudaGetLastError() == cudaSuccess ? 1 : -1;
}

int launch_h2o_mass(const TokSpec &toks, const int *token_index, const H2oView &h, int budget, int sinks, int recent, int H, int Hkv,
                    const float *ml, const H2oStep &step, float *cand, int max_rows, cudaStream_t st) {
    if (Hkv < 1 || Hkv > 8 || H % Hkv || H / Hkv > 16) return -1;
    H2oParams p;
    p.h = h; p.budget = budget; p.sinks = sinks; p.recent = recent; p.H = H; p.Hkv = Hkv; p.ml = ml; p.step = step; p.cand = reinterpret_cast<float4 *>(cand);
    for (int i = 0; i < toks.n; i++) p.token_index[i] = token_index[i];
    dim3 grid((max_rows + kH2oRowsPerCta - 1) / kH2oRowsPerCta, toks.n);
    h2o_mass_kernel<<<grid, kH2oThreads, 0, st>>>(toks, p);
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
