// Causal prefill attention over the paged KV store (rows already appended by the caller):
// token t of the run attends to rows [0, row0 + t] and is multiplied by sigmoid(gate).
// Math of the Metal kernel prefill_causal_attn (metal_infer/shaders.metal:2228-2315).
//
// This version runs every token of the run as an independent decode problem on the split-KV
// kernel of attn_decode.cu (one CTA per (KV head, token), the 16 grouped query heads as the MMA M
// dimension), followed by the normalise + gate kernel.  K/V tiles are re-read from L2 per token.
#include "fm_internal.h"

namespace fm {

int launch_attn_prefill(const KvView &kv, const RopeParams &rope, int seq, int start_pos, int row0, int n,
                        int H, const float *q_proj_out, const float *q, const float *gate,
                        const uint16_t *q_norm_w, float eps, float *work_o, float *work_ml, float *out,
                        cudaStream_t st) {
    TokSpec t;
    t.mode = 1; t.n = n; t.seq0 = seq; t.pos0 = start_pos; t.row0 = row0;
    const int D = kv.D;
    if (launch_attn_decode(kv, rope, t, H, q_proj_out, q, q_norm_w, eps, work_o, work_ml, 1, st) < 0) return -1;
    if (launch_attn_merge(work_o, work_ml, 1, D, 2, (long long)H * D, (long long)H * 2, D, 2, n, H, D,
                          q_proj_out, gate, out, nullptr, st) < 0)
        return -1;
    return 2;
}

}  // namespace fm
