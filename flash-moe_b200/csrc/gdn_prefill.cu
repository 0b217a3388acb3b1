// GatedDeltaNet over a run of n tokens of one sequence.
#include "fm_internal.h"

namespace fm {

size_t gdn_prefill_work_bytes(const GdnDims &, int, int) { return 0; }

// Token-by-token version: one fused decode launch per token (same arithmetic as n decode steps).
int launch_gdn_prefill(const GdnDims &g, int n, int chunk, int step0, float *conv_state, float *ssm_state,
                       const float *qkv, const float *z, const float *beta, const float *alpha,
                       const uint16_t *conv_w, const float *A_log, const uint16_t *dt_bias,
                       const uint16_t *norm_w, float *out, void *work, size_t work_bytes, cudaStream_t st) {
    (void)chunk; (void)work; (void)work_bytes;
    const size_t vd = (size_t)g.Hv * g.dv;
    int launches = 0;
    for (int t = 0; t < n; t++) {
        TokSpec ts;
        ts.mode = 0; ts.n = 1; ts.seq[0] = 0; ts.pos[0] = step0 + t; ts.row[0] = 0;
        const int r = launch_gdn_decode(g, ts, conv_state, ssm_state, 0, 0, qkv + (size_t)t * g.conv_dim, z + t * vd,
                                        beta + (size_t)t * g.Hv, alpha + (size_t)t * g.Hv, conv_w, A_log, dt_bias,
                                        norm_w, out + t * vd, st);
        if (r < 0) return -1;
        launches += r;
    }
    return launches;
}

}  // namespace fm
