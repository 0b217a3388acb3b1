"""Error metrics shared by the parity tests."""
import numpy as np


def rel_errors(a, r):
    """Returns (gated, max_over_max, rms_rel) for result `a` against reference `r`.

    gated        = max_i |a_i - r_i| / max(|r_i|, rms(r))   -- the figure tests gate on
    max_over_max = max|a - r| / max|r|
    rms_rel      = ||a - r|| / ||r||                         -- the reference's own validation metric
                                                               (metal_infer/batched_prefill.h:1282-1299)
    """
    a = np.asarray(a, np.float64).ravel()
    r = np.asarray(r, np.float64).ravel()
    d = np.abs(a - r)
    rms = np.sqrt(np.mean(r * r)) if r.size else 0.0
    den = np.maximum(np.abs(r), rms)
    den[den == 0] = 1.0
    gated = float((d / den).max()) if r.size else 0.0
    mom = float(d.max() / max(np.abs(r).max(), 1e-30)) if r.size else 0.0
    rr = float(np.sqrt((d * d).sum()) / max(np.sqrt((r * r).sum()), 1e-30)) if r.size else 0.0
    return gated, mom, rr
