"""Output projection (4-bit affine weights) + residual + post-attention RMS-norm through the C-ABI against the CPU
checker (the reference's cpu_dequant_matvec / residual add / cpu_rms_norm)."""
import numpy as np
import pytest

from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3


def make_weights(synth, seed, out_dim, in_dim):
    rng = np.random.default_rng(seed)
    w = rng.integers(0, 2 ** 32, size=(out_dim, in_dim // 8), dtype=np.uint64).astype(np.uint32)
    sc = np.abs(synth.normal(seed, "s", (out_dim, in_dim // 64), std=0.004)) + 0.001
    scales = synth.to_bf16_bits(sc)
    biases = synth.to_bf16_bits(-7.5 * synth.bf16_bits_to_f32(scales) + synth.normal(seed, "b", (out_dim, in_dim // 64), std=0.001))
    return w, scales, biases


@pytest.mark.parametrize("n,out_dim,in_dim", [(1, 4096, 8192), (5, 4096, 8192), (64, 4096, 8192), (70, 256, 1024), (8, 64, 512)])
def test_out_proj_norm_matches_checker(pkg, port, synth, n, out_dim, in_dim):
    w, scales, biases = make_weights(synth, 5 + n, out_dim, in_dim)
    x = synth.normal(5 + n, "x", (n, in_dim)); res = synth.normal(5 + n, "r", (n, out_dim))
    nw = synth.to_bf16_bits(1.0 + synth.normal(5 + n, "nw", (out_dim,), std=0.1))
    want_mid, want_post = port.out_proj_norm(w, scales, biases, x, res, nw)
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seq_len=128, max_batch_tokens=64)
    c = pkg.Context(cfg, host_pointers=True)
    dev = c.proj_upload(w, scales, biases)
    h_mid = np.empty((n, out_dim), np.float32); h_post = np.empty_like(h_mid)
    c.out_proj_norm(dev, n, x, res, nw, h_mid, h_post)
    g1, _, r1 = rel_errors(h_mid, want_mid); g2, _, r2 = rel_errors(h_post, want_post)
    print("out_proj n", n, out_dim, in_dim, "h_mid gated", g1, "rms-rel", r1, "h_post gated", g2)
    assert g1 <= TOL and g2 <= TOL
    # without residual and norm weight
    want_mid2, _ = port.out_proj_norm(w, scales, biases, x[:1], None, nw)
    h2 = np.empty((1, out_dim), np.float32)
    c.out_proj_norm(dev, 1, x[:1].copy(), None, None, h2, None)
    g3, _, _ = rel_errors(h2, want_mid2)
    assert g3 <= TOL
    c.proj_free(dev)
    with pytest.raises(pkg.FmError):
        c.out_proj_norm(dev, 1, x[:1].copy(), None, None, h2, None)   # freed weights: refused, not dereferenced
    c.close()
