"""CPU checks of the checker itself: the plain-C restatement against the reference project's own
CPU code (bit-exact) and both against the committed golden vectors."""
from pathlib import Path

import numpy as np
import pytest

from oracle.oracle_py import make_dims

GOLD = Path(__file__).resolve().parent / "golden"
ATTN_CASES = ["attn_h8_d256_ctx37", "attn_h16_d256_ctx130_bf16", "attn_h4_d64_ctx0"]
GDN_CASES = ["gdn_v8_k4_d32", "gdn_v4_k1_d128"]


def run_attn_fixture(orc, f, threads=1):
    dims = make_dims(num_attn_heads=int(f["heads"]), num_kv_heads=int(f["kv_heads"]),
                     head_dim=int(f["head_dim"]), rotary_dim=int(f["rot"]), rope_theta=float(f["theta"]))
    ctx, steps = int(f["ctx"]), int(f["steps"])
    kv_dim = dims.num_kv_heads * dims.head_dim
    kc = np.zeros((ctx + steps, kv_dim), np.float32); vc = np.zeros_like(kc)
    kc[:ctx] = f["k0"]; vc[:ctx] = f["v0"]
    qn = f["qn"] if f["qn"].size else None
    kn = f["kn"] if f["kn"].size else None
    out, ln = orc.attn_run(dims, kc, vc, ctx, f["q"], f["gate"], f["k"], f["v"], qn, kn, threads=threads)
    return out, kc[ctx:ln], vc[ctx:ln], ln


def run_gdn_fixture(orc, f, threads=1):
    vh, kh, dk, dv = int(f["v_heads"]), int(f["k_heads"]), int(f["dk"]), int(f["dv"])
    dims = make_dims(linear_num_v_heads=vh, linear_num_k_heads=kh, linear_key_dim=dk, linear_value_dim=dv)
    conv_dim = 2 * kh * dk + vh * dv
    conv = np.zeros((3, conv_dim), np.float32)
    ssm = f["s0"].copy() if f["s0"].size else np.zeros((vh, dv, dk), np.float32)
    out = orc.gdn_run(dims, conv, ssm, f["qkv"], f["z"], f["beta"], f["alpha"], f["conv_w"],
                      f["A_log"], f["dt_bias"], f["norm_w"], threads=threads)
    return out, conv, ssm


@pytest.mark.parametrize("case", ATTN_CASES)
@pytest.mark.parametrize("threads", [1, 3])
def test_port_matches_attn_golden(port, case, threads):
    f = np.load(GOLD / f"{case}.npz")
    out, kt, vt, ln = run_attn_fixture(port, f, threads)
    assert ln == int(f["len_final"])
    np.testing.assert_array_equal(kt, f["k_final_tail"])
    np.testing.assert_array_equal(vt, f["v_final_tail"])
    np.testing.assert_array_equal(out, f["out"])


@pytest.mark.parametrize("case", GDN_CASES)
@pytest.mark.parametrize("threads", [1, 4])
def test_port_matches_gdn_golden(port, case, threads):
    f = np.load(GOLD / f"{case}.npz")
    out, conv, ssm = run_gdn_fixture(port, f, threads)
    np.testing.assert_array_equal(conv, f["conv_final"])
    np.testing.assert_array_equal(ssm, f["ssm_final"])
    np.testing.assert_array_equal(out, f["out"])


@pytest.mark.parametrize("case", ATTN_CASES)
def test_reference_reproduces_attn_golden(ref, case):
    f = np.load(GOLD / f"{case}.npz")
    for threads in (1, 2):
        out, kt, vt, ln = run_attn_fixture(ref, f, threads)
        np.testing.assert_array_equal(out, f["out"])
        np.testing.assert_array_equal(kt, f["k_final_tail"])


@pytest.mark.parametrize("case", GDN_CASES)
def test_reference_reproduces_gdn_golden(ref, case):
    f = np.load(GOLD / f"{case}.npz")
    for threads in (1, 2):
        out, conv, ssm = run_gdn_fixture(ref, f, threads)
        np.testing.assert_array_equal(out, f["out"])
        np.testing.assert_array_equal(ssm, f["ssm_final"])


def test_port_equals_reference_config1_slice(port, ref, synth):
    """Production head shape (32 q / 2 kv heads x 256, RoPE on 64 dims, theta 1e7) at a context the
    CPU finishes in a second; positions far from zero so the rotation matters."""
    dims = make_dims()
    ctx, steps = 300, 2
    k0, v0 = synth.attn_cache(3, ctx, bf16=False)
    q, g, k, v = synth.attn_step_inputs(3, steps)
    res = []
    for orc in (port, ref):
        kc = np.zeros((ctx + steps, 512), np.float32); vc = np.zeros_like(kc)
        kc[:ctx] = k0; vc[:ctx] = v0
        out, ln = orc.attn_run(dims, kc, vc, ctx, q, g, k, v, start_pos=100000)
        res.append((out, kc.copy()))
    np.testing.assert_array_equal(res[0][0], res[1][0])
    np.testing.assert_array_equal(res[0][1], res[1][1])


@pytest.mark.parametrize("mode,factor", [(1, 4.0), (2, 4.0), (3, 4.0)])
def test_port_equals_reference_rope_scaling(port, ref, synth, mode, factor):
    dims = make_dims(num_attn_heads=4, num_kv_heads=1, rope_scaling_mode=mode,
                     rope_scale_factor=factor, max_seq_len=4096)
    ctx, steps = 20, 2
    k0, v0 = synth.attn_cache(5, ctx, 1, 256, bf16=False)
    q, g, k, v = synth.attn_step_inputs(5, steps, 4, 1, 256)
    res = []
    for orc in (port, ref):
        kc = np.zeros((ctx + steps, 256), np.float32); vc = np.zeros_like(kc)
        kc[:ctx] = k0; vc[:ctx] = v0
        out, _ = orc.attn_run(dims, kc, vc, ctx, q, g, k, v, start_pos=9000)
        res.append(out)
    np.testing.assert_array_equal(res[0], res[1])


def test_port_equals_reference_gdn_production_shape(port, ref, synth):
    dims = make_dims()
    w = synth.gdn_weights(7)
    qkv, z, beta, alpha = synth.gdn_step_inputs(7, 4)
    res = []
    for orc in (port, ref):
        conv = np.zeros((3, 12288), np.float32)
        ssm = synth.gdn_state(7).copy()
        out = orc.gdn_run(dims, conv, ssm, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"],
                          w["norm_w"], threads=2)
        res.append((out, ssm, conv))
    for a, b in zip(res[0], res[1]):
        np.testing.assert_array_equal(a, b)


def test_overflow_is_reported(port):
    dims = make_dims(num_attn_heads=2, num_kv_heads=1, head_dim=64, rotary_dim=16)
    kc = np.zeros((2, 64), np.float32); vc = np.zeros_like(kc)
    x = np.ones((1, 128), np.float32); kv = np.ones((1, 64), np.float32)
    with pytest.raises(RuntimeError):
        port.attn_run(dims, kc, vc, 2, x, x, kv, kv)


def test_first_token_attends_to_itself_only(port):
    """Empty cache: softmax over one row is 1, so out = v * sigmoid(gate)."""
    dims = make_dims(num_attn_heads=2, num_kv_heads=1, head_dim=64, rotary_dim=16)
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 128)).astype(np.float32)
    g = rng.standard_normal((1, 128)).astype(np.float32)
    k = rng.standard_normal((1, 64)).astype(np.float32)
    v = rng.standard_normal((1, 64)).astype(np.float32)
    kc = np.zeros((1, 64), np.float32); vc = np.zeros_like(kc)
    out, ln = port.attn_run(dims, kc, vc, 0, q, g, k, v)
    want = np.tile(v, (1, 2)) * (1.0 / (1.0 + np.exp(-g)))
    assert ln == 1
    np.testing.assert_allclose(out, want, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("window", [5, 37])
def test_port_equals_reference_sliding_window(port, ref, synth, window):
    """Circular KV cache of `window` rows (metal_infer/layer_forward.h:600-601, 649-650, 673-677): 3 * window
    steps from an empty cache wrap the buffer twice; restatement and reference agree bit for bit, and once
    wrapped the output equals plain attention over the last `window` tokens."""
    heads, kvh, D = 8, 2, 256
    steps = 3 * window
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh, sliding_window=window)
    q, g, k, v = synth.attn_step_inputs(21, steps, heads=heads, kv_heads=kvh)
    res = []
    for orc in (port, ref):
        kc = np.zeros((window, kvh * D), np.float32); vc = np.zeros_like(kc)
        out, ln = orc.attn_run(dims, kc, vc, 0, q, g, k, v, threads=2)
        assert ln == steps
        res.append((out, kc, vc))
    np.testing.assert_array_equal(res[0][0], res[1][0])
    np.testing.assert_array_equal(res[0][1], res[1][1])
    # last step against an unbounded cache that holds only the last `window` tokens (already rotated rows
    # are position-independent, so they can be replayed as a prefix)
    plain = make_dims(num_attn_heads=heads, num_kv_heads=kvh)
    kc = np.zeros((steps, kvh * D), np.float32); vc = np.zeros_like(kc)
    full, _ = port.attn_run(plain, kc, vc, 0, q, g, k, v)
    k_last, v_last = kc[steps - window:steps - 1].copy(), vc[steps - window:steps - 1].copy()
    kc2 = np.zeros((window, kvh * D), np.float32); vc2 = np.zeros_like(kc2)
    kc2[:window - 1] = k_last; vc2[:window - 1] = v_last
    last, _ = port.attn_run(plain, kc2, vc2, window - 1, q[-1:], g[-1:], k[-1:], v[-1:], start_pos=steps - 1)
    np.testing.assert_allclose(res[0][0][-1], last[0], rtol=2e-5, atol=2e-6)
