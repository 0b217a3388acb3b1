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


# ---- cache policies: FP8 store and H2O eviction -------------------------------------------------
def test_fp8_codec_port_equals_reference(port, ref, synth):
    """Bytes and scales of the FP8 E4M3 cache codec (metal_infer/fp8.h:19-118), including the values the
    reference encodes oddly: magnitudes in [2^-9, 2^-6) of the scaled range, values one ulp either side of a
    power of two, zeros, an all-zero row, the clamp at 448."""
    rows = synth.normal(31, "fp8rows", (64, 512))
    rows[1] = 0.0
    rows[2, :] = np.linspace(-1.0, 1.0, 512, dtype=np.float32) * 240.0            # scale exactly 1
    tiny = np.float32(2.0) ** np.arange(-12, -4, dtype=np.float32)
    rows[3, :8] = tiny; rows[3, 8:16] = -tiny; rows[3, 16] = 240.0
    pw = np.float32(2.0) ** np.arange(-8, 8, dtype=np.float32)
    rows[4, :16] = pw; rows[4, 16:32] = np.nextafter(pw, np.float32(0)); rows[4, 32:48] = np.nextafter(pw, np.float32(1e9))
    rows[4, 48] = 240.0
    rows[5, :256] = np.linspace(0.0, 0.02, 256, dtype=np.float32); rows[5, 256] = 240.0; rows[5, 257:] = 0.0
    b0, s0 = ref.fp8_encode_rows(rows)
    b1, s1 = port.fp8_encode_rows(rows)
    np.testing.assert_array_equal(b0, b1)
    np.testing.assert_array_equal(s0, s1)
    assert (b0 >= 0xFA).any(), "the sample must reach the reference's negative-mantissa bytes"
    allb = np.arange(256, dtype=np.uint8).reshape(1, 256)
    d0, d1 = ref.fp8_decode_rows(allb, np.array([0.37], np.float32)), port.fp8_decode_rows(allb, np.array([0.37], np.float32))
    np.testing.assert_array_equal(d0, d1)            # NaN at 0x7F in both (array_equal treats NaNs as equal)
    assert d0[0, 0xFF] == np.float32(-480.0) * np.float32(0.37)


def _run_cache(orc, dims, kv_dim, capacity, q, g, k, v, threads=1, **cache_kw):
    from oracle.oracle_py import Cache
    c = Cache(capacity, kv_dim, **cache_kw)
    out = orc.attn_run_cache(dims, c, q, g, k, v, threads=threads)
    return out, c


def test_port_equals_reference_fp8_cache(port, ref, synth):
    """Decode steps on an FP8 cache from empty: outputs, stored bytes and scales agree bit for bit (the port
    also with its per-head loop threaded: it keeps a dequantisation buffer per head)."""
    heads, kvh, D, steps = 8, 2, 256, 40
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh)
    q, g, k, v = synth.attn_step_inputs(41, steps, heads=heads, kv_heads=kvh)
    kn = synth.to_bf16_bits(1.0 + synth.normal(41, "kn", (D,), std=0.1))
    from oracle.oracle_py import Cache
    res = []
    for orc, threads in ((ref, 1), (port, 1), (port, 3)):
        c = Cache(steps, kvh * D, fp8=True)
        out = orc.attn_run_cache(dims, c, q, g, k, v, k_norm_w=kn, threads=threads)
        res.append((out, c))
    for out, c in res[1:]:
        np.testing.assert_array_equal(out, res[0][0])
        np.testing.assert_array_equal(c.k8, res[0][1].k8)
        np.testing.assert_array_equal(c.v8, res[0][1].v8)
        np.testing.assert_array_equal(c.k_scales, res[0][1].k_scales)
        np.testing.assert_array_equal(c.v_scales, res[0][1].v_scales)


@pytest.mark.parametrize("fp8", [False, True])
def test_port_equals_reference_h2o(port, ref, synth, fp8):
    """Heavy-hitter eviction (metal_infer/layer_forward.h:248-383): budget 24 with 4 sinks (so 5 recent, 15 heavy
    hitters), 70 steps from empty -- the cache is compacted on every step past the budget.  Outputs, kept rows,
    accumulated mass and original positions agree bit for bit."""
    heads, kvh, D, steps, budget = 8, 2, 256, 70, 24
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh)
    q, g, k, v = synth.attn_step_inputs(43, steps, heads=heads, kv_heads=kvh)
    from oracle.oracle_py import Cache
    res = []
    for orc in (ref, port):
        c = Cache(budget + 1, kvh * D, fp8=fp8, h2o_budget=budget, h2o_sinks=4)
        out = orc.attn_run_cache(dims, c, q, g, k, v, threads=2)
        assert c.len == steps and c.num_valid == budget
        res.append((out, c))
    (o0, c0), (o1, c1) = res
    np.testing.assert_array_equal(o0, o1)
    np.testing.assert_array_equal(c0.token_positions[:budget], c1.token_positions[:budget])
    np.testing.assert_array_equal(c0.accum[:budget], c1.accum[:budget])
    if fp8:
        np.testing.assert_array_equal(c0.k8[:budget], c1.k8[:budget])
        np.testing.assert_array_equal(c0.v_scales[:budget], c1.v_scales[:budget])
    else:
        np.testing.assert_array_equal(c0.k[:budget], c1.k[:budget])
        np.testing.assert_array_equal(c0.v[:budget], c1.v[:budget])
    assert list(c0.token_positions[:4]) == [0, 1, 2, 3]              # the sinks stay
    assert list(c0.token_positions[budget - 5:budget]) == list(range(steps - 5, steps))   # and the recent rows


@pytest.mark.parametrize("case", ["attn_fp8_h8_d256", "attn_h2o_h8_d256"])
def test_cache_policy_golden(port, ref, case):
    f = np.load(GOLD / f"{case}.npz")
    from oracle.oracle_py import Cache
    heads, kvh, D = int(f["heads"]), int(f["kv_heads"]), 256
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh)
    for orc in (port, ref):
        c = Cache(int(f["capacity"]), kvh * D, fp8=bool(f["fp8"]), h2o_budget=int(f["h2o_budget"]), h2o_sinks=4)
        out = orc.attn_run_cache(dims, c, f["q"], f["gate"], f["k"], f["v"])
        np.testing.assert_array_equal(out, f["out"])
        if bool(f["fp8"]):
            np.testing.assert_array_equal(c.k8, f["k8"])
            np.testing.assert_array_equal(c.k_scales, f["k_scales"])
        if int(f["h2o_budget"]):
            np.testing.assert_array_equal(c.token_positions, f["token_positions"])
            np.testing.assert_array_equal(c.accum, f["accum"])


def test_port_equals_reference_out_proj_norm(port, ref, synth):
    """Output projection from the 4-bit affine format + residual + post-attention RMS-norm: bit for bit."""
    rng = np.random.default_rng(3)
    out_dim, in_dim = 96, 1024
    w = rng.integers(0, 2 ** 32, size=(out_dim, in_dim // 8), dtype=np.uint64).astype(np.uint32)
    scales = synth.to_bf16_bits(np.abs(synth.normal(3, "s", (out_dim, in_dim // 64), std=0.01)) + 0.002)
    biases = synth.to_bf16_bits(-7.5 * synth.bf16_bits_to_f32(scales) + synth.normal(3, "b", (out_dim, in_dim // 64), std=0.002))
    x = synth.normal(3, "x", (3, in_dim)); res = synth.normal(3, "r", (3, out_dim))
    nw = synth.to_bf16_bits(1.0 + synth.normal(3, "nw", (out_dim,), std=0.1))
    a = ref.out_proj_norm(w, scales, biases, x, res, nw)
    b = port.out_proj_norm(w, scales, biases, x, res, nw)
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])
