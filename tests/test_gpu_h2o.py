"""Heavy-hitter (H2O) eviction of the KV store through the C-ABI against the CPU checker running the reference's
H2O cache (metal_infer/layer_forward.h:248-383, 591-727): outputs of every step, and after the last step the rows
kept (their original token positions), their contents in cache order and their accumulated attention mass."""
import numpy as np
import pytest

from gpu_util import attn_ctx
from oracle.oracle_py import Cache, host_threads, make_dims
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.mark.parametrize("heads,kv_heads,budget,steps,fp8", [(8, 2, 24, 70, False), (32, 2, 100, 260, False), (32, 2, 100, 180, True),
                                                           (32, 2, 700, 760, False)])
def test_h2o_decode_matches_checker(pkg, port, synth, heads, kv_heads, budget, steps, fp8):
    kvd = kv_heads * 256
    q, g, k, v = synth.attn_step_inputs(300 + budget, steps, heads=heads, kv_heads=kv_heads)
    if not fp8:
        k, v = synth.round_bf16(k), synth.round_bf16(v)
    qn = synth.to_bf16_bits(1.0 + synth.normal(5, "qn", (256,), std=0.1))
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kv_heads, store_bf16=0 if fp8 else 1)
    cache = Cache(budget + 1, kvd, fp8=fp8, h2o_budget=budget, h2o_sinks=4)
    want = port.attn_run_cache(dims, cache, q, g, k, v, qn, None, start_pos=0, threads=host_threads())
    c = attn_ctx(pkg, heads, kv_heads, max_seq_len=4096, h2o_budget=budget, h2o_num_sinks=4,
                 kv_dtype=pkg.binding.FM_KV_FP8_E4M3 if fp8 else pkg.binding.FM_KV_BF16)
    got = np.empty_like(want)
    for t in range(steps):
        c.attn_decode(0, [0], [t], got[t:t + 1], q=q[t:t + 1].copy(), gate=g[t:t + 1].copy(), k=k[t:t + 1].copy(), v=v[t:t + 1].copy(),
                      q_norm_w=qn)
    assert c.kv_len(0, 0) == steps
    n = min(steps, budget)
    acc = np.zeros(n, np.float32); tp = np.zeros(n, np.int32)
    assert c.h2o_export(0, 0, acc, tp, n) == n
    ke = np.zeros((n, kvd), np.float32); ve = np.zeros_like(ke)
    assert c.kv_export(0, 0, ke, ve, n) == n
    c.close()
    worst = 0.0
    for t in range(steps):
        gated, _, _ = rel_errors(got[t], want[t])
        worst = max(worst, gated)
    print("H2O budget", budget, "steps", steps, "fp8", fp8, "worst gated", worst)
    assert cache.num_valid == n
    np.testing.assert_array_equal(tp, cache.token_positions[:n])          # the same rows survive, in the same order
    np.testing.assert_allclose(acc, cache.accum[:n], rtol=2e-3, atol=1e-5)
    if fp8:
        np.testing.assert_array_equal(ve, port.fp8_decode_rows(cache.v8[:n], cache.v_scales[:n]))
    else:
        np.testing.assert_array_equal(ve, cache.v[:n])
        np.testing.assert_allclose(ke, cache.k[:n], rtol=2 ** -7, atol=1e-6)
    assert worst <= TOL
    assert list(tp[:4]) == [0, 1, 2, 3]


def test_h2o_batched_and_limits(pkg, port, synth):
    """Two sequences of different ages in one call; entry points that cannot serve an H2O store say so."""
    budget = 40
    c = attn_ctx(pkg, 32, 2, max_seq_len=1024, max_seqs=2, h2o_budget=budget)
    dims = make_dims(store_bf16=1)
    caches = [Cache(budget + 1, 512, h2o_budget=budget) for _ in range(2)]
    ins = [synth.attn_step_inputs(70 + s, 90) for s in range(2)]
    ins = [(q, g, synth.round_bf16(k), synth.round_bf16(v)) for q, g, k, v in ins]
    for t in range(30):   # sequence 1 starts 30 tokens ahead
        q, g, k, v = ins[1]
        o = np.empty((1, 8192), np.float32)
        c.attn_decode(0, [1], [t], o, q=q[t:t + 1].copy(), gate=g[t:t + 1].copy(), k=k[t:t + 1].copy(), v=v[t:t + 1].copy())
        port.attn_run_cache(dims, caches[1], q[t:t + 1], g[t:t + 1], k[t:t + 1], v[t:t + 1], start_pos=t, threads=host_threads())
    worst = 0.0
    for t in range(60):
        t0, t1 = t, t + 30
        qq = np.concatenate([ins[0][0][t0:t0 + 1], ins[1][0][t1:t1 + 1]]); gg = np.concatenate([ins[0][1][t0:t0 + 1], ins[1][1][t1:t1 + 1]])
        kk = np.concatenate([ins[0][2][t0:t0 + 1], ins[1][2][t1:t1 + 1]]); vv = np.concatenate([ins[0][3][t0:t0 + 1], ins[1][3][t1:t1 + 1]])
        o = np.empty((2, 8192), np.float32)
        c.attn_decode(0, [0, 1], [t0, t1], o, q=qq, gate=gg, k=kk, v=vv)
        for s, tt in ((0, t0), (1, t1)):
            w = port.attn_run_cache(dims, caches[s], ins[s][0][tt:tt + 1], ins[s][1][tt:tt + 1], ins[s][2][tt:tt + 1], ins[s][3][tt:tt + 1],
                                    start_pos=tt, threads=host_threads())
            worst = max(worst, rel_errors(o[s], w[0])[0])
    print("batched H2O worst gated", worst)
    assert worst <= TOL
    for s in range(2):
        n = caches[s].num_valid
        tp = np.zeros(n, np.int32)
        assert c.h2o_export(0, s, None, tp, n) == n
        np.testing.assert_array_equal(tp, caches[s].token_positions[:n])
    q, g, k, v = ins[0]
    o = np.empty((4, 8192), np.float32)
    with pytest.raises(pkg.FmError) as e:
        c.attn_prefill(0, 0, 60, 4, o, q=q[:4].copy(), gate=g[:4].copy(), k=k[:4].copy(), v=v[:4].copy())
    assert e.value.status == pkg.binding.FM_ERR_UNSUPPORTED
    with pytest.raises(pkg.FmError) as e:
        c.kv_append_rope(0, [0], [60], k[:1].copy(), v[:1].copy())
    assert e.value.status == pkg.binding.FM_ERR_UNSUPPORTED
    with pytest.raises(pkg.FmError) as e:
        c.seq_fork(0, 1)
    assert e.value.status == pkg.binding.FM_ERR_UNSUPPORTED
    c.reset(0)
    assert c.kv_len(0, 0) == 0
    c.close()
