"""Prefill entry points against sequential CPU steps (needs a B200)."""
import numpy as np
import pytest

from gpu_util import attn_ctx, gdn_ctx, oracle_attn
from oracle.oracle_py import make_dims
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3
TOL_GDN = 5e-3


@pytest.mark.parametrize("n,prefix", [(1, 0), (70, 0), (128, 0), (129, 0), (256, 0), (100, 150), (300, 1000), (2048, 0)])
def test_attn_prefill_matches_sequential_steps(pkg, port, synth, n, prefix):
    """Causal prefill of n tokens after `prefix` cached rows against n sequential CPU steps;
    bf16-representable q, k, v as in the bf16 prefill configuration, the checker rounding the
    rotated k rows to bf16 as the store does."""
    k0, v0 = synth.attn_cache(70 + n, prefix)
    q, g, k, v = synth.attn_step_inputs(70 + n, n, bf16=True)
    c = attn_ctx(pkg, 32, 2, max_seq_len=prefix + n + 10, max_batch=max(64, n))
    c.kv_import(0, 0, k0, v0, prefix)
    out = np.empty((n, 8192), np.float32)
    c.attn_prefill(0, 0, prefix, n, out, q=q, gate=g, k=k, v=v)
    L = c.kv_len(0, 0)
    assert L == prefix + n
    ke = np.zeros((L, 512), np.float32); ve = np.zeros_like(ke)
    c.kv_export(0, 0, ke, ve, L)
    c.close()
    ref_out, kc, vc = oracle_attn(port, 32, 2, k0, v0, q, g, k, v, start_pos=prefix)
    np.testing.assert_allclose(ke, kc, rtol=2 ** -7, atol=1e-6)
    gated, mom, rr = rel_errors(out, ref_out)
    print("prefill n", n, "prefix", prefix, "gated", gated, "rms-rel", rr)
    assert gated <= TOL


def test_attn_prefill_in_small_calls(pkg, port, synth):
    """A 4096-token prompt fed 32 tokens at a time (the reference's batch, MAX_PFB_GPU, metal_infer/shaders.metal:2130)
    with a few decode steps in the middle: the result equals 4096 sequential CPU steps, and the cost of a call does not
    grow with the rows already cached beyond what attending to them takes (each cached row is converted into the
    kernel's operand workspace once, not once per call)."""
    import time
    import torch
    T, step = 4096, 32
    q, g, k, v = synth.attn_step_inputs(91, T, bf16=True)
    dev = torch.device("cuda:0")
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seq_len=T + 8, max_batch_tokens=64)
    c = pkg.Context(cfg)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    tq, tg, tk, tv = (torch.from_numpy(a).to(dev) for a in (q, g, k, v))
    out = torch.empty((T, 8192), device=dev)
    times = []
    t = 0
    while t < T:
        if t == 2048:  # two decode steps in the middle of the prompt: the workspace has to pick their rows up
            for _ in range(2):
                c.attn_decode(0, [0], [t], out[t:t + 1], q=tq[t:t + 1], gate=tg[t:t + 1], k=tk[t:t + 1], v=tv[t:t + 1])
                t += 1
            continue
        n = min(step, T - t)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        c.attn_prefill(0, 0, t, n, out[t:t + n], q=tq[t:t + n], gate=tg[t:t + n], k=tk[t:t + n], v=tv[t:t + n])
        torch.cuda.synchronize()
        times.append((t, time.perf_counter() - t0))
        t += n
    got = out.cpu().numpy()
    c.close()
    ref_out, _, _ = oracle_attn(port, 32, 2, np.zeros((0, 512), np.float32), np.zeros((0, 512), np.float32), q, g, k, v, start_pos=0,
                                threads=16)
    gated, _, rr = rel_errors(got, ref_out)
    print("prefill in 32-token calls: gated", gated, "rms-rel", rr)
    assert gated <= TOL
    early = np.median([d for t_, d in times if 256 <= t_ < 768]); late = np.median([d for t_, d in times if t_ >= 3584])
    print("seconds per call: early %.2e late %.2e" % (early, late))
    assert late <= 3.0 * early + 30e-6


@pytest.mark.parametrize("sizes", [(1,), (63,), (64,), (65,), (200,), (100, 70, 3), (4096,)])
def test_gdn_prefill_matches_sequential_steps(pkg, port, synth, sizes):
    """Chunked GatedDeltaNet prefill against sequential CPU steps: output, final recurrent state and
    conv history; bf16-representable inputs, fp32 state ~ N(0, 0.02^2).  (4096,) is the full chunked
    prefill configuration (sequence 4096, chunk 64, 16 qk / 64 v heads x 128); several sizes in a
    row exercise continuation across calls, and a decode step continues from the prefilled state."""
    n = sum(sizes)
    dims = make_dims()
    w = synth.gdn_weights(8)
    qkv, z, beta, alpha = synth.gdn_step_inputs(8, n, bf16=True)
    s0 = synth.gdn_state(8)
    conv_ref = np.zeros((3, 12288), np.float32); ssm_ref = s0.copy()
    out_ref = port.gdn_run(dims, conv_ref, ssm_ref, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"],
                           w["norm_w"], threads=16)
    c = gdn_ctx(pkg, max_batch=max(sizes))
    c.state_import(0, 0, None, s0)
    out = np.empty((n, 8192), np.float32)
    t = 0
    for m in sizes:
        c.gdn_prefill(0, 0, m, qkv[t:t + m].copy(), z[t:t + m].copy(), beta[t:t + m].copy(), alpha[t:t + m].copy(),
                      out[t:t + m], w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
        t += m
    conv = np.empty((3, 12288), np.float32); ssm = np.empty((64, 128, 128), np.float32)
    c.state_export(0, 0, conv, ssm)
    q1, z1, b1, a1 = synth.gdn_step_inputs(9, 1)
    o1 = np.empty((1, 8192), np.float32)
    c.gdn_decode(0, [0], q1, z1, b1, a1, o1, w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
    c.close()
    r1 = port.gdn_run(dims, conv_ref.copy(), ssm_ref.copy(), q1, z1, b1, a1, w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
    np.testing.assert_array_equal(conv, conv_ref)
    gs, _, rs = rel_errors(ssm, ssm_ref)
    go, _, ro = rel_errors(out, out_ref)
    g1, _, _ = rel_errors(o1, r1)
    print("gdn prefill", sizes, "state", gs, rs, "out", go, ro, "next step", g1)
    assert gs <= TOL_GDN and go <= TOL_GDN and g1 <= TOL_GDN


@pytest.mark.parametrize("shards", [2, 4])
def test_attn_prefill_on_a_sequence_sharded_store(pkg, port, synth, shards):
    """A prompt prefilled in three calls on every shard of a sequence-sharded store (each shard is given the run's
    k and v, keeps the rows of its own pages and attends over the whole prompt): every shard returns the checker's
    output, the shards' rows put together are the checker's cache, and a decode step whose partial results are merged
    by log-sum-exp continues from there."""
    sizes = (130, 64, 107)
    n = sum(sizes)
    q, g, k, v = synth.attn_step_inputs(55, n + 1, bf16=True)
    empty = np.zeros((0, 512), np.float32)
    ref_out, kc, vc = oracle_attn(port, 32, 2, empty, empty, q, g, k, v, start_pos=0)
    ctxs = [attn_ctx(pkg, 32, 2, max_seq_len=n + 70, max_batch=256, shard=(r, shards)) for r in range(shards)]
    ke = np.zeros((n, 512), np.float32); ve = np.zeros_like(ke)
    for r, c in enumerate(ctxs):
        out = np.empty((n, 8192), np.float32)
        t = 0
        for m in sizes:
            c.attn_prefill(0, 0, t, m, out[t:t + m], q=q[t:t + m].copy(), gate=g[t:t + m].copy(), k=k[t:t + m].copy(), v=v[t:t + m].copy())
            t += m
        gated, _, rr = rel_errors(out, ref_out[:n])
        print("shard", r, "of", shards, "prefill gated", gated)
        assert gated <= TOL
        assert c.kv_len(0, 0) == n
        c.kv_export(0, 0, ke, ve, n)          # fills the rows this shard owns
    np.testing.assert_allclose(ke, kc[:n], rtol=2 ** -7, atol=1e-6)
    np.testing.assert_array_equal(ve, vc[:n])
    parts_o, parts_ml = [], []
    for c in ctxs:
        o = np.empty((1, 32, 256), np.float32); ml = np.empty((1, 32, 2), np.float32)
        c.attn_decode_partial(0, [0], [n], o, ml, q=q[n:n + 1].copy(), k=k[n:n + 1].copy(), v=v[n:n + 1].copy())
        parts_o.append(o); parts_ml.append(ml)
    out1 = np.empty((1, 8192), np.float32)
    ctxs[0].attn_merge_gate(shards, np.stack(parts_o), np.stack(parts_ml), 1, out1, gate=g[n:n + 1].copy())
    gated, _, _ = rel_errors(out1, ref_out[n:n + 1])
    print("decode step after the sharded prefill: gated", gated)
    assert gated <= TOL
    # a prompt that does not start at the sequence's first token cannot be served from one shard's rows
    with pytest.raises(pkg.FmError) as e:
        ctxs[1].attn_prefill(0, 0, n + 1, 4, np.empty((4, 8192), np.float32), q=q[:4].copy(), gate=g[:4].copy(), k=k[:4].copy(), v=v[:4].copy())
    assert e.value.status == pkg.binding.FM_ERR_UNSUPPORTED
    for c in ctxs:
        c.close()
