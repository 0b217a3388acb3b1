"""Sliding-window KV store (circular buffer of W rows) through the C-ABI against the CPU checker run with the
same window (needs a B200).  The reference's rule: row = token count % W, attention over the last
min(count, W) tokens (metal_infer/layer_forward.h:600-601, 649-650, 673-677)."""
import numpy as np
import pytest

from gpu_util import attn_ctx
from oracle.oracle_py import make_dims
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.mark.parametrize("window,steps", [(200, 470), (64, 200), (1000, 1100)])
def test_decode_with_sliding_window_matches_checker(pkg, port, synth, window, steps):
    """From an empty store through two wraps (window not a multiple of the page size in the first case); every
    step's output is compared, and the store's rows equal the checker's circular buffer up to bf16 rounding."""
    heads, kvh = 32, 2
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh, sliding_window=window, store_bf16=1)
    q, g, k, v = synth.attn_step_inputs(31, steps)
    kc = np.zeros((window, kvh * 256), np.float32); vc = np.zeros_like(kc)
    ref, ln = port.attn_run(dims, kc, vc, 0, q, g, k, v, threads=8)
    assert ln == steps
    c = attn_ctx(pkg, heads, kvh, max_seq_len=4096, sliding_window=window)
    worst = 0.0
    for t in range(steps):
        out = np.empty((1, heads * 256), np.float32)
        c.attn_decode(0, [0], [t], out, q=q[t:t + 1].copy(), gate=g[t:t + 1].copy(), k=k[t:t + 1].copy(), v=v[t:t + 1].copy())
        gated, _, _ = rel_errors(out[0], ref[t])
        worst = max(worst, gated)
        assert gated <= TOL, (t, gated)
    assert c.kv_len(0, 0) == steps                      # the count keeps growing, as kv->len does
    ke = np.zeros((window, kvh * 256), np.float32); ve = np.zeros_like(ke)
    assert c.kv_export(0, 0, ke, ve, window) == window  # rows in store order
    c.close()
    np.testing.assert_allclose(ke, kc, rtol=2 ** -7, atol=1e-6)
    np.testing.assert_allclose(ve, vc, rtol=2 ** -7, atol=1e-6)
    print("window", window, "steps", steps, "worst gated", worst)


def test_window_batch_and_limits(pkg, port, synth):
    """Two sequences at different fill levels in one call; prefill that would wrap is refused; a window larger than
    max_seq_len is rejected at creation."""
    heads, kvh, window = 32, 2, 130
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh, sliding_window=window, store_bf16=1)
    c = attn_ctx(pkg, heads, kvh, max_seq_len=1024, max_seqs=2, max_batch=128, sliding_window=window)
    steps = [150, 40]
    ins = [synth.attn_step_inputs(41 + s, steps[s], tag=f"s{s}") for s in range(2)]
    refs = []
    for s in range(2):
        q, g, k, v = ins[s]
        kc = np.zeros((window, kvh * 256), np.float32); vc = np.zeros_like(kc)
        refs.append(port.attn_run(dims, kc, vc, 0, q, g, k, v, threads=8)[0])
    for t in range(max(steps)):
        seqs = [s for s in range(2) if t < steps[s]]
        st = lambda i: np.ascontiguousarray(np.stack([ins[s][i][t] for s in seqs]))
        out = np.empty((len(seqs), heads * 256), np.float32)
        c.attn_decode(0, seqs, [t] * len(seqs), out, q=st(0), gate=st(1), k=st(2), v=st(3))
        for j, s in enumerate(seqs):
            gated, _, _ = rel_errors(out[j], refs[s][t])
            assert gated <= TOL, (t, s, gated)
    q, g, k, v = synth.attn_step_inputs(43, 100)
    with pytest.raises(pkg.FmError) as e:
        c.attn_prefill(0, 1, 40, 100, np.empty((100, heads * 256), np.float32), q=q, gate=g, k=k, v=v)
    assert e.value.status == pkg.binding.FM_ERR_UNSUPPORTED
    c.close()
    with pytest.raises(pkg.FmError):
        attn_ctx(pkg, heads, kvh, max_seq_len=128, sliding_window=500)


def test_window_on_a_sequence_sharded_store(pkg, port, synth):
    """Sliding window of 300 rows held by two sequence-shard contexts (alternating pages of the circular buffer):
    every step both compute their partial result, merged by log-sum-exp + gate, through a wrap of the window."""
    heads, kvh, window, steps = 32, 2, 300, 420
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh, sliding_window=window, store_bf16=1)
    q, g, k, v = synth.attn_step_inputs(51, steps)
    kc = np.zeros((window, kvh * 256), np.float32); vc = np.zeros_like(kc)
    ref, _ = port.attn_run(dims, kc, vc, 0, q, g, k, v, threads=8)
    shards = [attn_ctx(pkg, heads, kvh, max_seq_len=2048, shard=(r, 2), sliding_window=window) for r in range(2)]
    merger = attn_ctx(pkg, heads, kvh, max_seq_len=128)
    worst = 0.0
    for t in range(steps):
        po, pml = [], []
        for c in shards:
            o = np.empty((1, heads, 256), np.float32); ml = np.empty((1, heads, 2), np.float32)
            c.attn_decode_partial(0, [0], [t], o, ml, q=q[t:t + 1].copy(), k=k[t:t + 1].copy(), v=v[t:t + 1].copy())
            po.append(o); pml.append(ml)
        out = np.empty((1, heads * 256), np.float32)
        merger.attn_merge_gate(2, np.stack(po), np.stack(pml), 1, out, gate=g[t:t + 1].copy())
        gated, _, _ = rel_errors(out[0], ref[t])
        worst = max(worst, gated)
        assert gated <= TOL, (t, gated)
    for c in shards + [merger]:
        c.close()
    print("sharded window worst gated", worst)
