"""fm_seq_fork: a sequence continues from another's prefix, sharing its full KV pages (needs a B200).
Both branches are checked against the CPU checker run separately from the same prefix, page accounting is
checked through resets."""
import numpy as np
import pytest

from gpu_util import oracle_attn
from oracle.oracle_py import make_dims
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3


def test_fork_shares_prefix_pages_and_branches_diverge(pkg, port, synth):
    heads, kvh, L, steps = 32, 2, 150, 70   # 2 full pages + 22 rows; 70 steps cross a page boundary
    cfg = pkg.default_config(num_attn_heads=heads, num_kv_heads=kvh, num_full_layers=2, num_linear_layers=1, max_seqs=3,
                             max_seq_len=512)
    c = pkg.Context(cfg, host_pointers=True)
    total = c.kv_free_pages()
    k0, v0 = synth.attn_cache(71, L)
    for layer in range(2):
        c.kv_import(layer, 0, k0, v0, L)
    # recurrent state of the source: a few GatedDeltaNet steps
    w = synth.gdn_weights(8)
    qkv, z, beta, alpha = synth.gdn_step_inputs(72, 5)
    go = np.empty((1, 8192), np.float32)
    for t in range(3):
        c.gdn_decode(0, [0], qkv[t:t + 1].copy(), z[t:t + 1].copy(), beta[t:t + 1].copy(), alpha[t:t + 1].copy(), go,
                     w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
    assert c.kv_free_pages() == total - 2 * 3
    c.seq_fork(0, 1)
    assert c.kv_free_pages() == total - 2 * 3 - 2 * 1   # only the partly filled page of each layer is new
    assert c.kv_len(0, 1) == L and c.kv_len(1, 1) == L
    # the two branches see different tokens
    branches = {0: synth.attn_step_inputs(73, steps, tag="a"), 1: synth.attn_step_inputs(74, steps, tag="b")}
    refs = {}
    for s, (q, g, k, v) in branches.items():
        refs[s] = oracle_attn(port, heads, kvh, k0, v0, q, g, synth.round_bf16(k), synth.round_bf16(v))[0]
    worst = 0.0
    for t in range(steps):
        for s, (q, g, k, v) in branches.items():
            for layer in range(2):
                out = np.empty((1, heads * 256), np.float32)
                c.attn_decode(layer, [s], [L + t], out, q=q[t:t + 1].copy(), gate=g[t:t + 1].copy(),
                              k=synth.round_bf16(k[t:t + 1]), v=synth.round_bf16(v[t:t + 1]))
                gated, _, _ = rel_errors(out[0], refs[s][t])
                worst = max(worst, gated)
                assert gated <= TOL, (t, s, layer, gated)
    # the forked recurrent state continues exactly like the source's
    outs = []
    for s in (0, 1):
        o = np.empty((1, 8192), np.float32)
        c.gdn_decode(0, [s], qkv[3:4].copy(), z[3:4].copy(), beta[3:4].copy(), alpha[3:4].copy(), o,
                     w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
        outs.append(o)
    np.testing.assert_array_equal(outs[0], outs[1])
    # dropping the source leaves the fork intact (its shared pages stay alive)
    c.reset(0)
    q, g, k, v = branches[1]
    extra = synth.attn_step_inputs(75, 1, tag="c")
    kc = np.zeros((L + steps + 1, kvh * 256), np.float32); vc = np.zeros_like(kc)
    kc[:L] = k0; vc[:L] = v0
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kvh, store_bf16=1)
    port.attn_run(dims, kc, vc, L, q, g, synth.round_bf16(k), synth.round_bf16(v), threads=8)
    ref, _ = port.attn_run(dims, kc, vc, L + steps, extra[0], extra[1], synth.round_bf16(extra[2]), synth.round_bf16(extra[3]), threads=8)
    out = np.empty((1, heads * 256), np.float32)
    c.attn_decode(0, [1], [L + steps], out, q=extra[0], gate=extra[1], k=synth.round_bf16(extra[2]), v=synth.round_bf16(extra[3]))
    gated, _, _ = rel_errors(out[0], ref[0])
    assert gated <= TOL
    c.reset(1)
    assert c.kv_free_pages() == total
    c.close()
    print("fork: worst gated", worst)
