"""GatedDeltaNet decode through the C-ABI against the CPU checker (needs a B200)."""
from pathlib import Path

import numpy as np
import pytest

from gpu_util import gdn_ctx
from oracle.oracle_py import make_dims
from parity import rel_errors

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"

# tolerance of the task statement: 5e-3 on the recurrent state after 1000 steps
TOL_STATE = 5e-3
TOL_OUT = 5e-3


def test_golden_gdn(pkg):
    f = np.load(GOLD / "gdn_v4_k1_d128.npz")
    c = gdn_ctx(pkg, 4, 1)
    n = int(f["steps"])
    outs = []
    for t in range(n):
        out = np.empty((1, 512), np.float32)
        c.gdn_decode(0, [0], f["qkv"][t:t + 1].copy(), f["z"][t:t + 1].copy(), f["beta"][t:t + 1].copy(),
                     f["alpha"][t:t + 1].copy(), out, f["conv_w"], f["A_log"], f["dt_bias"], f["norm_w"])
        outs.append(out)
    conv = np.empty((3, 768), np.float32); ssm = np.empty((4, 128, 128), np.float32)
    c.state_export(0, 0, conv, ssm)
    c.close()
    np.testing.assert_array_equal(conv, f["conv_final"])
    g1, _, r1 = rel_errors(np.concatenate(outs), f["out"])
    g2, _, r2 = rel_errors(ssm, f["ssm_final"])
    print("golden gdn out", g1, r1, "state", g2, r2)
    assert g1 <= 1e-4 and g2 <= 1e-4


def test_config2_1000_steps(pkg, port, synth):
    """1000 sequential tokens at the production shape (16 q/k heads, 64 v heads, 128x128 fp32 state
    ~ N(0, 0.02^2)); state and outputs against the CPU recurrence."""
    n = 1000
    dims = make_dims()
    w = synth.gdn_weights(0)
    qkv, z, beta, alpha = synth.gdn_step_inputs(0, n)
    s0 = synth.gdn_state(0)
    conv_ref = np.zeros((3, 12288), np.float32); ssm_ref = s0.copy()
    out_ref = port.gdn_run(dims, conv_ref, ssm_ref, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"],
                           w["norm_w"], threads=8)
    c = gdn_ctx(pkg)
    c.state_import(0, 0, None, s0)
    outs = np.empty((n, 8192), np.float32)
    for t in range(n):
        c.gdn_decode(0, [0], qkv[t:t + 1].copy(), z[t:t + 1].copy(), beta[t:t + 1].copy(), alpha[t:t + 1].copy(),
                     outs[t:t + 1], w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
    conv = np.empty((3, 12288), np.float32); ssm = np.empty((64, 128, 128), np.float32)
    c.state_export(0, 0, conv, ssm)
    c.close()
    np.testing.assert_array_equal(conv, conv_ref)
    gs, _, rs = rel_errors(ssm, ssm_ref)
    go, _, ro = rel_errors(outs, out_ref)
    print("config2 state gated", gs, "rms-rel", rs, "| out gated", go, "rms-rel", ro)
    assert gs <= TOL_STATE and go <= TOL_OUT


def test_batched_sequences_and_layers(pkg, port, synth):
    """Batch of 5 sequences (uses the whole-head-per-CTA variants) on the second of two layers; the
    first layer's state stays zero."""
    B, n = 5, 6
    dims = make_dims()
    w = synth.gdn_weights(3)
    c = gdn_ctx(pkg, max_seqs=B, layers=2)
    refs, states = [], []
    ins = [synth.gdn_step_inputs(40 + s, n) for s in range(B)]
    for s in range(B):
        conv = np.zeros((3, 12288), np.float32); ssm = synth.gdn_state(40 + s).copy()
        c.state_import(1, s, None, ssm)
        refs.append(port.gdn_run(dims, conv, ssm, *ins[s], w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"], threads=8))
        states.append(ssm)
    for t in range(n):
        pack = lambda j: np.ascontiguousarray(np.stack([ins[s][j][t] for s in range(B)]))
        out = np.empty((B, 8192), np.float32)
        c.gdn_decode(1, list(range(B)), pack(0), pack(1), pack(2), pack(3), out, w["conv_w"], w["A_log"],
                     w["dt_bias"], w["norm_w"])
        for s in range(B):
            g, _, _ = rel_errors(out[s], refs[s][t])
            assert g <= 1e-4, (t, s, g)
    for s in range(B):
        ssm = np.empty((64, 128, 128), np.float32)
        c.state_export(1, s, None, ssm)
        g, _, _ = rel_errors(ssm, states[s])
        assert g <= 1e-4
    z0 = np.ones((64, 128, 128), np.float32)
    c.state_export(0, 0, None, z0)
    assert not z0.any()
    c.close()


def test_large_batch_whole_head_variant(pkg, port, synth):
    B = 9  # 64 heads x 9 >= 512 CTAs: one CTA per head
    dims = make_dims()
    w = synth.gdn_weights(4)
    c = gdn_ctx(pkg, max_seqs=B)
    qkv, z, beta, alpha = synth.gdn_step_inputs(50, B)
    out = np.empty((B, 8192), np.float32)
    for s in range(B):
        c.state_import(0, s, None, synth.gdn_state(60 + s))
    c.gdn_decode(0, list(range(B)), qkv, z, beta, alpha, out, w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
    for s in range(B):
        conv = np.zeros((3, 12288), np.float32); ssm = synth.gdn_state(60 + s).copy()
        r = port.gdn_run(dims, conv, ssm, qkv[s:s + 1], z[s:s + 1], beta[s:s + 1], alpha[s:s + 1], w["conv_w"],
                         w["A_log"], w["dt_bias"], w["norm_w"], threads=8)
        g, _, _ = rel_errors(out[s], r)
        assert g <= 1e-4
    c.close()


@pytest.mark.parametrize("B,defaults", [(24, False), (8, True), (64, False)])
def test_streamed_states_many_pairs(pkg, port, synth, B, defaults):
    """64 heads x B >= 512 (head, sequence) pairs: the persistent form that streams the states through shared memory.
    Several steps per sequence (ring slots and stages are reused, 1536 pairs do not divide by the SM count), outputs of
    every step and the final recurrent and conv states against the checker; once with the reference's defaults for
    absent A_log / dt_bias / norm weight."""
    n = 5 if B < 64 else 2
    dims = make_dims()
    w = synth.gdn_weights(11)
    wa = (w["conv_w"], None, None, None) if defaults else (w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
    c = gdn_ctx(pkg, max_seqs=B)
    refs, states, convs = [], [], []
    ins = [synth.gdn_step_inputs(300 + s, n) for s in range(B)]
    for s in range(B):
        conv = np.zeros((3, 12288), np.float32); ssm = synth.gdn_state(300 + s).copy()
        c.state_import(0, s, None, ssm)
        refs.append(port.gdn_run(dims, conv, ssm, *ins[s], *wa, threads=8))
        states.append(ssm); convs.append(conv)
    for t in range(n):
        pack = lambda j: np.ascontiguousarray(np.stack([ins[s][j][t] for s in range(B)]))
        out = np.empty((B, 8192), np.float32)
        c.gdn_decode(0, list(range(B)), pack(0), pack(1), pack(2), pack(3), out, *wa)
        for s in range(B):
            g, _, _ = rel_errors(out[s], refs[s][t])
            assert g <= 1e-4, (t, s, g)
    for s in range(0, B, max(1, B // 8)):
        ssm = np.empty((64, 128, 128), np.float32); conv = np.empty((3, 12288), np.float32)
        c.state_export(0, s, conv, ssm)
        g, _, _ = rel_errors(ssm, states[s])
        assert g <= 1e-4
        assert np.array_equal(conv, convs[s])
    c.close()


def test_steps_of_different_layers_may_overlap(pkg, port, synth):
    """fm_set_layer_overlap: with device pointers, the steps of three layers are issued round-robin, each launch a
    programmatic dependent of the previous one (it fetches its state before the previous launch has finished and waits
    for it before touching its inputs).  Every layer's outputs and final state against the checker."""
    import torch
    dev = torch.device("cuda:0")
    layers, n = 3, 6
    dims = make_dims()
    cfg = pkg.default_config(num_full_layers=0, num_linear_layers=layers, max_seqs=1, max_batch_tokens=64)
    c = pkg.Context(cfg)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    c.set_layer_overlap(True)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a.view(np.int16) if a.dtype == np.uint16 else a)).to(dev)
    ws = [synth.gdn_weights(20 + l) for l in range(layers)]
    wd = [{k: t(v) for k, v in w.items()} for w in ws]
    ins = [synth.gdn_step_inputs(400 + l, n) for l in range(layers)]
    refs, states = [], []
    for l in range(layers):
        conv = np.zeros((3, 12288), np.float32); ssm = synth.gdn_state(400 + l).copy()
        c.state_import(l, 0, None, t(ssm))
        refs.append(port.gdn_run(dims, conv, ssm, *ins[l], ws[l]["conv_w"], ws[l]["A_log"], ws[l]["dt_bias"], ws[l]["norm_w"], threads=8))
        states.append(ssm)
    dins = [[t(a) for a in ins[l]] for l in range(layers)]
    outs = [[torch.empty((1, 8192), device=dev) for _ in range(n)] for _ in range(layers)]
    for st in range(n):
        for l in range(layers):
            qkv, z, beta, alpha = (a[st:st + 1] for a in dins[l])
            c.gdn_decode(l, [0], qkv, z, beta, alpha, outs[l][st], wd[l]["conv_w"], wd[l]["A_log"], wd[l]["dt_bias"], wd[l]["norm_w"])
    c.synchronize()
    for l in range(layers):
        for st in range(n):
            g, _, _ = rel_errors(outs[l][st].cpu().numpy(), refs[l][st])
            assert g <= 1e-4, (l, st, g)
        ssm = torch.empty((64, 128, 128), device=dev)
        c.state_export(l, 0, None, ssm)
        c.synchronize()
        g, _, _ = rel_errors(ssm.cpu().numpy(), states[l])
        assert g <= 1e-4
    c.close()


def test_reset_and_reference_defaults(pkg, port, synth):
    """NULL A_log / dt_bias / norm weight mean A = 1, bias 0, no output norm, as in the reference;
    fm_reset returns the layer to the zero state."""
    dims = make_dims(linear_num_v_heads=8, linear_num_k_heads=2)
    c = gdn_ctx(pkg, 8, 2)
    w = synth.gdn_weights(6, 8, 2)
    qkv, z, beta, alpha = synth.gdn_step_inputs(6, 3, 8, 2)
    for rep in range(2):
        conv = np.zeros((3, 1536), np.float32); ssm = np.zeros((8, 128, 128), np.float32)
        ref = port.gdn_run(dims, conv, ssm, qkv, z, beta, alpha, w["conv_w"], None, None, None)
        for t in range(3):
            out = np.empty((1, 1024), np.float32)
            c.gdn_decode(0, [0], qkv[t:t + 1].copy(), z[t:t + 1].copy(), beta[t:t + 1].copy(), alpha[t:t + 1].copy(), out,
                         w["conv_w"], None, None, None)
            g, _, _ = rel_errors(out, ref[t])
            assert g <= 1e-4
        c.reset(0)
    c.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_head_sharded_contexts_reproduce_the_full_layer(pkg, port, synth, world):
    """GatedDeltaNet across GPUs shards by value head with no exchange: `world` contexts, each holding 64 / world value
    heads and 16 / world key heads (pkg.sharding.gdn_head_slice / gdn_slice_inputs), run a chunked prefill and decode
    steps on their slices; outputs and final states concatenated over the ranks equal the checker's full layer."""
    from oracle.oracle_py import make_dims
    sh = pkg.sharding
    n_pf, n_dec = 150, 5
    n = n_pf + n_dec
    dims = make_dims()
    w = synth.gdn_weights(12)
    w["dt_bias"] = synth.to_bf16_bits(synth.normal(12, "dtb", (64,), std=0.5))
    qkv, z, beta, alpha = synth.gdn_step_inputs(12, n, bf16=True)
    s0 = synth.gdn_state(12)
    conv_ref = np.zeros((3, 12288), np.float32); ssm_ref = s0.copy()
    out_ref = port.gdn_run(dims, conv_ref, ssm_ref, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"], threads=16)
    out = np.empty((n, 8192), np.float32); ssm = np.empty((64, 128, 128), np.float32)
    for r in range(world):
        v0, nv, k0, nk = sh.gdn_head_slice(r, world)
        sl = sh.gdn_slice_inputs(r, world, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"])
        c = gdn_ctx(pkg, v_heads=nv, k_heads=nk, max_batch=256)
        c.state_import(0, 0, None, np.ascontiguousarray(s0[v0:v0 + nv]))
        o = np.empty((n, nv * 128), np.float32)
        c.gdn_prefill(0, 0, n_pf, sl["qkv"][:n_pf].copy(), sl["z"][:n_pf].copy(), sl["beta"][:n_pf].copy(), sl["alpha"][:n_pf].copy(),
                      o[:n_pf], sl["conv_w"], sl["A_log"], sl["dt_bias"], w["norm_w"])
        for t in range(n_pf, n):
            c.gdn_decode(0, [0], sl["qkv"][t:t + 1].copy(), sl["z"][t:t + 1].copy(), sl["beta"][t:t + 1].copy(), sl["alpha"][t:t + 1].copy(),
                         o[t:t + 1], sl["conv_w"], sl["A_log"], sl["dt_bias"], w["norm_w"])
        c.state_export(0, 0, None, ssm[v0:v0 + nv])
        c.close()
        out[:, v0 * 128:(v0 + nv) * 128] = o
    go, _, _ = rel_errors(out, out_ref)
    gs, _, _ = rel_errors(ssm, ssm_ref)
    print("head-sharded over", world, "contexts: out", go, "state", gs)
    assert go <= TOL_OUT and gs <= TOL_STATE
