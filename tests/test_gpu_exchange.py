"""Peer-memory exchange of decode partials (needs a B200).  Two sequence-shard contexts live on the
one test GPU and use each other's exchange buffers as "peers"; both push before either merges, so no
kernel ever waits for a launch that comes after it on the same GPU."""
import numpy as np
import pytest

from gpu_util import oracle_attn
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _contexts(pkg, torch, n, L):
    dev = torch.device("cuda:0")
    ctxs, bufs = [], []
    for r in range(n):
        cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seqs=2, max_seq_len=L + 64,
                                 seq_shard_rank=r, seq_shard_count=n)
        c = pkg.Context(cfg)
        c.set_stream(torch.cuda.current_stream().cuda_stream)
        ctxs.append(c)
        bufs.append(torch.empty(c.exchange_bytes(n) // 4, dtype=torch.float32, device=dev))
    for r, c in enumerate(ctxs):
        c.exchange_attach(r, [b.data_ptr() for b in bufs])
    return ctxs, bufs, dev


@pytest.mark.parametrize("nshards", [2, 4])
def test_exchange_matches_single_context(pkg, port, synth, nshards):
    import torch
    L, steps = 1500, 3
    ctxs, bufs, dev = _contexts(pkg, torch, nshards, L)
    k0, v0 = synth.attn_cache(61, L)
    q, g, k, v = synth.attn_step_inputs(61, steps)
    k, v = synth.round_bf16(k), synth.round_bf16(v)
    ref_out, _, _ = oracle_attn(port, 32, 2, k0, v0, q, g, k, v)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    for c in ctxs:
        c.kv_import(0, 0, t(k0), t(v0), L)
    outs = [torch.empty((1, 8192), device=dev) for _ in ctxs]
    for s in range(steps):
        qs, gs, ks, vs = t(q[s:s + 1]), t(g[s:s + 1]), t(k[s:s + 1]), t(v[s:s + 1])
        for c in ctxs:
            c.attn_decode_exchange_push(0, [0], [L + s], q=qs, k=ks, v=vs)
        for c, o in zip(ctxs, outs):
            c.attn_decode_exchange_merge(1, o, gate=gs)
        torch.cuda.synchronize()
        for c, o in zip(ctxs, outs):
            c.synchronize()
            gated, _, rr = rel_errors(o.cpu().numpy(), ref_out[s])
            assert gated <= TOL, (s, gated)
            assert c.kv_len(0, 0) == L + s + 1
    print("exchange", nshards, "shards gated", gated, "rms-rel", rr)
    for c in ctxs:
        c.close()


def test_missing_peer_times_out_and_context_survives(pkg, synth):
    """Only one of two shards pushes: its merge waits for the other's step, gives up after about half
    a second, reports FM_ERR_TIMEOUT with zeros in the output, and the next complete step works."""
    import torch
    L = 300
    ctxs, bufs, dev = _contexts(pkg, torch, 2, L)
    k0, v0 = synth.attn_cache(62, L)
    q, g, k, v = synth.attn_step_inputs(62, 2)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    for c in ctxs:
        c.kv_import(0, 0, t(k0), t(v0), L)
    out = torch.full((1, 8192), 7.0, device=dev)
    a, b = ctxs
    a.attn_decode_exchange_push(0, [0], [L], q=t(q[:1]), k=t(k[:1]), v=t(v[:1]))
    a.attn_decode_exchange_merge(1, out, gate=t(g[:1]))     # b never pushed step 1
    with pytest.raises(pkg.FmError) as e:
        a.synchronize()
    assert e.value.status == pkg.binding.FM_ERR_TIMEOUT
    assert not out.cpu().numpy().any()
    # b catches up with step 1, then both run step 2 normally
    b.attn_decode_exchange_push(0, [0], [L], q=t(q[:1]), k=t(k[:1]), v=t(v[:1]))
    ob = torch.empty((1, 8192), device=dev)
    b.attn_decode_exchange_merge(1, ob, gate=t(g[:1]))
    b.synchronize()
    for c in ctxs:
        c.attn_decode_exchange_push(0, [0], [L + 1], q=t(q[1:2]), k=t(k[1:2]), v=t(v[1:2]))
    oa = torch.empty((1, 8192), device=dev)
    a.attn_decode_exchange_merge(1, oa, gate=t(g[1:2]))
    b.attn_decode_exchange_merge(1, ob, gate=t(g[1:2]))
    a.synchronize(); b.synchronize()
    np.testing.assert_array_equal(oa.cpu().numpy(), ob.cpu().numpy())
    assert np.isfinite(oa.cpu().numpy()).all() and oa.abs().max().item() > 0
    for c in ctxs:
        c.close()
