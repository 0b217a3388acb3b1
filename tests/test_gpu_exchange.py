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


@pytest.mark.parametrize("lens", [(1400, 900), (60, 40)])
def test_whole_step_in_one_launch_single_rank_group(pkg, port, synth, lens):
    """fm_attn_decode_exchange with a group of one rank: the decode launch pushes its rows to its own
    buffer, sees its own unit flags and merges -- the one-launch path of the sharded step, which must
    reproduce the plain step."""
    import torch
    dev = torch.device("cuda:0")
    steps = 3
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seqs=2, max_seq_len=max(lens) + 64)
    c = pkg.Context(cfg)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    buf = torch.empty(c.exchange_bytes(1) // 4, dtype=torch.float32, device=dev)
    c.exchange_attach(0, [buf.data_ptr()])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    refs = []
    for s in range(2):
        k0, v0 = synth.attn_cache(63, lens[s], tag=f"s{s}")
        q, g, k, v = synth.attn_step_inputs(63, steps, tag=f"s{s}")
        k, v = synth.round_bf16(k), synth.round_bf16(v)
        c.kv_import(0, s, t(k0), t(v0), lens[s])
        refs.append((q, g, k, v, oracle_attn(port, 32, 2, k0, v0, q, g, k, v)[0]))
    launches0 = c.launch_count()
    for st in range(steps):
        out = torch.empty((2, 8192), device=dev)
        stack = lambda i: t(np.stack([refs[s][i][st] for s in range(2)]))
        c.attn_decode_exchange(0, [0, 1], [lens[0] + st, lens[1] + st], out, q=stack(0), gate=stack(1), k=stack(2), v=stack(3))
        c.synchronize()
        for s in range(2):
            gated, _, _ = rel_errors(out[s].cpu().numpy(), refs[s][4][st])
            assert gated <= TOL, (st, s, gated)
    assert c.launch_count() - launches0 == steps  # one launch per step
    c.close()


def test_whole_step_times_out_without_the_peer(pkg, synth):
    """Group of two, the second rank never runs: the one-launch step waits about half a second for the
    peer's unit flags, reports FM_ERR_TIMEOUT with zeros in the output, and the context stays usable."""
    import torch
    dev = torch.device("cuda:0")
    L = 300
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seqs=1, max_seq_len=L + 64,
                             seq_shard_rank=0, seq_shard_count=2)
    c = pkg.Context(cfg)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    bufs = [torch.zeros(c.exchange_bytes(2) // 4, dtype=torch.float32, device=dev) for _ in range(2)]
    c.exchange_attach(0, [b.data_ptr() for b in bufs])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    k0, v0 = synth.attn_cache(64, L)
    q, g, k, v = synth.attn_step_inputs(64, 1)
    c.kv_import(0, 0, t(k0), t(v0), L)
    out = torch.full((1, 8192), 7.0, device=dev)
    c.attn_decode_exchange(0, [0], [L], out, q=t(q), gate=t(g), k=t(k), v=t(v))
    with pytest.raises(pkg.FmError) as e:
        c.synchronize()
    assert e.value.status == pkg.binding.FM_ERR_TIMEOUT
    assert not out.cpu().numpy().any()
    c.synchronize()  # the error is reported once; the context answers again
    assert c.kv_len(0, 0) == L + 1
    c.close()
