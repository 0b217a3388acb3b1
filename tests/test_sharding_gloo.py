"""Multi-rank host logic on CPU (gloo, world size 2 and 4): the mesh, page ownership and the
log-sum-exp merge of per-shard partial results reproduce the single-rank CPU checker; GatedDeltaNet layers sliced by
value head (each rank steps its heads, no exchange) reproduce the whole layer."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _partial(q, K, V, rows, scale):
    """Un-normalised attention of one head over a subset of rows: (o, max, sum) in the exp2 domain."""
    if not rows:
        return np.zeros(V.shape[1], np.float64), -1e30, 0.0
    s = (K[rows].astype(np.float64) @ q.astype(np.float64)) * scale * np.log2(np.e)
    m = s.max()
    p = np.exp2(s - m)
    return p @ V[rows].astype(np.float64), m, p.sum()


def _worker(rank, world, port, L, out_file):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from __graft_entry__ import load_package
    pkg = load_package()
    synth, sh = pkg.synth, pkg.sharding
    mesh = sh.mesh_for(world)
    hg, ss = mesh.coords(rank)
    H, HKV, D = 32, 2, 256
    Hl = H // mesh.head_groups
    k0, v0 = synth.attn_cache(3, L)                       # rows as the store holds them (no rotation here)
    q, gate, _, _ = synth.attn_step_inputs(3, 1)
    kv_h = hg if mesh.head_groups == 2 else None          # which KV head this rank holds (None: both)
    rows = sh.owned_rows(L, 64, ss, mesh.seq_shards)
    o = np.zeros((Hl, D)); ml = np.zeros((Hl, 2))
    for hl in range(Hl):
        h = hg * Hl + hl
        kvh = h // 16
        assert kv_h is None or kvh == kv_h
        o[hl], ml[hl, 0], ml[hl, 1] = _partial(q[0, h * D:(h + 1) * D], k0[:, kvh * D:(kvh + 1) * D],
                                               v0[:, kvh * D:(kvh + 1) * D], rows, 1.0 / 16.0)
    # all-gather inside the sequence group, merge by log-sum-exp, apply the gate
    groups = [dist.new_group(mesh.seq_group_ranks(g)) for g in range(mesh.head_groups)]
    grp = groups[hg]
    to = [torch.zeros(Hl, D, dtype=torch.float64) for _ in range(mesh.seq_shards)]
    tm = [torch.zeros(Hl, 2, dtype=torch.float64) for _ in range(mesh.seq_shards)]
    dist.all_gather(to, torch.from_numpy(o), group=grp)
    dist.all_gather(tm, torch.from_numpy(ml), group=grp)
    O = np.stack([t.numpy() for t in to]); ML = np.stack([t.numpy() for t in tm])
    M = ML[:, :, 0].max(axis=0)
    w = np.exp2(ML[:, :, 0] - M)
    merged = (w[:, :, None] * O).sum(axis=0) / (w * ML[:, :, 1]).sum(axis=0)[:, None]
    g = gate[0, hg * Hl * D:(hg + 1) * Hl * D].reshape(Hl, D)
    mine = merged / (1.0 + np.exp(-g))
    # every rank of a sequence group holds the same merged heads; collect one copy per head group
    full = [torch.zeros(Hl, D, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(full, torch.from_numpy(mine))
    if rank == 0:
        res = np.concatenate([full[r].numpy() for r in range(mesh.head_groups)]).reshape(-1)
        np.save(out_file, res)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_partials_merge_to_the_single_rank_answer(tmp_path, port, synth, world):
    from oracle.oracle_py import make_dims
    L = 1000
    out_file = str(tmp_path / "merged.npy")
    mp.spawn(_worker, args=(world, _free_port(), L, out_file), nprocs=world, join=True)
    got = np.load(out_file)
    # single-rank checker on the same cache: no new row (attend over L rows), no rotation
    k0, v0 = synth.attn_cache(3, L)
    q, gate, _, _ = synth.attn_step_inputs(3, 1)
    dims = make_dims(rotary_dim=0)
    kc = np.zeros((L, 512), np.float32); vc = np.zeros_like(kc)
    kc[:L - 1] = k0[:L - 1]; vc[:L - 1] = v0[:L - 1]
    want, ln = port.attn_run(dims, kc, vc, L - 1, q, gate, k0[L - 1:L], v0[L - 1:L], start_pos=0)
    assert ln == L
    np.testing.assert_allclose(got, want.reshape(-1), rtol=2e-4, atol=2e-6)


def test_mesh_and_ownership(pkg):
    sh = pkg.sharding
    assert (sh.mesh_for(1).head_groups, sh.mesh_for(1).seq_shards) == (1, 1)
    assert (sh.mesh_for(2).head_groups, sh.mesh_for(2).seq_shards) == (2, 1)
    assert (sh.mesh_for(8).head_groups, sh.mesh_for(8).seq_shards) == (2, 4)
    m = sh.mesh_for(8)
    assert sorted(sum((m.seq_group_ranks(g) for g in range(2)), [])) == list(range(8))
    assert {m.coords(r) for r in range(8)} == {(g, s) for g in range(2) for s in range(4)}
    # every row has exactly one owner, and shares differ by at most one page
    L = 1000
    owners = [sh.owned_rows(L, 64, s, 4) for s in range(4)]
    assert sorted(sum(owners, [])) == list(range(L))
    assert max(map(len, owners)) - min(map(len, owners)) <= 64
    assert sh.owned_rows(0, 64, 0, 4) == []
    assert sh.gdn_head_slice(3, 8) == (24, 8, 6, 2)
    with pytest.raises(ValueError):
        sh.mesh_for(3)


def _gdn_worker(rank, world, port, steps, out_file):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from __graft_entry__ import load_package
    from oracle.oracle_py import Oracle, make_dims
    pkg = load_package()
    synth, sh = pkg.synth, pkg.sharding
    w = synth.gdn_weights(9)
    qkv, z, beta, alpha = synth.gdn_step_inputs(9, steps)
    v0, nv, k0, nk = sh.gdn_head_slice(rank, world)
    mine = sh.gdn_slice_inputs(rank, world, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"])
    dims = make_dims(linear_num_v_heads=nv, linear_num_k_heads=nk)
    conv = np.zeros((3, 2 * nk * 128 + nv * 128), np.float32)
    ssm = np.ascontiguousarray(synth.gdn_state(9)[v0:v0 + nv])
    out = Oracle("port").gdn_run(dims, conv, ssm, mine["qkv"], mine["z"], mine["beta"], mine["alpha"], mine["conv_w"],
                                 mine["A_log"], mine["dt_bias"], w["norm_w"])
    outs = [torch.zeros(steps, nv * 128) for _ in range(world)]
    states = [torch.zeros(nv, 128, 128) for _ in range(world)]
    dist.all_gather(outs, torch.from_numpy(np.ascontiguousarray(out, dtype=np.float32)))
    dist.all_gather(states, torch.from_numpy(ssm))
    if rank == 0:
        np.savez(out_file, out=np.concatenate([o.numpy() for o in outs], axis=1), ssm=np.concatenate([s_.numpy() for s_ in states]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gdn_layers_sliced_by_value_head_reproduce_the_whole_layer(tmp_path, port, synth, world):
    from oracle.oracle_py import make_dims
    steps = 3
    out_file = str(tmp_path / "gdn.npz")
    mp.spawn(_gdn_worker, args=(world, _free_port(), steps, out_file), nprocs=world, join=True)
    got = np.load(out_file)
    w = synth.gdn_weights(9)
    qkv, z, beta, alpha = synth.gdn_step_inputs(9, steps)
    conv = np.zeros((3, 12288), np.float32); ssm = synth.gdn_state(9).copy()
    want = port.gdn_run(make_dims(), conv, ssm, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"], w["norm_w"])
    np.testing.assert_array_equal(got["out"], np.asarray(want, dtype=np.float32))   # heads never mix: bit for bit
    np.testing.assert_array_equal(got["ssm"], ssm)
