"""One rank of the multi-GPU decode parity run (started by test_gpu_multi.py under torch.distributed.run).

Every rank holds all heads and one sequence shard of every layer's KV store; a token goes through
all layers in one fm_attn_decode_layers call whose launches exchange their partial results over
peer memory.  Each rank compares its gated output with the CPU checker."""
import json
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm
    from __graft_entry__ import load_package
    from gpu_util import oracle_attn
    from oracle.oracle_py import Oracle
    from parity import rel_errors

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pkg = load_package()
    synth, port = pkg.synth, Oracle("port")
    H, HKV, D = 32, 2, 256
    lens, layers, steps = (2500, 900), 5, 4
    B = len(lens)
    cfg = pkg.default_config(num_full_layers=layers, num_linear_layers=0, max_seqs=B, max_seq_len=max(lens) + steps + 64,
                             seq_shard_rank=rank, seq_shard_count=world, device=local)
    c = pkg.Context(cfg)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    xbuf = symm.empty(c.exchange_bytes(world) // 4, dtype=torch.float32, device=dev)
    hdl = symm.rendezvous(xbuf, group=dist.group.WORLD)
    c.exchange_attach(hdl.rank, list(hdl.buffer_ptrs))
    torch.cuda.synchronize()
    dist.barrier()

    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    caches, steps_in = {}, {}
    for l in range(layers):
        for s, L in enumerate(lens):
            k0, v0 = synth.attn_cache(500 + l, L, tag=f"s{s}")
            caches[l, s] = (k0, v0)
            c.kv_import(l, s, t(k0), t(v0), L)
            q, g, k, v = synth.attn_step_inputs(500 + l, steps, tag=f"s{s}")
            steps_in[l, s] = (q, g, synth.round_bf16(k), synth.round_bf16(v))
    sq, skv, so = B * H * 2 * D, B * HKV * D, B * H * D
    outs = []
    for st in range(steps):
        qp = np.empty((layers, B, H, 2, D), np.float32)
        kk = np.empty((layers, B, HKV * D), np.float32); vv = np.empty_like(kk)
        for l in range(layers):
            for s in range(B):
                q, g, k, v = steps_in[l, s]
                qp[l, s, :, 0] = q[st].reshape(H, D); qp[l, s, :, 1] = g[st].reshape(H, D)
                kk[l, s] = k[st]; vv[l, s] = v[st]
        out = torch.empty((layers, B, H * D), device=dev)
        c.attn_decode_layers(0, layers, list(range(B)), [L + st for L in lens], out, t(qp), t(kk), t(vv), sq, skv, so,
                             exchange=True)
        outs.append(out)
    c.synchronize()
    outs = [o.cpu().numpy() for o in outs]
    worst = 0.0
    for l in range(layers):
        for s, L in enumerate(lens):
            k0, v0 = caches[l, s]
            q, g, k, v = steps_in[l, s]
            ref, _, _ = oracle_attn(port, H, HKV, k0, v0, q, g, k, v)
            for st in range(steps):
                gated, _, _ = rel_errors(outs[st][l, s], ref[st])
                worst = max(worst, gated)
            assert c.kv_len(l, s) == L + steps
    res = torch.tensor([worst], device=dev)
    dist.all_reduce(res, op=dist.ReduceOp.MAX)
    dist.barrier()
    c.close()
    if rank == 0:
        print(json.dumps({"world": world, "worst_gated": float(res.item())}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
