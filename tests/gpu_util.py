"""Helpers for the GPU parity tests: contexts in host-pointer mode driven with numpy arrays."""
import numpy as np

from oracle.oracle_py import make_dims


def attn_ctx(pkg, heads=32, kv_heads=2, max_seq_len=8192, max_seqs=1, max_batch=64, layers=1,
             shard=(0, 1), rot=64, theta=1e7, **kw):
    cfg = pkg.default_config(num_attn_heads=heads, num_kv_heads=kv_heads, rotary_dim=rot,
                             rope_theta=theta, num_full_layers=layers, num_linear_layers=0,
                             max_seqs=max_seqs, max_seq_len=max_seq_len, max_batch_tokens=max_batch,
                             seq_shard_rank=shard[0], seq_shard_count=shard[1], **kw)
    return pkg.Context(cfg, host_pointers=True)


def gdn_ctx(pkg, v_heads=64, k_heads=16, max_seqs=1, max_batch=64, layers=1):
    cfg = pkg.default_config(linear_num_v_heads=v_heads, linear_num_k_heads=k_heads,
                             num_full_layers=0, num_linear_layers=layers, max_seqs=max_seqs,
                             max_batch_tokens=max_batch)
    return pkg.Context(cfg, host_pointers=True)


def oracle_attn(orc, heads, kv_heads, k0, v0, q, gate, k, v, qn=None, kn=None, start_pos=None,
                rot=64, theta=1e7, threads=8, store_bf16=1, **dims_kw):
    """Runs the CPU checker for n steps after a cache prefix; returns (out, k_rows, v_rows).
    store_bf16=1: the checker rounds each appended row to bf16 like the KV store under test does,
    so the comparison isolates the attention arithmetic from the store's own rounding."""
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kv_heads, head_dim=256, rotary_dim=rot,
                     rope_theta=theta, store_bf16=store_bf16, **dims_kw)
    ctx, n = k0.shape[0], q.shape[0]
    kc = np.zeros((ctx + n, kv_heads * 256), np.float32); vc = np.zeros_like(kc)
    kc[:ctx] = k0; vc[:ctx] = v0
    out, ln = orc.attn_run(dims, kc, vc, ctx, q, gate, k, v, qn, kn, start_pos=start_pos, threads=threads)
    return out, kc, vc
