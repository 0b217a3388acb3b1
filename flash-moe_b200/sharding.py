"""Host-side layout of the path across several GPUs (one process per GPU).

Full attention has 2 KV heads: up to 2 head groups (16 query heads + 1 KV head each, no exchange
inside the attention path), and inside a head group the sequence is split page-wise: global page
p of a sequence lives on sequence shard p % shards (round-robin keeps the shards' shares equal at
every context length).  GatedDeltaNet shards by value head only (the state never moves).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Mesh:
    world: int
    head_groups: int
    seq_shards: int

    def coords(self, rank: int):
        """(head group, sequence shard) of a rank; ranks of one head group form a sequence group."""
        return rank % self.head_groups, rank // self.head_groups

    def seq_group_ranks(self, head_group: int):
        return [r for r in range(self.world) if r % self.head_groups == head_group]


def mesh_for(world: int, kv_heads: int = 2) -> Mesh:
    if world < 1 or (world & (world - 1)) != 0:
        raise ValueError(f"world size {world}: a power of two is expected")
    hg = min(kv_heads, world)
    return Mesh(world, hg, world // hg)


def owned_rows(length: int, page_size: int, shard: int, shards: int):
    """Cache rows of a sequence of `length` rows that sequence shard `shard` holds."""
    rows = []
    for page in range(shard, (length + page_size - 1) // page_size, shards):
        rows.extend(range(page * page_size, min((page + 1) * page_size, length)))
    return rows


def gdn_head_slice(rank: int, world: int, v_heads: int = 64, k_heads: int = 16):
    """(first v head, v heads, first k head, k heads) of a rank; the 4:1 v:k mapping is preserved."""
    if v_heads % world or k_heads % world:
        raise ValueError("head counts must divide by the world size")
    nv, nk = v_heads // world, k_heads // world
    return rank * nv, nv, rank * nk, nk


def gdn_slice_inputs(rank: int, world: int, qkv, z, beta, alpha, conv_w=None, A_log=None, dt_bias=None,
                     v_heads: int = 64, k_heads: int = 16, dk: int = 128, dv: int = 128):
    """The part of one GatedDeltaNet layer's inputs and per-head weights that a rank holding
    `gdn_head_slice(rank, world)` needs: qkv [n][q | k | v] -> the rank's q, k and v heads in the same
    q | k | v order, z [n][Hv*dv], beta / alpha [n][Hv], conv_w [conv_dim][ks] rows, A_log / dt_bias [Hv].
    (The output-norm weight [dv] is shared by all heads.)  Arrays are numpy; copies are returned."""
    import numpy as np
    v0, nv, k0, nk = gdn_head_slice(rank, world, v_heads, k_heads)
    tk, tv = k_heads * dk, v_heads * dv
    qs = slice(k0 * dk, (k0 + nk) * dk)
    ks = slice(tk + k0 * dk, tk + (k0 + nk) * dk)
    vs = slice(2 * tk + v0 * dv, 2 * tk + (v0 + nv) * dv)
    cat = lambda a, axis: np.ascontiguousarray(np.concatenate([a[..., qs] if axis else a[qs], a[..., ks] if axis else a[ks],
                                                               a[..., vs] if axis else a[vs]], axis=-1 if axis else 0))
    out = dict(qkv=cat(qkv, 1), z=np.ascontiguousarray(z[..., v0 * dv:(v0 + nv) * dv]),
               beta=np.ascontiguousarray(beta[..., v0:v0 + nv]), alpha=np.ascontiguousarray(alpha[..., v0:v0 + nv]))
    if conv_w is not None:
        out["conv_w"] = cat(conv_w, 0)
    if A_log is not None:
        out["A_log"] = np.ascontiguousarray(A_log[v0:v0 + nv])
    if dt_bias is not None:
        out["dt_bias"] = np.ascontiguousarray(dt_bias[v0:v0 + nv])
    return out
