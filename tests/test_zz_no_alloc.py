"""fm_attn_decode_static -- the decode step for callers that are not allowed to allocate device
memory (a plugin inside another engine's fixed memory plan, a serving loop that bans allocator
calls once running).  Such a caller cannot create a context, so it hands the library its own KV
pages and page table; the split-KV partial results go to a fixed array inside the library.

The test lays out a small paged bf16 KV store by hand, runs the step through the C-ABI twice in a
row (the second call reuses the scratch the first one dirtied) and compares each result with the
CPU checker and with the ordinary entry point, fm_attn_decode, run on a context that imported the
same rows.  The bound is the 2e-3 of the attention parity tests.  This file is named to be collected
last.
"""
import numpy as np
import pytest

from gpu_util import oracle_attn
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3
H, HKV, D, PAGE = 32, 2, 256, 64


def build_store(torch, dev, synth, port, lens, max_pages, seed, pos, q, g, qn):
    """A caller-owned paged store (pages handed out in an arbitrary order) holding `lens[s]` rows per sequence,
    and the checker's answer for a decode step over exactly those rows.  The checker always appends the step's
    row, so the last row of each sequence is produced by it (normalised, rotated, rounded to bf16 like the
    store) and copied into the pages; the entry point under test then attends without appending."""
    B = len(lens)
    n_pages = B * max_pages
    pages = torch.zeros((n_pages, 2, HKV, PAGE, D), dtype=torch.bfloat16, device=dev)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    table = perm.reshape(B, max_pages).contiguous().to(dev)
    want = np.empty((B, H * D), np.float32)
    rows = []
    for s, L in enumerate(lens):
        k0, v0 = synth.attn_cache(seed * 1000 + s, L - 1)       # bf16-representable rows
        _, _, kn, vn = synth.attn_step_inputs(seed * 1000 + s, 1)
        ref, kc, vc = oracle_attn(port, H, HKV, k0, v0, q[s:s + 1], g[s:s + 1], kn, vn, qn, None, start_pos=pos[s])
        want[s] = ref[0]
        rows.append((kc, vc))
        kt, vt = torch.from_numpy(kc).to(dev), torch.from_numpy(vc).to(dev)
        for r0 in range(0, L, PAGE):
            n = min(PAGE, L - r0)
            pg = int(perm[s * max_pages + r0 // PAGE])
            pages[pg, 0, :, :n] = kt[r0:r0 + n].reshape(n, HKV, D).permute(1, 0, 2).bfloat16()
            pages[pg, 1, :, :n] = vt[r0:r0 + n].reshape(n, HKV, D).permute(1, 0, 2).bfloat16()
    return pages, table, want, rows


@pytest.mark.parametrize("lens,interleaved", [([1000, 130], False), ([5000, 64, 1], True),
                                              ([37 + 5 * i for i in range(64)], False)])
def test_static_scratch_decode_matches_checker(pkg, synth, port, lens, interleaved):
    import torch
    dev = torch.device("cuda:0")
    B = len(lens)
    max_pages = (max(lens) + PAGE - 1) // PAGE + 2
    qn_bits = synth.to_bf16_bits(1.0 + synth.normal(9, "qn", (D,), std=0.1))
    qn = torch.from_numpy(qn_bits.view(np.int16)).to(dev)
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seqs=B, max_seq_len=max_pages * PAGE)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    for call in range(2):   # two calls in a row: the second reuses the scratch the first one dirtied
        q, g, _, _ = synth.attn_step_inputs(40 + call, B)
        pos = [L + 5 for L in lens]
        pages, table, want, rows = build_store(torch, dev, synth, port, lens, max_pages, 3 + call, pos, q, g, qn_bits)
        qt, gt = torch.from_numpy(q).to(dev), torch.from_numpy(g).to(dev)
        got = torch.full((B, H * D), float("nan"), device=dev)
        if interleaved:
            qp = torch.stack([qt.reshape(B, H, D), gt.reshape(B, H, D)], dim=2).reshape(B, H * 2 * D).contiguous()
            pkg.binding.attn_decode_static(pages, table, max_pages, lens, pos, got, q_proj_out=qp, q_norm_w=qn,
                                           stream=torch.cuda.current_stream().cuda_stream)
        else:
            pkg.binding.attn_decode_static(pages, table, max_pages, lens, pos, got, q=qt, gate=gt, q_norm_w=qn,
                                           stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        gated, _, rr = rel_errors(got.cpu().numpy(), want)
        print("call", call, "vs checker: gated", gated, "rms-rel", rr)
        assert gated <= TOL
        # the ordinary entry point on a context holding the same rows (k = NULL: nothing appended)
        for s, L in enumerate(lens):
            ctx.kv_import(0, s, torch.from_numpy(rows[s][0]).to(dev), torch.from_numpy(rows[s][1]).to(dev), L)
        other = torch.empty((B, H * D), device=dev)
        ctx.attn_decode(0, list(range(B)), pos, other, q=qt, gate=gt, q_norm_w=qn)
        torch.cuda.synchronize()
        gated2, _, _ = rel_errors(got.cpu().numpy(), other.cpu().numpy())
        print("call", call, "vs fm_attn_decode: gated", gated2)
        assert gated2 <= TOL
    ctx.close()


def test_static_scratch_rejects_oversize(pkg):
    import torch
    dev = torch.device("cuda:0")
    pages = torch.zeros((1, 2, 2, 64, 256), dtype=torch.bfloat16, device=dev)
    table = torch.zeros((1, 1), dtype=torch.int32, device=dev)
    out = torch.empty((1, 8192), device=dev)
    q = torch.zeros((1, 8192), device=dev)
    with pytest.raises(pkg.FmError) as e:   # 65 sequences: beyond the per-call batch limit
        pkg.binding.attn_decode_static(pages, table, 1, [1] * 65, [0] * 65, out, q=q, gate=q)
    assert e.value.status == pkg.binding.FM_ERR_INVALID and "batch" in e.value.text
    with pytest.raises(pkg.FmError) as e:   # 64 sequences x 256 heads > 8192 partial rows
        pkg.binding.attn_decode_static(pages, table, 1, [1] * 64, [0] * 64, out, q=q, gate=q,
                                       num_attn_heads=256, num_kv_heads=16)
    assert e.value.status == pkg.binding.FM_ERR_CAPACITY and "scratch" in e.value.text
    with pytest.raises(pkg.FmError) as e:   # a length the page table cannot hold
        pkg.binding.attn_decode_static(pages, table, 1, [65], [0], out, q=q, gate=q)
    assert e.value.status == pkg.binding.FM_ERR_INVALID
    for bad in (dict(num_attn_heads=0), dict(num_attn_heads=-2), dict(rope_theta=0.0)):
        with pytest.raises(pkg.FmError) as e:   # no heads / a non-positive RoPE base: refused before any arithmetic
            pkg.binding.attn_decode_static(pages, table, 1, [1], [0], out, q=q, gate=q, **bad)
        assert e.value.status == pkg.binding.FM_ERR_INVALID
