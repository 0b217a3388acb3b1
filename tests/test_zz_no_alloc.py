"""fm_attn_decode_static -- the decode step for callers that are not allowed to allocate device
memory (a plugin inside another engine's fixed memory plan, a serving loop that bans allocator
calls once running).  Such a caller cannot create a context, so it hands the library its own KV
pages and page table; the split-KV partial results go to a fixed array inside the library.

The test lays out a small paged bf16 KV store by hand, runs the step through the C-ABI twice in a
row (the second call reuses the scratch the first one dirtied) and compares each result with the
ordinary entry point, fm_attn_decode, run on a context that imported the same rows.  Both paths
run the same kernels on the same bf16 values, so the results must agree to rounding noise; the
bound used is the 2e-3 of the attention parity tests.  This file is named to be collected last.
"""
import numpy as np
import pytest

from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3


def test_static_scratch_decode_matches_context_decode(pkg, synth):
    import torch
    dev = torch.device("cuda:0")
    H, HKV, D, PAGE = 32, 2, 256, 64
    lens = [1000, 130]           # two sequences, the second ending mid-page
    B = len(lens)
    max_pages = 20
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seqs=B, max_seq_len=max_pages * PAGE)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)

    # caller-owned store: pages handed out in an arbitrary order, layout [page][K|V][head][row][dim]
    n_pages = B * max_pages
    pages = torch.zeros((n_pages, 2, HKV, PAGE, D), dtype=torch.bfloat16, device=dev)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).to(torch.int32)
    table = perm.reshape(B, max_pages).contiguous().to(dev)
    for s, L in enumerate(lens):
        k0, v0 = synth.attn_cache(500 + s, L)              # bf16-representable rows
        kt = torch.from_numpy(k0).to(dev); vt = torch.from_numpy(v0).to(dev)
        ctx.kv_import(0, s, kt, vt, L)
        for r0 in range(0, L, PAGE):
            n = min(PAGE, L - r0)
            pg = int(perm[s * max_pages + r0 // PAGE])
            pages[pg, 0, :, :n] = kt[r0:r0 + n].reshape(n, HKV, D).permute(1, 0, 2).bfloat16()
            pages[pg, 1, :, :n] = vt[r0:r0 + n].reshape(n, HKV, D).permute(1, 0, 2).bfloat16()
    qn = torch.from_numpy(synth.to_bf16_bits(1.0 + synth.normal(9, "qn", (D,), std=0.1)).view(np.int16)).to(dev)

    for call in range(2):
        q, g, _, _ = synth.attn_step_inputs(40 + call, B)
        qt = torch.from_numpy(q).to(dev); gt = torch.from_numpy(g).to(dev)
        pos = [L + 5 for L in lens]
        want = torch.empty((B, H * D), device=dev)
        ctx.attn_decode(0, list(range(B)), pos, want, q=qt, gate=gt, q_norm_w=qn)   # k = NULL: nothing appended
        got = torch.full((B, H * D), float("nan"), device=dev)
        pkg.binding.attn_decode_static(pages, table, max_pages, lens, pos, got, q=qt, gate=gt, q_norm_w=qn,
                                       stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        gated, _, rr = rel_errors(got.cpu().numpy(), want.cpu().numpy())
        print("call", call, "gated", gated, "rms-rel", rr)
        assert gated <= TOL
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
