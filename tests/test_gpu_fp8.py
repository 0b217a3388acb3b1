"""The FP8 E4M3 KV store (FmConfig.kv_dtype = FM_KV_FP8_E4M3) through the C-ABI against the CPU checker run with
the reference's FP8 cache (g_use_fp8_kv; metal_infer/fp8.h, metal_infer/layer_forward.h:609-616, 679-712).

Two bars.  The stored bytes and scales are byte / integer work: bit-exact against the checker's codec, quirks of
the reference's encoder included.  The attention output over an FP8 cache is compared with the checker reading
THE SAME bytes, at the 2e-3 of the other attention tests: what is checked is the kernel's arithmetic, not the
quantisation -- the reference's own FP8 path sits about 1e-1 (rms-relative) from its fp32 path on N(0,1) rows,
mostly because of the values its encoder misplaces, and that distance is a property of the format, not of this
library."""
import numpy as np
import pytest

from gpu_util import attn_ctx
from oracle.oracle_py import Cache, host_threads, make_dims
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3


def fp8_ctx(pkg, heads=32, kv_heads=2, max_seq_len=8192, max_seqs=1, **kw):
    return attn_ctx(pkg, heads, kv_heads, max_seq_len=max_seq_len, max_seqs=max_seqs, kv_dtype=pkg.binding.FM_KV_FP8_E4M3, **kw)


def awkward_rows(synth, n, kv_dim=512):
    """N(0,1) rows plus the values the reference encodes oddly (see tests/test_oracle.py)."""
    rows = synth.normal(31, "fp8rows", (n, kv_dim))
    rows[1] = 0.0
    rows[2, :] = np.linspace(-1.0, 1.0, kv_dim, dtype=np.float32) * 240.0
    tiny = np.float32(2.0) ** np.arange(-12, -4, dtype=np.float32)
    rows[3, :8] = tiny; rows[3, 8:16] = -tiny; rows[3, 16] = 240.0
    pw = np.float32(2.0) ** np.arange(-8, 8, dtype=np.float32)
    rows[4, :16] = pw; rows[4, 16:32] = np.nextafter(pw, np.float32(0)); rows[4, 32:48] = np.nextafter(pw, np.float32(1e9))
    rows[4, 48] = 240.0
    rows[5, :256] = np.linspace(0.0, 0.02, 256, dtype=np.float32); rows[5, 256] = 240.0; rows[5, 257:] = 0.0
    return rows


def test_import_quantises_like_the_reference(pkg, port, synth):
    """fm_kv_import of fp32 rows into an FP8 store: bytes and scales equal the checker's codec bit for bit; fp32
    export decodes them the reference's way; the raw export / import pair round-trips exactly."""
    n = 200
    k = awkward_rows(synth, n); v = synth.normal(32, "fp8v", (n, 512)) * 3.0
    c = fp8_ctx(pkg, max_seq_len=256)
    c.kv_import(0, 0, k, v, n)
    k8 = np.zeros((n, 512), np.uint8); v8 = np.zeros_like(k8); ks = np.zeros(n, np.float32); vs = np.zeros(n, np.float32)
    assert c.kv_export_fp8(0, 0, k8, v8, ks, vs, n) == n
    wk8, wks = port.fp8_encode_rows(k); wv8, wvs = port.fp8_encode_rows(v)
    np.testing.assert_array_equal(k8, wk8); np.testing.assert_array_equal(ks, wks)
    np.testing.assert_array_equal(v8, wv8); np.testing.assert_array_equal(vs, wvs)
    assert (k8 >= 0xFA).any()
    kf = np.zeros((n, 512), np.float32); vf = np.zeros_like(kf)
    assert c.kv_export(0, 0, kf, vf, n) == n
    np.testing.assert_array_equal(kf, port.fp8_decode_rows(wk8, wks))
    np.testing.assert_array_equal(vf, port.fp8_decode_rows(wv8, wvs))
    c.reset(0)
    c.kv_import_fp8(0, 0, k8, v8, ks, vs, n)
    k8b = np.zeros_like(k8); v8b = np.zeros_like(k8); ksb = np.zeros_like(ks); vsb = np.zeros_like(vs)
    assert c.kv_export_fp8(0, 0, k8b, v8b, ksb, vsb, n) == n
    np.testing.assert_array_equal(k8b, k8); np.testing.assert_array_equal(vsb, vs)
    c.close()


def run_fp8_decode(pkg, port, synth, heads, kv_heads, ctx, steps, seed, norm=False, batchless=True):
    """Prefix of `ctx` quantised rows (from the checker's codec), then `steps` decode steps with append."""
    kvd = kv_heads * 256
    k0 = synth.normal(seed, "k0", (ctx, kvd)); v0 = synth.normal(seed, "v0", (ctx, kvd))
    q, g, k, v = synth.attn_step_inputs(seed, steps, heads=heads, kv_heads=kv_heads)
    qn = synth.to_bf16_bits(1.0 + synth.normal(seed, "qn", (256,), std=0.1)) if norm else None
    kn = synth.to_bf16_bits(1.0 + synth.normal(seed, "kn", (256,), std=0.1)) if norm else None
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kv_heads)
    cache = Cache(ctx + steps, kvd, fp8=True)
    if ctx:
        cache.k8[:ctx], cache.k_scales[:ctx] = port.fp8_encode_rows(k0)
        cache.v8[:ctx], cache.v_scales[:ctx] = port.fp8_encode_rows(v0)
    cache.c.len = ctx
    c = fp8_ctx(pkg, heads, kv_heads, max_seq_len=ctx + steps + 8)
    if ctx:
        c.kv_import_fp8(0, 0, cache.k8[:ctx].copy(), cache.v8[:ctx].copy(), cache.k_scales[:ctx].copy(), cache.v_scales[:ctx].copy(), ctx)
    want = port.attn_run_cache(dims, cache, q, g, k, v, qn, kn, start_pos=ctx + 11, threads=host_threads())
    got = np.empty_like(want)
    for t in range(steps):
        c.attn_decode(0, [0], [ctx + 11 + t], got[t:t + 1], q=q[t:t + 1].copy(), gate=g[t:t + 1].copy(), k=k[t:t + 1].copy(),
                      v=v[t:t + 1].copy(), q_norm_w=qn, k_norm_w=kn)
    n = ctx + steps
    k8 = np.zeros((n, kvd), np.uint8); v8 = np.zeros_like(k8); ks = np.zeros(n, np.float32); vs = np.zeros(n, np.float32)
    assert c.kv_export_fp8(0, 0, k8, v8, ks, vs, n) == n
    c.close()
    return got, want, (k8, v8, ks, vs), cache


@pytest.mark.parametrize("ctx", [0, 1, 63, 64, 200, 1000, 5000])
def test_fp8_decode_matches_checker(pkg, port, synth, ctx):
    steps = 3
    got, want, (k8, v8, ks, vs), cache = run_fp8_decode(pkg, port, synth, 32, 2, ctx, steps, 700 + ctx)
    for t in range(steps):
        gated, _, rr = rel_errors(got[t], want[t])
        print("ctx", ctx, "step", t, "gated", gated, "rms-rel", rr)
        assert gated <= TOL
    # the prefix is untouched; V of the appended rows involves no arithmetic before the codec: bit-exact
    np.testing.assert_array_equal(k8[:ctx], cache.k8[:ctx])
    np.testing.assert_array_equal(v8, cache.v8); np.testing.assert_array_equal(vs, cache.v_scales)
    # K of the appended rows went through RoPE first; the device's sin / cos differ from libm's in the last bit,
    # which can move a value across a rounding boundary of the 3-bit mantissa: nearly all bytes equal, the rest
    # one code apart
    new = slice(ctx, ctx + steps)
    np.testing.assert_allclose(ks[new], cache.k_scales[new], rtol=1e-6)
    differ = k8[new] != cache.k8[new]
    assert differ.mean() <= 0.01
    a, b = port.fp8_decode_rows(k8[new], ks[new]), port.fp8_decode_rows(cache.k8[new], cache.k_scales[new])
    ok = ~differ | (np.abs(a - b) <= 0.13 * np.abs(b) + 1e-6) | (cache.k8[new] >= 0xFA) | (k8[new] >= 0xFA)
    assert ok.all()


def test_fp8_decode_with_norm_weights_and_few_heads(pkg, port, synth):
    got, want, _, _ = run_fp8_decode(pkg, port, synth, 8, 2, 333, 4, 811, norm=True)
    gated, _, rr = rel_errors(got, want)
    print("norm, 8 heads: gated", gated, "rms-rel", rr)
    assert gated <= TOL


def test_fp8_batched_ragged_sequences(pkg, port, synth):
    lens = [0, 5, 64, 65, 300, 1000, 129, 2047]
    B = len(lens)
    c = fp8_ctx(pkg, max_seq_len=2100, max_seqs=B)
    q, g, k, v = synth.attn_step_inputs(9, B)
    dims = make_dims()
    refs = []
    for s, L in enumerate(lens):
        cache = Cache(L + 1, 512, fp8=True)
        if L:
            k0 = synth.normal(900 + s, "k0", (L, 512)); v0 = synth.normal(900 + s, "v0", (L, 512))
            cache.k8[:L], cache.k_scales[:L] = port.fp8_encode_rows(k0)
            cache.v8[:L], cache.v_scales[:L] = port.fp8_encode_rows(v0)
            c.kv_import(0, s, k0, v0, L)           # the library's own quantiser this time
        cache.c.len = L
        refs.append(port.attn_run_cache(dims, cache, q[s:s + 1], g[s:s + 1], k[s:s + 1], v[s:s + 1], start_pos=L, threads=host_threads()))
    out = np.empty((B, 8192), np.float32)
    c.attn_decode(0, list(range(B)), lens, out, q=q, gate=g, k=k, v=v)
    for s, L in enumerate(lens):
        gated, _, _ = rel_errors(out[s], refs[s])
        print("seq", s, "len", L, "gated", gated)
        assert gated <= TOL
        assert c.kv_len(0, s) == L + 1
    c.close()


@pytest.mark.parametrize("batch,ctx", [(1, 32768), (8, 32768)])
def test_fp8_quoted_sizes_against_checker(pkg, port, batch, ctx):
    """Long contexts (every split on its own SM at batch 1; the bench's launch shape at batch 8), rows quantised by
    the library, read back raw and handed to the checker."""
    import torch
    dev = torch.device("cuda:0")
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seqs=batch, max_seq_len=ctx + 64,
                             kv_dtype=pkg.binding.FM_KV_FP8_E4M3)
    c = pkg.Context(cfg)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device=dev); gen.manual_seed(77 + batch)
    q = torch.randn((batch, 8192), device=dev, generator=gen); g = torch.randn((batch, 8192), device=dev, generator=gen)
    k = torch.randn((batch, 512), device=dev, generator=gen); v = torch.randn((batch, 512), device=dev, generator=gen)
    dims = make_dims()
    refs = []
    for s in range(batch):
        K = torch.randn((ctx, 512), device=dev, generator=gen); V = torch.randn((ctx, 512), device=dev, generator=gen)
        c.kv_import(0, s, K, V, ctx)
        cache = Cache(ctx + 1, 512, fp8=True)
        k8 = torch.zeros((ctx, 512), dtype=torch.uint8, device=dev); v8 = torch.zeros_like(k8)
        ks = torch.zeros(ctx, device=dev); vs = torch.zeros(ctx, device=dev)
        assert c.kv_export_fp8(0, s, k8, v8, ks, vs, ctx) == ctx
        torch.cuda.synchronize()
        cache.k8[:ctx] = k8.cpu().numpy(); cache.v8[:ctx] = v8.cpu().numpy()
        cache.k_scales[:ctx] = ks.cpu().numpy(); cache.v_scales[:ctx] = vs.cpu().numpy()
        cache.c.len = ctx
        refs.append(port.attn_run_cache(dims, cache, q[s:s + 1].cpu().numpy(), g[s:s + 1].cpu().numpy(), k[s:s + 1].cpu().numpy(),
                                        v[s:s + 1].cpu().numpy(), start_pos=ctx, threads=host_threads()))
    out = torch.empty((batch, 8192), device=dev)
    c.attn_decode(0, list(range(batch)), [ctx] * batch, out, q=q, gate=g, k=k, v=v)
    c.synchronize()
    got = out.cpu().numpy()
    for s in range(batch):
        gated, _, rr = rel_errors(got[s], refs[s])
        print("batch", batch, "ctx", ctx, "seq", s, "gated", gated, "rms-rel", rr)
        assert gated <= TOL
    c.close()


def test_fp8_prefill_is_refused(pkg, synth):
    c = fp8_ctx(pkg, max_seq_len=256)
    q, g, k, v = synth.attn_step_inputs(1, 4)
    out = np.empty((4, 8192), np.float32)
    with pytest.raises(pkg.FmError) as e:
        c.attn_prefill(0, 0, 0, 4, out, q=q, gate=g, k=k, v=v)
    assert e.value.status == pkg.binding.FM_ERR_UNSUPPORTED
    c.close()
