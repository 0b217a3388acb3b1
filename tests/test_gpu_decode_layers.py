"""fm_attn_decode_layers: one call steps a token through several layers, consecutive launches
overlapping (needs a B200).  Every layer of every step is checked against the CPU checker run on
that layer alone, so a launch that ran ahead of data it depends on would show."""
import numpy as np
import pytest

from gpu_util import oracle_attn
from parity import rel_errors

pytestmark = pytest.mark.gpu
TOL = 2e-3
H, HKV, D = 32, 2, 256


@pytest.mark.parametrize("lens,layers,steps,host", [((3000, 1200, 4500), 6, 4, False), ((64,), 3, 3, False),
                                                    ((20000,), 4, 2, False), ((700, 2100), 5, 3, True),
                                                    ((700, 2100), 5, 2, "pinned"), ((900,), 1, 2, "pinned"),
                                                    ((900, 100), 2, 2, True), ((300,), 9, 2, "pinned")])
def test_layers_call_matches_layer_by_layer_checker(pkg, port, synth, lens, layers, steps, host):
    """host=True: the same call with pageable host arrays (staged through the library's page-locked buffer);
    host="pinned": page-locked caller arrays, copied directly.  Either way the copies run on the library's copy stream
    in groups (first layers | rest; all but the last layer's outputs | last), whatever the number of layers."""
    import torch
    dev = torch.device("cuda:0")
    B = len(lens)
    cfg = pkg.default_config(num_full_layers=layers, num_linear_layers=0, max_seqs=B,
                             max_seq_len=max(lens) + steps + 64)
    c = pkg.Context(cfg)
    c.set_stream(torch.cuda.current_stream().cuda_stream)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    caches, steps_in = {}, {}
    for l in range(layers):
        for s, L in enumerate(lens):
            k0, v0 = synth.attn_cache(300 + l, L, tag=f"s{s}")
            caches[l, s] = (k0, v0)
            c.kv_import(l, s, t(k0), t(v0), L)
            q, g, k, v = synth.attn_step_inputs(300 + l, steps, tag=f"s{s}")
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
        if host:
            c.set_pointer_mode(pkg.binding.FM_PTR_HOST)
            out = np.empty((layers, B, H * D), np.float32)
            if host == "pinned":
                pin = lambda a: torch.empty(a.shape, dtype=torch.float32, pin_memory=True).copy_(torch.from_numpy(a)).numpy()
                qp, kk, vv = pin(qp), pin(kk), pin(vv)
                out = torch.empty((layers, B, H * D), dtype=torch.float32, pin_memory=True).numpy()
            c.attn_decode_layers(0, layers, list(range(B)), [L + st for L in lens], out, qp, kk, vv, sq, skv, so)
            c.set_pointer_mode(pkg.binding.FM_PTR_DEVICE)
        else:
            out = torch.empty((layers, B, H * D), device=dev)
            c.attn_decode_layers(0, layers, list(range(B)), [L + st for L in lens], out, t(qp), t(kk), t(vv), sq, skv, so)
        outs.append(out)
    c.synchronize()
    outs = [o if host else o.cpu().numpy() for o in outs]
    worst = 0.0
    for l in range(layers):
        for s, L in enumerate(lens):
            k0, v0 = caches[l, s]
            q, g, k, v = steps_in[l, s]
            ref, _, _ = oracle_attn(port, H, HKV, k0, v0, q, g, k, v)
            for st in range(steps):
                gated, _, _ = rel_errors(outs[st][l, s], ref[st])
                worst = max(worst, gated)
                assert gated <= TOL, (l, s, st, gated)
            assert c.kv_len(l, s) == L + steps
    print("decode_layers", lens, layers, "layers worst gated", worst)
    c.close()
