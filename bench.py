"""Benchmark of the attention hot path: gated GQA decode attention over the paged bf16 KV store.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): one decode token for `batch` sequences at context `ctx` through the
`layers` full-attention layers of the hybrid stack (append of the new K/V row + attention over the
whole context + sigmoid gate), production shapes 32 q / 2 kv heads x 256, RoPE on 64 dims.
Metric: KV-cache bytes streamed per second (K and V rows of every layer and sequence, bf16), the
figure the HBM roofline bounds.  Synthetic N(0,1) data, bf16-representable.

N > 1 (launched by torchrun, one rank per GPU): the same workload sharded by KV head (2 groups) and
along the sequence (N/2 shards, pages round-robin); partial softmax results are all-gathered inside
each sequence group with NCCL and merged by log-sum-exp.  Strong scaling: total work is fixed.

--impl reference times the reference project's own CPU attention code (oracle/_ref, else the C
restatement) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

H, HKV, D = 32, 2, 256
KV_BYTES_PER_ROW = 2 * HKV * D * 2  # K and V, bf16, both KV heads (set_kv_dtype changes it for an FP8 store)
KV_DTYPE = "bf16"


def set_kv_dtype(name: str):
    """bf16: 2 bytes per element.  fp8: one E4M3 byte per element plus the row's two fp32 scales."""
    global KV_BYTES_PER_ROW, KV_DTYPE
    KV_DTYPE = name
    KV_BYTES_PER_ROW = 2 * HKV * D * 2 if name == "bf16" else 2 * HKV * D + 8


def algorithmic_bytes_per_layer_seq(L: int) -> int:
    """K+V rows once, q / gate / out once, the appended row."""
    return L * KV_BYTES_PER_ROW + 3 * H * D * 4 + KV_BYTES_PER_ROW


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle.oracle_py import Oracle, host_threads, make_dims, ref_available
    from __graft_entry__ import load_package
    synth = load_package().synth
    kind = "reference" if ref_available() else "port"
    orc = Oracle(kind)
    threads = host_threads()
    L = args.ctx
    cap = L + args.steps + args.warmup + 1
    dims = make_dims()
    rng = np.random.default_rng(0)
    # the arithmetic does not depend on the values; a fast generator keeps set-up short
    kc = np.zeros((cap, HKV * D), np.float32); vc = np.zeros_like(kc)
    kc[:L] = rng.standard_normal((L, HKV * D), dtype=np.float32)
    vc[:L] = rng.standard_normal((L, HKV * D), dtype=np.float32)
    q, g, k, v = synth.attn_step_inputs(0, args.steps + args.warmup)
    ln = L
    for t in range(args.warmup):
        _, ln = orc.attn_run(dims, kc, vc, ln, q[t:t + 1], g[t:t + 1], k[t:t + 1], v[t:t + 1], threads=threads)
    t0 = time.perf_counter()
    for t in range(args.warmup, args.warmup + args.steps):
        _, ln = orc.attn_run(dims, kc, vc, ln, q[t:t + 1], g[t:t + 1], k[t:t + 1], v[t:t + 1], threads=threads)
    dt = time.perf_counter() - t0
    ms = dt * 1e3 / args.steps
    value = (L + args.warmup + (args.steps + 1) / 2) * KV_BYTES_PER_ROW / (ms * 1e-3) / 1e9
    sample = (f"1 layer x 1 sequence of the workload per step (context {L}, append + attention + gate), "
              f"reference CPU code with its per-head loop on {threads} OpenMP threads; value = the same rows "
              "counted as bf16 KV bytes per second")
    line = {
        "impl": "reference", "metric": "decode_attn_kv_stream", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(args), "batch": args.batch, "ctx": L, "layers": args.layers},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_name(args):
    return (f"gated GQA decode attention, batch {args.batch}, context {args.ctx}, {args.layers} full-attention "
            f"layers, {H}q/{HKV}kv heads x {D}, {'bf16' if KV_DTYPE == 'bf16' else 'FP8 E4M3 (per-row scales)'} paged KV")


# ---------------------------------------------------------------------------------------------
def cpu_baseline(args, synth):
    """The reference's CPU code on the host cores, on one (layer, sequence) of the workload."""
    from oracle.oracle_py import Oracle, host_threads, make_dims, ref_available
    kind = "reference" if ref_available() else "port"
    orc = Oracle(kind)
    threads = host_threads()
    L = args.ctx
    reps = 3
    rng = np.random.default_rng(0)
    kc = np.zeros((L + reps + 1, HKV * D), np.float32); vc = np.zeros_like(kc)
    kc[:L] = rng.standard_normal((L, HKV * D), dtype=np.float32)
    vc[:L] = rng.standard_normal((L, HKV * D), dtype=np.float32)
    q, g, k, v = synth.attn_step_inputs(0, reps + 1)
    dims = make_dims()
    _, ln = orc.attn_run(dims, kc, vc, L, q[:1], g[:1], k[:1], v[:1], threads=threads)
    t0 = time.perf_counter()
    for t in range(1, reps + 1):
        _, ln = orc.attn_run(dims, kc, vc, ln, q[t:t + 1], g[t:t + 1], k[t:t + 1], v[t:t + 1], threads=threads)
    dt = (time.perf_counter() - t0) / reps
    return {"value": L * KV_BYTES_PER_ROW / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "ms_per_layer_seq": dt * 1e3,
            "sample": (f"{reps} decode steps of 1 layer x 1 sequence at context {L} (of {args.layers} layers x "
                       f"{args.batch} sequences per step), per-head loop on {threads} OpenMP threads; rows counted "
                       "as bf16 KV bytes so the ratio to `value` is a speed ratio")}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    synth = pkg.synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    # mesh: KV-head groups x sequence shards
    mesh = pkg.sharding.mesh_for(world, HKV)
    hg, ss = mesh.head_groups, mesh.seq_shards
    my_hg, my_ss = mesh.coords(rank)
    seq_group = None
    if ss > 1:
        for g_ in range(hg):
            grp = dist.new_group(mesh.seq_group_ranks(g_))
            if g_ == my_hg:
                seq_group = grp
    Hl, Hkvl = H // hg, HKV // hg
    B, L, NL = args.batch, args.ctx, args.layers
    total_steps = 2 * args.steps + args.warmup + args.e2e_steps + 4
    cfg = pkg.default_config(num_attn_heads=Hl, num_kv_heads=Hkvl, num_full_layers=NL, num_linear_layers=0,
                             max_seqs=B, max_seq_len=L + total_steps + 64, max_batch_tokens=max(B, 64),
                             seq_shard_rank=my_ss, seq_shard_count=ss, device=local,
                             kv_dtype=pkg.binding.FM_KV_FP8_E4M3 if KV_DTYPE == "fp8" else pkg.binding.FM_KV_BF16)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)

    gen = torch.Generator(device=dev); gen.manual_seed(1234 + rank)
    for layer in range(NL):
        for s in range(B):
            K = torch.randn((L, Hkvl * D), device=dev, generator=gen).bfloat16().float()
            V = torch.randn((L, Hkvl * D), device=dev, generator=gen).bfloat16().float()
            ctx.kv_import(layer, s, K, V, L)
    del K, V
    # the step's inputs are those of the head group: the same on every rank of a sequence group
    gen = torch.Generator(device=dev); gen.manual_seed(99991 + my_hg)
    qp = torch.randn((NL, B, Hl * 2 * D), device=dev, generator=gen)
    kn = torch.randn((NL, B, Hkvl * D), device=dev, generator=gen)
    vn = torch.randn((NL, B, Hkvl * D), device=dev, generator=gen)
    out = torch.empty((NL, B, Hl * D), device=dev)
    seqs = list(range(B))
    o_part = torch.empty((B, Hl, D), device=dev); ml_part = torch.empty((B, Hl, 2), device=dev)
    o_all = torch.empty((ss, B, Hl, D), device=dev); ml_all = torch.empty((ss, B, Hl, 2), device=dev)
    cur = [L]
    p2p = ss > 1 and args.exchange == "p2p"
    if p2p:
        # exchange buffers the ranks of a sequence group map for each other (symmetric memory);
        # the library then moves the partial results itself with peer stores, no collective call
        import torch.distributed._symmetric_memory as symm
        xbuf = symm.empty(ctx.exchange_bytes(ss) // 4, dtype=torch.float32, device=dev)
        hdl = symm.rendezvous(xbuf, group=seq_group)
        ctx.exchange_attach(hdl.rank, list(hdl.buffer_ptrs))
        torch.cuda.synchronize()
        dist.barrier()

    sq, skv, so = B * Hl * 2 * D, B * Hkvl * D, B * Hl * D  # floats between consecutive layers

    def step():
        pos = [cur[0]] * B
        if ss == 1 or p2p:
            # the layer loop runs inside the library, as in a C host (one call per token)
            ctx.attn_decode_layers(0, NL, seqs, pos, out, qp, kn, vn, sq, skv, so, exchange=p2p)
            cur[0] += 1
            return
        for layer in range(NL):
            ctx.attn_decode_partial(layer, seqs, pos, o_part, ml_part, q_proj_out=qp[layer], k=kn[layer], v=vn[layer])
            dist.all_gather_into_tensor(o_all, o_part, group=seq_group)
            dist.all_gather_into_tensor(ml_all, ml_part, group=seq_group)
            ctx.attn_merge_gate(ss, o_all, ml_all, B, out[layer], q_proj_out=qp[layer])
        cur[0] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.15)
    launches0 = ctx.launch_count()
    L_first = cur[0]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = ctx.launch_count() - launches0
    # the same K steps once more with an event pair around every decode launch: the per-launch
    # duration the roofline uses.  Kept out of the region above because the event records sit
    # between consecutive launches and lengthen the step they measure.
    ctx.profile_read()
    ctx.profile_enable(True)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for _ in range(args.steps):
        step()
    p1.record()
    barrier()
    ms_profiled = p0.elapsed_time(p1) / args.steps
    n_kern, kern_ms = ctx.profile_read()
    ctx.profile_enable(False)
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms_total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    L_mean = L_first + (args.steps + 1) / 2  # rows attended, averaged over the timed steps
    kv_bytes_step = L_mean * KV_BYTES_PER_ROW * B * NL  # whole job, all ranks
    value = kv_bytes_step / (ms_step * 1e-3) / 1e9

    # roofline of the dominant kernel (split-KV decode) on this rank
    peak, peak_kind = load_peaks()
    alg_bytes_launch = algorithmic_bytes_per_layer_seq(int(L_mean)) * B / world
    traffic_scale = 1.0 if KV_DTYPE == "bf16" else None  # the ncu capture below is of the bf16 kernel
    # The timed region holds nothing but launches of this kernel, consecutive ones overlapping at their
    # ends: its average launch duration is the region's device time over the launches in it.  The same
    # launches bracketed one by one (second pass) include each launch's start-up and drain.
    n_dec = NL * args.steps  # one decode launch per layer and step (an exchange adds its merge launch to the same slot)
    kern_s = ms_total * 1e-3 / n_dec
    iso_s = kern_ms * 1e-3 / max(n_kern, 1)
    achieved = alg_bytes_launch / kern_s / 1e9
    roofline = {"bound": "hbm", "kernel": "attn_decode_kernel", "achieved": achieved, "peak": peak,
                "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
                "unit": "GB/s", "frac": achieved / peak if achieved else None,
                "us_per_launch": kern_s * 1e6, "launches_timed": n_dec,
                "us_per_launch_bracketed_alone": iso_s * 1e6, "ms_per_step_with_launch_events": ms_profiled,
                "algorithmic_bytes_per_launch": alg_bytes_launch,
                "traffic": TRAFFIC_NCU_1SEQ_128K * (B / world) * (L_mean / 131073.0) if traffic_scale else None,
                "traffic_source": "ncu capture at batch 1, scaled by sequences x rows per launch" if traffic_scale else None}

    # ---- end to end through the C-ABI with host buffers (rank-local copies inside the timed region) ----
    e2e = None
    if args.e2e_steps > 0:
        ctx.set_pointer_mode(pkg.binding.FM_PTR_HOST)
        # page-locked host buffers, as a serving host keeps for its projections
        pin = lambda t_: torch.empty(t_.shape, dtype=t_.dtype, pin_memory=True).copy_(t_).numpy()
        h_qp, h_k, h_v = pin(qp), pin(kn), pin(vn)
        h_out = torch.empty((NL, B, Hl * D), dtype=torch.float32, pin_memory=True).numpy()
        h_o = np.empty((B, Hl, D), np.float32); h_ml = np.empty((B, Hl, 2), np.float32)

        def step_host():
            pos = [cur[0]] * B
            if ss == 1 or p2p:
                ctx.attn_decode_layers(0, NL, seqs, pos, h_out, h_qp, h_k, h_v, sq, skv, so, exchange=p2p)
                cur[0] += 1
                return
            for layer in range(NL):
                ctx.attn_decode_partial(layer, seqs, pos, h_o, h_ml, q_proj_out=h_qp[layer], k=h_k[layer], v=h_v[layer])
                o_part.copy_(torch.from_numpy(h_o)); ml_part.copy_(torch.from_numpy(h_ml))
                dist.all_gather_into_tensor(o_all, o_part, group=seq_group)
                dist.all_gather_into_tensor(ml_all, ml_part, group=seq_group)
                ctx.set_pointer_mode(pkg.binding.FM_PTR_DEVICE)
                ctx.attn_merge_gate(ss, o_all, ml_all, B, out[layer], q_proj_out=qp[layer])
                ctx.set_pointer_mode(pkg.binding.FM_PTR_HOST)
                h_out[layer] = out[layer].cpu().numpy()
            cur[0] += 1

        step_host()
        barrier()
        L_e = cur[0]
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            step_host()
        barrier()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item()) / args.e2e_steps
        L_em = L_e + (args.e2e_steps + 1) / 2
        e2e = {"value": L_em * KV_BYTES_PER_ROW * B * NL / dt / 1e9, "unit": "GB/s",
               "ms_per_step": dt * 1e3,
               "h2d_bytes_per_step": int(NL * B * (Hl * 2 * D + 2 * Hkvl * D) * 4 * world),
               "d2h_bytes_per_step": int(NL * B * Hl * D * 4 * world),
               "note": "fm_attn_decode_layers in host-pointer mode: every step copies q_proj_out, k, v of all layers "
                       "from page-locked host memory to the device and the gated outputs back; the KV cache is resident state"}
        ctx.set_pointer_mode(pkg.binding.FM_PTR_DEVICE)

    # ---- correctness of what was timed: one more step of the same workload, one (layer, sequence) of it against
    # the CPU checker on every rank (each rank holds one KV-head group; the ranks of a sequence group put their
    # shards of the cache together first).  Outside every timed region.
    parity = None
    if not args.no_check:
        parity = parity_check(args, pkg, torch, dist, ctx, step, cur, qp, kn, vn, out, dev, world, ss, seq_group, Hl, Hkvl)

    extra = {}
    if world > 1 and not args.no_extra and 16 % world == 0:
        # GatedDeltaNet decode sharded by value head over the ranks (no exchange inside the path): every rank steps its
        # 64 / N value heads; the time of a layer step is the slowest rank's
        ctx.close()
        ctx = None
        torch.cuda.empty_cache()
        extra = _probe_gdn_decode_sharded(pkg, torch, dist, dev, peak, rank, world)
        if ss == 1:
            # batch 64 x 131072 rows does not fit one GPU (258 GB of bf16 KV); split by KV head it does
            extra.update(_probe_attn_b64_head_sharded(pkg, torch, dist, dev, peak, rank, world, Hl, Hkvl))
    if rank == 0 and world == 1 and not args.no_extra:
        ctx.close()
        ctx = None
        torch.cuda.empty_cache()
        extra = extra_measurements(pkg, torch, dev, peak)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and KV_DTYPE == "bf16":  # the CPU leg times the reference's fp32 cache
        cpu = cpu_baseline(args, synth)

    if rank == 0:
        line = {
            "metric": "decode_attn_kv_stream", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if KV_DTYPE == "bf16" else "fp8_e4m3",
            "data": "synthetic",
            "config": {"workload": workload_name(args), "batch": B, "ctx": L, "layers": NL,
                       "parallelism": f"kv-head groups {hg} x sequence shards {ss}",
                       "exchange": ("none" if ss == 1 else "peer stores + flags (fm_attn_decode_exchange)" if p2p
                                    else "NCCL all-gather + fm_attn_merge_gate"),
                       "l2": "inputs larger than L2 (KV streamed per step: %.1f GB)" % (kv_bytes_step / 1e9)},
            "us_per_layer": ms_step * 1e3 / NL,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "clocks": clocks, "parity": parity, "extra": extra,
        }
        print(json.dumps(line))
    if ctx is not None:
        ctx.close()
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        sys.exit(3)


PARITY_TOL = 2e-3


def parity_check(args, pkg, torch, dist, ctx, step, cur, qp, kn, vn, out, dev, world, ss, seq_group, Hl, Hkvl):
    """Runs one more step of the timed workload and compares the last layer's output for the last sequence with
    the CPU checker fed the same cache rows and inputs (tolerance of the attention parity tests).  The checker
    is used as a checker only; nothing here is timed."""
    from oracle.oracle_py import Oracle, host_threads, make_dims
    B, NL = args.batch, args.layers
    layer, s = NL - 1, B - 1
    n = ctx.kv_len(layer, s)
    pos = cur[0]
    x = qp[layer, s].cpu().numpy().reshape(Hl, 2, D)
    q, gate = np.ascontiguousarray(x[:, 0].reshape(1, -1)), np.ascontiguousarray(x[:, 1].reshape(1, -1))
    k, v = kn[layer, s:s + 1].cpu().numpy(), vn[layer, s:s + 1].cpu().numpy()
    if KV_DTYPE == "fp8":
        from oracle.oracle_py import Cache
        k8 = torch.zeros((n, Hkvl * D), dtype=torch.uint8, device=dev); v8 = torch.zeros_like(k8)
        ks = torch.zeros(n, device=dev); vs = torch.zeros(n, device=dev)
        ctx.kv_export_fp8(layer, s, k8, v8, ks, vs, n)   # on a sequence-sharded store: the rows this rank owns
        torch.cuda.synchronize()
        if ss > 1:
            for t_ in (k8, v8, ks, vs):
                dist.all_reduce(t_, group=seq_group)
        cache = Cache(n + 1, Hkvl * D, fp8=True)
        cache.k8[:n] = k8.cpu().numpy(); cache.v8[:n] = v8.cpu().numpy()
        cache.k_scales[:n] = ks.cpu().numpy(); cache.v_scales[:n] = vs.cpu().numpy()
        cache.c.len = n
        del k8, v8
        step()
        torch.cuda.synchronize()
        got = out[layer, s].cpu().numpy()
        want = Oracle("port").attn_run_cache(make_dims(num_attn_heads=Hl, num_kv_heads=Hkvl), cache, q, gate, k, v, start_pos=pos,
                                             threads=host_threads())
    else:
        kd = torch.zeros((n + 1, Hkvl * D), device=dev); vd = torch.zeros_like(kd)
        ctx.kv_export(layer, s, kd, vd, n + 1)          # on a sequence-sharded store: the rows this rank owns
        torch.cuda.synchronize()
        if ss > 1:
            dist.all_reduce(kd, group=seq_group); dist.all_reduce(vd, group=seq_group)
        kc, vc = kd.cpu().numpy(), vd.cpu().numpy()
        del kd, vd
        step()
        torch.cuda.synchronize()
        got = out[layer, s].cpu().numpy()
        dims = make_dims(num_attn_heads=Hl, num_kv_heads=Hkvl, store_bf16=1)
        want, _ = Oracle("port").attn_run(dims, kc, vc, n, q, gate, k, v, start_pos=pos, threads=host_threads())
    a, r = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    err = float((np.abs(a - r) / np.maximum(np.abs(r), np.sqrt(np.mean(r * r)))).max())
    t = torch.tensor([err], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    err = float(t.item())
    return {"gated": err, "tol": PARITY_TOL, "ok": bool(err <= PARITY_TOL), "rows": n + 1,
            "checked": f"layer {layer}, sequence {s} of one more step of the timed workload, on every rank (max over ranks), "
                       "against the CPU checker"}


# DRAM bytes (read + write) of one attn_decode_kernel launch for ONE sequence at 131073 rows, from
# the committed ncu capture (profiles/attn_decode_kernel_b1_ctx128k_ncu.md): 268.76 MB + 4.43 MB.
# Traffic grows in proportion to rows x sequences, so the bench launch is scaled from it.  Captured on the kernel
# as of commit 946021c (wide merges as a dependent launch; its own traffic, a few hundred KB, is not included); refresh
# when the kernel's memory behaviour changes.
TRAFFIC_NCU_1SEQ_128K = 272.57e6


PROBE_REPS = None  # --probe with an explicit --steps: that many timed repetitions (short runs for profiling)


def extra_measurements(pkg, torch, dev, peak, only=None):
    """Batch-1 context sweep (us per layer and KV GB/s), prefill attention TFLOP/s, GatedDeltaNet decode
    and chunked prefill.  `only` runs a single one of them (used when profiling one kernel)."""
    res = {}
    gen = torch.Generator(device=dev); gen.manual_seed(7)
    want = lambda name: only is None or only == name
    if want("sweep"):
        res.update(_probe_sweep(pkg, torch, dev, peak, gen))
    if want("prefill"):
        res.update(_probe_prefill(pkg, torch, dev, gen))
    if want("gdn_decode"):
        res.update(_probe_gdn_decode(pkg, torch, dev, peak, gen))
    if want("gdn_prefill"):
        res.update(_probe_gdn_prefill(pkg, torch, dev, gen))
    if want("out_proj"):
        res.update(_probe_out_proj(pkg, torch, dev, peak))
    if want("kv_policies"):
        res.update(_probe_kv_policies(pkg, torch, dev, peak, gen))
    if want("hybrid"):
        res.update(_probe_hybrid(pkg, torch, dev, peak, gen))
    return res


def _probe_out_proj(pkg, torch, dev, peak):
    """o_proj / out_proj from the reference's 4-bit format + residual + post-attention norm, 4096 x 8192, cycling 16 weight
    sets (300 MB) so that the weights come from HBM; bytes = packed weights + scales + biases."""
    res = {}
    out_dim, in_dim, nsets = 4096, 8192, 16
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seq_len=128, max_batch_tokens=64)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(0)
    w = rng.integers(0, 2 ** 32, size=(out_dim, in_dim // 8), dtype=np.uint64).astype(np.uint32)
    sc = pkg.synth.to_bf16_bits(np.full((out_dim, in_dim // 64), 0.004, np.float32))
    bi = pkg.synth.to_bf16_bits(np.full((out_dim, in_dim // 64), -0.03, np.float32))
    sets = [ctx.proj_upload(w, sc, bi) for _ in range(nsets)]
    nw = torch.ones(out_dim, dtype=torch.bfloat16, device=dev)
    wbytes = out_dim * in_dim // 2 + 2 * out_dim * (in_dim // 64) * 2
    for n in (1, 8, 64):
        x = torch.randn((n, in_dim), device=dev); r = torch.randn((n, out_dim), device=dev)
        hm = torch.empty((n, out_dim), device=dev); hp = torch.empty_like(hm)
        import ctypes as C
        ptr = lambda t_: C.c_void_p(t_.data_ptr())
        calls = [(C.byref(d), C.c_int(n), ptr(x), ptr(r), ptr(nw), ptr(hm), ptr(hp)) for d in sets]  # arguments converted once
        fn, h = ctx.lib.fm_out_proj_norm, ctx.h

        def run():
            for a in calls:
                fn(h, *a)
        reps = PROBE_REPS or 10
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        us_host = e0.elapsed_time(e1) * 1e3 / (reps * nsets)
        us, note = us_host, None
        try:  # the same pass as one CUDA graph: one host call per projection is bounded by the host's call rate
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                ctx.set_stream(torch.cuda.current_stream().cuda_stream)
                run()
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * nsets)
            del g
        except Exception as exc:  # noqa: BLE001
            note = f"graph capture failed: {exc}"[:200]
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        res[f"out_proj_q4_n{n}"] = {"us": us, "us_host_launched": us_host, "weight_gbps": wbytes / us / 1e3,
                                     "frac_of_peak": wbytes / us / 1e3 / peak, "weight_bytes": wbytes,
                                     "issued_as": note or "one CUDA graph of the calls' launches"}
    for d in sets:
        ctx.proj_free(d)
    ctx.close()
    return res


def _probe_kv_policies(pkg, torch, dev, peak, gen):
    """The decode step under the reference's cache policies, batch 8, 32768 rows attended, 8 layers cycled (the bf16 store
    is 4.3 GB per pass: far more than L2), one fm_attn_decode call per layer: the bf16 store as the yardstick, the FP8
    store, a sliding window of 32768 rows (circular store, already wrapped), and H2O eviction with a budget of 32768
    rows (every step evicts; the figure includes the mass / eviction launch)."""
    res = {}
    B, L, NL = 8, 32768, 8
    K = torch.randn((L, HKV * D), device=dev, generator=gen).bfloat16().float()
    qp = torch.randn((NL, B, H * 2 * D), device=dev, generator=gen)
    kn = torch.randn((NL, B, HKV * D), device=dev, generator=gen)
    out = torch.empty((NL, B, H * D), device=dev)
    seq_arr = np.arange(B, dtype=np.int32)
    pos_arr = np.zeros(B, dtype=np.int32)
    variants = (("bf16", {}, 2048), ("fp8", {"kv_dtype": pkg.binding.FM_KV_FP8_E4M3}, 1032),
                ("sliding_window", {"sliding_window": L}, 2048), ("h2o", {"h2o_budget": L, "h2o_num_sinks": 4}, 2048))
    for name, extra_cfg, row_bytes in variants:
        cfg = pkg.default_config(num_full_layers=NL, num_linear_layers=0, max_seqs=B, max_seq_len=L + 256, max_batch_tokens=64, **extra_cfg)
        ctx = pkg.Context(cfg)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        for layer in range(NL):
            for s_ in range(B):
                ctx.kv_import(layer, s_, K, K, L - 1 if name == "h2o" else L)
        calls = [ctx.prepared("fm_attn_decode", l, seq_arr, pos_arr, B, qp[l], None, None, kn[l], kn[l], None, None, out[l]) for l in range(NL)]
        pos = L
        launches0 = ctx.launch_count()

        def token():
            pos_arr[:] = pos
            for f in calls:
                f()
        for _ in range(3):
            token(); pos += 1
        torch.cuda.synchronize()
        reps = PROBE_REPS or 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            token(); pos += 1
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * NL)
        rows_bytes = B * L * row_bytes
        res[name] = {"us_per_layer": us, "kv_gbps": rows_bytes / us / 1e3, "frac_of_peak": rows_bytes / us / 1e3 / peak,
                     "launches_per_layer": (ctx.launch_count() - launches0) / ((reps + 3) * NL)}
        ctx.close()
        del ctx
        torch.cuda.empty_cache()
    return {"decode_b8_32k_cache_policies": res}


def _probe_hybrid(pkg, torch, dev, peak, gen):
    """One decode token through the token-mixing part of the full hybrid stack: 60 layers arranged as 15 x (3
    GatedDeltaNet + 1 gated GQA), each layer's entry point called in model order (the projections and MoE between
    them are outside this library).  Batch x context combinations that fit one GPU."""
    res = {}
    tw = _gdn_weights(pkg, torch, dev)
    out = {}
    for B, L in ((1, 32768), (1, 131072), (8, 32768), (8, 131072), (64, 32768)):
        cfg = pkg.default_config(num_full_layers=15, num_linear_layers=45, max_seqs=B, max_seq_len=L + 64,
                                 max_batch_tokens=max(B, 64))
        ctx = pkg.Context(cfg)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        ctx.set_layer_overlap(True)  # consecutive calls step different layers, as in the model
        K = torch.randn((L, HKV * D), device=dev, generator=gen).bfloat16().float()
        for layer in range(15):
            for s in range(B):
                ctx.kv_import(layer, s, K, K, L)
        del K
        qp = torch.randn((B, H * 2 * D), device=dev, generator=gen)
        kn = torch.randn((B, HKV * D), device=dev, generator=gen)
        ao = torch.empty((B, H * D), device=dev)
        qkv = torch.randn((B, 12288), device=dev, generator=gen)
        z = torch.randn((B, 8192), device=dev, generator=gen)
        be = torch.randn((B, 64), device=dev, generator=gen)
        al = torch.randn((B, 64), device=dev, generator=gen)
        go = torch.empty((B, 8192), device=dev)
        # the calls of one token, arguments converted once (a C host pays no per-call conversion either)
        seq_arr = np.arange(B, dtype=np.int32)
        pos_arr = np.full(B, L, dtype=np.int32)
        calls = []
        for blk in range(15):
            for j in range(3):
                calls.append(ctx.prepared("fm_gdn_decode", 3 * blk + j, seq_arr, B, qkv, z, be, al, tw["conv_w"], tw["A_log"],
                                          tw["dt_bias"], tw["norm_w"], go))
            calls.append(ctx.prepared("fm_attn_decode", blk, seq_arr, pos_arr, B, qp, None, None, kn, kn, None, None, ao))

        def token():
            for f in calls:
                f()
            pos_arr[:] += 1

        for _ in range(3):
            token()
        torch.cuda.synchronize()
        reps = 10 if B * L <= 262144 else 4
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            token()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        # the same token as one CUDA graph of its 60+ launches, replayed (every replay repeats the captured step: the
        # same rows are attended and the same row rewritten, so the time is that of a step and the state stands still)
        ms_graph, graph_note = None, None
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                ctx.set_stream(torch.cuda.current_stream().cuda_stream)
                token()
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
            for _ in range(2):
                g.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            ms_graph = e0.elapsed_time(e1) / reps
            del g
        except Exception as exc:  # noqa: BLE001
            graph_note = f"graph capture failed: {exc}"[:200]
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        kv_bytes = 15 * B * (L + 4) * KV_BYTES_PER_ROW
        gdn_bytes = 45 * (B * (2 * 4194304 + 2 * 147456 + (12288 + 8192 + 128 + 8192) * 4) + 98304 + 768)
        out[f"b{B}_ctx{L}"] = {"ms_per_token": ms, "ms_per_token_as_one_cuda_graph": ms_graph or graph_note,
                               "bytes_per_token": kv_bytes + gdn_bytes,
                               "gbps": (kv_bytes + gdn_bytes) / ms / 1e6, "frac_of_peak": (kv_bytes + gdn_bytes) / ms / 1e6 / peak}
        ctx.close()
        del ctx
        torch.cuda.empty_cache()
    res["hybrid_stack_token_mixing"] = out
    return res


def _probe_sweep(pkg, torch, dev, peak, gen):
    res = {}
    # ---- batch-1 decode sweep; 32 layers so that even the 4K case streams more than L2 per pass ----
    NL = 32
    sweep = {}
    Lmax = 131072
    cfg = pkg.default_config(num_full_layers=NL, num_linear_layers=0, max_seqs=1, max_seq_len=Lmax + 4096)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    K = torch.randn((Lmax, HKV * D), device=dev, generator=gen).bfloat16().float()
    V = torch.randn((Lmax, HKV * D), device=dev, generator=gen).bfloat16().float()
    qp = torch.randn((NL, 1, H * 2 * D), device=dev, generator=gen)
    kn = torch.randn((NL, 1, HKV * D), device=dev, generator=gen)
    out = torch.empty((NL, 1, H * D), device=dev)
    sq, skv, so = H * 2 * D, HKV * D, H * D

    seq_arr = np.zeros(1, dtype=np.int32)
    pos_arr = np.zeros(1, dtype=np.int32)
    # model order: one fm_attn_decode call per layer, each an ordinary launch that starts when the previous one has
    # finished (in the model, layer l+1's projections depend on layer l's output)
    calls = [ctx.prepared("fm_attn_decode", l, seq_arr, pos_arr, 1, qp[l], None, None, kn[l], kn[l], None, None, out[l])
             for l in range(NL)]

    def token(pos):
        pos_arr[0] = pos
        for f in calls:
            f()

    def token_overlapped(pos):  # one C call for all layers: consecutive layers' launches overlap (needs every layer's
        ctx.attn_decode_layers(0, NL, [0], [pos], out, qp, kn, kn, sq, skv, so)  # inputs up front: a throughput figure)

    def timed(fn, pos, reps):
        for _ in range(3):
            fn(pos); pos += 1
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for r in range(reps):
            fn(pos); pos += 1
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * NL), pos

    for L in (4096, 8192, 16384, 32768, 65536, 131072):
        for layer in range(NL):
            ctx.kv_import(layer, 0, K, V, L)
        reps = 6 if L >= 65536 else 20
        us_layer, pos = timed(token, L, reps)
        us_overlapped, pos = timed(token_overlapped, pos, reps)
        kvb = 2 * (L + 4 + reps / 2) * HKV * D * 2
        sweep[str(L)] = {"us_per_layer": us_layer, "kv_gbps": kvb / us_layer / 1e3, "frac_of_peak": kvb / us_layer / 1e3 / peak,
                         "how": "one fm_attn_decode call per layer in model order (no overlap between layers)",
                         "us_per_layer_all_layers_in_one_call": us_overlapped,
                         "kv_gbps_all_layers_in_one_call": kvb / us_overlapped / 1e3}
    res["decode_b1_sweep"] = sweep
    ctx.close()
    del K, V
    torch.cuda.empty_cache()
    return res


def _probe_prefill(pkg, torch, dev, gen):
    res = {}
    # ---- causal prefill attention, T = 2048, empty cache ----
    T = 2048
    cfg = pkg.default_config(num_full_layers=1, num_linear_layers=0, max_seqs=1, max_seq_len=T + 64, max_batch_tokens=T)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    q = torch.randn((T, H * D), device=dev, generator=gen).bfloat16().float()
    g = torch.randn((T, H * D), device=dev, generator=gen)
    k = torch.randn((T, HKV * D), device=dev, generator=gen).bfloat16().float()
    v = torch.randn((T, HKV * D), device=dev, generator=gen).bfloat16().float()
    o = torch.empty((T, H * D), device=dev)
    times = []
    for it in range(4):
        ctx.reset(0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.attn_prefill(0, 0, 0, T, o, q=q, gate=g, k=k, v=v)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = min(times[1:])
    flops = 4 * H * D * T * (T + 1) / 2
    ctx.profile_read(); ctx.profile_enable(True)
    ctx.reset(0)
    ctx.attn_prefill(0, 0, 0, T, o, q=q, gate=g, k=k, v=v)
    n_k, k_ms = ctx.profile_read(); ctx.profile_enable(False)
    res["prefill_attn_T2048"] = {"ms": ms, "tflops": flops / ms / 1e9, "algorithmic_gflop": flops / 1e9,
                                 "ms_launches_bracketed": k_ms, "tflops_launches_bracketed": flops / k_ms / 1e9}
    ctx.close()
    return res


def _gdn_weights(pkg, torch, dev):
    w = pkg.synth.gdn_weights(0)
    return {k_: torch.from_numpy(v_.view(np.int16) if v_.dtype == np.uint16 else v_).to(dev) for k_, v_ in w.items()}


def _probe_gdn_decode(pkg, torch, dev, peak, gen):
    """GatedDeltaNet decode step, one launch per layer, cycling layers so that the states read exceed L2:
    batch 1 over the 45 layers (180 MiB), batch 8 over 45 layers, batch 64 over 8 layers (2 GiB)."""
    res = {}
    tw = _gdn_weights(pkg, torch, dev)
    for B, NL, reps in ((1, 45, 20), (8, 45, 10), (64, 8, 10)):
        cfg = pkg.default_config(num_full_layers=0, num_linear_layers=NL, max_seqs=B, max_batch_tokens=max(B, 64))
        ctx = pkg.Context(cfg)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        qkv = torch.randn((B, 12288), device=dev, generator=gen)
        z = torch.randn((B, 8192), device=dev, generator=gen)
        be = torch.randn((B, 64), device=dev, generator=gen)
        al = torch.randn((B, 64), device=dev, generator=gen)
        go = torch.empty((B, 8192), device=dev)
        seq_arr = np.arange(B, dtype=np.int32)
        calls = [ctx.prepared("fm_gdn_decode", li, seq_arr, B, qkv, z, be, al, tw["conv_w"], tw["A_log"], tw["dt_bias"],
                              tw["norm_w"], go) for li in range(NL)]

        def gdn_pass():
            for f in calls:
                f()

        for _ in range(3):
            gdn_pass()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            gdn_pass()
        e1.record()
        torch.cuda.synchronize()
        us_host = e0.elapsed_time(e1) * 1e3 / (reps * NL)
        # host-launched once more with fm_set_layer_overlap (consecutive calls step different layers: a step may be
        # launched under the previous one's tail)
        ctx.set_layer_overlap(True)
        for _ in range(3):
            gdn_pass()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            gdn_pass()
        e1.record()
        torch.cuda.synchronize()
        us_host_overlap = e0.elapsed_time(e1) * 1e3 / (reps * NL)
        ctx.set_layer_overlap(False)
        # the same pass as one CUDA graph (how a serving loop would issue it): at batch 1 a launch per host call is
        # bounded by the host's call rate, not by the kernel
        us = us_host
        graph_note = None
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                ctx.set_stream(torch.cuda.current_stream().cuda_stream)
                gdn_pass()
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * NL)
            del g
        except Exception as exc:  # noqa: BLE001
            graph_note = f"graph capture failed: {exc}"[:200]
            ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        # per sequence: state read + written, conv ring rows, inputs and output; weights once per launch
        gdn_bytes = B * (2 * 4194304 + 2 * 147456 + (12288 + 8192 + 128 + 8192) * 4) + 98304 + 768
        res[f"gdn_decode_b{B}"] = {"us_per_layer": us, "us_per_layer_host_launched": us_host,
                                   "us_per_layer_host_launched_layer_overlap": us_host_overlap, "state_gbps": gdn_bytes / us / 1e3,
                                   "frac_of_peak": gdn_bytes / us / 1e3 / peak, "algorithmic_bytes_per_layer": gdn_bytes,
                                   "layers_cycled": NL, "issued_as": graph_note or "one CUDA graph of the layers' launches"}
        ctx.close()
        del ctx
        torch.cuda.empty_cache()
    return res


def _probe_gdn_decode_sharded(pkg, torch, dist, dev, peak, rank, world):
    res = {}
    sh = pkg.sharding
    v0, nv, k0, nk = sh.gdn_head_slice(rank, world)
    w = pkg.synth.gdn_weights(0)
    zeros = np.zeros((1, 12288), np.float32)
    sl = sh.gdn_slice_inputs(rank, world, zeros, np.zeros((1, 8192), np.float32), np.zeros((1, 64), np.float32),
                             np.zeros((1, 64), np.float32), w["conv_w"], w["A_log"], w["dt_bias"])
    tw = {k_: torch.from_numpy(v_.view(np.int16) if v_.dtype == np.uint16 else v_).to(dev)
          for k_, v_ in dict(conv_w=sl["conv_w"], A_log=sl["A_log"], dt_bias=sl["dt_bias"], norm_w=w["norm_w"]).items()}
    gen = torch.Generator(device=dev); gen.manual_seed(11 + rank)
    conv_dim = 2 * nk * 128 + nv * 128
    for B, NL, reps in ((8, 45, 10), (64, 8, 10)):
        cfg = pkg.default_config(num_full_layers=0, num_linear_layers=NL, max_seqs=B, max_batch_tokens=max(B, 64),
                                 linear_num_v_heads=nv, linear_num_k_heads=nk, device=dev.index)
        ctx = pkg.Context(cfg)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        qkv = torch.randn((B, conv_dim), device=dev, generator=gen)
        z = torch.randn((B, nv * 128), device=dev, generator=gen)
        be = torch.randn((B, nv), device=dev, generator=gen)
        al = torch.randn((B, nv), device=dev, generator=gen)
        go = torch.empty((B, nv * 128), device=dev)
        seq_arr = np.arange(B, dtype=np.int32)
        calls = [ctx.prepared("fm_gdn_decode", li, seq_arr, B, qkv, z, be, al, tw["conv_w"], tw["A_log"], tw["dt_bias"],
                              tw["norm_w"], go) for li in range(NL)]
        for _ in range(3):
            for f in calls:
                f()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for f in calls:
                f()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / (reps * NL)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item())
        gdn_bytes = B * (2 * 4194304 + 2 * 147456 + (12288 + 8192 + 128 + 8192) * 4) + 98304 + 768  # the whole layer, all ranks
        res[f"gdn_decode_head_sharded_b{B}"] = {"us_per_layer": us, "state_gbps_all_ranks": gdn_bytes / us / 1e3,
                                                "frac_of_peak_per_gpu": gdn_bytes / us / 1e3 / peak / world,
                                                "v_heads_per_rank": nv, "layers_cycled": NL}
        ctx.close()
        del ctx
        torch.cuda.empty_cache()
    return res


def _probe_attn_b64_head_sharded(pkg, torch, dist, dev, peak, rank, world, Hl, Hkvl):
    """The largest cell of the hybrid configuration, batch 64 x context 131072: each rank holds one KV-head group (no
    exchange inside the path).  Three layers are filled and stepped in one call (26 GB of rows per rank and step, far
    more than L2; all 15 would take minutes to fill); the time is the slowest rank's, per layer and times 15."""
    B, L, NL = 64, 131072, 3
    need = B * (L + 128) * NL * Hkvl * D * 2 * 2 + (8 << 30)
    free, _ = torch.cuda.mem_get_info(dev)
    if free < need:
        return {"decode_b64_ctx131072_head_sharded": f"skipped: {need >> 30} GiB needed, {free >> 30} GiB free"}
    cfg = pkg.default_config(num_attn_heads=Hl, num_kv_heads=Hkvl, num_full_layers=NL, num_linear_layers=0, max_seqs=B,
                             max_seq_len=L + 64, max_batch_tokens=64, device=dev.index,
                             kv_dtype=pkg.binding.FM_KV_FP8_E4M3 if KV_DTYPE == "fp8" else pkg.binding.FM_KV_BF16)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device=dev); gen.manual_seed(4321 + rank)
    K = torch.randn((L, Hkvl * D), device=dev, generator=gen).bfloat16().float()
    for layer in range(NL):
        for s_ in range(B):
            ctx.kv_import(layer, s_, K, K, L)
    del K
    qp = torch.randn((NL, B, Hl * 2 * D), device=dev, generator=gen)
    kn = torch.randn((NL, B, Hkvl * D), device=dev, generator=gen)
    out = torch.empty((NL, B, Hl * D), device=dev)
    sq, skv, so = B * Hl * 2 * D, B * Hkvl * D, B * Hl * D
    seqs = list(range(B))
    pos = L

    def token(p_):
        ctx.attn_decode_layers(0, NL, seqs, [p_] * B, out, qp, kn, kn, sq, skv, so)
    for _ in range(2):
        token(pos); pos += 1
    torch.cuda.synchronize()
    dist.barrier()
    reps = 3
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        token(pos); pos += 1
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    kv_bytes = NL * B * (L + 3) * KV_BYTES_PER_ROW  # whole job: both KV heads
    ctx.close()
    del ctx
    torch.cuda.empty_cache()
    return {"decode_b64_ctx131072_head_sharded": {"ms_per_layer": ms / NL, "ms_per_token_15_layers": ms / NL * 15, "layers_stepped": NL,
                                                  "kv_gbps_all_ranks": kv_bytes / ms / 1e6,
                                                  "frac_of_peak_per_gpu": kv_bytes / ms / 1e6 / world / peak, "ranks": world}}


def _probe_gdn_prefill(pkg, torch, dev, gen):
    res = {}
    tw = _gdn_weights(pkg, torch, dev)
    # ---- chunked GatedDeltaNet prefill, T = 4096, chunk 64 ----
    T = 4096
    cfg = pkg.default_config(num_full_layers=0, num_linear_layers=1, max_seqs=1, max_batch_tokens=T)
    ctx = pkg.Context(cfg)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    qkv = torch.randn((T, 12288), device=dev, generator=gen).bfloat16().float()
    z = torch.randn((T, 8192), device=dev, generator=gen).bfloat16().float()
    be = torch.randn((T, 64), device=dev, generator=gen)
    al = torch.randn((T, 64), device=dev, generator=gen)
    go = torch.empty((T, 8192), device=dev)
    times = []
    for it in range(4):
        ctx.reset(0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.gdn_prefill(0, 0, T, qkv, z, be, al, go, tw["conv_w"], tw["A_log"], tw["dt_bias"], tw["norm_w"])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = min(times[1:])
    gflop = 64 * 64 * (4 * 64 * 64 * 128 + 2 * 64 * 64 * 128 + 64 * 64 * 128 + 6 * 64 * 128 * 128) / 1e9
    res["gdn_prefill_T4096"] = {"ms": ms, "tflops": gflop / ms, "algorithmic_gflop": gflop,
                                "sequential_form_gflop": 7 * 2 ** 20 * T / 1e9}
    ctx.close()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--layers", type=int, default=15)
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-extra", action="store_true", help="skip the context sweep / prefill / GatedDeltaNet figures")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of one step's output with the CPU checker")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8"], help="element type of the KV store")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="how sequence shards exchange partial results: the library's peer-memory kernels, or NCCL all-gathers")
    ap.add_argument("--probe", default=None, choices=["sweep", "prefill", "gdn_decode", "gdn_prefill", "hybrid", "out_proj", "kv_policies"],
                    help="run only one of the extra measurements and print it (for profiling one kernel)")
    args = ap.parse_args()
    set_kv_dtype(args.kv)
    if args.probe:
        global PROBE_REPS
        if any(a == "--steps" or a.startswith("--steps=") for a in sys.argv):
            PROBE_REPS = args.steps
        import torch
        from __graft_entry__ import load_package
        torch.cuda.set_device(0)
        peak, _ = load_peaks()
        print(json.dumps({"probe": args.probe, **extra_measurements(load_package(), torch, torch.device("cuda", 0), peak, args.probe)}))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
