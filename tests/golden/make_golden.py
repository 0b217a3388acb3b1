"""Produce the golden vectors under tests/golden/ from the reference project's own CPU code.

Needs oracle/_ref/libfm_ref.so (built by oracle/build_oracle.py on a machine that has a
reference checkout).  Inputs are stored next to the outputs so that checking a fixture does not
depend on regenerating the inputs.  Run: python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from __graft_entry__ import load_package  # noqa: E402
from oracle.oracle_py import Oracle, make_dims  # noqa: E402

synth = load_package().synth
OUT = Path(__file__).resolve().parent


def attn_case(name, seed, heads, kv_heads, head_dim, rot, theta, ctx, steps, norm, bf16, cap_extra=0):
    ref = Oracle("reference")
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim,
                     rotary_dim=rot, rope_theta=theta)
    kv_dim = kv_heads * head_dim
    k0, v0 = synth.attn_cache(seed, ctx, kv_heads, head_dim, bf16=bf16)
    q, g, k, v = synth.attn_step_inputs(seed, steps, heads, kv_heads, head_dim, bf16=bf16)
    qn = kn = None
    if norm:
        qn = synth.to_bf16_bits(1.0 + synth.normal(seed, "qn", (head_dim,), std=0.1))
        kn = synth.to_bf16_bits(1.0 + synth.normal(seed, "kn", (head_dim,), std=0.1))
    cap = ctx + steps + cap_extra
    kc = np.zeros((cap, kv_dim), np.float32); vc = np.zeros((cap, kv_dim), np.float32)
    kc[:ctx] = k0; vc[:ctx] = v0
    out, ln = ref.attn_run(dims, kc, vc, ctx, q, g, k, v, qn, kn)
    np.savez_compressed(
        OUT / f"{name}.npz", kind="attn", heads=heads, kv_heads=kv_heads, head_dim=head_dim,
        rot=rot, theta=np.float32(theta), ctx=ctx, steps=steps, k0=k0, v0=v0, q=q, gate=g, k=k, v=v,
        qn=qn if norm else np.zeros(0, np.uint16), kn=kn if norm else np.zeros(0, np.uint16),
        out=out, k_final_tail=kc[ctx:ln], v_final_tail=vc[ctx:ln], len_final=ln)
    print(name, out.shape, float(np.abs(out).max()))


def gdn_case(name, seed, v_heads, k_heads, dk, dv, steps, zero_state, bf16):
    ref = Oracle("reference")
    dims = make_dims(linear_num_v_heads=v_heads, linear_num_k_heads=k_heads, linear_key_dim=dk,
                     linear_value_dim=dv)
    conv_dim = 2 * k_heads * dk + v_heads * dv
    w = synth.gdn_weights(seed, v_heads, k_heads, dk, dv)
    w["dt_bias"] = synth.to_bf16_bits(synth.normal(seed, "dtb", (v_heads,), std=0.5))
    w["norm_w"] = synth.to_bf16_bits(1.0 + synth.normal(seed, "nw", (dv,), std=0.1))
    s0 = np.zeros((v_heads, dv, dk), np.float32) if zero_state else synth.gdn_state(seed, v_heads, dk, dv)
    qkv, z, beta, alpha = synth.gdn_step_inputs(seed, steps, v_heads, k_heads, dk, dv, bf16=bf16)
    conv = np.zeros((3, conv_dim), np.float32)
    ssm = s0.copy()
    out = ref.gdn_run(dims, conv, ssm, qkv, z, beta, alpha, w["conv_w"], w["A_log"], w["dt_bias"],
                      w["norm_w"])
    np.savez_compressed(
        OUT / f"{name}.npz", kind="gdn", v_heads=v_heads, k_heads=k_heads, dk=dk, dv=dv, steps=steps,
        s0=s0 if not zero_state else np.zeros(0, np.float32), qkv=qkv, z=z, beta=beta, alpha=alpha,
        conv_w=w["conv_w"], A_log=w["A_log"], dt_bias=w["dt_bias"], norm_w=w["norm_w"],
        out=out, conv_final=conv, ssm_final=ssm)
    print(name, out.shape, float(np.abs(out).max()), float(np.sqrt((ssm ** 2).mean())))


def cache_policy_case(name, seed, heads, kv_heads, steps, fp8, h2o_budget):
    """Decode steps from an empty cache with the FP8 store and / or H2O eviction switched on."""
    from oracle.oracle_py import Cache
    ref = Oracle("reference")
    dims = make_dims(num_attn_heads=heads, num_kv_heads=kv_heads)
    q, g, k, v = synth.attn_step_inputs(seed, steps, heads, kv_heads, 256)
    capacity = h2o_budget + 1 if h2o_budget else steps
    c = Cache(capacity, kv_heads * 256, fp8=fp8, h2o_budget=h2o_budget, h2o_sinks=4)
    out = ref.attn_run_cache(dims, c, q, g, k, v)
    z = np.zeros(0, np.float32)
    np.savez_compressed(
        OUT / f"{name}.npz", kind="attn_cache", heads=heads, kv_heads=kv_heads, steps=steps, fp8=fp8,
        h2o_budget=h2o_budget, capacity=capacity, q=q, gate=g, k=k, v=v, out=out,
        k8=c.k8 if fp8 else z, v8=c.v8 if fp8 else z, k_scales=c.k_scales if fp8 else z,
        v_scales=c.v_scales if fp8 else z, token_positions=c.token_positions if h2o_budget else z,
        accum=c.accum if h2o_budget else z)
    print(name, out.shape, float(np.abs(out).max()))


if __name__ == "__main__":
    cache_policy_case("attn_fp8_h8_d256", 14, 8, 2, 12, fp8=True, h2o_budget=0)
    cache_policy_case("attn_h2o_h8_d256", 15, 8, 2, 30, fp8=False, h2o_budget=16)
    # decode steps at the production head size, few heads (fp32 inputs, with norm weights)
    attn_case("attn_h8_d256_ctx37", 11, 8, 2, 256, 64, 1e7, 37, 3, norm=True, bf16=False)
    # bf16-representable inputs, GQA group 16 as in the production model, ragged context
    attn_case("attn_h16_d256_ctx130_bf16", 12, 16, 1, 256, 64, 1e7, 130, 2, norm=False, bf16=True)
    # small odd shape from an empty cache (first token attends to itself only)
    attn_case("attn_h4_d64_ctx0", 13, 4, 1, 64, 32, 1e4, 0, 5, norm=True, bf16=False)
    gdn_case("gdn_v8_k4_d32", 21, 8, 4, 32, 32, 6, zero_state=False, bf16=False)
    gdn_case("gdn_v4_k1_d128", 22, 4, 1, 128, 128, 5, zero_state=True, bf16=True)
