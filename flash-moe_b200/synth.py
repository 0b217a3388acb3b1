"""Seeded synthetic inputs with the shapes and value distributions of the
decode / prefill workloads this library is measured on.

A counter-based generator (splitmix64 over ``(seed, stream, index)`` followed
by Box-Muller) so that any slice of any tensor can be produced independently
and identically on every machine; no global RNG state is involved.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _stream_key(seed: int, stream: str) -> np.uint64:
    h = np.uint64(1469598103934665603)
    with np.errstate(over="ignore"):
        for ch in stream.encode():
            h = ((h ^ np.uint64(ch)) * np.uint64(1099511628211)) & _M64
        return _splitmix64(np.array([h ^ np.uint64(seed * 0x9E3779B97F4A7C15 & 0xFFFFFFFFFFFFFFFF)],
                                    dtype=np.uint64))[0]


def uniform(seed: int, stream: str, shape, lo: float = 0.0, hi: float = 1.0, offset: int = 0) -> np.ndarray:
    """U(lo, hi) as float32; `offset` is the flat index of the first element."""
    n = int(np.prod(shape))
    idx = np.arange(offset, offset + n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        bits = _splitmix64(idx * np.uint64(2) + _stream_key(seed, stream))
    u = ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))
    return (lo + (hi - lo) * u).astype(np.float32).reshape(shape)


def normal(seed: int, stream: str, shape, std: float = 1.0, offset: int = 0) -> np.ndarray:
    """N(0, std^2) as float32 (Box-Muller on two counter-derived uniforms)."""
    n = int(np.prod(shape))
    idx = np.arange(offset, offset + n, dtype=np.uint64)
    key = _stream_key(seed, stream)
    with np.errstate(over="ignore"):
        b1 = _splitmix64(idx * np.uint64(2) + key)
        b2 = _splitmix64(idx * np.uint64(2) + np.uint64(1) + key)
    u1 = ((b1 >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))
    u2 = ((b2 >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (std * z).astype(np.float32).reshape(shape)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round fp32 to bf16 (nearest even); returns uint16 bit patterns."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)
    return r.astype(np.uint16).reshape(x.shape)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32).reshape(b.shape)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 values that are exactly representable in bf16."""
    return bf16_bits_to_f32(to_bf16_bits(x))


# --------------------------------------------------------------------------
# Workload builders
# --------------------------------------------------------------------------

def attn_dims(heads=32, kv_heads=2, head_dim=256, rotary_dim=64, theta=1e7, eps=1e-6):
    return dict(num_attn_heads=heads, num_kv_heads=kv_heads, head_dim=head_dim,
                rotary_dim=rotary_dim, rope_theta=theta, rms_norm_eps=eps)


def gdn_dims(v_heads=64, k_heads=16, key_dim=128, value_dim=128, conv=4, eps=1e-6):
    return dict(linear_num_v_heads=v_heads, linear_num_k_heads=k_heads, linear_key_dim=key_dim,
                linear_value_dim=value_dim, conv_kernel_size=conv, rms_norm_eps=eps)


def attn_cache(seed: int, ctx: int, kv_heads=2, head_dim=256, bf16=True, tag=""):
    """K, V rows [ctx][kv_heads*head_dim] ~ N(0,1), taken as already rotated."""
    k = normal(seed, f"kcache{tag}", (ctx, kv_heads * head_dim))
    v = normal(seed, f"vcache{tag}", (ctx, kv_heads * head_dim))
    return (round_bf16(k), round_bf16(v)) if bf16 else (k, v)


def attn_step_inputs(seed: int, n: int, heads=32, kv_heads=2, head_dim=256, bf16=False, tag=""):
    """q, gate [n][heads*head_dim]; k, v [n][kv_heads*head_dim] ~ N(0,1)."""
    q = normal(seed, f"q{tag}", (n, heads * head_dim))
    g = normal(seed, f"gate{tag}", (n, heads * head_dim))
    k = normal(seed, f"k{tag}", (n, kv_heads * head_dim))
    v = normal(seed, f"v{tag}", (n, kv_heads * head_dim))
    if bf16:
        q, g, k, v = (round_bf16(a) for a in (q, g, k, v))
    return q, g, k, v


def gdn_weights(seed: int, v_heads=64, k_heads=16, key_dim=128, value_dim=128, conv=4):
    conv_dim = 2 * k_heads * key_dim + v_heads * value_dim
    return dict(
        conv_w=to_bf16_bits(normal(seed, "conv_w", (conv_dim, conv), std=0.1)),
        A_log=uniform(seed, "A_log", (v_heads,), -2.0, 0.0),
        dt_bias=to_bf16_bits(np.zeros((v_heads,), np.float32)),
        norm_w=to_bf16_bits(np.ones((value_dim,), np.float32)),
    )


def gdn_state(seed: int, v_heads=64, key_dim=128, value_dim=128, std=0.02, tag=""):
    return normal(seed, f"ssm{tag}", (v_heads, value_dim, key_dim), std=std)


def gdn_step_inputs(seed: int, n: int, v_heads=64, k_heads=16, key_dim=128, value_dim=128,
                    bf16=False, tag=""):
    conv_dim = 2 * k_heads * key_dim + v_heads * value_dim
    qkv = normal(seed, f"qkv{tag}", (n, conv_dim))
    z = normal(seed, f"z{tag}", (n, v_heads * value_dim))
    beta = normal(seed, f"beta{tag}", (n, v_heads))
    alpha = normal(seed, f"alpha{tag}", (n, v_heads))
    if bf16:
        qkv, z = round_bf16(qkv), round_bf16(z)
    return qkv, z, beta, alpha
