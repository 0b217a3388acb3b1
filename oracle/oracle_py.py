"""ctypes binding of the CPU checkers -- TEST INFRASTRUCTURE ONLY.

Importable from tests/, the smoke check and the bench's CPU-baseline leg;
never from the product package.  ``Oracle("port")`` is the plain-C
restatement, ``Oracle("reference")`` the reference project's own CPU code
(present only when ``oracle/_ref/libfm_ref.so`` was built).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


class FmoDims(C.Structure):
    _fields_ = [
        ("num_attn_heads", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int),
        ("rotary_dim", C.c_int), ("rope_theta", C.c_float), ("rms_norm_eps", C.c_float),
        ("rope_scaling_mode", C.c_int), ("rope_scale_factor", C.c_float), ("max_seq_len", C.c_int),
        ("linear_num_v_heads", C.c_int), ("linear_num_k_heads", C.c_int),
        ("linear_key_dim", C.c_int), ("linear_value_dim", C.c_int), ("conv_kernel_size", C.c_int),
        ("store_bf16", C.c_int), ("sliding_window", C.c_int),
    ]


class FmoCache(C.Structure):
    _fields_ = [
        ("k_cache", C.POINTER(C.c_float)), ("v_cache", C.POINTER(C.c_float)),
        ("k8", C.POINTER(C.c_uint8)), ("v8", C.POINTER(C.c_uint8)),
        ("k_scales", C.POINTER(C.c_float)), ("v_scales", C.POINTER(C.c_float)),
        ("len", C.c_int), ("capacity", C.c_int), ("use_fp8", C.c_int), ("window_size", C.c_int),
        ("h2o_budget", C.c_int), ("h2o_num_sinks", C.c_int), ("h2o_num_recent", C.c_int),
        ("h2o_num_valid", C.c_int),
        ("attn_scores_accum", C.POINTER(C.c_float)), ("token_positions", C.POINTER(C.c_int)),
    ]


class Cache:
    """A KV cache with the reference's optional policies, backed by numpy arrays the caller can read:
    fp32 rows (k, v) or FP8 bytes + per-row scales (k8, v8, k_scales, v_scales); sliding window; H2O
    (accum, token_positions, num_valid).  num_recent follows kv_cache_new(): (budget - sinks) // 4."""

    def __init__(self, capacity: int, kv_dim: int, fp8: bool = False, window: int = 0, h2o_budget: int = 0,
                 h2o_sinks: int = 4):
        self.capacity, self.kv_dim, self.fp8 = capacity, kv_dim, fp8
        f32p, u8p, i32p = C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.POINTER(C.c_int)
        self.k = np.zeros((capacity, kv_dim), np.float32) if not fp8 else None
        self.v = np.zeros((capacity, kv_dim), np.float32) if not fp8 else None
        self.k8 = np.zeros((capacity, kv_dim), np.uint8) if fp8 else None
        self.v8 = np.zeros((capacity, kv_dim), np.uint8) if fp8 else None
        self.k_scales = np.zeros((capacity,), np.float32) if fp8 else None
        self.v_scales = np.zeros((capacity,), np.float32) if fp8 else None
        self.accum = np.zeros((capacity,), np.float32) if h2o_budget > 0 else None
        self.token_positions = np.zeros((capacity,), np.int32) if h2o_budget > 0 else None
        p = lambda a, t: a.ctypes.data_as(t) if a is not None else None
        self.c = FmoCache(p(self.k, f32p), p(self.v, f32p), p(self.k8, u8p), p(self.v8, u8p), p(self.k_scales, f32p),
                          p(self.v_scales, f32p), 0, capacity, 1 if fp8 else 0, window, h2o_budget, h2o_sinks,
                          (h2o_budget - h2o_sinks) // 4 if h2o_budget > 0 else 0, 0, p(self.accum, f32p),
                          p(self.token_positions, i32p))

    @property
    def len(self):
        return self.c.len

    @property
    def num_valid(self):
        return self.c.h2o_num_valid


def make_dims(**kw) -> FmoDims:
    d = dict(num_attn_heads=32, num_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1e7,
             rms_norm_eps=1e-6, rope_scaling_mode=0, rope_scale_factor=1.0, max_seq_len=262144,
             linear_num_v_heads=64, linear_num_k_heads=16, linear_key_dim=128,
             linear_value_dim=128, conv_kernel_size=4, store_bf16=0, sliding_window=0)
    d.update(kw)
    return FmoDims(**d)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _u16(a):
    if a is None:
        return None, None
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint16))


def ref_available() -> bool:
    return (HERE / "_ref" / "libfm_ref.so").exists()


class Oracle:
    def __init__(self, kind: str = "port"):
        if kind == "reference":
            path, self.prefix = HERE / "_ref" / "libfm_ref.so", "fmr_"
        elif kind == "port":
            path, self.prefix = HERE / "libfm_oracle.so", "fmo_"
            if not path.exists():
                import importlib.util
                spec = importlib.util.spec_from_file_location("build_oracle", HERE / "build_oracle.py")
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                mod.build_port()
        else:
            raise ValueError(kind)
        self.kind = kind
        self.lib = C.CDLL(str(path))
        for name in ("attn_step", "attn_run", "gdn_step", "gdn_run", "attn_step_cache"):
            getattr(self.lib, self.prefix + name).restype = C.c_int
        for name in ("fp8_encode_rows", "fp8_decode_rows", "out_proj_norm"):
            getattr(self.lib, self.prefix + name).restype = None

    # -- cache policies: FP8 store, sliding window, H2O ------------------------
    def attn_run_cache(self, dims: FmoDims, cache: Cache, q, gate, k, v, q_norm_w=None, k_norm_w=None,
                       start_pos=None, threads: int = 1):
        """n decode steps on a Cache (updated in place).  Returns out [n][q_dim]."""
        q, _ = _f32(q); gate, _ = _f32(gate); k, _ = _f32(k); v, _ = _f32(v)
        q, gate, k, v = (np.atleast_2d(a) for a in (q, gate, k, v))
        n = q.shape[0]
        out = np.empty((n, dims.num_attn_heads * dims.head_dim), np.float32)
        _a, qn = _u16(q_norm_w); _b, kn = _u16(k_norm_w)
        if start_pos is None:
            start_pos = cache.len
        f32p = C.POINTER(C.c_float)
        fn = getattr(self.lib, self.prefix + "attn_step_cache")
        for t in range(n):
            rc = fn(C.byref(dims), C.byref(cache.c), q[t].ctypes.data_as(f32p), gate[t].ctypes.data_as(f32p),
                    k[t].ctypes.data_as(f32p), v[t].ctypes.data_as(f32p), qn, kn, C.c_int(start_pos + t),
                    out[t].ctypes.data_as(f32p), C.c_int(threads))
            if rc != 0:
                raise RuntimeError("KV cache overflow in oracle")
        return out

    def out_proj_norm(self, w, scales, biases, x, residual, norm_w, eps=1e-6, group_size=64):
        """x [n][in], residual [n][out] or None -> (h_mid, h_post) [n][out]."""
        w = np.ascontiguousarray(w, np.uint32); scales = np.ascontiguousarray(scales, np.uint16)
        biases = np.ascontiguousarray(biases, np.uint16); norm_w = np.ascontiguousarray(norm_w, np.uint16)
        x = np.atleast_2d(np.ascontiguousarray(x, np.float32))
        out_dim, in_dim = w.shape[0], w.shape[1] * 8
        n = x.shape[0]
        h_mid = np.empty((n, out_dim), np.float32); h_post = np.empty_like(h_mid)
        fn = getattr(self.lib, self.prefix + "out_proj_norm")
        f32p, u16p = C.POINTER(C.c_float), C.POINTER(C.c_uint16)
        for t in range(n):
            r = None if residual is None else np.ascontiguousarray(residual[t], np.float32)
            fn(w.ctypes.data_as(C.POINTER(C.c_uint32)), scales.ctypes.data_as(u16p), biases.ctypes.data_as(u16p), C.c_int(out_dim),
               C.c_int(in_dim), C.c_int(group_size), x[t].ctypes.data_as(f32p), None if r is None else r.ctypes.data_as(f32p),
               norm_w.ctypes.data_as(u16p), C.c_float(eps), h_mid[t].ctypes.data_as(f32p), h_post[t].ctypes.data_as(f32p))
        return h_mid, h_post

    def fp8_encode_rows(self, rows):
        rows, rp = _f32(rows)
        n, kv_dim = rows.shape
        b = np.empty((n, kv_dim), np.uint8); sc = np.empty((n,), np.float32)
        getattr(self.lib, self.prefix + "fp8_encode_rows")(rp, C.c_int(n), C.c_int(kv_dim),
                                                            b.ctypes.data_as(C.POINTER(C.c_uint8)),
                                                            sc.ctypes.data_as(C.POINTER(C.c_float)))
        return b, sc

    def fp8_decode_rows(self, b, sc):
        b = np.ascontiguousarray(b, np.uint8); sc = np.ascontiguousarray(sc, np.float32)
        n, kv_dim = b.shape
        out = np.empty((n, kv_dim), np.float32)
        getattr(self.lib, self.prefix + "fp8_decode_rows")(b.ctypes.data_as(C.POINTER(C.c_uint8)),
                                                            sc.ctypes.data_as(C.POINTER(C.c_float)), C.c_int(n),
                                                            C.c_int(kv_dim), out.ctypes.data_as(C.POINTER(C.c_float)))
        return out

    # -- full attention ------------------------------------------------------
    def attn_run(self, dims: FmoDims, k_cache, v_cache, length: int, q, gate, k, v,
                 q_norm_w=None, k_norm_w=None, start_pos=None, threads: int = 1):
        """Run n decode steps. k_cache / v_cache are float32 [capacity][kv_dim] arrays updated in
        place. Returns (out [n][q_dim], new length)."""
        assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous
        assert v_cache.dtype == np.float32 and v_cache.flags.c_contiguous
        q, qp = _f32(q); gate, gp = _f32(gate); k, kp = _f32(k); v, vp = _f32(v)
        n = q.shape[0] if q.ndim == 2 else 1
        qd = dims.num_attn_heads * dims.head_dim
        out = np.empty((n, qd), np.float32)
        ln = C.c_int(length)
        _a, qn = _u16(q_norm_w); _b, kn = _u16(k_norm_w)
        if start_pos is None:
            start_pos = length
        rc = getattr(self.lib, self.prefix + "attn_run")(
            C.byref(dims), k_cache.ctypes.data_as(C.POINTER(C.c_float)),
            v_cache.ctypes.data_as(C.POINTER(C.c_float)), C.byref(ln), C.c_int(k_cache.shape[0]),
            qp, gp, kp, vp, qn, kn, C.c_int(start_pos), C.c_int(n),
            out.ctypes.data_as(C.POINTER(C.c_float)), C.c_int(threads))
        if rc != 0:
            raise RuntimeError("KV cache overflow in oracle")
        return out, ln.value

    # -- GatedDeltaNet -------------------------------------------------------
    def gdn_run(self, dims: FmoDims, conv_state, ssm_state, qkv, z, beta, alpha, conv_w, A_log,
                dt_bias, norm_w, threads: int = 1):
        """Run n steps; conv_state / ssm_state float32 arrays updated in place. Returns out."""
        for a in (conv_state, ssm_state):
            assert a.dtype == np.float32 and a.flags.c_contiguous
        qkv, qp = _f32(qkv); z, zp = _f32(z); beta, bp = _f32(beta); alpha, ap = _f32(alpha)
        n = qkv.shape[0] if qkv.ndim == 2 else 1
        vd = dims.linear_num_v_heads * dims.linear_value_dim
        out = np.empty((n, vd), np.float32)
        _a, cw = _u16(conv_w); _b, db = _u16(dt_bias); _c, nw = _u16(norm_w)
        if A_log is not None:
            A_log, alp = _f32(A_log)
        else:
            alp = None
        getattr(self.lib, self.prefix + "gdn_run")(
            C.byref(dims), conv_state.ctypes.data_as(C.POINTER(C.c_float)),
            ssm_state.ctypes.data_as(C.POINTER(C.c_float)), qp, zp, bp, ap, cw, alp, db, nw,
            C.c_int(n), out.ctypes.data_as(C.POINTER(C.c_float)), C.c_int(threads))
        return out


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1
