"""ctypes binding of libfm_b200.so (the C-ABI of include/fm_attn.h) for tests and benches.

The product is the shared library; this module only turns numpy arrays / torch tensors into the
pointers the C-ABI takes.  There is no fallback: if the library is missing, importing fails.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libfm_b200.so"

FM_OK, FM_ERR_INVALID, FM_ERR_CAPACITY, FM_ERR_NOMEM, FM_ERR_CUDA, FM_ERR_TIMEOUT, FM_ERR_UNSUPPORTED = range(7)
FM_PTR_DEVICE, FM_PTR_HOST = 0, 1
FM_KV_BF16, FM_KV_FP8_E4M3 = 0, 1

EXPORTS = [
    "fm_default_config", "fm_create", "fm_destroy", "fm_last_error", "fm_set_stream",
    "fm_set_pointer_mode", "fm_set_layer_overlap", "fm_synchronize", "fm_reset", "fm_seq_fork", "fm_kv_free_pages", "fm_kv_len", "fm_kv_append_rope",
    "fm_attn_decode", "fm_attn_decode_partial", "fm_attn_merge_gate", "fm_attn_prefill",
    "fm_gdn_decode", "fm_gdn_prefill", "fm_kv_export", "fm_kv_import", "fm_state_export",
    "fm_state_import", "fm_launch_count", "fm_profile_enable", "fm_profile_read",
    "fm_attn_decode_static", "fm_exchange_bytes", "fm_exchange_attach", "fm_attn_decode_exchange_push",
    "fm_attn_decode_exchange_merge", "fm_attn_decode_exchange", "fm_attn_decode_layers",
    "fm_kv_export_fp8", "fm_kv_import_fp8", "fm_h2o_export", "fm_proj_upload", "fm_proj_free", "fm_out_proj_norm",
]


class FmConfig(C.Structure):
    _fields_ = [
        ("num_attn_heads", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int),
        ("rotary_dim", C.c_int), ("rope_theta", C.c_float), ("rms_norm_eps", C.c_float),
        ("rope_scaling_mode", C.c_int), ("rope_scale_factor", C.c_float),
        ("rope_orig_max_pos", C.c_int), ("num_full_layers", C.c_int),
        ("linear_num_v_heads", C.c_int), ("linear_num_k_heads", C.c_int),
        ("linear_key_dim", C.c_int), ("linear_value_dim", C.c_int), ("conv_kernel_size", C.c_int),
        ("num_linear_layers", C.c_int),
        ("max_seqs", C.c_int), ("max_seq_len", C.c_int), ("page_size", C.c_int),
        ("kv_pool_pages", C.c_int64), ("max_batch_tokens", C.c_int),
        ("seq_shard_rank", C.c_int), ("seq_shard_count", C.c_int), ("device", C.c_int),
        ("sliding_window", C.c_int), ("kv_dtype", C.c_int), ("h2o_budget", C.c_int), ("h2o_num_sinks", C.c_int),
    ]


class FmStaticDecodeArgs(C.Structure):
    _fields_ = [
        ("kv_pages", C.c_void_p), ("page_table", C.c_void_p), ("max_pages_per_seq", C.c_int),
        ("kv_len", C.POINTER(C.c_int)), ("pos", C.POINTER(C.c_int)), ("batch", C.c_int),
        ("num_attn_heads", C.c_int), ("num_kv_heads", C.c_int), ("rotary_dim", C.c_int),
        ("rope_theta", C.c_float), ("rms_norm_eps", C.c_float),
        ("q_proj_out", C.c_void_p), ("q", C.c_void_p), ("gate", C.c_void_p),
        ("q_norm_w", C.c_void_p), ("out", C.c_void_p), ("stream", C.c_void_p),
    ]


class FmProjWeights(C.Structure):
    _fields_ = [("format", C.c_int), ("out_dim", C.c_int), ("in_dim", C.c_int), ("group_size", C.c_int),
                ("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p)]


class FmError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"fm status {status}: {text}")
        self.status = status
        self.text = text


def load_library() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is not built: run `python flash-moe_b200/build.py` "
                          "(there is no CPU or PyTorch fallback for this library)")
    lib = C.CDLL(str(LIB_PATH))
    lib.fm_last_error.restype = C.c_char_p
    lib.fm_last_error.argtypes = [C.c_void_p]
    lib.fm_launch_count.restype = C.c_int64
    lib.fm_launch_count.argtypes = [C.c_void_p]
    lib.fm_kv_free_pages.restype = C.c_int64
    lib.fm_kv_free_pages.argtypes = [C.c_void_p]
    lib.fm_destroy.restype = None
    lib.fm_destroy.argtypes = [C.c_void_p]
    lib.fm_default_config.restype = None
    lib.fm_exchange_bytes.restype = C.c_size_t
    lib.fm_exchange_bytes.argtypes = [C.c_void_p, C.c_int]
    lib.fm_proj_free.restype = None
    return lib


def _ptr(a):
    """Pointer of a numpy array, a torch tensor, or None."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        assert a.flags.c_contiguous
        return C.c_void_p(a.ctypes.data)
    # torch tensor
    assert a.is_contiguous()
    return C.c_void_p(a.data_ptr())


def _ints(a):
    arr = np.ascontiguousarray(np.atleast_1d(np.asarray(a)), dtype=np.int32)
    return arr, arr.ctypes.data_as(C.POINTER(C.c_int))


def default_config(**kw) -> FmConfig:
    lib = load_library()
    cfg = FmConfig()
    lib.fm_default_config(C.byref(cfg))
    for k, v in kw.items():
        if not hasattr(cfg, k):
            raise AttributeError(k)
        setattr(cfg, k, v)
    return cfg


class Context:
    """One FmCtx.  Arrays given to the methods must match the pointer mode: numpy (host) arrays in
    FM_PTR_HOST mode, CUDA torch tensors in FM_PTR_DEVICE mode."""

    def __init__(self, cfg: FmConfig | None = None, host_pointers: bool = False, **kw):
        self.lib = load_library()
        self.cfg = cfg if cfg is not None else default_config(**kw)
        h = C.c_void_p()
        st = self.lib.fm_create(C.byref(self.cfg), C.byref(h))
        if st != FM_OK:
            raise FmError(st, self.lib.fm_last_error(None).decode())
        self.h = h
        if host_pointers:
            self.set_pointer_mode(FM_PTR_HOST)

    def close(self):
        if getattr(self, "h", None):
            self.lib.fm_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st != FM_OK:
            raise FmError(st, self.lib.fm_last_error(self.h).decode())

    def last_error(self) -> str:
        return self.lib.fm_last_error(self.h).decode()

    def set_stream(self, stream_ptr: int):
        self._check(self.lib.fm_set_stream(self.h, C.c_void_p(stream_ptr)))

    def set_layer_overlap(self, on: bool):
        self._check(self.lib.fm_set_layer_overlap(self.h, C.c_int(1 if on else 0)))

    def set_pointer_mode(self, mode: int):
        self._check(self.lib.fm_set_pointer_mode(self.h, C.c_int(mode)))

    def synchronize(self):
        self._check(self.lib.fm_synchronize(self.h))

    def reset(self, seq: int = -1):
        self._check(self.lib.fm_reset(self.h, C.c_int(seq)))

    def prepared(self, entry: str, *args):
        """A zero-argument callable for `entry(ctx, *args)` with the arguments converted once: Python ints become
        C ints, int32 numpy arrays `const int *` (mutate them in place between calls, e.g. positions), other arrays
        and tensors pointers.  For callers that step layers in a tight loop and do not want the per-call
        conversions of the convenience methods in the way."""
        fn = getattr(self.lib, entry)
        conv, keep = [], []
        for a in args:
            if a is None:
                conv.append(None)
            elif isinstance(a, (int, np.integer)):
                conv.append(C.c_int(int(a)))
            elif isinstance(a, np.ndarray) and a.dtype == np.int32:
                assert a.flags.c_contiguous
                keep.append(a)
                conv.append(a.ctypes.data_as(C.POINTER(C.c_int)))
            else:
                keep.append(a)
                conv.append(_ptr(a))
        h, check = self.h, self._check

        def call(_conv=tuple(conv), _keep=keep):
            check(fn(h, *_conv))
        return call

    def seq_fork(self, src: int, dst: int):
        self._check(self.lib.fm_seq_fork(self.h, C.c_int(src), C.c_int(dst)))

    def kv_free_pages(self) -> int:
        return self.lib.fm_kv_free_pages(self.h)

    def kv_len(self, fa_idx: int, seq: int = 0) -> int:
        return self.lib.fm_kv_len(self.h, C.c_int(fa_idx), C.c_int(seq))

    def launch_count(self) -> int:
        return self.lib.fm_launch_count(self.h)

    def profile_enable(self, on: bool = True):
        self._check(self.lib.fm_profile_enable(self.h, C.c_int(1 if on else 0)))

    def profile_read(self):
        """(launches, total milliseconds) of the bracketed dominant-kernel launches since the last read."""
        n = C.c_int(0); ms = C.c_double(0.0)
        self._check(self.lib.fm_profile_read(self.h, C.byref(n), C.byref(ms)))
        return n.value, ms.value

    def kv_append_rope(self, fa_idx, seq, pos, k, v, k_norm_w=None):
        s, sp = _ints(seq); p, pp = _ints(pos)
        self._check(self.lib.fm_kv_append_rope(self.h, C.c_int(fa_idx), sp, pp, C.c_int(len(s)),
                                               _ptr(k), _ptr(v), _ptr(k_norm_w)))

    def attn_decode(self, fa_idx, seq, pos, out, q_proj_out=None, q=None, gate=None, k=None, v=None,
                    q_norm_w=None, k_norm_w=None):
        s, sp = _ints(seq); p, pp = _ints(pos)
        self._check(self.lib.fm_attn_decode(self.h, C.c_int(fa_idx), sp, pp, C.c_int(len(s)),
                                            _ptr(q_proj_out), _ptr(q), _ptr(gate), _ptr(k), _ptr(v),
                                            _ptr(q_norm_w), _ptr(k_norm_w), _ptr(out)))

    def attn_decode_partial(self, fa_idx, seq, pos, o_part, ml_part, q_proj_out=None, q=None, k=None,
                            v=None, q_norm_w=None, k_norm_w=None):
        s, sp = _ints(seq); p, pp = _ints(pos)
        self._check(self.lib.fm_attn_decode_partial(self.h, C.c_int(fa_idx), sp, pp, C.c_int(len(s)),
                                                    _ptr(q_proj_out), _ptr(q), _ptr(k), _ptr(v),
                                                    _ptr(q_norm_w), _ptr(k_norm_w), _ptr(o_part),
                                                    _ptr(ml_part)))

    def attn_merge_gate(self, nparts, o_parts, ml_parts, batch, out, q_proj_out=None, gate=None):
        self._check(self.lib.fm_attn_merge_gate(self.h, C.c_int(nparts), _ptr(o_parts), _ptr(ml_parts),
                                                _ptr(q_proj_out), _ptr(gate), C.c_int(batch), _ptr(out)))

    def exchange_bytes(self, nranks: int) -> int:
        return self.lib.fm_exchange_bytes(self.h, C.c_int(nranks))

    def exchange_attach(self, my_index: int, peer_ptrs):
        """peer_ptrs: device addresses (ints) of every rank's exchange buffer as mapped in this process."""
        arr = (C.c_void_p * len(peer_ptrs))(*[C.c_void_p(int(p)) for p in peer_ptrs])
        self._check(self.lib.fm_exchange_attach(self.h, C.c_int(len(peer_ptrs)), C.c_int(my_index), arr))

    def attn_decode_exchange_push(self, fa_idx, seq, pos, q_proj_out=None, q=None, k=None, v=None, q_norm_w=None,
                                  k_norm_w=None):
        s, sp = _ints(seq); p, pp = _ints(pos)
        self._check(self.lib.fm_attn_decode_exchange_push(self.h, C.c_int(fa_idx), sp, pp, C.c_int(len(s)), _ptr(q_proj_out),
                                                          _ptr(q), _ptr(k), _ptr(v), _ptr(q_norm_w), _ptr(k_norm_w)))

    def attn_decode_exchange_merge(self, batch, out, q_proj_out=None, gate=None):
        self._check(self.lib.fm_attn_decode_exchange_merge(self.h, C.c_int(batch), _ptr(q_proj_out), _ptr(gate), _ptr(out)))

    def attn_decode_exchange(self, fa_idx, seq, pos, out, q_proj_out=None, q=None, gate=None, k=None, v=None,
                             q_norm_w=None, k_norm_w=None):
        s, sp = _ints(seq); p, pp = _ints(pos)
        self._check(self.lib.fm_attn_decode_exchange(self.h, C.c_int(fa_idx), sp, pp, C.c_int(len(s)), _ptr(q_proj_out),
                                                     _ptr(q), _ptr(gate), _ptr(k), _ptr(v), _ptr(q_norm_w),
                                                     _ptr(k_norm_w), _ptr(out)))

    def attn_decode_layers(self, first_layer, n_layers, seq, pos, out, q_proj_out, k, v, stride_q, stride_kv, stride_out,
                           q_norm_w=None, k_norm_w=None, exchange=False):
        """All layers of one token in one call; strides in floats between consecutive layers."""
        s, sp = _ints(seq); p, pp = _ints(pos)
        self._check(self.lib.fm_attn_decode_layers(self.h, C.c_int(first_layer), C.c_int(n_layers), sp, pp, C.c_int(len(s)),
                                                   _ptr(q_proj_out), C.c_size_t(stride_q), _ptr(k), _ptr(v), C.c_size_t(stride_kv),
                                                   _ptr(q_norm_w), _ptr(k_norm_w), _ptr(out), C.c_size_t(stride_out),
                                                   C.c_int(1 if exchange else 0)))

    def attn_prefill(self, fa_idx, seq, start_pos, n, out, q_proj_out=None, q=None, gate=None, k=None,
                     v=None, q_norm_w=None, k_norm_w=None):
        self._check(self.lib.fm_attn_prefill(self.h, C.c_int(fa_idx), C.c_int(seq), C.c_int(start_pos),
                                             C.c_int(n), _ptr(q_proj_out), _ptr(q), _ptr(gate), _ptr(k),
                                             _ptr(v), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(out)))

    def gdn_decode(self, li, seq, qkv, z, beta, alpha, out, conv_w=None, A_log=None, dt_bias=None,
                   norm_w=None):
        s, sp = _ints(seq)
        self._check(self.lib.fm_gdn_decode(self.h, C.c_int(li), sp, C.c_int(len(s)), _ptr(qkv), _ptr(z),
                                           _ptr(beta), _ptr(alpha), _ptr(conv_w), _ptr(A_log),
                                           _ptr(dt_bias), _ptr(norm_w), _ptr(out)))

    def gdn_prefill(self, li, seq, n, qkv, z, beta, alpha, out, conv_w=None, A_log=None, dt_bias=None,
                    norm_w=None, chunk=0):
        self._check(self.lib.fm_gdn_prefill(self.h, C.c_int(li), C.c_int(seq), C.c_int(n), C.c_int(chunk),
                                            _ptr(qkv), _ptr(z), _ptr(beta), _ptr(alpha), _ptr(conv_w),
                                            _ptr(A_log), _ptr(dt_bias), _ptr(norm_w), _ptr(out)))

    def kv_export(self, fa_idx, seq, k, v, max_rows) -> int:
        n = C.c_int(0)
        self._check(self.lib.fm_kv_export(self.h, C.c_int(fa_idx), C.c_int(seq), _ptr(k), _ptr(v),
                                          C.c_int(max_rows), C.byref(n)))
        return n.value

    def kv_import(self, fa_idx, seq, k, v, length):
        self._check(self.lib.fm_kv_import(self.h, C.c_int(fa_idx), C.c_int(seq), _ptr(k), _ptr(v),
                                          C.c_int(length)))

    def kv_export_fp8(self, fa_idx, seq, k8, v8, k_scales, v_scales, max_rows) -> int:
        n = C.c_int(0)
        self._check(self.lib.fm_kv_export_fp8(self.h, C.c_int(fa_idx), C.c_int(seq), _ptr(k8), _ptr(v8), _ptr(k_scales),
                                              _ptr(v_scales), C.c_int(max_rows), C.byref(n)))
        return n.value

    def kv_import_fp8(self, fa_idx, seq, k8, v8, k_scales, v_scales, length):
        self._check(self.lib.fm_kv_import_fp8(self.h, C.c_int(fa_idx), C.c_int(seq), _ptr(k8), _ptr(v8), _ptr(k_scales),
                                              _ptr(v_scales), C.c_int(length)))

    def h2o_export(self, fa_idx, seq, accum, token_positions, max_rows) -> int:
        n = C.c_int(0)
        self._check(self.lib.fm_h2o_export(self.h, C.c_int(fa_idx), C.c_int(seq), _ptr(accum), _ptr(token_positions),
                                           C.c_int(max_rows), C.byref(n)))
        return n.value

    def proj_upload(self, w, scales, biases) -> "FmProjWeights":
        """4-bit affine weights (numpy: w uint32 [out][in/8], scales / biases uint16 bf16 bits [out][in/64]) -> device."""
        out_dim, in_dim = w.shape[0], w.shape[1] * 8
        host = FmProjWeights(0, out_dim, in_dim, 64, w.ctypes.data, scales.ctypes.data, biases.ctypes.data)
        dev = FmProjWeights()
        self._check(self.lib.fm_proj_upload(self.h, C.byref(host), C.byref(dev)))
        return dev

    def proj_free(self, dev):
        self.lib.fm_proj_free(self.h, C.byref(dev))

    def out_proj_norm(self, dev, n, x, residual, norm_w, h_mid, h_post):
        self._check(self.lib.fm_out_proj_norm(self.h, C.byref(dev), C.c_int(n), _ptr(x), _ptr(residual), _ptr(norm_w), _ptr(h_mid), _ptr(h_post)))

    def state_export(self, li, seq, conv, ssm):
        self._check(self.lib.fm_state_export(self.h, C.c_int(li), C.c_int(seq), _ptr(conv), _ptr(ssm)))

    def state_import(self, li, seq, conv, ssm):
        self._check(self.lib.fm_state_import(self.h, C.c_int(li), C.c_int(seq), _ptr(conv), _ptr(ssm)))


def attn_decode_static(kv_pages, page_table, max_pages_per_seq, kv_len, pos, out, q_proj_out=None, q=None,
                       gate=None, q_norm_w=None, num_attn_heads=32, num_kv_heads=2, rotary_dim=64,
                       rope_theta=1e7, rms_norm_eps=1e-6, stream=0):
    """fm_attn_decode_static: the decode step for callers that may not allocate device memory (no
    context; the caller passes the KV pages and page table as device tensors).  Raises FmError."""
    lib = load_library()
    ln, lnp = _ints(kv_len); ps, psp = _ints(pos)
    p = lambda t: None if t is None else t.data_ptr()
    args = FmStaticDecodeArgs(p(kv_pages), p(page_table), max_pages_per_seq, lnp, psp, len(ln),
                              num_attn_heads, num_kv_heads, rotary_dim, rope_theta, rms_norm_eps,
                              p(q_proj_out), p(q), p(gate), p(q_norm_w), p(out), stream)
    err = C.create_string_buffer(256)
    st = lib.fm_attn_decode_static(C.byref(args), err, C.c_size_t(256))
    if st != FM_OK:
        raise FmError(st, err.value.decode())
