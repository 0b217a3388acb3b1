"""The shared library loads and exports every entry point the header declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "fm_attn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fm_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_documented_surface():
    names = declared_functions()
    for must in ["fm_create", "fm_destroy", "fm_kv_append_rope", "fm_attn_decode", "fm_attn_prefill",
                 "fm_gdn_decode", "fm_gdn_prefill", "fm_kv_export", "fm_kv_import", "fm_state_export",
                 "fm_state_import", "fm_reset", "fm_last_error"]:
        assert must in names


def test_library_exports_every_declared_symbol(pkg):
    lib = ctypes.CDLL(str(pkg.binding.LIB_PATH))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/fm_attn.h but not exported"
    assert set(pkg.binding.EXPORTS) == set(declared_functions())


def test_config_struct_matches_header(pkg):
    """Field order of the ctypes mirror follows the C struct."""
    text = (ROOT / "include" / "fm_attn.h").read_text()
    body = re.search(r"typedef struct FmConfig \{(.*?)\} FmConfig;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b(?:int|float|int64_t)\s+([a-z_0-9]+)\s*;", body)
    assert fields == [f[0] for f in pkg.FmConfig._fields_]


def test_default_config_is_the_production_model(pkg):
    cfg = pkg.default_config()
    assert (cfg.num_attn_heads, cfg.num_kv_heads, cfg.head_dim, cfg.rotary_dim) == (32, 2, 256, 64)
    assert (cfg.linear_num_v_heads, cfg.linear_num_k_heads, cfg.linear_key_dim, cfg.linear_value_dim) == (64, 16, 128, 128)
    assert (cfg.num_full_layers, cfg.num_linear_layers, cfg.page_size) == (15, 45, 64)


def test_create_without_gpu_fails_loudly(pkg):
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present")
    import pytest
    with pytest.raises(pkg.FmError) as e:
        pkg.Context()
    assert "no CUDA device" in str(e.value) or "CUDA" in str(e.value)
