"""The C host layer (include/fm_compat.h, flash-moe_b200/host/fm_compat.c): it compiles as plain C
against the C-ABI (checked on CPU), and a C program in the reference's calling style reproduces the
CPU checker on a B200."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "flash-moe_b200"


def build_c_test(tmp_path):
    exe = tmp_path / "test_compat"
    cmd = ["gcc", "-std=gnu11", "-O2", "-Wall", "-Werror", "-ffp-contract=off", "-fopenmp", f"-I{ROOT / 'include'}", f"-I{ROOT / 'oracle'}",
           str(ROOT / "tests" / "c" / "test_compat.c"), str(PKG / "host" / "fm_compat.c"), str(ROOT / "oracle" / "fm_oracle.c"),
           f"-L{PKG}", "-lfm_b200", f"-Wl,-rpath,{PKG}", "-lm", "-o", str(exe)]
    subprocess.check_call(cmd)
    return exe


def test_c_host_layer_compiles_and_links(pkg, tmp_path):
    assert pkg.binding.LIB_PATH.exists()
    build_c_test(tmp_path)


@pytest.mark.gpu
def test_c_host_program_matches_the_checker(pkg, tmp_path):
    exe = build_c_test(tmp_path)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL PASS" in r.stdout
    assert "ERROR: KV cache overflow" in r.stderr  # the reference's message on a full cache
