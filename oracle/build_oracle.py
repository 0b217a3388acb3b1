"""Build the CPU checkers used by the tests and by the bench's CPU baseline.

TEST INFRASTRUCTURE ONLY. Nothing under the product package may import, link
or execute anything produced here.

Two shared libraries are produced:

* ``oracle/libfm_oracle.so`` -- the plain-C restatement in ``fm_oracle.c``
  (always built; needs only gcc).
* ``oracle/_ref/libfm_ref.so`` -- the reference project's own CPU code for the
  attention / GatedDeltaNet path, compiled from the reference checkout where
  it lies.  The reference is one Objective-C unity build, so the plain-C
  regions that make up this path are cut out by line range into a *temporary*
  directory, ``#include``d by ``ref_harness.c`` and compiled; the temporary
  directory is deleted afterwards, so only the ``.so`` remains.  Every cut is
  guarded by sentinel strings and fails loudly if the reference moved.
  Built only when a reference checkout is present (``FM_REFERENCE_DIR`` or
  the default location); on a machine without one the prebuilt ``.so`` is used.

Usage: ``python oracle/build_oracle.py [--force]``
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = Path(os.environ.get("FM_REFERENCE_DIR", "/root/reference"))
REF_OUT = HERE / "_ref"

# Portable x86-64 code (the library is built on one machine and run on
# another), no FMA contraction so that the restatement and the reference
# round identically.
CFLAGS = ["-O2", "-std=gnu11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
          "-fno-fast-math", "-Wall", "-Wno-unused-function", "-Wno-unused-variable",
          "-Wno-unused-but-set-variable"]

# (slice name, file relative to the reference root, first line, last line,
#  text that must appear on the first line, text that must appear on the last line)
SLICES = [
    ("ref_config_struct.inc", "metal_infer/config.h", 9, 77, "typedef struct {", "static ModelConfig cfg;"),
    ("ref_fp8.inc", "metal_infer/fp8.h", 13, 118, "static int g_use_fp8_kv", "}"),
    ("ref_bf16.inc", "metal_infer/weights.h", 9, 21, "static float bf16_to_f32", "}"),
    ("ref_cpu_kernels.inc", "metal_infer/cpu_kernels.h", 196, 387, "4-bit dequant matvec", "}"),
    ("ref_rope.inc", "metal_infer/layer_forward.h", 22, 115, "static inline float rope_scaled_freq", "}"),
    ("ref_kv.inc", "metal_infer/layer_forward.h", 121, 236, "typedef struct {", "}"),
    ("ref_h2o.inc", "metal_infer/layer_forward.h", 248, 383, "static void kv_cache_h2o_accumulate_scores", "}"),
    ("ref_las.inc", "metal_infer/layer_forward.h", 414, 432, "typedef struct {", "}"),
    ("ref_gdn_helpers.inc", "metal_infer/layer_forward.h", 778, 797, "RMS norm without weights", "}"),
    # full attention: norm -> RoPE -> append -> SDPA -> sigmoid gate (function body)
    ("ref_fa_core.inc", "metal_infer/layer_forward.h", 556, 735, "Q/K RMSNorm", "}"),
    # the same body cut in three so the harness can thread the per-head loop
    ("ref_fa_pre.inc", "metal_infer/layer_forward.h", 556, 660, "Q/K RMSNorm", ""),
    ("ref_fa_head_body.inc", "metal_infer/layer_forward.h", 662, 716, "int kv_h = h / heads_per_kv;", "free(scores);"),
    ("ref_fa_post.inc", "metal_infer/layer_forward.h", 719, 735, "H2O: accumulate attention scores", "}"),
    # GatedDeltaNet: conv -> shift -> normalise -> decay/beta -> recurrence -> gated norm
    ("ref_gdn_core.inc", "metal_infer/layer_forward.h", 886, 1025, "Conv1d step", "}"),
    ("ref_gdn_pre.inc", "metal_infer/layer_forward.h", 886, 966, "Conv1d step", ""),
    ("ref_gdn_head_body.inc", "metal_infer/layer_forward.h", 968, 1008, "int kh = vh / k_heads_per_v;", "}"),
    ("ref_gdn_post.inc", "metal_infer/layer_forward.h", 1011, 1025, "RMSNormGated", "}"),
]


def _cut(tmp: Path) -> None:
    cache: dict[str, list[str]] = {}
    for name, rel, first, last, head, tail in SLICES:
        lines = cache.setdefault(rel, (REF_DIR / rel).read_text().splitlines())
        chunk = lines[first - 1:last]
        if head not in chunk[0]:
            raise SystemExit(f"reference moved: {rel}:{first} lacks {head!r}: {chunk[0]!r}")
        if tail and tail not in chunk[-1]:
            raise SystemExit(f"reference moved: {rel}:{last} lacks {tail!r}: {chunk[-1]!r}")
        (tmp / name).write_text("\n".join(chunk) + "\n")


def build_port(force: bool = False) -> Path:
    out = HERE / "libfm_oracle.so"
    src = HERE / "fm_oracle.c"
    if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["gcc", *CFLAGS, str(src), "-o", str(out), "-lm"])
    return out


def build_ref(force: bool = False) -> Path | None:
    out = REF_OUT / "libfm_ref.so"
    src = HERE / "ref_harness.c"
    if not (REF_DIR / "metal_infer" / "layer_forward.h").exists():
        return out if out.exists() else None
    if not force and out.exists() and out.stat().st_mtime >= max(src.stat().st_mtime,
                                                                   Path(__file__).stat().st_mtime):
        return out
    REF_OUT.mkdir(exist_ok=True)
    tmp = Path(tempfile.mkdtemp(prefix="fm_ref_slices_"))
    try:
        _cut(tmp)
        subprocess.check_call(["gcc", *CFLAGS, f"-I{tmp}", str(src), "-o", str(out), "-lm"])
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return out


def main() -> None:
    force = "--force" in sys.argv
    print("port:", build_port(force))
    print("ref :", build_ref(force))


if __name__ == "__main__":
    main()
