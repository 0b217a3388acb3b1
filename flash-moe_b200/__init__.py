"""Blackwell-native attention hot path of Flash-MoE behind a C-ABI (see include/fm_attn.h)."""
from . import synth  # noqa: F401
