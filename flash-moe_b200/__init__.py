"""Blackwell-native attention hot path of Flash-MoE behind a C-ABI (see include/fm_attn.h)."""
from . import sharding, synth  # noqa: F401
from . import binding  # noqa: F401,E402
from .binding import Context, FmConfig, FmError, default_config  # noqa: F401,E402
