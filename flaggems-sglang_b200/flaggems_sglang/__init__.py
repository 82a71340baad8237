"""Alias so that ``import flaggems_sglang`` resolves to the B200 implementation
of the fused-MoE entry points."""
from flaggems_sglang_b200 import *  # noqa: F401,F403
from flaggems_sglang_b200 import __all__, __version__, device, vendor_name, ops  # noqa: F401
