"""Alias package: ``import flaggems_sglang`` resolves to the B200 implementation of the
fused-MoE entry points, under the module paths the reference exposes them at
(src/flaggems_sglang/__init__.py:7-10, src/flaggems_sglang/ops/__init__.py:1-4)."""
from flaggems_sglang_b200 import *  # noqa: F401,F403
from flaggems_sglang_b200 import __all__, __version__, device, vendor_name  # noqa: F401

from . import ops, testing  # noqa: F401,E402
