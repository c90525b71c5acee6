"""Drop-in module name: ``import flaggems_vllm`` resolves the fused-MoE
operators to the B200 kernels of ``flaggems_vllm_b200`` (same names, same
signatures), so callers written against FlagGems-vllm need no change."""

from flaggems_vllm_b200 import *  # noqa: F401,F403
from flaggems_vllm_b200 import __all__, __version__, device, vendor_name  # noqa: F401
