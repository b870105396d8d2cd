"""miniattn — B200 (sm_100a) FlashAttention-2 forward operator behind the Python operator
surface of ShlokVFX/Mini-Attention.  Importing the package loads libminiattn.so; there is no
other backend and no CPU fallback."""
from . import _lib
from .ops import flash_attn_fwd, carry_state, flash_attn_fwd_host, flash_attn_fwd_int8qk, Int8QK, merge_partials, device_status, check_device_status, selftest_wait
from .compat import forward, ext
from .variants import MHA, GQA_Flash, MQA_Flash
from . import kernel_configs, parallel

__all__ = ["flash_attn_fwd", "carry_state", "flash_attn_fwd_host", "flash_attn_fwd_int8qk", "Int8QK", "merge_partials", "parallel", "device_status", "check_device_status", "selftest_wait", "version", "forward", "ext",
           "MHA", "GQA_Flash", "MQA_Flash", "kernel_configs"]


def version() -> str:
    return _lib.lib.miniattn_version().decode()
