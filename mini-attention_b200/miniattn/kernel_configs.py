"""Compatibility mirror of the reference's kernel-config helper module
(kernels/flash_attn/cuda/sm_120/py/flash_helpers/kernel_configs.py).

Reference callers build a ``FlashForwardKernelConfig`` and pass it as the first argument of
``ext.forward`` (flash_attention.cu:19-35,60-65).  The B200 kernels have one tcgen05 tiling, so
of the 13 fields only ``dtype``, ``d_head``, ``B_r`` and ``B_c`` still carry meaning (they drive
the same argument checks as the reference launcher); the mma.sync tuning knobs (async copy,
eager loads, swizzling, fragment-streaming depths, register double buffering, exp2 softmax)
are accepted and ignored.  Like the reference module this file does not import torch at
module level.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, replace
from enum import IntEnum
from typing import List


class DType(IntEnum):
    """Values are torch's ScalarType codes, as in the reference (kernel_configs.py:9-13)."""

    FP16 = 5
    BF16 = 15

    def to_torch_dtype(self):
        import torch

        return torch.float16 if self == DType.FP16 else torch.bfloat16

    @classmethod
    def from_string(cls, text: str) -> "DType":
        text = text.strip()
        if text.lstrip("-").isdigit():
            return cls(int(text))
        try:
            return cls[text.upper()]
        except KeyError:
            raise ValueError(f"Invalid dtype string {text!r}; valid: {[m.name for m in cls]}") from None


@dataclass(frozen=True, order=True)
class FlashForwardKernelConfig:
    """Same 13 fields, in the same order, as kernel_configs.py:106-120."""

    dtype: DType
    d_head: int
    B_r: int
    B_c: int
    n_warps: int
    async_copy: bool
    eager_load_blocks: bool
    swizzled: bool
    Q_mma_load_K_tiles: int
    K_mma_load_K_tiles: int
    V_mma_load_K_tiles: int
    mma_double_buffer_loads: bool
    optimized_softmax: bool

    def short_form(self, include_d_head: bool = True, include_tup: bool = True) -> str:
        head = f"{self.d_head}, " if include_d_head else ""
        base = f"({DType(self.dtype).name}, {head}{self.B_r}, {self.B_c}, {self.n_warps}): " if include_tup else ""
        parts = [name for flag, name in ((self.async_copy, "async"), (self.eager_load_blocks, "eager"),
                                         (self.swizzled, "swizzled")) if flag]
        parts.append(f"load_{self.Q_mma_load_K_tiles}_{self.K_mma_load_K_tiles}_{self.V_mma_load_K_tiles}_tiles")
        if self.mma_double_buffer_loads:
            parts.append("buffer")
        if self.optimized_softmax:
            parts.append("opt_softmax")
        return base + "+".join(parts)

    __str__ = short_form

    def kernel_name(self) -> str:
        return "flash_forward_kernel"

    def attn_flop(self, n_samples: int, n_heads: int, seq_len: int) -> int:
        return calc_self_attn_flop(n_samples, n_heads, seq_len, self.d_head)


def calc_self_attn_flop(n_samples: int, n_heads: int, seq_len: int, d_head: int) -> int:
    """4*N^2*D matmul flops plus 6*N^2 softmax flops per head (kernel_configs.py:102-103)."""
    return n_samples * n_heads * (4 * seq_len**2 * d_head + 6 * seq_len**2)


def attention_matmul_flop(batch: int, heads: int, seq_len: int, d_head: int, causal: bool = False) -> float:
    """The benchmark's flop count: 4*B*H*N^2*D, halved for causal
    (kernels/flash_attn/cuda/sm86/ncu_metrics.py:95-97)."""
    f = 4.0 * batch * heads * seq_len * seq_len * d_head
    return f / 2 if causal else f


def _cfg(async_copy, eager, swizzled, q, k, v, dbuf, osm) -> FlashForwardKernelConfig:
    return FlashForwardKernelConfig(DType.FP16, 128, 64, 64, 4, async_copy, eager, swizzled, q, k, v, dbuf, osm)


def get_kernel_progression_configs(all_block_sizes: bool = False) -> List[FlashForwardKernelConfig]:
    """The K1..K7 progression of the reference (kernel_configs.py:426-454)."""
    base = [
        _cfg(True, False, False, 0, 0, 0, False, False),  # K1
        _cfg(True, False, True, 0, 0, 0, False, False),   # K2 + swizzle
        _cfg(True, True, True, 0, 0, 0, False, False),    # K3 + eager K/V loads
        _cfg(True, True, True, 2, 2, 2, False, False),    # K4 fragment streaming
        _cfg(True, True, True, 2, 2, 2, True, False),     # K5 + register double buffer
        _cfg(True, True, True, 2, 2, 2, True, True),      # K6 + exp2 softmax
        _cfg(True, True, True, 0, 2, 2, False, True),     # K7 Q resident in registers
    ]
    if not all_block_sizes:
        return base
    out = []
    for cfg in base:
        for B_r in (128, 64):
            for B_c in (128, 64, 32):
                for n_warps in (4, 8):
                    if (B_r < 128 and n_warps == 8) or B_r < B_c:
                        continue
                    out.append(replace(cfg, B_r=B_r, B_c=B_c, n_warps=n_warps))
    return out


def get_kernel_configs(kernels_key: str = "") -> List[FlashForwardKernelConfig]:
    """Selection by key or the KERNELS environment variable (kernel_configs.py:465-485).
    Only the progression keys exist here: there is no autotuning set on B200."""
    key = kernels_key or os.environ.get("KERNELS", "")
    if key.startswith("prog"):
        return get_kernel_progression_configs(all_block_sizes="all" in key)
    raise ValueError(f"Invalid kernels env key: {key}")
