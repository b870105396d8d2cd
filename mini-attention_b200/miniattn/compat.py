"""Drop-in for the reference's CUDA operator surface.

* ``forward(q, k, v)``  — the module-level operator of every generated inline module
  (kernels/flash_attn/cuda/sm86/inline/fp16_k1_sm86.py:265-269): (B,N,H,D) tensors in,
  ``torch.empty_like(q)`` out.
* ``ext.forward(kernel_cfg, q, k, v, o, benchmark=False) -> (Tensor, ms)`` — the pybind entry
  of the reference extension (kernels/flash_attn/cuda/sm_120/kernel/flash_attention.cu:37-40,
  134-138) with the same checks and the same RuntimeError behaviour (``:41-80``): CUDA and
  contiguous inputs, fp16/bf16 with equal dtypes, dtype matching the config, identical shapes,
  sequence length a multiple of the config's B_r and B_c.  With ``benchmark=True`` the launch is
  bracketed by CUDA events and the elapsed milliseconds are returned (``:111-131``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .kernel_configs import DType, FlashForwardKernelConfig, get_kernel_progression_configs
from .ops import flash_attn_fwd

# K7, the reference's best progression kernel, stands in as the default config object.
_CFG = get_kernel_progression_configs()[6]


class _Ext:
    """Stand-in for the JIT-loaded extension module object (`_ext`) of the reference."""

    @staticmethod
    def forward(
        kernel_cfg: Optional[FlashForwardKernelConfig],
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        o: Optional[torch.Tensor] = None,
        benchmark: bool = False,
    ) -> Tuple[torch.Tensor, float]:
        for name, t in (("q", q), ("k", k), ("v", v)):
            if not t.is_cuda:
                raise RuntimeError(f"{name} must be a CUDA tensor")
            if not t.is_contiguous():
                raise RuntimeError(f"{name} must be contiguous")
        if q.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("Only fp16 and bf16 are supported")
        if not (q.dtype == k.dtype == v.dtype):
            raise RuntimeError("Input tensors must have the same data type")
        if not (q.shape == k.shape == v.shape) or q.dim() != 4:
            raise RuntimeError("q, k, v must be 4-D (batch, seq_len, n_heads, d_head) with identical shapes")
        if kernel_cfg is not None:
            if DType(kernel_cfg.dtype).to_torch_dtype() != q.dtype:
                raise RuntimeError("Kernel configuration dtype does not match input dtype")
            if kernel_cfg.d_head != q.shape[3]:
                raise RuntimeError("Kernel configuration d_head does not match input head dim")
            n = q.shape[1]
            if n % kernel_cfg.B_r != 0 or n % kernel_cfg.B_c != 0:
                raise RuntimeError("Sequence length must be a multiple of the block sizes B_r and B_c")
        if o is None:
            o = torch.empty_like(q)
        elif not o.is_cuda or not o.is_contiguous() or o.shape != q.shape or o.dtype != q.dtype:
            raise RuntimeError("o must be a contiguous CUDA tensor shaped and typed like q")
        ms = 0.0
        if benchmark:
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            flash_attn_fwd(q, k, v, layout="bnhd", out=o)
            stop.record()
            stop.synchronize()
            ms = start.elapsed_time(stop)
        else:
            flash_attn_fwd(q, k, v, layout="bnhd", out=o)
        return o, ms


ext = _Ext()


def forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Flash attention forward. q/k/v: (B, N, H, D) fp16 or bf16 CUDA tensors; non-causal,
    softmax scale 1/sqrt(D) (the reference operator's fixed behaviour)."""
    out = torch.empty_like(q)
    ext.forward(_CFG if q.dtype == torch.float16 and q.shape[3] == _CFG.d_head and q.shape[1] % 64 == 0 else None,
                q.contiguous(), k.contiguous(), v.contiguous(), out, False)
    return out
