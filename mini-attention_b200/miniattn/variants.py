"""MHA / GQA / MQA attention variants of kernels/standard/pytorch with the core attention
call replaced by the B200 kernel.  Projections stay ordinary ``nn.Linear`` layers (they are
not on the hot path); parameter names match the reference modules so state dicts load
unchanged.

* ``MHA``        kernels/standard/pytorch/mha.py:9-55   (returns ``(output, weights)`` like the
                 reference; ``mask`` = None or all ones runs the non-causal kernel, a
                 lower-triangular mask the causal kernel; any other mask raises, because there is
                 no eager path behind the fused kernel.  The weights the reference returns are
                 rebuilt from the kernel's log-sum-exp, ``exp(q k^T * scale - lse)``; the
                 constructor flag ``need_weights=False`` skips that and returns ``(output, None)``)
* ``GQA_Flash``  kernels/standard/pytorch/gqa.py:7-51   (causal; K/V heads are broadcast inside
                 the kernel instead of ``repeat_interleave``)
* ``MQA_Flash``  kernels/standard/pytorch/mqa.py:8-47   (causal; single K/V head)
"""
from __future__ import annotations

import torch
import torch.nn as nn

import math

from .ops import flash_attn_fwd


def _attend(q, k, v, causal, return_lse=False):
    """q: (B,S,Hq,dh) view, k/v: (B,S,Hkv,dh) views -> (B,S,Hq*dh) [, lse (B,Hq,S)]."""
    dt = q.dtype
    if dt not in (torch.float16, torch.bfloat16):
        raise RuntimeError("the B200 attention kernels take fp16 or bf16 activations")
    res = flash_attn_fwd(q, k, v, causal=causal, layout="bnhd", return_lse=return_lse)
    o = res[0] if return_lse else res
    o = o.reshape(o.shape[0], o.shape[1], -1)
    return (o, res[1]) if return_lse else o


class MHA(nn.Module):
    def __init__(self, d_model: int, n_heads: int, dropout: float = 0.0, need_weights: bool = True):
        super().__init__()
        assert d_model % n_heads == 0
        if dropout != 0.0:
            raise RuntimeError("attention dropout is not supported by the fused kernel")
        self.d_model, self.n_heads, self.d_h = d_model, n_heads, d_model // n_heads
        self.need_weights = need_weights
        self.w_q = nn.Linear(d_model, d_model)
        self.w_k = nn.Linear(d_model, d_model)
        self.w_v = nn.Linear(d_model, d_model)
        self.w_o = nn.Linear(d_model, d_model)

    def forward(self, x: torch.Tensor, mask: torch.Tensor = None):
        """Returns ``(output, weights)`` as kernels/standard/pytorch/mha.py:55 does; ``weights``
        is (B, n_heads, S, S) in x's dtype, or None when the module was built with
        ``need_weights=False``.  ``mask`` follows the reference's convention (0 = hidden,
        mha.py:43-44)."""
        B, S, _ = x.shape
        causal = False
        if mask is not None:
            if mask.shape[-2:] != (S, S):
                raise RuntimeError(f"mask must end in ({S}, {S}), got {tuple(mask.shape)}")
            m = (mask != 0).reshape(-1, S, S)
            if not bool(m.all()):  # an all-ones mask hides nothing: the non-causal kernel
                tril = torch.tril(torch.ones(S, S, device=mask.device, dtype=torch.bool))
                if not bool((m == tril).all()):
                    raise RuntimeError("only no mask, an all-ones mask or a lower-triangular (causal) mask is "
                                       "supported: there is no eager path behind the fused kernel")
                causal = True
        q = self.w_q(x).view(B, S, self.n_heads, self.d_h)
        k = self.w_k(x).view(B, S, self.n_heads, self.d_h)
        v = self.w_v(x).view(B, S, self.n_heads, self.d_h)
        if not self.need_weights:
            return self.w_o(_attend(q, k, v, causal)), None
        o, lse = _attend(q, k, v, causal, return_lse=True)
        # weights = softmax(q k^T / sqrt(d_h) [+ mask]) rebuilt from the kernel's log-sum-exp
        scores = torch.matmul(q.transpose(1, 2).float(), k.permute(0, 2, 3, 1).float()) / math.sqrt(self.d_h)
        weights = torch.exp(scores - lse.unsqueeze(-1))
        if causal:
            weights = weights.masked_fill(~torch.tril(torch.ones(S, S, device=x.device, dtype=torch.bool)), 0.0)
        return self.w_o(o), weights.to(x.dtype)


class GQA_Flash(nn.Module):
    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int):
        super().__init__()
        assert d_model % n_heads == 0 and n_heads % n_kv_heads == 0
        self.d_model, self.n_heads, self.n_kv_heads = d_model, n_heads, n_kv_heads
        self.head_dim = d_model // n_heads
        self.group_size = n_heads // n_kv_heads
        self.w_q = nn.Linear(d_model, d_model)
        self.kv = nn.Linear(d_model, 2 * self.head_dim * n_kv_heads)
        self.w_o = nn.Linear(d_model, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, _ = x.shape
        q = self.w_q(x).view(B, S, self.n_heads, self.head_dim)
        kv = self.kv(x).view(B, S, 2, self.n_kv_heads, self.head_dim)
        return self.w_o(_attend(q, kv[:, :, 0], kv[:, :, 1], True))


class MQA_Flash(nn.Module):
    def __init__(self, d_model: int, n_heads: int):
        super().__init__()
        assert d_model % n_heads == 0
        self.d_model, self.n_heads, self.head_dim = d_model, n_heads, d_model // n_heads
        self.w_q = nn.Linear(d_model, d_model)
        self.k_v = nn.Linear(d_model, 2 * self.head_dim)
        self.w_o = nn.Linear(d_model, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, _ = x.shape
        q = self.w_q(x).view(B, S, self.n_heads, self.head_dim)
        kv = self.k_v(x).view(B, S, 2, 1, self.head_dim)
        return self.w_o(_attend(q, kv[:, :, 0], kv[:, :, 1], True))
