"""MHA / GQA / MQA attention variants of kernels/standard/pytorch with the core attention
call replaced by the B200 kernel.  Projections stay ordinary ``nn.Linear`` layers (they are
not on the hot path); parameter names match the reference modules so state dicts load
unchanged.

* ``MHA``        kernels/standard/pytorch/mha.py:9-55   (non-causal; ``mask`` = lower-triangular
                 selects the causal kernel, any other mask is rejected; attention weights are
                 not materialised, so ``forward`` returns only the output)
* ``GQA_Flash``  kernels/standard/pytorch/gqa.py:7-51   (causal; K/V heads are broadcast inside
                 the kernel instead of ``repeat_interleave``)
* ``MQA_Flash``  kernels/standard/pytorch/mqa.py:8-47   (causal; single K/V head)
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .ops import flash_attn_fwd


def _attend(q, k, v, causal):
    """q: (B,S,Hq,dh) view, k/v: (B,S,Hkv,dh) views -> (B,S,Hq*dh)."""
    dt = q.dtype
    if dt not in (torch.float16, torch.bfloat16):
        raise RuntimeError("the B200 attention kernels take fp16 or bf16 activations")
    o = flash_attn_fwd(q, k, v, causal=causal, layout="bnhd")
    return o.reshape(o.shape[0], o.shape[1], -1)


class MHA(nn.Module):
    def __init__(self, d_model: int, n_heads: int, dropout: float = 0.0):
        super().__init__()
        assert d_model % n_heads == 0
        if dropout != 0.0:
            raise RuntimeError("attention dropout is not supported by the fused kernel")
        self.d_model, self.n_heads, self.d_h = d_model, n_heads, d_model // n_heads
        self.w_q = nn.Linear(d_model, d_model)
        self.w_k = nn.Linear(d_model, d_model)
        self.w_v = nn.Linear(d_model, d_model)
        self.w_o = nn.Linear(d_model, d_model)

    def forward(self, x: torch.Tensor, mask: torch.Tensor = None) -> torch.Tensor:
        B, S, _ = x.shape
        causal = False
        if mask is not None:
            tril = torch.tril(torch.ones(S, S, device=mask.device, dtype=mask.dtype))
            if mask.shape[-2:] != (S, S) or not torch.equal(mask.reshape(-1, S, S)[0], tril) or \
                    not bool((mask.reshape(-1, S, S) == tril).all()):
                raise RuntimeError("only a lower-triangular (causal) mask is supported")
            causal = True
        q = self.w_q(x).view(B, S, self.n_heads, self.d_h)
        k = self.w_k(x).view(B, S, self.n_heads, self.d_h)
        v = self.w_v(x).view(B, S, self.n_heads, self.d_h)
        return self.w_o(_attend(q, k, v, causal))


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
