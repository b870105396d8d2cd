"""Pins the CPU oracle to outputs of the reference repository's own PyTorch code.

Every fixture under tests/golden/ was produced by running a reference function (see
tests/golden/make_golden.py); the oracle's restatement must reproduce each of them.
"""
import math

import pytest
import torch

from conftest import golden_names, load_golden
from oracle.attention_oracle import attention_reference, sdpa_reference_bnhd


def _tol(dtype):
    # both sides round the same fp32 result to `dtype`; allow one unit of rounding slack
    return {torch.float16: 1e-3, torch.bfloat16: 8e-3, torch.float32: 2e-6}[dtype]


@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith("triton_reference")])
def test_triton_file_reference(name):
    g = load_golden(name)
    out = attention_reference(g["q"], g["k"], g["v"], causal=bool(g["causal"]))
    assert out.dtype == g["out"].dtype
    err = (out.float() - g["out"].float()).abs().max().item()
    assert err <= _tol(out.dtype), err


def test_standard_attention():
    g = load_golden("standard_attention_fp32")
    q, k, v = (g[x].unsqueeze(1) for x in ("q", "k", "v"))  # (B,S,D) -> (B,1,S,D)
    out = attention_reference(q, k, v).squeeze(1)
    assert (out - g["out"]).abs().max().item() <= 2e-6


def test_reference_test_recipe_full_size():
    """tests/test_correctness.py of the reference: seed 42, (B,N,H,D)=(2,512,8,128) fp16."""
    g = load_golden("sdpa_bnhd_test_correctness")
    torch.manual_seed(int(g["seed"]))
    q = torch.randn(int(g["B"]), int(g["N"]), int(g["H"]), int(g["D"]), dtype=torch.float16)
    k = torch.randn_like(q)
    v = torch.randn_like(q)
    out = sdpa_reference_bnhd(q, k, v)[:, :: int(g["row_step"])]
    err = (out.float() - g["out_rows"].float()).abs().max().item()
    assert err <= float(g["tolerance"]), err  # the reference's own 1e-3 budget


def test_reference_test_recipe_small():
    g = load_golden("sdpa_bnhd_small")
    out = sdpa_reference_bnhd(g["q"], g["k"], g["v"])
    assert (out.float() - g["out"].float()).abs().max().item() <= 1e-3


@pytest.mark.parametrize("name", ["gqa_core", "mqa_core"])
def test_gqa_mqa_core(name):
    g = load_golden(name)
    assert g["q"].shape[1] == g["k"].shape[1] * int(g["group"])
    out = attention_reference(g["q"], g["k"], g["v"], causal=bool(g["causal"]))
    assert (out - g["out"]).abs().max().item() <= 5e-6


@pytest.mark.parametrize("name", ["mha_core_full", "mha_core_masked"])
def test_mha_core(name):
    g = load_golden(name)
    out, lse = attention_reference(g["q"], g["k"], g["v"], causal=bool(g["causal"]), return_lse=True)
    assert (out - g["out"]).abs().max().item() <= 5e-6
    # log-sum-exp against the weights the module returned: w_ij = exp(s_ij - lse_i)
    s = (g["q"] @ g["k"].transpose(-1, -2)) / math.sqrt(g["q"].shape[-1])
    w = torch.exp(s - lse.unsqueeze(-1))
    if g["causal"]:
        w = torch.tril(w)
    assert (w - g["weights"]).abs().max().item() <= 1e-5


def test_mha_module_end_to_end():
    """The reference MHA module run whole (projections, masked softmax, both return values):
    the oracle reproduces its output and its weights from the stored parameters."""
    g = load_golden("mha_module")
    assert g["ones_equals_full"] == 1
    x = g["x"]
    H, dh = 2, 64
    lin = lambda n: x @ g[f"{n}__weight"].t() + g[f"{n}__bias"]  # noqa: E731
    q, k, v = (lin(n).view(1, 64, H, dh).transpose(1, 2) for n in ("w_q", "w_k", "w_v"))
    for tag, causal in (("full", False), ("masked", True)):
        o, lse = attention_reference(q, k, v, causal=causal, return_lse=True)
        y = o.transpose(1, 2).reshape(1, 64, H * dh) @ g["w_o__weight"].t() + g["w_o__bias"]
        assert (y - g[f"y_{tag}"]).abs().max().item() <= 1e-5
        w = torch.exp((q @ k.transpose(-1, -2)) / math.sqrt(dh) - lse.unsqueeze(-1))
        if causal:
            w = torch.tril(w)
        assert (w - g[f"weights_{tag}"]).abs().max().item() <= 1e-5
