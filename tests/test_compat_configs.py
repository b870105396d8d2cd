"""The kernel-config mirror reproduces the reference's K1..K7 progression exactly
(fixture written from the reference module by tests/golden/make_golden.py)."""
import dataclasses
import json
from pathlib import Path

import pytest

from miniattn import kernel_configs as kc

GOLD = json.loads((Path(__file__).parent / "golden" / "kernel_progression.json").read_text())


def test_progression_matches_reference():
    cfgs = kc.get_kernel_progression_configs()
    assert [c.short_form() for c in cfgs] == GOLD["short_forms"]
    assert [[int(x) for x in dataclasses.astuple(c)] for c in cfgs] == GOLD["fields"]
    assert len(kc.get_kernel_progression_configs(all_block_sizes=True)) == GOLD["n_all_block_sizes"]
    assert cfgs[0].attn_flop(2, 8, 512) == GOLD["attn_flop_2_8_512"]


def test_selection_key(monkeypatch):
    assert kc.get_kernel_configs("prog") == kc.get_kernel_progression_configs()
    monkeypatch.setenv("KERNELS", "progall")
    assert len(kc.get_kernel_configs()) == GOLD["n_all_block_sizes"]
    with pytest.raises(ValueError):
        kc.get_kernel_configs("nope")


def test_dtype_enum():
    import torch
    assert kc.DType.from_string("fp16") is kc.DType.FP16 and kc.DType.from_string("15") is kc.DType.BF16
    assert kc.DType.BF16.to_torch_dtype() is torch.bfloat16
    assert kc.attention_matmul_flop(2, 8, 512, 128) == 4 * 2 * 8 * 512 * 512 * 128
