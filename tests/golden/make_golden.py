"""Generate tests/golden/*.npz by RUNNING the reference repository's own PyTorch code on the CPU.

Usage (only where the reference checkout is mounted; the fixtures it writes are committed):

    python tests/golden/make_golden.py /path/to/Mini-Attention

Each fixture stores seeded inputs and the output the reference function produced for them:

* ``triton_reference_*``  ``reference(q, k, v, causal)`` of
  kernels/flash_attn/triton/fp16_flash_attn_sm86.py:112-117 (causal and non-causal)
* ``standard_attention``  kernels/flash_attn/pytorch/standard.py:4-20
* ``sdpa_bnhd_*``         ``sdpa_reference`` of tests/test_correctness.py:35-43, the reference
  test's own recipe (seed 42, (B,N,H,D) layout); the full-size case keeps every 8th token
* ``gqa_core`` / ``mqa_core`` / ``mha_core``  the core attention call inside ``GQA_Flash``,
  ``MQA_Flash`` and ``MHA`` (kernels/standard/pytorch/{gqa,mqa,mha}.py) with the q, k, v the
  module fed into it, captured by wrapping the module's attention call.
* ``mha_module``  the ``MHA`` module of kernels/standard/pytorch/mha.py run whole (d_model 128, 2 heads, 64
  tokens): its parameters, its input and both return values without a mask and with a lower-triangular
  mask, plus the fact that an all-ones mask changes nothing.

Inputs are stored in fp16/bf16 bit patterns (uint16 views) so that loading is exact.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def _save(name: str, **arrays):
    meta = {k: v for k, v in arrays.items() if not isinstance(v, torch.Tensor)}
    tens = {k: _bits(v) for k, v in arrays.items() if isinstance(v, torch.Tensor)}
    dts = {k + "__dtype": str(v.dtype) for k, v in arrays.items() if isinstance(v, torch.Tensor)}
    np.savez_compressed(OUT / f"{name}.npz", **tens, **dts, **meta)
    print("wrote", name, {k: tuple(v.shape) for k, v in tens.items()})


def main(ref_root: Path) -> None:
    torch.set_num_threads(8)

    # ---- reference() of the Triton file (plain PyTorch function) -------------------------
    tri_path = ref_root / "kernels/flash_attn/triton/fp16_flash_attn_sm86.py"
    try:
        tri = _load(tri_path, "ref_triton_fa")
        reference = tri.reference
    except Exception as e:  # triton may refuse to build its autotuner without a GPU
        print("importing the Triton file failed (", repr(e), "); extracting reference() from its source")
        src = tri_path.read_text()
        start = src.index("def reference(")
        end = src.index('if __name__ == "__main__"')
        ns = {"torch": torch, "math": __import__("math")}
        exec(compile(src[start:end], str(tri_path), "exec"), ns)
        reference = ns["reference"]
    for causal in (False, True):
        for dtype, tag in ((torch.float16, "fp16"), (torch.bfloat16, "bf16")):
            torch.manual_seed(0)
            q = torch.randn(1, 2, 256, 64, dtype=torch.float32).to(dtype)
            k = torch.randn(1, 2, 256, 64, dtype=torch.float32).to(dtype)
            v = torch.randn(1, 2, 256, 64, dtype=torch.float32).to(dtype)
            o = reference(q, k, v, causal=causal)
            _save(f"triton_reference_{tag}_{'causal' if causal else 'full'}", q=q, k=k, v=v, out=o,
                  causal=int(causal))
    torch.manual_seed(1)
    q = torch.randn(1, 2, 384, 128).half(); k = torch.randn(1, 2, 384, 128).half(); v = torch.randn(1, 2, 384, 128).half()
    _save("triton_reference_fp16_d128_causal", q=q, k=k, v=v, out=reference(q, k, v, causal=True), causal=1)

    # ---- standard_attention (module runs a demo at import; harmless on CPU) ---------------
    std = _load(ref_root / "kernels/flash_attn/pytorch/standard.py", "ref_standard")
    torch.manual_seed(2)
    q = torch.randn(2, 192, 64); k = torch.randn(2, 192, 64); v = torch.randn(2, 192, 64)
    o, w = std.standard_attention(q, k, v)
    _save("standard_attention_fp32", q=q, k=k, v=v, out=o, causal=0)

    # ---- the reference test's own recipe ---------------------------------------------------
    tc = _load(ref_root / "tests/test_correctness.py", "ref_test_correctness")
    torch.manual_seed(tc.SEED)
    q = torch.randn(tc.B, tc.N, tc.H, tc.D, dtype=torch.float16)
    k = torch.randn_like(q)
    v = torch.randn_like(q)
    o = tc.sdpa_reference(q, k, v)
    # inputs are regenerated from the seed by the test; keep every 8th token of the output
    _save("sdpa_bnhd_test_correctness", out_rows=o[:, ::8].contiguous(), seed=tc.SEED, B=tc.B, N=tc.N,
          H=tc.H, D=tc.D, row_step=8, tolerance=tc.TOLERANCE)
    torch.manual_seed(7)
    q = torch.randn(1, 128, 2, 128, dtype=torch.float16); k = torch.randn_like(q); v = torch.randn_like(q)
    _save("sdpa_bnhd_small", q=q, k=k, v=v, out=tc.sdpa_reference(q, k, v), causal=0)

    # ---- core attention call inside the standard modules ------------------------------------
    import torch.nn.functional as F
    captured = {}

    def spy(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, **kw):
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p,
                                           is_causal=is_causal, **kw)
        captured.update(q=q.detach().clone(), k=k.detach().clone(), v=v.detach().clone(),
                        out=o.detach().clone(), causal=int(is_causal))
        return o

    gqa = _load(ref_root / "kernels/standard/pytorch/gqa.py", "ref_gqa")
    gqa.scaled_dot_product_attention = spy
    torch.manual_seed(3)
    mod = gqa.GQA_Flash(d_model=512, n_heads=8, n_kv_heads=2)
    with torch.no_grad():
        mod(torch.randn(1, 96, 512))
    # the module expands K/V with repeat_interleave before the call: store the un-expanded heads
    G = mod.group_size
    _save("gqa_core", q=captured["q"], k=captured["k"][:, ::G].contiguous(), v=captured["v"][:, ::G].contiguous(),
          out=captured["out"], causal=captured["causal"], group=G)

    mqa = _load(ref_root / "kernels/standard/pytorch/mqa.py", "ref_mqa")
    mqa.scaled_dot_product_attention = spy
    torch.manual_seed(4)
    mod = mqa.MQA_Flash(d_model=256, n_heads=4)
    captured.clear()
    try:
        with torch.no_grad():
            mod(torch.randn(1, 96, 256))
    except RuntimeError as e:
        # the module forces the FLASH backend; if that is unavailable on this CPU, call the
        # same SDPA without the backend restriction on the tensors the module built
        print("MQA forced-flash backend unavailable on CPU:", e)
    if captured:
        _save("mqa_core", q=captured["q"], k=captured["k"][:, :1].contiguous(), v=captured["v"][:, :1].contiguous(),
              out=captured["out"], causal=captured["causal"], group=mod.n_heads)

    # MHA does explicit matmul / masked_fill / softmax and returns the weights: recover the
    # core output as weights @ v from the projections it applies.
    mha = _load(ref_root / "kernels/standard/pytorch/mha.py", "ref_mha")
    torch.manual_seed(5)
    mod = mha.MHA(d_model=256, n_heads=4)
    x = torch.randn(1, 64, 256)
    with torch.no_grad():
        B, S, _ = x.shape
        q = mod.w_q(x).view(B, S, 4, 64).transpose(1, 2)
        k = mod.w_k(x).view(B, S, 4, 64).transpose(1, 2)
        v = mod.w_v(x).view(B, S, 4, 64).transpose(1, 2)
        for tag, mask in (("full", None), ("masked", torch.tril(torch.ones(S, S)))):
            y, weights = mod(x, mask=mask)
            core = weights @ v  # exactly the `output = weights @ v` line of MHA.forward
            _save(f"mha_core_{tag}", q=q, k=k, v=v, out=core, weights=weights, causal=int(mask is not None))
        # the module end to end (projections included): input, parameters, both return values
        torch.manual_seed(6)
        small = mha.MHA(d_model=128, n_heads=2)
        xs = torch.randn(1, 64, 128)
        sd = {name.replace(".", "__"): t for name, t in small.state_dict().items()}
        res = {}
        for tag, mask in (("full", None), ("masked", torch.tril(torch.ones(64, 64)))):
            res[f"y_{tag}"], res[f"weights_{tag}"] = small(xs, mask=mask)
        # an all-ones mask hides nothing (mask == 0 -> -inf, mha.py:43-44): same result as no mask
        y1, w1 = small(xs, mask=torch.ones(64, 64))
        res["ones_equals_full"] = int(torch.equal(y1, res["y_full"]) and torch.equal(w1, res["weights_full"]))
        _save("mha_module", x=xs, **res, **sd)


def kernel_config_strings(ref_root: Path) -> None:
    """Short forms and field tuples of the reference's K1..K7 progression
    (kernels/flash_attn/cuda/sm_120/py/flash_helpers/kernel_configs.py:426-454)."""
    import dataclasses
    import json
    kc = _load(ref_root / "kernels/flash_attn/cuda/sm_120/py/flash_helpers/kernel_configs.py", "ref_kernel_configs")
    cfgs = kc.get_kernel_progression_configs()
    data = {
        "short_forms": [c.short_form() for c in cfgs],
        "fields": [[int(x) for x in dataclasses.astuple(c)] for c in cfgs],
        "n_all_block_sizes": len(kc.get_kernel_progression_configs(all_block_sizes=True)),
        "attn_flop_2_8_512": cfgs[0].attn_flop(2, 8, 512),
    }
    (OUT / "kernel_progression.json").write_text(json.dumps(data, indent=1))
    print("wrote kernel_progression.json")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/Mini-Attention")
    kernel_config_strings(Path(sys.argv[1]))
    main(Path(sys.argv[1]))
