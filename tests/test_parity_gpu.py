"""Parity of the CUDA path (called through the C ABI via miniattn) with the CPU oracle, the
golden fixtures produced by the reference's own PyTorch code, and size-independent properties
at the full BASELINE sizes.

Tolerances (max |out - reference|): fp16 2e-3, bf16 1e-2 — the north-star bars; they are
spelled out in conftest.TOL.
"""
import math

import pytest
import torch

import miniattn
from conftest import TOL, golden_names, load_golden
from oracle.attention_oracle import (attention_reference, attention_reference_rows, make_inputs,
                                     sdpa_reference_bnhd)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
KERNELS = ["ws", "simple"]


def run(q, k, v, **kw):
    out = miniattn.flash_attn_fwd(q.to(DEV), k.to(DEV), v.to(DEV), **kw)
    if isinstance(out, tuple):
        res = tuple(o.cpu() for o in out)
    else:
        res = out.cpu()
    assert miniattn.device_status(DEV) == 0, "a bounded device wait ran out"
    return res


def maxerr(a, b):
    return (a.float() - b.float()).abs().max().item()


# ------------------------------------------------------------------ small-case sweep
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize(
    "B,Hq,Hkv,Nq,Nk,D",
    [
        (1, 1, 1, 128, 128, 128),
        (1, 2, 2, 256, 256, 64),
        (2, 4, 1, 384, 384, 128),   # MQA
        (1, 8, 2, 512, 512, 128),   # GQA, 4 query heads per KV head
        (1, 2, 2, 200, 333, 128),   # ragged: neither length is a multiple of the tile
        (1, 3, 3, 1, 77, 64),       # a single query row
        (1, 2, 1, 640, 96, 64),     # more queries than keys
        (2, 2, 2, 129, 1, 128),     # a single key
    ],
)
def test_small_cases(kernel, dtype, causal, B, Hq, Hkv, Nq, Nk, D):
    q, k, v = make_inputs(B, Hq, Hkv, Nq, Nk, D, dtype, seed=Nq * 7 + Nk)
    ref, ref_lse = attention_reference(q, k, v, causal=causal, return_lse=True, out_dtype=torch.float32)
    out, lse = run(q, k, v, causal=causal, kernel=kernel, return_lse=True)
    assert out.dtype == dtype
    assert maxerr(out, ref) <= TOL[dtype]
    finite = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), finite)
    assert (lse[finite] - ref_lse[finite]).abs().max().item() <= 2e-3


@pytest.mark.parametrize("kernel", KERNELS)
def test_softmax_scale_and_layouts(kernel):
    q, k, v = make_inputs(2, 4, 4, 256, 256, 128, torch.float16, seed=11)
    ref = attention_reference(q, k, v, softmax_scale=0.05, out_dtype=torch.float32)
    assert maxerr(run(q, k, v, softmax_scale=0.05, kernel=kernel), ref) <= TOL[torch.float16]
    # (B,N,H,D) tensors, as the reference CUDA operator takes them
    qn, kn, vn = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    out = run(qn, kn, vn, softmax_scale=0.05, layout="bnhd", kernel=kernel)
    assert maxerr(out.transpose(1, 2), ref) <= TOL[torch.float16]
    # strided views: every other head of a wider tensor, no copy
    wide = torch.randn(2, 8, 256, 128, dtype=torch.float16)
    qs = wide[:, ::2]
    ref2 = attention_reference(qs, k, v, out_dtype=torch.float32)
    out2 = miniattn.flash_attn_fwd(wide.to(DEV)[:, ::2], k.to(DEV), v.to(DEV), kernel=kernel).cpu()
    assert maxerr(out2, ref2) <= TOL[torch.float16]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kernel", KERNELS)
def test_causal_offsets(kernel, dtype):
    """Global positions shift the diagonal (what a ring step needs); rows that see no key give
    exact zeros and lse = -inf (in bf16 a masked score's 2^-126 does not round to zero: the rows
    must come out zero all the same)."""
    q, k, v = make_inputs(1, 2, 2, 256, 384, 128, dtype, seed=5)
    for q_pos0, k_pos0 in ((128, 0), (0, 128), (300, 100), (0, 400)):
        ref, ref_lse = attention_reference(q, k, v, causal=True, q_pos0=q_pos0, k_pos0=k_pos0,
                                           return_lse=True, out_dtype=torch.float32)
        out, lse = run(q, k, v, causal=True, q_pos0=q_pos0, k_pos0=k_pos0, kernel=kernel, return_lse=True)
        assert maxerr(out, ref) <= TOL[dtype], (q_pos0, k_pos0)
        dark = ~torch.isfinite(ref_lse)
        assert float(out[dark].abs().max() if dark.any() else 0.0) == 0.0
        finite = torch.isfinite(ref_lse)
        assert torch.equal(torch.isfinite(lse), finite)
        if finite.any():
            assert (lse[finite] - ref_lse[finite]).abs().max().item() <= 2e-3


# ------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith("triton_reference")])
def test_golden_triton_reference(kernel, name):
    g = load_golden(name)
    out = run(g["q"], g["k"], g["v"], causal=bool(g["causal"]), kernel=kernel)
    assert maxerr(out, g["out"]) <= TOL[g["q"].dtype]


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("name", ["gqa_core", "mqa_core", "mha_core_full", "mha_core_masked"])
def test_golden_standard_modules(kernel, name):
    """Core attention call of GQA_Flash / MQA_Flash / MHA: fp32 fixtures, run here in fp16."""
    g = load_golden(name)
    out = run(g["q"].half(), g["k"].half(), g["v"].half(), causal=bool(g["causal"]), kernel=kernel)
    assert maxerr(out, g["out"]) <= 3e-3  # fp16 tolerance + rounding of the fp32 inputs to fp16


def test_golden_reference_test_recipe():
    """The reference's tests/test_correctness.py through the compat operator: seed 42,
    (B,N,H,D) = (2,512,8,128) fp16, its own tolerance 1e-3."""
    g = load_golden("sdpa_bnhd_test_correctness")
    torch.manual_seed(int(g["seed"]))
    q = torch.randn(int(g["B"]), int(g["N"]), int(g["H"]), int(g["D"]), dtype=torch.float16)
    k = torch.randn_like(q)
    v = torch.randn_like(q)
    out = miniattn.forward(q.to(DEV), k.to(DEV), v.to(DEV)).cpu()
    assert maxerr(out[:, :: int(g["row_step"])], g["out_rows"]) < float(g["tolerance"])
    cfg = miniattn.kernel_configs.get_kernel_progression_configs()[6]
    o2, ms = miniattn.ext.forward(cfg, q.to(DEV), k.to(DEV), v.to(DEV), None, True)
    assert ms > 0 and torch.equal(o2.cpu(), out)
    g2 = load_golden("sdpa_bnhd_small")
    assert maxerr(miniattn.forward(g2["q"].to(DEV), g2["k"].to(DEV), g2["v"].to(DEV)).cpu(), g2["out"]) < 1e-3


def test_compat_error_behaviour():
    q = torch.zeros(1, 96, 2, 128, dtype=torch.float16, device=DEV)
    cfg = miniattn.kernel_configs.get_kernel_progression_configs()[0]
    with pytest.raises(RuntimeError, match="multiple of the block sizes"):
        miniattn.ext.forward(cfg, q, q, q, None, False)
    with pytest.raises(RuntimeError, match="contiguous"):
        miniattn.ext.forward(cfg, q.transpose(1, 2), q, q, None, False)
    with pytest.raises(RuntimeError, match="dtype"):
        miniattn.ext.forward(cfg, q.bfloat16(), q.bfloat16(), q.bfloat16(), None, False)
    with pytest.raises(RuntimeError, match="same data type"):
        miniattn.ext.forward(None, q, q.bfloat16(), q, None, False)


# ------------------------------------------------------------------ BASELINE configurations
def test_config1_full_oracle():
    """MHA fp16 B=2 H=8 N=512 D=128, seed 0, (B,H,N,D)."""
    q, k, v = make_inputs(2, 8, 8, 512, 512, 128, torch.float16, seed=0)
    ref = attention_reference(q, k, v, out_dtype=torch.float32)
    for kernel in KERNELS:
        assert maxerr(run(q, k, v, kernel=kernel), ref) <= TOL[torch.float16]


@pytest.mark.parametrize("N", [1024, 2048, 4096, 8192])
def test_config2_sweep(N):
    """Config 2 at every N: sampled rows against the exact oracle, plus the two kernels agree."""
    q, k, v = make_inputs(2, 8, 8, N, N, 128, torch.float16, seed=0)
    rows = torch.cat([torch.tensor([0, 1, 127, 128, N // 2, N - 129, N - 128, N - 1]),
                      torch.randint(0, N, (120,), generator=torch.Generator().manual_seed(N))]).unique()
    ref_rows = attention_reference_rows(q, k, v, rows)
    out = run(q, k, v, kernel="ws")
    assert maxerr(out[:, :, rows], ref_rows) <= TOL[torch.float16]
    out_s = run(q, k, v, kernel="simple")
    assert maxerr(out, out_s) <= TOL[torch.float16]


def test_config3_gqa_causal_bf16():
    """GQA causal bf16 B=4 Hq=32 Hkv=8 N=4096 D=128: sampled rows vs the oracle."""
    q, k, v = make_inputs(4, 32, 8, 4096, 4096, 128, torch.bfloat16, seed=0)
    rows = torch.cat([torch.tensor([0, 1, 127, 128, 255, 256, 2047, 4095]),
                      torch.randint(0, 4096, (56,), generator=torch.Generator().manual_seed(3))]).unique()
    ref_rows = attention_reference_rows(q, k, v, rows, causal=True)
    out = run(q, k, v, causal=True)
    assert maxerr(out[:, :, rows], ref_rows) <= TOL[torch.bfloat16]


# ------------------------------------------------------------------ properties at full size
@pytest.mark.parametrize("causal", [False, True])
def test_properties_full_size(causal):
    N, D = 8192, 128
    q, k, v = make_inputs(1, 4, 4, N, N, D, torch.float16, seed=9)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    # V constant per channel -> every output row equals that constant
    const = torch.linspace(-2, 2, D, dtype=torch.float16, device=DEV).expand(1, 4, N, D).contiguous()
    out = miniattn.flash_attn_fwd(qd, kd, const, causal=causal)
    assert maxerr(out, const) <= 2e-3
    # K = 0 -> uniform weights: O = mean of the visible V rows (prefix mean when causal)
    out = miniattn.flash_attn_fwd(qd, torch.zeros_like(kd), vd, causal=causal).float()
    if causal:
        expect = vd.float().cumsum(dim=2) / torch.arange(1, N + 1, device=DEV).view(1, 1, N, 1)
    else:
        expect = vd.float().mean(dim=2, keepdim=True).expand_as(out)
    assert maxerr(out, expect) <= 2e-3
    # linearity in V: O(V1 + V2) = O(V1) + O(V2)
    v2 = torch.randn_like(vd)
    o1 = miniattn.flash_attn_fwd(qd, kd, vd, causal=causal).float()
    o2 = miniattn.flash_attn_fwd(qd, kd, v2, causal=causal).float()
    o12 = miniattn.flash_attn_fwd(qd, kd, (vd.float() + v2.float()).half(), causal=causal).float()
    assert maxerr(o12, o1 + o2) <= 6e-3
    if not causal:
        # permuting the keys (with their values) leaves the result unchanged
        perm = torch.randperm(N, device=DEV)
        o_perm = miniattn.flash_attn_fwd(qd, kd[:, :, perm].contiguous(), vd[:, :, perm].contiguous()).float()
        assert maxerr(o_perm, o1) <= 2e-3
    # a huge logit on one key -> the output is that key's value row
    kk = kd.clone()
    qq = qd.clone()
    qq[:, :, :, 0] = 40.0
    kk[:, :, :, 0] = 0.0
    kk[:, :, 5, 0] = 40.0
    o_hot = miniattn.flash_attn_fwd(qq, kk, vd, causal=causal, softmax_scale=1.0).float()
    assert maxerr(o_hot[:, :, 5:], vd[:, :, 5:6].float().expand(-1, -1, N - 5, -1)) <= 2e-3
    assert miniattn.device_status(DEV) == 0


def test_bounded_wait_self_test():
    """A device-side wait that nothing satisfies gives up, reports bit 30 and leaves the context usable."""
    assert miniattn.selftest_wait(20.0) == (1 << 30)
    q, k, v = make_inputs(1, 1, 1, 128, 128, 128, torch.float16, seed=1)
    assert maxerr(run(q, k, v), attention_reference(q, k, v, out_dtype=torch.float32)) <= 2e-3


def test_variant_modules_match_reference_math():
    """MHA / GQA_Flash / MQA_Flash modules vs the same module math done with the oracle."""
    torch.manual_seed(0)
    x = torch.randn(2, 256, 512).half()
    for mod, hq, hkv in ((miniattn.GQA_Flash(512, 8, 2), 8, 2), (miniattn.MQA_Flash(512, 4), 4, 1)):
        mod = mod.half()
        y = mod.to(DEV)(x.to(DEV)).float().cpu()
        mod = mod.cpu().float()
        xf = x.float()
        dh = 512 // hq
        q = mod.w_q(xf).view(2, 256, hq, dh).transpose(1, 2)
        kvp = (mod.kv if hasattr(mod, "kv") else mod.k_v)(xf).view(2, 256, 2, hkv, dh)
        kk, vv = kvp[:, :, 0].transpose(1, 2), kvp[:, :, 1].transpose(1, 2)
        o = attention_reference(q.half(), kk.half(), vv.half(), causal=True, out_dtype=torch.float32)
        y_ref = mod.w_o(o.transpose(1, 2).reshape(2, 256, 512))
        assert maxerr(y, y_ref.detach()) <= 2e-2


def test_mha_module_against_reference_module():
    """MHA through the module, against what the reference's own MHA module returned for the same
    parameters and input (fixture written by tests/golden/make_golden.py): both return values,
    no mask / lower-triangular mask / all-ones mask; any other mask raises."""
    g = load_golden("mha_module")
    mha = miniattn.MHA(128, 2)
    mha.load_state_dict({k.replace("__", "."): v for k, v in g.items() if k.startswith("w_")})
    mha = mha.half().to(DEV)
    x = g["x"].half().to(DEV)
    S = x.shape[1]
    tril = torch.tril(torch.ones(S, S, device=DEV))
    for tag, mask in (("full", None), ("masked", tril), ("full", torch.ones(S, S, device=DEV))):
        y, w = mha(x, mask=mask)   # the reference's arity: `output, weights = mha(x)`
        assert y.shape == (1, S, 128) and w.shape == (1, 2, S, S) and w.dtype == x.dtype
        # fp16 activations and projections against the fp32 module
        assert maxerr(y.cpu(), g[f"y_{tag}"]) <= 1e-2
        assert maxerr(w.cpu(), g[f"weights_{tag}"]) <= 2e-3
    y, w = miniattn.MHA(128, 2, need_weights=False).half().to(DEV)(x)
    assert w is None and y.shape == (1, S, 128)
    with pytest.raises(RuntimeError, match="no eager path"):
        mha(x, mask=torch.triu(torch.ones(S, S, device=DEV)))
    assert miniattn.device_status(DEV) == 0


def test_host_buffer_pipeline():
    """flash_attn_fwd_host: pinned host tensors in and out, chunked copies overlapped with compute."""
    q, k, v = make_inputs(2, 8, 2, 512, 512, 128, torch.float16, seed=21)
    ref = attention_reference(q, k, v, causal=True, out_dtype=torch.float32)
    qh, kh, vh = q.pin_memory(), k.pin_memory(), v.pin_memory()
    for _ in range(2):  # second call reuses the cached pipeline
        out = miniattn.flash_attn_fwd_host(qh, kh, vh, causal=True, n_chunks=3)
        torch.cuda.synchronize()
        assert not out.is_cuda and maxerr(out, ref) <= TOL[torch.float16]
    with pytest.raises(RuntimeError, match="pinned"):
        miniattn.flash_attn_fwd_host(q, kh, vh)


def test_random_shapes_against_oracle():
    """Seeded sweep over shapes, head groupings, offsets and dtypes (both kernels)."""
    g = torch.Generator().manual_seed(2024)

    def ri(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=g).item())

    for case in range(36):
        D = (64, 128)[ri(0, 1)]
        dtype = (torch.float16, torch.bfloat16)[ri(0, 1)]
        Hkv = ri(1, 3)
        Hq = Hkv * ri(1, 3)
        B = ri(1, 2)
        Nq, Nk = ri(1, 700), ri(1, 900)
        causal = bool(ri(0, 1))
        q_pos0, k_pos0 = (ri(0, 300), ri(0, 300)) if causal and ri(0, 1) else (0, 0)
        scale = None if ri(0, 1) else 0.02 * ri(1, 8)
        q, k, v = make_inputs(B, Hq, Hkv, Nq, Nk, D, dtype, seed=1000 + case)
        ref = attention_reference(q, k, v, causal=causal, softmax_scale=scale, q_pos0=q_pos0, k_pos0=k_pos0,
                                  out_dtype=torch.float32)
        for kernel in KERNELS:
            out = run(q, k, v, causal=causal, softmax_scale=scale, q_pos0=q_pos0, k_pos0=k_pos0, kernel=kernel)
            # with very few keys the outputs are as large as single V rows (|x| up to ~4), so the
            # bound scales with the magnitude: TOL for |ref| <= 1, relative TOL above
            bad = (out.float() - ref).abs() > TOL[dtype] * ref.abs().clamp_min(1.0)
            assert not bool(bad.any()), (case, kernel, B, Hq, Hkv, Nq, Nk, D, causal, q_pos0, k_pos0)


def test_last_wave_single_tile_ctas():
    """160 tile pairs on 148 SMs: the 12 pairs of the last wave run as 24 single-tile CTAs."""
    q, k, v = make_inputs(1, 10, 5, 4096, 1024, 128, torch.float16, seed=77)
    rows = torch.randint(0, 4096, (80,), generator=torch.Generator().manual_seed(7)).unique()
    for causal in (False, True):
        ref = attention_reference_rows(q, k, v, rows, causal=causal)
        out = run(q, k, v, causal=causal, kernel="ws")
        simple = run(q, k, v, causal=causal, kernel="simple")
        if causal:  # rows past the last key see every key; the row oracle masks with kj > row already
            pass
        assert maxerr(out[:, :, rows], ref) <= TOL[torch.float16]
        assert maxerr(out, simple) <= TOL[torch.float16]


@pytest.mark.parametrize("causal", [False, True])
def test_one_wave_single_tile_ctas(causal):
    """32 tile pairs for 148 SMs (config 2 at N = 512): a launch of less than half a wave runs every
    pair as two single-tile CTAs; with a carried state the second tile's CTA finds its own rows."""
    q, k, v = make_inputs(2, 8, 8, 512, 512, 128, torch.float16, seed=12)
    ref = attention_reference(q, k, v, causal=causal, out_dtype=torch.float32)
    out = run(q, k, v, causal=causal, kernel="ws")
    assert maxerr(out, ref) <= TOL[torch.float16]
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    state = miniattn.carry_state(qd)
    miniattn.flash_attn_fwd(qd, kd[:, :, :256], vd[:, :, :256], causal=causal, carry=state, carry_out=True)
    out2 = miniattn.flash_attn_fwd(qd, kd[:, :, 256:], vd[:, :, 256:], causal=causal, k_pos0=256, carry=state,
                                   carry_in=True)
    assert miniattn.device_status(DEV) == 0
    assert maxerr(out2.cpu(), ref) <= TOL[torch.float16]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("causal", [False, True])
def test_head_dim_96(dtype, kernel, causal):
    """D = 96 (the reference instantiates D = 128 only, flash_attention.cu:77-80): ragged lengths,
    GQA, both kernels, against the oracle; scale defaults to 1/sqrt(96)."""
    q, k, v = make_inputs(2, 4, 2, 333, 200 if not causal else 333, 96, dtype, seed=96)
    ref, ref_lse = attention_reference(q, k, v, causal=causal, return_lse=True, out_dtype=torch.float32)
    out, lse = run(q, k, v, causal=causal, kernel=kernel, return_lse=True)
    assert out.shape == q.shape and maxerr(out, ref) <= TOL[dtype]
    assert maxerr(lse, ref_lse) <= 2e-3
    # (B,N,H,D) layout: token stride 4*96 elements
    qb, kb, vb = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    outb = run(qb, kb, vb, causal=causal, kernel=kernel, layout="bnhd")
    assert maxerr(outb.transpose(1, 2), ref) <= TOL[dtype]


def test_head_dim_96_balanced_launch():
    """A D = 96 launch the planner cuts (few long items): partials and merge run at the kernel's
    padded head dim."""
    q, k, v = make_inputs(1, 1, 1, 4096, 4096, 96, torch.float16, seed=97)
    rows = torch.tensor([0, 1, 127, 128, 2047, 2048, 4000, 4095])
    ref = attention_reference_rows(q, k, v, rows, causal=True)
    out = run(q, k, v, causal=True)
    assert maxerr(out[:, :, rows], ref) <= TOL[torch.float16]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 96, 128])
def test_carried_state_chain(dtype, D):
    """Key blocks fed one call at a time with the rows' running state carried in the library's
    buffer (carry_out / carry_in): equals the single call over all keys, and the oracle.  Ragged
    block sizes, GQA, a causal diagonal that hides the later blocks from the early rows."""
    q, k, v = make_inputs(1, 4, 2, 300, 700, D, dtype, seed=31 + D)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    for causal, q_pos0 in ((False, 0), (True, 100)):
        ref, ref_lse = attention_reference(q, k, v, causal=causal, q_pos0=q_pos0, return_lse=True,
                                           out_dtype=torch.float32)
        single = miniattn.flash_attn_fwd(qd, kd, vd, causal=causal, q_pos0=q_pos0)
        state = miniattn.carry_state(qd)
        cuts = [0, 128, 391, 700]   # key blocks [0,128) [128,391) [391,700)
        res = None
        for i in range(3):
            kb, vb = kd[:, :, cuts[i]:cuts[i + 1]], vd[:, :, cuts[i]:cuts[i + 1]]
            res = miniattn.flash_attn_fwd(qd, kb, vb, causal=causal, q_pos0=q_pos0, k_pos0=cuts[i],
                                          carry=state, carry_in=i > 0, carry_out=i < 2, return_lse=i == 2)
            assert (res is None) == (i < 2)
        out, lse = res
        assert miniattn.device_status(DEV) == 0
        assert maxerr(out.cpu(), ref) <= TOL[dtype]
        assert maxerr(out, single) <= (5e-4 if dtype == torch.float16 else 4e-3)
        assert maxerr(lse.cpu(), ref_lse) <= 2e-3


def test_carried_state_rows_without_keys():
    """A chain whose first block is entirely in the rows' future (state = nothing seen yet) and a
    chain that ends on such a block: rows keep what the other blocks gave them."""
    q, k, v = make_inputs(1, 2, 2, 256, 512, 128, torch.float16, seed=77)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ref = attention_reference(q, k[:, :, :256], v[:, :, :256], causal=True, out_dtype=torch.float32)
    for order in ((1, 0), (0, 1)):   # block 1 = keys 256..511, hidden from every row
        state = miniattn.carry_state(qd)
        out = None
        for i, blk in enumerate(order):
            out = miniattn.flash_attn_fwd(qd, kd[:, :, 256 * blk:256 * blk + 256], vd[:, :, 256 * blk:256 * blk + 256],
                                          causal=True, k_pos0=256 * blk, carry=state, carry_in=i > 0, carry_out=i < 1)
        assert maxerr(out.cpu(), ref) <= TOL[torch.float16]
    assert miniattn.device_status(DEV) == 0


def test_carried_state_on_a_row_range():
    """A state buffer made for 512 query rows serves calls on rows [0,256), [256,512) and on all of
    them (carry_rows): what the ring launcher does with its two resident blocks."""
    q, k, v = make_inputs(1, 2, 2, 512, 768, 128, torch.float16, seed=41)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ref = attention_reference(q, k, v, out_dtype=torch.float32)
    state = miniattn.carry_state(qd)
    lo, hi = qd[:, :, :256], qd[:, :, 256:]
    k0, v0, k1, v1, k2, v2 = kd[:, :, :256], vd[:, :, :256], kd[:, :, 256:512], vd[:, :, 256:512], kd[:, :, 512:], vd[:, :, 512:]
    miniattn.flash_attn_fwd(lo, k0, v0, carry=state, carry_out=True, carry_rows=(0, 512))
    miniattn.flash_attn_fwd(hi, k0, v0, carry=state, carry_out=True, carry_rows=(256, 512))
    miniattn.flash_attn_fwd(qd, k1, v1, carry=state, carry_in=True, carry_out=True, carry_rows=(0, 512))  # both halves at once
    out = torch.empty_like(qd)
    miniattn.flash_attn_fwd(lo, k2, v2, carry=state, carry_in=True, out=out[:, :, :256], carry_rows=(0, 512))
    miniattn.flash_attn_fwd(hi, k2, v2, carry=state, carry_in=True, out=out[:, :, 256:], carry_rows=(256, 512))
    assert miniattn.device_status(DEV) == 0
    assert maxerr(out.cpu(), ref) <= TOL[torch.float16]
    with pytest.raises(RuntimeError, match="multiple of 128"):
        miniattn.flash_attn_fwd(qd[:, :, 100:356], k0, v0, carry=state, carry_out=True, carry_rows=(100, 512))


def test_repeated_calls_reuse_the_parameter_block_safely():
    """The operator caches the parameter block of a call by pointers, shapes, strides and flags.
    Calls that hit the cache must still return fresh outputs, honour changed flags, and see new
    values written into the same input tensors."""
    q, k, v = make_inputs(1, 2, 2, 256, 256, 128, torch.float16, seed=61)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ref = attention_reference(q, k, v, out_dtype=torch.float32)
    ref_c = attention_reference(q, k, v, causal=True, out_dtype=torch.float32)
    a = miniattn.flash_attn_fwd(qd, kd, vd)
    b = miniattn.flash_attn_fwd(qd, kd, vd)                       # cache hit, no `out` given
    assert a.data_ptr() != b.data_ptr() and torch.equal(a, b)
    c = miniattn.flash_attn_fwd(qd, kd, vd, causal=True)          # same tensors, other flag
    o2, lse2 = miniattn.flash_attn_fwd(qd, kd, vd, return_lse=True)
    o3, lse3 = miniattn.flash_attn_fwd(qd, kd, vd, return_lse=True)   # fresh lse per call
    assert lse2.data_ptr() != lse3.data_ptr() and torch.equal(lse2, lse3)
    assert maxerr(a.cpu(), ref) <= TOL[torch.float16] and maxerr(c.cpu(), ref_c) <= TOL[torch.float16]
    assert maxerr(o3.cpu(), ref) <= TOL[torch.float16]
    # new values in the same storage
    q2, _, _ = make_inputs(1, 2, 2, 256, 256, 128, torch.float16, seed=62)
    qd.copy_(q2)
    d = miniattn.flash_attn_fwd(qd, kd, vd)
    assert maxerr(d.cpu(), attention_reference(q2, k, v, out_dtype=torch.float32)) <= TOL[torch.float16]
    # a caller-provided output is written in place, every time
    out = torch.zeros_like(qd)
    for _ in range(2):
        out.zero_()
        assert miniattn.flash_attn_fwd(qd, kd, vd, out=out) is out
        assert maxerr(out, d) == 0
    # a view with the same base pointer but other strides is another problem
    wide = torch.randn(1, 4, 256, 128, dtype=torch.float16, device=DEV)
    e = miniattn.flash_attn_fwd(wide[:, :2], kd, vd)
    f = miniattn.flash_attn_fwd(wide[:, ::2], kd, vd)
    assert maxerr(e.cpu(), attention_reference(wide[:, :2].cpu(), k, v, out_dtype=torch.float32)) <= TOL[torch.float16]
    assert maxerr(f.cpu(), attention_reference(wide[:, ::2].cpu(), k, v, out_dtype=torch.float32)) <= TOL[torch.float16]
    with pytest.raises(RuntimeError, match="same data type"):
        miniattn.flash_attn_fwd(qd, kd.bfloat16(), vd)
    miniattn.check_device_status(DEV)   # raises if any bounded wait ran out
