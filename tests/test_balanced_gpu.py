"""Balanced launches (miniattn_fwd_balanced): the key range of some work items is cut over several
CTAs whose partial results the last-arriving CTA merges.  Parity with the oracle and with the
plain launch, through the Python operator and through the C ABI with caller-provided scratch."""
import ctypes as C

import pytest
import torch

import miniattn
from miniattn import _lib
from miniattn.ops import _balance_scratch, _prepare, plan_info
from conftest import TOL
from oracle.attention_oracle import attention_reference, make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = [
    # B, Hq, Hkv, Nq, Nk, D, dtype, causal
    (1, 2, 2, 512, 512, 128, torch.float16, False),
    (1, 4, 4, 2048, 2048, 128, torch.float16, False),       # every item cut in two
    (2, 8, 8, 1024, 1024, 128, torch.float16, False),       # short items: the planner leaves them whole
    (1, 4, 2, 1000, 1300, 128, torch.bfloat16, True),       # ragged, GQA, pieces past a row's diagonal
    (1, 4, 4, 2048, 2048, 64, torch.float16, False),
    (1, 3, 1, 640, 3000, 64, torch.bfloat16, True),
    (1, 1, 1, 4096, 4096, 128, torch.float16, False),       # many pieces per item
    (1, 4, 4, 4096, 4096, 128, torch.float16, True),
    (2, 8, 8, 4096, 4096, 128, torch.float16, False),       # headline shape: whole round + pieces
]


def sms():
    return torch.cuda.get_device_properties(0).multi_processor_count


@pytest.mark.parametrize("case", CASES)
def test_balanced_matches_oracle_and_plain_launch(case):
    B, Hq, Hkv, Nq, Nk, D, dtype, causal = case
    q, k, v = make_inputs(B, Hq, Hkv, Nq, Nk, D, dtype, seed=77)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    info, _ = plan_info(B, Hq, Nq, Nk, D, causal=causal, sm_count=sms())
    plain, lse_p = miniattn.flash_attn_fwd(qd, kd, vd, causal=causal, return_lse=True, balance=False)
    for _ in range(2):  # the second launch finds the arrival counters as the first left them
        bal, lse_b = miniattn.flash_attn_fwd(qd, kd, vd, causal=causal, return_lse=True, balance=True)
    torch.cuda.synchronize()
    assert miniattn.device_status(DEV) == 0
    ref = attention_reference(q, k, v, causal=causal, out_dtype=torch.float32)
    assert (bal.float().cpu() - ref).abs().max().item() <= TOL[dtype]
    # same arithmetic up to the order of fp32 sums and one more rounding of the weights
    assert (bal.float() - plain.float()).abs().max().item() <= (5e-4 if dtype == torch.float16 else 4e-3)
    fin = torch.isfinite(lse_p)
    assert bool((torch.isfinite(lse_b) == fin).all())
    assert (lse_b[fin] - lse_p[fin]).abs().max().item() <= 1e-5
    if info.split:
        for t in _balance_scratch.values():
            assert int(t[:16384].view(torch.int32).abs().sum().item()) == 0, "arrival counters must be left zero"


def test_headline_shapes_take_the_balanced_path():
    """The probe shapes must exercise the cut-item path on this GPU, not fall back to the plain launch."""
    n = sms()
    assert plan_info(2, 8, 4096, 4096, sm_count=n)[0].split == 1
    assert plan_info(1, 1, 4096, 4096, sm_count=n)[0].n_cut_items > 0


def test_c_abi_scratch_contract():
    q, k, v = make_inputs(1, 4, 4, 2048, 2048, 128, torch.float16, seed=5)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    p, out, _ = _prepare(qd, kd, vd, False, None, "bhnd", False, None, "auto", 0, 0)
    need = _lib.lib.miniattn_fwd_balanced_scratch_bytes(C.byref(p))
    assert need > 16384
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    small = torch.zeros(need - 256, dtype=torch.uint8, device=DEV)
    rc = _lib.lib.miniattn_fwd_balanced(C.byref(p), C.c_void_p(small.data_ptr()), C.c_size_t(small.numel()), stream)
    assert rc == _lib.EINVAL and "scratch" in _lib.last_error()
    buf = torch.zeros(need + 256, dtype=torch.uint8, device=DEV)
    rc = _lib.lib.miniattn_fwd_balanced(C.byref(p), C.c_void_p(buf.data_ptr() + 16), C.c_size_t(need), stream)
    assert rc == _lib.EINVAL and "aligned" in _lib.last_error()
    rc = _lib.lib.miniattn_fwd_balanced(C.byref(p), C.c_void_p(buf.data_ptr()), C.c_size_t(buf.numel()), stream)
    assert rc == _lib.OK
    ref = attention_reference(q, k, v, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert (out.float().cpu() - ref).abs().max().item() <= TOL[torch.float16]
    # scratch == NULL: the plain launch
    out.zero_()
    rc = _lib.lib.miniattn_fwd_balanced(C.byref(p), None, C.c_size_t(0), stream)
    assert rc == _lib.OK
    torch.cuda.synchronize()
    assert (out.float().cpu() - ref).abs().max().item() <= TOL[torch.float16]
    assert miniattn.device_status(DEV) == 0


def test_repeated_balanced_launches_stay_one_rounding_from_the_plain_launch():
    """Which piece of a cut item arrives last varies from launch to launch (other work on the GPU,
    clocks), so the fp32 merge order does too; a missing fence or a stale counter would show up as
    an occasional large error.  200 launches with a second stream busy beside them."""
    q, k, v = make_inputs(1, 4, 4, 2048, 2048, 128, torch.float16, seed=9)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    assert plan_info(1, 4, 2048, 2048, 128, sm_count=sms())[0].n_cut_items > 0
    plain, lse_p = miniattn.flash_attn_fwd(qd, kd, vd, return_lse=True, balance=False)
    side = torch.cuda.Stream()
    worst = worst_lse = 0.0
    for i in range(200):
        if i % 3 == 2:
            with torch.cuda.stream(side):
                miniattn.flash_attn_fwd(qd[:, :1, :512], kd[:, :1, :512], vd[:, :1, :512], balance=False)
        o, lse = miniattn.flash_attn_fwd(qd, kd, vd, return_lse=True, balance=True)
        worst = max(worst, (o.float() - plain.float()).abs().max().item())
        worst_lse = max(worst_lse, (lse - lse_p).abs().max().item())
    torch.cuda.synchronize()
    assert miniattn.device_status(DEV) == 0
    assert worst <= 5e-4 and worst_lse <= 1e-5


@pytest.mark.parametrize("causal", [False, True])
def test_head_groups_when_k_and_v_outgrow_l2(causal):
    """8 heads x 16384 keys x D=128: 67 MB of K and V, so the work items walk the heads in groups
    (a share of L2 each) instead of all at once.  Plain and balanced launches against the kernel
    that has its own, fixed order and against the exact oracle on sampled rows."""
    from oracle.attention_oracle import attention_reference_rows
    B, H, N, D = 1, 8, 16384, 128
    info, _ = plan_info(B, H, N, N, D, causal=causal, sm_count=sms())
    assert 0 < info.head_group < B * H and (B * H) % info.head_group == 0
    q, k, v = make_inputs(B, H, H, N, N, D, torch.float16, seed=3)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    simple = miniattn.flash_attn_fwd(qd, kd, vd, causal=causal, kernel="simple")
    plain = miniattn.flash_attn_fwd(qd, kd, vd, causal=causal, balance=False)
    bal = miniattn.flash_attn_fwd(qd, kd, vd, causal=causal, balance=True)
    assert miniattn.device_status(DEV) == 0
    assert (plain.float() - simple.float()).abs().max().item() <= TOL[torch.float16]
    assert (bal.float() - plain.float()).abs().max().item() <= 5e-4
    rows = torch.tensor([0, 1, 127, 128, 255, 256, N // 2 - 1, N // 2, N - 257, N - 256, N - 129, N - 1])
    ref = attention_reference_rows(q, k, v, rows, causal=causal)
    assert (bal[:, :, rows.to(DEV)].float().cpu() - ref).abs().max().item() <= TOL[torch.float16]
