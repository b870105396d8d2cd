"""Merge kernel and launchers on one GPU: the merge kernel against the oracle's merge, the ring
driver with all ranks emulated on the device (same schedule, kernels and merges as the
multi-process ring, no communication) and shard mode run rank after rank."""
import pytest
import torch

import miniattn
from miniattn import parallel as par
from conftest import TOL
from oracle.attention_oracle import attention_reference, attention_reference_rows, make_inputs, merge_partials

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
def test_merge_kernel_matches_oracle(dtype, D):
    g = torch.Generator().manual_seed(D)
    rows = (3, 5, 77)  # 1155 rows: not a multiple of the rows per block
    acc_o = torch.randn(*rows, D, generator=g)
    acc_lse = torch.randn(*rows, generator=g) * 4
    part_o = torch.randn(*rows, D, generator=g).to(dtype)
    part_lse = torch.randn(*rows, generator=g) * 4
    acc_lse[0, 0, :5] = float("-inf")      # empty running result
    part_lse[0, 1, :5] = float("-inf")     # empty partial
    acc_lse[0, 2, :5] = float("-inf")
    part_lse[0, 2, :5] = float("-inf")     # both empty -> zeros, -inf
    ref_o, ref_lse = merge_partials(acc_o, acc_lse, part_o, part_lse)
    a_o, a_l = acc_o.to(DEV), acc_lse.to(DEV)
    out = torch.empty(*rows, D, dtype=dtype, device=DEV)
    miniattn.merge_partials(a_o, a_l, part_o.to(DEV), part_lse.to(DEV), out=out)
    assert (a_o.cpu() - ref_o).abs().max().item() < 1e-5
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(a_l.cpu()), fin)
    assert (a_l.cpu()[fin] - ref_lse[fin]).abs().max().item() < 1e-5
    # `out` is the merged value rounded to the 16-bit dtype: within one rounding step of it
    rel = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert bool(((out.float().cpu() - ref_o).abs() <= rel * ref_o.abs().clamp_min(1.0)).all())
    # init=True overwrites the accumulators with the partial
    miniattn.merge_partials(a_o, a_l, part_o.to(DEV), part_lse.to(DEV), init=True)
    assert torch.equal(a_o.cpu(), part_o.float()) and torch.equal(a_l.cpu(), part_lse)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ring_emulated_on_gpu_scaled_down_config5(world):
    """Config 5 scaled to N=8192 (B=1, H=4, D=128, fp16, causal): the ring result must agree
    with the single-launch kernel and with the exact oracle on sampled rows."""
    N = 8192
    q, k, v = make_inputs(1, 4, 4, N, N, 128, torch.float16, seed=5)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = par.ring_forward_emulated(qd, kd, vd, world, causal=True).cpu()
    single = miniattn.flash_attn_fwd(qd, kd, vd, causal=True).cpu()
    assert miniattn.device_status(DEV) == 0
    assert (out.float() - single.float()).abs().max().item() <= TOL[torch.float16]
    L = N // (2 * world)
    rows = torch.tensor(sorted({0, 1, L - 1, L, L + 1, N // 2 - 1, N // 2, N - L - 1, N - L, N - 1}
                               | set(torch.randint(0, N, (64,), generator=torch.Generator().manual_seed(world)).tolist())))
    ref = attention_reference_rows(q, k, v, rows, causal=True)
    assert (out[:, :, rows].float() - ref).abs().max().item() <= TOL[torch.float16]


def test_ring_emulated_non_causal_bf16_gqa():
    q, k, v = make_inputs(1, 4, 2, 2048, 2048, 64, torch.bfloat16, seed=8)
    out = par.ring_forward_emulated(q.to(DEV), k.to(DEV), v.to(DEV), 4, causal=False).cpu()
    ref = attention_reference(q, k, v, out_dtype=torch.float32)
    assert (out.float() - ref).abs().max().item() <= TOL[torch.bfloat16]


def test_shard_mode_rank_by_rank():
    q, k, v = make_inputs(2, 8, 2, 512, 512, 128, torch.bfloat16, seed=2)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.zeros_like(qd)
    for r in range(4):
        par.sharded_forward(qd, kd, vd, causal=True, rank=r, world=4, out=out)
    ref = attention_reference(q, k, v, causal=True, out_dtype=torch.float32)
    assert (out.float().cpu() - ref).abs().max().item() <= TOL[torch.bfloat16]
