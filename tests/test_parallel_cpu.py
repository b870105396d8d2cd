"""Host-side logic of the multi-GPU launchers, on CPU: shard partition, ring schedule, and the
ring driver itself run (a) with all ranks emulated in one process and (b) as two real gloo ranks
exchanging K/V pairs, with the CPU oracle standing in for the CUDA kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from miniattn import parallel as par
from oracle.attention_oracle import attention_reference, make_inputs, merge_partials


def cpu_attn(q, k, v, causal, q_pos0, k_pos0, softmax_scale):
    return attention_reference(q, k, v, causal=causal, q_pos0=q_pos0, k_pos0=k_pos0,
                               softmax_scale=softmax_scale, return_lse=True)


class CpuAccumulator:
    def __init__(self, like):
        self.o = None
        self.lse = None

    def add(self, o, lse, out=None):
        if self.o is None:
            self.o, self.lse = o.float(), lse.clone()
        else:
            self.o, self.lse = merge_partials(self.o, self.lse, o, lse)
        if out is not None:
            out.copy_(self.o.to(out.dtype))


@pytest.mark.parametrize("B,Hkv,world", [(4, 8, 8), (4, 8, 4), (2, 3, 4), (1, 1, 2), (3, 5, 7)])
def test_shard_partition_is_exact(B, Hkv, world):
    seen = []
    sizes = []
    for r in range(world):
        units = par.shard_units(B, Hkv, world, r)
        sizes.append(len(units))
        seen += units
        # the grouped form covers the same units
        flat = [(b, h) for b, h0, h1 in par.shard_slices(B, Hkv, world, r) for h in range(h0, h1)]
        assert flat == units
    assert sorted(seen) == [(b, h) for b in range(B) for h in range(Hkv)]
    assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ring_schedule_covers_causal_pairs_once_and_is_balanced(world):
    for r in range(world):
        pairs = []
        for s in range(world):
            tasks = par.ring_step_tasks(r, world, s, causal=True)
            weight = sum(0.5 if t.causal else 1.0 for t in tasks)
            assert weight == 2.0 or (s == 0 and weight == 2.0)  # two block-pairs of work every step
            pairs += [(t.q_block, t.kv_block, t.causal) for t in tasks]
        owned = par.ring_owner_blocks(r, world)
        want = [(qb, kb, kb == qb) for qb in owned for kb in range(2 * world) if kb <= qb]
        assert sorted(pairs) == sorted(want)
    # non-causal: every (owned q block, kv block) pair exactly once
    pairs = [(t.q_block, t.kv_block) for s in range(world) for t in par.ring_step_tasks(0, world, s, causal=False)]
    assert sorted(pairs) == [(qb, kb) for qb in sorted(par.ring_owner_blocks(0, world)) for kb in range(2 * world)]


def test_zigzag_roundtrip():
    x = torch.arange(2 * 3 * 16 * 4).view(2, 3, 16, 4)
    for world in (1, 2, 4):
        assert torch.equal(par.zigzag_merge(par.zigzag_split(x, world)), x)


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("causal", [True, False])
def test_ring_emulated_matches_full_attention(world, causal):
    q, k, v = make_inputs(1, 2, 2, 64, 64, 16, torch.float32, seed=world)
    ref = attention_reference(q, k, v, causal=causal)
    out = par.ring_forward_emulated(q, k, v, world, causal=causal, attn_fn=cpu_attn, accumulator=CpuAccumulator)
    assert (out - ref).abs().max().item() < 1e-5


def test_sharded_forward_cpu():
    q, k, v = make_inputs(2, 6, 3, 32, 32, 16, torch.float32, seed=3)
    ref = attention_reference(q, k, v, causal=True)

    def attn(q, k, v, causal, softmax_scale, out):
        out.copy_(attention_reference(q, k, v, causal=causal, softmax_scale=softmax_scale))

    out = torch.zeros_like(q)
    for r in range(4):
        par.sharded_forward(q, k, v, causal=True, rank=r, world=4, attn_fn=attn, out=out)
    assert (out - ref).abs().max().item() < 1e-6


def test_merge_is_associative_and_handles_empty_partials():
    g = torch.Generator().manual_seed(0)
    o = [torch.randn(5, 8, generator=g) for _ in range(3)]
    l = [torch.randn(5, generator=g) * 3 for _ in range(3)]
    l[1][2] = float("-inf")  # an empty partial for one row
    a, la = merge_partials(*merge_partials(o[0], l[0], o[1], l[1]), o[2], l[2])
    b, lb = merge_partials(o[0], l[0], *merge_partials(o[1], l[1], o[2], l[2]))
    assert (a - b).abs().max().item() < 1e-6 and (la - lb).abs().max().item() < 1e-6
    e, le = merge_partials(o[0], torch.full((5,), float("-inf")), o[1], torch.full((5,), float("-inf")))
    assert torch.all(e == 0) and torch.all(torch.isinf(le))


# ---------------------------------------------------------------- two real ranks over gloo
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ring_worker(rank, world, port, causal, fault, result_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = make_inputs(1, 2, 2, 96, 96, 16, torch.float32, seed=11)
        ref = attention_reference(q, k, v, causal=causal)
        qs, ks, vs = (par.zigzag_split(t, world) for t in (q, k, v))
        exchange = None
        if fault == "repeat":  # a hop that delivers the pair the rank already holds
            def exchange(kc, vc, kr, vr):
                kr.copy_(kc)
                vr.copy_(vc)

                class H:
                    def wait(self):
                        return None

                    def origin(self):
                        return rank

                return H()
        try:
            out = par.ring_forward(qs[rank], ks[rank], vs[rank], causal=causal, rank=rank, world=world,
                                   attn_fn=cpu_attn, accumulator=CpuAccumulator, exchange=exchange,
                                   verify_origin=True)
            err = (out - par.zigzag_split(ref, world)[rank]).abs().max().item()
            result_q.put((rank, "ok", err))
        except RuntimeError as e:
            result_q.put((rank, "error", str(e)))
    finally:
        dist.destroy_process_group()


def _run_ring(world, causal, fault=None):
    ctx = mp.get_context("spawn")
    result_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ring_worker, args=(r, world, port, causal, fault, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [result_q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results)


@pytest.mark.parametrize("causal", [True, False])
def test_ring_two_gloo_ranks(causal):
    for rank, status, err in _run_ring(2, causal):
        assert status == "ok" and err < 1e-5, (rank, status, err)


def test_ring_detects_a_repeated_hop():
    """Failure injected on the host: the exchange hands back the pair the rank already holds;
    the origin check must refuse it instead of silently merging the same keys twice."""
    for rank, status, msg in _run_ring(2, True, fault="repeat"):
        assert status == "error" and "expected rank" in msg


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("merge", [True, False])
def test_ring_launch_plan_covers_every_block_pair_once(world, causal, merge):
    """The carried-state launch plan of every rank: each (Q block, K/V block) pair of the schedule is
    covered by exactly one launch; a block's first launch has no state to read, all later ones do;
    exactly the last launch of a block writes its output; merged launches are unmasked rectangles."""
    n_launches = {True: 0, False: 0}
    for rank in range(world):
        remaining, started = [0, 0], [False, False]
        for s in range(world):
            for t in par.ring_step_tasks(rank, world, s, causal):
                remaining[t.q_half] += 1
        covered = []
        finished = [False, False]
        for s in range(world):
            tasks = par.ring_step_tasks(rank, world, s, causal)
            was_started = list(started)
            launches = par.ring_step_launches(tasks, remaining, started, merge)
            n_launches[merge] += len(launches)
            seen_in_step = [False, False]
            for ln in launches:
                if len(ln.q_halves) * len(ln.kv_halves) > 1:
                    assert merge and not ln.causal
                for qh in ln.q_halves:
                    assert not finished[qh], "a block was written out and then touched again"
                    assert ln.carry_in == (was_started[qh] or seen_in_step[qh])
                    for kh in ln.kv_halves:
                        covered.append((qh, s, kh))
                for qh in ln.q_halves:
                    seen_in_step[qh] = True
                    if ln.last:
                        finished[qh] = True
            want_step = sorted((t.q_half, s, t.kv_half) for t in tasks)
            assert sorted(c for c in covered if c[1] == s) == want_step
        assert remaining == [0, 0] and finished == [True, True]
    if merge and world > 1:
        # per rank: three launches in the first step, then one per step, plus one where the early
        # block ends before the late one (against 2 * world + 1 without merging)
        assert n_launches[True] <= (world + 3) * world
        if causal and world >= 4:
            assert n_launches[True] < (2 * world + 1) * world
