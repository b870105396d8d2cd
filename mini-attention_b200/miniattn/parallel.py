"""Multi-GPU launchers for the attention forward path (one process per GPU, torch.distributed).

The reference has no multi-GPU code; these launchers add the two modes the path shards into:

* **shard mode** — (batch x KV-head group) units are independent, so they are split across the
  ranks with no communication.  A unit is one KV head of one batch element together with the
  G = Hq/Hkv query heads it serves (kernels/standard/pytorch/gqa.py:38-39), so K/V are never
  duplicated.
* **ring (context-parallel) mode** — for sequences too long for one device.  The sequence is cut
  into 2*W blocks; rank r owns query/key/value blocks r and 2W-1-r ("zig-zag"), which balances
  causal work.  The K/V pair of each rank travels round the ring (send to r+1, receive from r-1)
  while the attention of the resident Q blocks against the visiting pair runs.  The rows' running
  (maximum, sum, un-normalised O) are carried from one attention launch to the next inside the
  kernel's epilogue (the split-KV merge of
  kernels/standard/pytorch/benchmark_mla_decode_torch.py:244-272, kept un-normalised until the
  last step), so a step is one launch per (Q block, K/V block) pair and nothing is rounded to
  16 bit on the way.  The two-launch form (normalised partial + log-sum-exp, merged by
  ``miniattn_merge_partials``) stays available: ``fused=False``.

The schedule functions are pure Python and are exercised on CPU ranks (gloo) in the tests; the
attention and merge callables are injectable so that the same driver runs on the CUDA kernels
(default) or, in tests, on a CPU stand-in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- shard mode
def shard_units(batch: int, n_kv_heads: int, world: int, rank: int) -> List[Tuple[int, int]]:
    """(batch index, KV head) units of `rank`: a contiguous, near-equal slice of the B*Hkv units
    (earlier ranks get the extra unit when the count does not divide)."""
    total = batch * n_kv_heads
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return [(u // n_kv_heads, u % n_kv_heads) for u in range(start, start + count)]


def shard_slices(batch: int, n_kv_heads: int, world: int, rank: int) -> List[Tuple[int, int, int]]:
    """The same units grouped per batch element: (batch index, first KV head, one-past-last)."""
    out: List[Tuple[int, int, int]] = []
    for b, hk in shard_units(batch, n_kv_heads, world, rank):
        if out and out[-1][0] == b and out[-1][2] == hk:
            out[-1] = (b, out[-1][1], hk + 1)
        else:
            out.append((b, hk, hk + 1))
    return out


def sharded_forward(q, k, v, *, causal=False, softmax_scale=None, rank=0, world=1, attn_fn=None, out=None):
    """Shard mode on full (B,Hq,N,D)/(B,Hkv,N,D) tensors resident on this rank's device: computes
    only this rank's (batch x KV-head group) units, as strided views (no copies), and writes them
    into `out` (other units are left untouched).  No communication."""
    if attn_fn is None:
        from .ops import flash_attn_fwd as attn_fn
    B, Hq, _, _ = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    if out is None:
        out = torch.empty_like(q)
    for b, h0, h1 in shard_slices(B, Hkv, world, rank):
        attn_fn(q[b:b + 1, h0 * G:h1 * G], k[b:b + 1, h0:h1], v[b:b + 1, h0:h1], causal=causal,
                softmax_scale=softmax_scale, out=out[b:b + 1, h0 * G:h1 * G])
    return out


# --------------------------------------------------------------------------- ring mode
@dataclass(frozen=True)
class RingTask:
    """One attention call of a ring step: resident Q block x visiting K/V block."""

    q_half: int      # 0 = early block (index r), 1 = late block (index 2W-1-r)
    kv_half: int     # 0 = early block of the visiting pair (index src), 1 = late (2W-1-src)
    q_block: int     # global block indices (positions = index * block_len)
    kv_block: int
    causal: bool     # True only on the diagonal (q_block == kv_block)


def ring_owner_blocks(rank: int, world: int) -> Tuple[int, int]:
    return rank, 2 * world - 1 - rank


def ring_step_tasks(rank: int, world: int, step: int, causal: bool = True) -> List[RingTask]:
    """Work of `rank` at ring step `step`, when it holds the K/V pair that started at
    src = (rank - step) mod world.  Causal: a (q block, kv block) pair is skipped when the keys
    lie entirely in the future, runs unmasked when they lie entirely in the past and runs the
    causal kernel on the diagonal.  Every rank gets two block-pairs of work per step (three
    half-weight ones at step 0), which is what keeps the ring balanced."""
    src = (rank - step) % world
    qb = ring_owner_blocks(rank, world)
    kb = ring_owner_blocks(src, world)
    tasks = []
    for qi in (0, 1):
        for ki in (0, 1):
            if not causal:
                tasks.append(RingTask(qi, ki, qb[qi], kb[ki], False))
            elif kb[ki] < qb[qi]:
                tasks.append(RingTask(qi, ki, qb[qi], kb[ki], False))
            elif kb[ki] == qb[qi]:
                tasks.append(RingTask(qi, ki, qb[qi], kb[ki], True))
    return tasks


def zigzag_split(x: torch.Tensor, world: int, dim: int = 2) -> List[torch.Tensor]:
    """Split the token axis into 2W blocks and give rank r blocks (r, 2W-1-r), concatenated."""
    blocks = x.chunk(2 * world, dim=dim)
    return [torch.cat([blocks[r], blocks[2 * world - 1 - r]], dim=dim) for r in range(world)]


def zigzag_merge(parts: Sequence[torch.Tensor], dim: int = 2) -> torch.Tensor:
    """Inverse of :func:`zigzag_split`."""
    world = len(parts)
    blocks: List[Optional[torch.Tensor]] = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = p.chunk(2, dim=dim)
        blocks[r], blocks[2 * world - 1 - r] = a, b
    return torch.cat(blocks, dim=dim)


def _gpu_attn(q, k, v, causal, q_pos0, k_pos0, softmax_scale):
    from .ops import flash_attn_fwd
    return flash_attn_fwd(q, k, v, causal=causal, q_pos0=q_pos0, k_pos0=k_pos0, softmax_scale=softmax_scale,
                          return_lse=True)


class _GpuAccumulator:
    """Running (o fp32, lse) of one resident Q block, merged with miniattn_merge_partials."""

    def __init__(self, like: torch.Tensor):
        self.acc_o = torch.empty(like.shape, dtype=torch.float32, device=like.device)
        self.acc_lse = torch.empty(like.shape[:-1], dtype=torch.float32, device=like.device)
        self.empty = True

    def add(self, o, lse, out=None):
        from .ops import merge_partials
        merge_partials(self.acc_o, self.acc_lse, o.contiguous(), lse, init=self.empty, out=out)
        self.empty = False


def ring_forward(
    q_local: torch.Tensor,
    k_local: torch.Tensor,
    v_local: torch.Tensor,
    *,
    causal: bool = True,
    softmax_scale: Optional[float] = None,
    rank: int = 0,
    world: int = 1,
    group=None,
    attn_fn: Optional[Callable] = None,
    accumulator: Optional[Callable] = None,
    exchange: Optional[Callable] = None,
    verify_origin: bool = False,
    fused: bool = True,
    merge_steps: bool = True,
) -> torch.Tensor:
    """Ring / context-parallel attention of this rank's zig-zag shard.

    q_local, k_local, v_local: (B, H, 2*L, D) — this rank's two blocks (early then late), L =
    N / (2*world).  Returns the attention output for the same rows, in the input dtype.
    `exchange(k, v, k_recv, v_recv)` starts the transfer of the visiting pair to rank+1 and of
    the next pair from rank-1 and returns a handle with ``wait()``; the default uses
    torch.distributed P2P (NCCL send/recv over NVLink) with double-buffered receive buffers, so
    the transfer of step s+1 overlaps the attention of step s.  With ``verify_origin`` the
    handle's ``origin()`` (rank the received pair started from) is compared with the schedule and
    a dropped or repeated hop raises ``RuntimeError`` (host-side check; it synchronises, so it is
    meant for tests and debugging).  ``attn_fn`` / ``accumulator`` replace the CUDA kernels (CPU
    stand-ins in the tests); with neither given and ``fused`` the running state is carried inside
    the attention kernel, otherwise each task yields a partial that the accumulator merges.
    """
    B, H, L2, D = q_local.shape
    L = L2 // 2
    fused = fused and attn_fn is None and accumulator is None
    attn_fn = attn_fn or _gpu_attn
    accumulator = accumulator or _GpuAccumulator
    if exchange is None and world > 1:
        exchange = _dist_exchange(rank, world, group)
    k_cur, v_cur = k_local.contiguous(), v_local.contiguous()
    bufs = [(torch.empty_like(k_cur), torch.empty_like(v_cur)) for _ in range(2 if world > 1 else 0)]
    q_blocks = (q_local[:, :, :L], q_local[:, :, L:])
    out = torch.empty_like(q_local)
    if fused:
        from .ops import carry_state, flash_attn_fwd
        # one state buffer for all 2L local rows; a launch on one block addresses its half of it
        # (needs the late block to start on a tile boundary, else one buffer per block)
        joint = L % 128 == 0
        if joint:
            state_all = carry_state(q_local)
            states = [state_all, state_all]
            rows_of = [(0, L2), (L, L2)]
        else:
            states = [carry_state(q_blocks[0]), carry_state(q_blocks[1])]
            rows_of = [None, None]
        started = [False, False]
    else:
        accs = [accumulator(q_blocks[0]), accumulator(q_blocks[1])]
    outs = (out[:, :, :L], out[:, :, L:])
    # number of partials each resident block will receive, to know which merge is the last one
    remaining = [0, 0]
    for s in range(world):
        for t in ring_step_tasks(rank, world, s, causal):
            remaining[t.q_half] += 1
    for s in range(world):
        handle = None
        if s + 1 < world:
            nk, nv = bufs[s % 2]
            handle = exchange(k_cur, v_cur, nk, nv)
        tasks = ring_step_tasks(rank, world, s, causal)
        if fused:
            # one launch per entry: state in (after a block's first task), state out or, on a block's
            # last task, the finished rows straight into the output
            for ln in ring_step_launches(tasks, remaining, started, joint and merge_steps):
                qh, kh = ln.q_halves, ln.kv_halves
                q_sel = q_local if len(qh) == 2 else q_blocks[qh[0]]
                k_sel = k_cur if len(kh) == 2 else k_cur[:, :, kh[0] * L:(kh[0] + 1) * L]
                v_sel = v_cur if len(kh) == 2 else v_cur[:, :, kh[0] * L:(kh[0] + 1) * L]
                out_sel = out if len(qh) == 2 else outs[qh[0]]
                if len(qh) == 2:
                    state, rows = state_all, (0, L2)
                else:
                    state, rows = states[qh[0]], rows_of[qh[0]]
                flash_attn_fwd(q_sel, k_sel, v_sel, causal=ln.causal, q_pos0=ln.q_block * L, k_pos0=ln.kv_block * L,
                               softmax_scale=softmax_scale, out=out_sel if ln.last else None, carry=state,
                               carry_in=ln.carry_in, carry_out=not ln.last, carry_rows=rows)
            tasks = []
        for t in tasks:
            kb = k_cur[:, :, t.kv_half * L:(t.kv_half + 1) * L]
            vb = v_cur[:, :, t.kv_half * L:(t.kv_half + 1) * L]
            remaining[t.q_half] -= 1
            last = remaining[t.q_half] == 0
            o, lse = attn_fn(q_blocks[t.q_half], kb, vb, t.causal, t.q_block * L, t.kv_block * L, softmax_scale)
            # the last merge of a block writes the finished rows straight into the output
            accs[t.q_half].add(o, lse, out=outs[t.q_half] if last else None)
        if handle is not None:
            handle.wait()
            k_cur, v_cur = bufs[s % 2]
            if verify_origin:
                got, want = handle.origin(), (rank - s - 1) % world
                if got != want:
                    raise RuntimeError(f"ring step {s + 1} on rank {rank}: received the K/V pair of rank {got}, "
                                       f"expected rank {want}")
    return out


@dataclass(frozen=True)
class RingLaunch:
    """One attention launch of a ring step in the carried-state form."""

    q_halves: Tuple[int, ...]    # resident Q blocks covered (0 = early, 1 = late); both = all 2L rows
    kv_halves: Tuple[int, ...]   # blocks of the visiting pair covered; both = all 2L keys
    causal: bool                 # True only for a single diagonal block pair
    q_block: int                 # global block indices of the first covered blocks (positions of a
    kv_block: int                # causal launch; ignored by an unmasked one)
    carry_in: bool               # the covered rows have a state from earlier launches
    last: bool                   # no later launch touches the covered rows: write the output


def ring_step_launches(tasks: Sequence[RingTask], remaining: List[int], started: List[bool],
                       merge: bool) -> List[RingLaunch]:
    """Launches of one ring step, and the bookkeeping that goes with them: `remaining[h]` (tasks
    resident block h still has to receive) and `started[h]` (block h has a state) are updated.
    With `merge` a step whose block pairs are all unmasked and form a full rectangle of
    (Q blocks) x (K/V blocks) — they share their Q block or their K/V block, or, without a mask,
    cover everything — becomes one launch over the contiguous union: half the state round trips
    where the Q block is shared, twice the work per CTA."""
    out: List[RingLaunch] = []
    if merge and _merge_step(tasks, remaining, started):
        qh = tuple(sorted({t.q_half for t in tasks}))
        kh = tuple(sorted({t.kv_half for t in tasks}))
        carry_in = all(started[h] for h in qh)
        for t in tasks:
            remaining[t.q_half] -= 1
        last = all(remaining[h] == 0 for h in qh)
        first = min(tasks, key=lambda t: (t.q_half, t.kv_half))
        out.append(RingLaunch(qh, kh, False, first.q_block, first.kv_block, carry_in, last))
        for h in qh:
            started[h] = True
        return out
    for t in tasks:
        remaining[t.q_half] -= 1
        out.append(RingLaunch((t.q_half,), (t.kv_half,), t.causal, t.q_block, t.kv_block, started[t.q_half],
                              remaining[t.q_half] == 0))
        started[t.q_half] = True
    return out


def _merge_step(tasks: Sequence[RingTask], remaining: Sequence[int], started: Sequence[bool]) -> bool:
    """Can the tasks of one ring step run as a single launch?  They must be unmasked and form a
    full rectangle of (Q blocks) x (K/V blocks); the Q blocks must agree on whether a state exists
    yet and on whether this step is their last."""
    if len(tasks) < 2 or any(t.causal for t in tasks):
        return False
    qh = sorted({t.q_half for t in tasks})
    kh = sorted({t.kv_half for t in tasks})
    if len(tasks) != len(qh) * len(kh):
        return False
    per_q = len(kh)
    if len({started[h] for h in qh}) != 1:
        return False
    return len({remaining[h] == per_q for h in qh}) == 1


def ring_process_group(ranks: Optional[Sequence[int]] = None):
    """A process group for :func:`ring_forward` whose NCCL stream has high priority.

    The attention kernel fills every SM with one CTA and keeps hundreds more queued, so the CTAs of
    a send/recv kernel on an ordinary stream are dispatched only as attention CTAs retire and the
    transfer starts late; on a high-priority stream they are dispatched first.  Measured on 8 GPUs
    (config 5, 268 MB per hop): 20.9 ms per ring pass with the default group, 20.0 ms with this one,
    18.3 ms for the same launches without any transfer.  Creating a group initialises a new NCCL
    communicator (seconds): make it once and pass it as ``group=``.  Collective over `ranks`
    (default: all)."""
    import torch.distributed as dist
    opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
    return dist.new_group(list(ranks) if ranks is not None else None, pg_options=opts)


class _P2PHandle:
    def __init__(self, works, tag_recv):
        self.works = works
        self.tag_recv = tag_recv

    def wait(self):
        for w in self.works:
            w.wait()

    def origin(self) -> int:
        return int(self.tag_recv.item())


def _dist_exchange(rank: int, world: int, group):
    import torch.distributed as dist

    nxt, prv = (rank + 1) % world, (rank - 1) % world

    state = {"tag": None}

    def exchange(k, v, k_recv, v_recv):
        # a one-element tag travels with the pair: the rank it started from
        if state["tag"] is None:
            state["tag"] = torch.full((1,), rank, dtype=torch.int64, device=k.device)
        tag_recv = torch.empty_like(state["tag"])
        ops = [dist.P2POp(dist.isend, k, nxt, group), dist.P2POp(dist.isend, v, nxt, group),
               dist.P2POp(dist.isend, state["tag"], nxt, group),
               dist.P2POp(dist.irecv, k_recv, prv, group), dist.P2POp(dist.irecv, v_recv, prv, group),
               dist.P2POp(dist.irecv, tag_recv, prv, group)]
        handle = _P2PHandle(dist.batch_isend_irecv(ops), tag_recv)
        state["tag"] = tag_recv
        return handle

    return exchange


def ring_forward_emulated(q, k, v, world: int, *, causal=True, softmax_scale=None, attn_fn=None,
                          accumulator=None, fused=True) -> torch.Tensor:
    """All `world` ranks of the ring run one after another in this process (no communication):
    the same schedule, kernels and merges as :func:`ring_forward`, for single-device checks."""
    qs, ks, vs = zigzag_split(q, world), zigzag_split(k, world), zigzag_split(v, world)
    outs = []
    for r in range(world):
        state = {"step": 0}

        def exchange(kc, vc, kr, vr, r=r, state=state):
            src = (r - state["step"] - 1) % world
            kr.copy_(ks[src])
            vr.copy_(vs[src])
            state["step"] += 1

            class _Done:
                def wait(self):
                    return None

            return _Done()

        outs.append(ring_forward(qs[r], ks[r], vs[r], causal=causal, softmax_scale=softmax_scale, rank=r,
                                 world=world, attn_fn=attn_fn, accumulator=accumulator, exchange=exchange,
                                 fused=fused))
    return zigzag_merge(outs)
