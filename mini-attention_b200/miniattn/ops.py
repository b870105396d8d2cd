"""Python operator surface of the B200 forward-attention kernels.

``flash_attn_fwd`` is the general entry ((B,H,N,D) or (B,N,H,D) tensors, causal,
GQA/MQA head broadcast, optional log-sum-exp).  It validates like the reference launcher
(kernels/flash_attn/cuda/sm_120/kernel/flash_attention.cu:41-80: CUDA tensors, equal
fp16/bf16 dtypes, agreeing shapes) and raises ``RuntimeError`` on violation, launches on the
current stream of the tensors' device and returns without synchronising.  torch is used for
device memory and streams only; the arithmetic runs in libminiattn.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple, Union

import torch

from . import _lib

_DTYPES = {torch.float16: _lib.FP16, torch.bfloat16: _lib.BF16}
_status_words: dict = {}
_balance_scratch: dict = {}   # (device index, stream) -> zero-initialised uint8 scratch tensor
# Parameter blocks of recent calls, keyed by everything that goes into one (pointers, shapes, strides,
# dtype, flags).  A training or serving loop calls the operator with the same tensors again and again;
# validating and filling the block costs more host time than a short-sequence kernel runs for.
_param_cache: dict = {}
_PARAM_CACHE_MAX = 256


def _status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def device_status(device: Union[torch.device, str, None] = None) -> int:
    """Synchronise and return (then clear) the wait-timeout bits kernels raised on `device`."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    t = _status_word(device)
    val = int(t.item())
    if val:
        t.zero_()
        # a launch that gave up may have left arrival counters of a balanced launch non-zero
        for key in [k for k in _balance_scratch if k[0] == device.index]:
            del _balance_scratch[key]
    return val


def check_device_status(device: Union[torch.device, str, None] = None) -> None:
    """Synchronise `device` and raise ``RuntimeError`` (MINIATTN_EDEVICE_WAIT, the waits named) if a
    bounded device-side wait of any launch since the last check ran out.  The operators launch
    asynchronously and never read the status word themselves, so a caller that wants the check calls
    this (or :func:`device_status`) where it synchronises anyway; results of the launches in between
    are undefined when it raises.  The word is cleared and the cached balanced-launch scratch of the
    device is dropped, so later launches start clean."""
    val = device_status(device)
    _lib.check(_lib.lib.miniattn_check_status(C.c_int32(val if val < (1 << 31) else val - (1 << 32))),
               "device status")


def _scratch_for(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """Scratch of a balanced launch: one buffer per (device, stream), zeroed when created (the
    kernels leave the arrival counters at its start zero again), grown on demand."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    t = _balance_scratch.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _balance_scratch[key] = t
    return t


def plan_info(B: int, Hq: int, Nq: int, Nk: int, D: int = 128, *, causal: bool = False, q_pos0: int = 0,
              k_pos0: int = 0, sm_count: int = 148):
    """The launch plan of a forward call on a GPU with `sm_count` SMs (host arithmetic only, no
    device needed): ``(info, pieces)`` with `info` a :class:`_lib.PlanInfo` and `pieces` the list
    of (item, t0, t1, part, nparts, slot) of the CTAs that follow the whole-item prefix."""
    p = _lib.FwdParams()
    p.B, p.Hq, p.Hkv, p.Nq, p.Nk, p.D = B, Hq, Hq, Nq, Nk, D
    p.causal = 1 if causal else 0
    p.q_pos0, p.k_pos0 = int(q_pos0), int(k_pos0)
    info = _lib.PlanInfo()
    cap = 1024
    arr = (_lib.PlanPiece * cap)()
    _lib.check(_lib.lib.miniattn_plan_fwd(C.byref(p), int(sm_count), C.byref(info), arr, cap), "miniattn_plan_fwd")
    pieces = [(e.item, e.t0, e.t1, e.part, e.nparts, e.slot) for e in arr[: info.n_pieces]]
    return info, pieces


def _bhn_strides(t: torch.Tensor, layout: str) -> Tuple[int, int, int]:
    if layout == "bhnd":
        return t.stride(0), t.stride(1), t.stride(2)
    return t.stride(0), t.stride(2), t.stride(1)


def _bhnd_shape(t: torch.Tensor, layout: str) -> Tuple[int, int, int, int]:
    if layout == "bhnd":
        return tuple(t.shape)  # type: ignore[return-value]
    b, n, h, d = t.shape
    return b, h, n, d


def _prepare(q, k, v, causal, softmax_scale, layout, return_lse, out, kernel, q_pos0, k_pos0, need_out=True):
    """Validate like the reference launcher and fill a FwdParams block.  Returns
    (params or None when the problem is empty, out, lse).  ``need_out=False``: a call that only
    stores carried state; no output tensor is allocated."""
    if layout not in ("bhnd", "bnhd"):
        raise RuntimeError(f"layout must be 'bhnd' or 'bnhd', got {layout!r}")
    if kernel not in _lib.KERNELS:
        raise RuntimeError(f"kernel must be one of {sorted(_lib.KERNELS)}, got {kernel!r}")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dim() != 4:
            raise RuntimeError(f"{name} must be 4-D, got {t.dim()}-D")
        if t.stride(-1) != 1 and t.numel() > 0:
            raise RuntimeError(f"{name} must be contiguous in the head dimension")
    if q.dtype not in _DTYPES:
        raise RuntimeError("Only fp16 and bf16 are supported")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError("Input tensors must have the same data type")
    if k.device != q.device or v.device != q.device:
        raise RuntimeError("Input tensors must be on the same device")
    B, Hq, Nq, D = _bhnd_shape(q, layout)
    Bk, Hkv, Nk, Dk = _bhnd_shape(k, layout)
    if _bhnd_shape(v, layout) != (Bk, Hkv, Nk, Dk):
        raise RuntimeError("k and v must have the same shape")
    if Bk != B or Dk != D:
        raise RuntimeError("q and k/v must agree in batch size and head dim")
    if Hkv == 0 or Hq % max(Hkv, 1) != 0:
        raise RuntimeError(f"number of query heads ({Hq}) must be a multiple of KV heads ({Hkv})")
    if out is None:
        if need_out:
            out = torch.empty_like(q)
    else:
        if out.shape != q.shape or out.dtype != q.dtype or out.device != q.device:
            raise RuntimeError("out must match q in shape, dtype and device")
        if out.stride(-1) != 1 and out.numel() > 0:
            raise RuntimeError("out must be contiguous in the head dimension")
    lse = torch.empty((B, Hq, Nq), dtype=torch.float32, device=q.device) if return_lse and need_out else None
    if q.numel() == 0:
        return None, out, lse
    p = _lib.FwdParams()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.o = out.data_ptr() if out is not None else None
    p.lse = lse.data_ptr() if lse is not None else None
    p.status = _status_word(q.device).data_ptr()
    p.q_stride[:] = _bhn_strides(q, layout)
    p.k_stride[:] = _bhn_strides(k, layout)
    p.v_stride[:] = _bhn_strides(v, layout)
    p.o_stride[:] = _bhn_strides(out if out is not None else q, layout)
    p.q_pos0, p.k_pos0 = int(q_pos0), int(k_pos0)
    p.B, p.Hq, p.Hkv, p.Nq, p.Nk, p.D = B, Hq, Hkv, Nq, Nk, D
    p.dtype = _DTYPES[q.dtype]
    p.causal = 1 if causal else 0
    p.softmax_scale = float(softmax_scale) if softmax_scale is not None else 0.0
    p.kernel = _lib.KERNELS[kernel]
    return p, out, lse


def flash_attn_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    layout: str = "bhnd",
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    kernel: str = "auto",
    q_pos0: int = 0,
    k_pos0: int = 0,
    balance: bool = True,
    carry: Optional[torch.Tensor] = None,
    carry_in: bool = False,
    carry_out: bool = False,
    carry_rows: Optional[Tuple[int, int]] = None,
):
    """O = softmax(Q K^T * scale [+ causal mask]) V on the GPU.

    q: (B,Hq,Nq,D) for ``layout="bhnd"`` or (B,Nq,Hq,D) for ``"bnhd"`` (the layout of the
    reference CUDA operator, flash_attention.cu:68-70); k, v likewise with Hkv heads where
    Hkv divides Hq (KV head g serves query heads g*G..g*G+G-1, as
    kernels/standard/pytorch/gqa.py:38-39).  Causal: key j is visible to query i iff
    ``k_pos0 + j <= q_pos0 + i`` (kernels/flash_attn/triton/fp16_flash_attn_sm86.py:74-75
    with both offsets 0).  Returns ``out`` or ``(out, lse)`` with lse fp32 (B,Hq,Nq) =
    natural-log of the softmax denominator.  ``balance`` (default on) launches through
    ``miniattn_fwd_balanced``: when the work items do not fill a whole number of rounds of one CTA
    per SM, the key range of some items is cut over several CTAs inside the one launch (scratch for
    their partial results is cached per device and stream).

    ``carry`` (a buffer from :func:`carry_state`) chains calls over the same q and successive key
    blocks, as the ring launcher does: with ``carry_out`` the rows' running (maximum, sum,
    un-normalised O) are stored in it and nothing is returned; with ``carry_in`` the stored state is
    folded into this call's result.  The last call of a chain (``carry_in`` only) returns the output.
    ``carry_rows=(first_row, total_rows)``: the buffer was made for a longer q of `total_rows` rows and
    this call's q is the row range of it that starts at `first_row` (a multiple of 128).

    The launch is asynchronous.  Every device-side wait is bounded; one that runs out sets a bit in a
    per-device status word instead of hanging — poll it with :func:`check_device_status` /
    :func:`device_status` after synchronising.
    """
    use_carry = bool(carry_in or carry_out)
    if use_carry and carry is None:
        raise RuntimeError("carry_in / carry_out need a carry buffer (carry_state)")
    # Fast path: the same tensors and flags as an earlier call.  Only a caller-provided `out` can be
    # part of the key; a fresh output (and lse) is allocated per call and patched into the block.
    try:
        key = (q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr() if out is not None else 0,
               q.shape, q.stride(), k.shape, k.stride(), v.stride(), out.stride() if out is not None else None,
               q.dtype, q.device.index, causal, softmax_scale, layout, return_lse, kernel, q_pos0, k_pos0, balance,
               carry.data_ptr() if carry is not None else 0, carry_in, carry_out, carry_rows)
        hit = _param_cache.get(key)
    except (AttributeError, TypeError):   # not tensors: let the validation below say so
        key, hit = None, None
    if hit is not None:
        p, need = hit
        lse = None
        if not carry_out and (out is None or return_lse):
            p = _lib.FwdParams.from_buffer_copy(p)   # the cached block stays as it is (other threads may hold it)
            if out is None:
                out = torch.empty_like(q)
                p.o = out.data_ptr()
            if return_lse:
                lse = torch.empty((p.B, p.Hq, p.Nq), dtype=torch.float32, device=q.device)
                p.lse = lse.data_ptr()
    else:
        out_given = out is not None
        p, out, lse = _prepare(q, k, v, causal, softmax_scale, layout, return_lse, out, kernel, q_pos0, k_pos0,
                               need_out=not carry_out)
        if p is not None and use_carry:
            if carry_rows is not None:
                first, total = carry_rows
                if first % 128 != 0 or first < 0 or first + p.Nq > total:
                    raise RuntimeError("carry_rows: the first row must be a multiple of 128 inside the state's rows")
                p.carry_tile0, p.carry_tiles = first // 128, (total + 127) // 128
                whole = _lib.FwdParams()
                whole.B, whole.Hq, whole.Hkv, whole.Nq, whole.Nk, whole.D = p.B, p.Hq, p.Hkv, total, p.Nk, p.D
                need_c = _lib.lib.miniattn_fwd_carry_bytes(C.byref(whole))
            else:
                need_c = _lib.lib.miniattn_fwd_carry_bytes(C.byref(p))
            if need_c < 0:
                _lib.check(int(need_c), "miniattn_fwd_carry_bytes")
            if not carry.is_cuda or carry.device != q.device or carry.numel() * carry.element_size() < need_c:
                raise RuntimeError(f"carry must be a CUDA buffer on q's device of at least {need_c} bytes")
            p.carry, p.carry_in, p.carry_out = carry.data_ptr(), int(bool(carry_in)), int(bool(carry_out))
        need = 0
        if p is not None and balance and not use_carry:
            with torch.cuda.device(q.device):
                need = int(_lib.lib.miniattn_fwd_balanced_scratch_bytes(C.byref(p)))
            if need < 0:
                _lib.check(need, "miniattn_fwd_balanced_scratch_bytes")
        # a freshly allocated output keeps the same strides from call to call (torch.empty_like)
        if p is not None and key is not None and (out_given or out is None or out.stride() == q.stride()):
            if len(_param_cache) >= _PARAM_CACHE_MAX:
                _param_cache.clear()
            _param_cache[key] = (p, need)
    if p is not None:
        dev_index = q.device.index
        if torch.cuda.current_device() == dev_index:
            rc = _launch_fwd(p, need, q.device, _current_raw_stream(dev_index))
        else:
            with torch.cuda.device(q.device):
                rc = _launch_fwd(p, need, q.device, _current_raw_stream(dev_index))
        _lib.check(rc, "miniattn_fwd")
    if carry_out:
        return None
    return (out, lse) if return_lse else out


def _current_raw_stream(device_index: int) -> int:
    """cudaStream_t of torch's current stream on the device, without building a Stream object (3 us
    of the 13 us a short-sequence call spends on the host)."""
    try:
        return torch._C._cuda_getCurrentRawStream(device_index)
    except AttributeError:
        return torch.cuda.current_stream(device_index).cuda_stream


def _launch_fwd(p, need: int, device: torch.device, stream: int) -> int:
    if need > 0:
        scratch = _scratch_for(device, stream, need)
        return _lib.lib.miniattn_fwd_balanced(C.byref(p), C.c_void_p(scratch.data_ptr()),
                                              C.c_size_t(scratch.numel()), C.c_void_p(stream))
    return _lib.lib.miniattn_fwd(C.byref(p), C.c_void_p(stream))


def carry_state(q: torch.Tensor, layout: str = "bhnd") -> torch.Tensor:
    """Device buffer for the running state of q's rows across a chain of ``flash_attn_fwd`` calls
    (``carry=...``).  Its layout is private to the library; its content is defined only between a
    ``carry_out`` call and the ``carry_in`` call that follows."""
    B, Hq, Nq, D = _bhnd_shape(q, layout)
    p = _lib.FwdParams()
    p.B, p.Hq, p.Hkv, p.Nq, p.Nk, p.D = B, Hq, Hq, Nq, Nq, D
    n = _lib.lib.miniattn_fwd_carry_bytes(C.byref(p))
    if n < 0:
        _lib.check(int(n), "miniattn_fwd_carry_bytes")
    return torch.empty(max(int(n), 256), dtype=torch.uint8, device=q.device)


class Int8QK:
    """Device buffers of the INT8-QK pre-pass for one problem shape: int8 Q and K, their
    per-128-token-block scales, the K channel means and the column-sum scratch."""

    def __init__(self, B, Hq, Hkv, Nq, Nk, D, device):
        nqb, nkb, nch = (Nq + 127) // 128, (Nk + 127) // 128, (Nk + 1023) // 1024
        self.shape = (B, Hq, Hkv, Nq, Nk, D)
        self.q8 = torch.empty((B, Hq, Nq, D), dtype=torch.int8, device=device)
        self.k8 = torch.empty((B, Hkv, Nk, D), dtype=torch.int8, device=device)
        self.q_scale = torch.empty((B, Hq, nqb), dtype=torch.float32, device=device)
        self.k_scale = torch.empty((B, Hkv, nkb), dtype=torch.float32, device=device)
        self.k_partial = torch.empty((B, Hkv, nch, D), dtype=torch.float32, device=device)
        self.k_mean = torch.empty((B, Hkv, D), dtype=torch.float32, device=device)

    def fill(self, p8: "_lib.Int8Params") -> None:
        p8.q8, p8.k8 = self.q8.data_ptr(), self.k8.data_ptr()
        p8.q_scale, p8.k_scale = self.q_scale.data_ptr(), self.k_scale.data_ptr()
        p8.k_partial, p8.k_mean = self.k_partial.data_ptr(), self.k_mean.data_ptr()


def flash_attn_fwd_int8qk(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    layout: str = "bhnd",
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    buffers: Optional[Int8QK] = None,
    quantize: bool = True,
    attend: bool = True,
    balance: bool = True,
):
    """INT8-QK attention: K is mean-smoothed, Q and K are quantised to int8 per block of 128
    tokens (pre-pass), Q8 K8^T runs on the int8 tensor cores, P V stays 16 bit.  `buffers` lets a
    caller reuse the pre-pass buffers across calls of the same shape (and inspect them);
    ``quantize=False`` skips the pre-pass (buffers already filled), ``attend=False`` runs the
    pre-pass only; ``balance`` as for :func:`flash_attn_fwd`."""
    p, out, lse = _prepare(q, k, v, causal, softmax_scale, layout, return_lse, out, "auto", 0, 0)
    if p is None:
        return (out, lse) if return_lse else out
    shape = (p.B, p.Hq, p.Hkv, p.Nq, p.Nk, p.D)
    if buffers is None:
        buffers = Int8QK(*shape, q.device)
    elif buffers.shape != shape or buffers.q8.device != q.device:
        raise RuntimeError("buffers were made for another problem shape or device")
    p8 = _lib.Int8Params()
    p8.fwd = p
    buffers.fill(p8)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        if quantize:
            _lib.check(_lib.lib.miniattn_quant_qk_int8(C.byref(p8), C.c_void_p(stream)), "miniattn_quant_qk_int8")
        if attend:
            need = _lib.lib.miniattn_fwd_balanced_scratch_bytes(C.byref(p)) if balance else 0
            if need < 0:
                _lib.check(int(need), "miniattn_fwd_balanced_scratch_bytes")
            if need > 0:
                scratch = _scratch_for(q.device, stream, int(need))
                rc = _lib.lib.miniattn_fwd_int8qk_balanced(C.byref(p8), C.c_void_p(scratch.data_ptr()),
                                                           C.c_size_t(scratch.numel()), C.c_void_p(stream))
            else:
                rc = _lib.lib.miniattn_fwd_int8qk(C.byref(p8), C.c_void_p(stream))
            _lib.check(rc, "miniattn_fwd_int8qk")
    return (out, lse) if return_lse else out


class HostPipeline:
    """Forward attention on HOST (pinned) tensors with the copies overlapped with compute.

    The (batch x KV-head group) units are independent, so the work is cut into chunks of units;
    chunk i+1 is copied host->device on one stream while chunk i runs on the compute stream and
    the output of chunk i-1 is copied back on a third stream.  Device staging tensors, streams and
    events are created once per problem shape and reused.  Inputs: q (B,Hq,N,D), k/v (B,Hkv,N,D)
    in pinned host memory; the result is written to ``out`` (pinned host tensor, same shape as q).
    """

    def __init__(self, q: torch.Tensor, k: torch.Tensor, device, n_chunks: int = 8):
        self.device = torch.device(device)
        B, Hq, Nq, D = q.shape
        Hkv = k.shape[1]
        self.G = Hq // Hkv
        self.qd = torch.empty(q.shape, dtype=q.dtype, device=self.device)
        self.kd = torch.empty(k.shape, dtype=k.dtype, device=self.device)
        self.vd = torch.empty(k.shape, dtype=k.dtype, device=self.device)
        self.od = torch.empty(q.shape, dtype=q.dtype, device=self.device)
        # chunks: runs of KV heads inside one batch element
        per = max(1, (B * Hkv + n_chunks - 1) // n_chunks)
        self.chunks = []
        for b in range(B):
            for h0 in range(0, Hkv, per):
                self.chunks.append((b, h0, min(Hkv, h0 + per)))
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.ev_in = [torch.cuda.Event() for _ in self.chunks]
        self.ev_done = [torch.cuda.Event() for _ in self.chunks]
        self._launches: dict = {}  # (causal, scale, kernel) -> per-chunk parameter blocks, filled once

    def _params(self, causal, softmax_scale, kernel):
        """Parameter blocks of the chunk launches: the staging tensors never move, so the blocks
        (and the scratch size of the balanced launch) are built once per (causal, scale, kernel)."""
        key = (bool(causal), softmax_scale, kernel)
        entry = self._launches.get(key)
        if entry is None:
            G = self.G
            blocks, need = [], 0
            for b, h0, h1 in self.chunks:
                p, _, _ = _prepare(self.qd[b:b + 1, h0 * G:h1 * G], self.kd[b:b + 1, h0:h1], self.vd[b:b + 1, h0:h1],
                                   causal, softmax_scale, "bhnd", False, self.od[b:b + 1, h0 * G:h1 * G], kernel, 0, 0)
                n = _lib.lib.miniattn_fwd_balanced_scratch_bytes(C.byref(p))
                if n < 0:
                    _lib.check(int(n), "miniattn_fwd_balanced_scratch_bytes")
                need = max(need, int(n))
                blocks.append(p)
            entry = self._launches[key] = (blocks, need)
        return entry

    def __call__(self, q, k, v, out, *, causal=False, softmax_scale=None, kernel="auto"):
        G = self.G
        main = torch.cuda.current_stream(self.device)
        blocks, need = self._params(causal, softmax_scale, kernel)
        scratch = _scratch_for(self.device, main.cuda_stream, need) if need > 0 else None
        sptr = C.c_void_p(scratch.data_ptr()) if scratch is not None else None
        ssize = C.c_size_t(scratch.numel() if scratch is not None else 0)
        stream = C.c_void_p(main.cuda_stream)
        self.s_in.wait_stream(main)   # staging buffers may still be in use by earlier work
        self.s_out.wait_stream(main)
        for i, (b, h0, h1) in enumerate(self.chunks):
            with torch.cuda.stream(self.s_in):
                self.qd[b, h0 * G:h1 * G].copy_(q[b, h0 * G:h1 * G], non_blocking=True)
                self.kd[b, h0:h1].copy_(k[b, h0:h1], non_blocking=True)
                self.vd[b, h0:h1].copy_(v[b, h0:h1], non_blocking=True)
                self.ev_in[i].record(self.s_in)
            main.wait_event(self.ev_in[i])
            _lib.check(_lib.lib.miniattn_fwd_balanced(C.byref(blocks[i]), sptr, ssize, stream), "miniattn_fwd_balanced")
            self.ev_done[i].record(main)
            self.s_out.wait_event(self.ev_done[i])
            with torch.cuda.stream(self.s_out):
                out[b, h0 * G:h1 * G].copy_(self.od[b, h0 * G:h1 * G], non_blocking=True)
        main.wait_stream(self.s_out)
        return out


_host_pipelines: dict = {}


def flash_attn_fwd_host(q, k, v, out=None, *, causal=False, softmax_scale=None, device=None, n_chunks=8,
                        kernel="auto"):
    """Forward attention with q, k, v and the result in pinned HOST memory ((B,H,N,D) layout).
    Host<->device copies are overlapped with the kernel chunk by chunk (see :class:`HostPipeline`);
    the call returns once everything is enqueued — synchronise before reading ``out``."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.is_cuda or not t.is_pinned():
            raise RuntimeError(f"{name} must be a pinned host tensor")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if out is None:
        out = torch.empty_like(q).pin_memory()
    key = (tuple(q.shape), tuple(k.shape), q.dtype, device.index, n_chunks)
    pipe = _host_pipelines.get(key)
    if pipe is None:
        pipe = _host_pipelines[key] = HostPipeline(q, k, device, n_chunks)
    with torch.cuda.device(device):
        return pipe(q, k, v, out, causal=causal, softmax_scale=softmax_scale, kernel=kernel)


def merge_partials(
    acc_o: torch.Tensor,
    acc_lse: torch.Tensor,
    part_o: torch.Tensor,
    part_lse: torch.Tensor,
    *,
    init: bool = False,
    out: Optional[torch.Tensor] = None,
) -> None:
    """In-place log-sum-exp merge of one ring-step partial into the running result.

    acc_o fp32 (..., N, D) and acc_lse fp32 (..., N) are updated; part_o is the fp16/bf16
    normalised partial with its part_lse.  ``init=True`` overwrites the accumulators with the
    partial; ``out`` (same dtype as part_o) additionally receives the merged result.  All
    tensors must be contiguous CUDA tensors of matching shapes, except ``out``, which may be a
    token-range view ``big[:, :, a:b]`` of a contiguous (B,H,N,D) tensor.
    """
    if part_o.dtype not in _DTYPES:
        raise RuntimeError("Only fp16 and bf16 partials are supported")
    if acc_o.dtype != torch.float32 or acc_lse.dtype != torch.float32 or part_lse.dtype != torch.float32:
        raise RuntimeError("acc_o, acc_lse and part_lse must be fp32")
    for t in (acc_o, acc_lse, part_o, part_lse):
        if not t.is_cuda or not t.is_contiguous() or t.device != acc_o.device:
            raise RuntimeError("merge_partials takes contiguous CUDA tensors on one device")
    slab_rows = slab_stride = 0
    if out is not None:
        if not out.is_cuda or out.device != acc_o.device:
            raise RuntimeError("out must be a CUDA tensor on the same device")
        if not out.is_contiguous():
            # accept (B,H,n,D) views whose (batch, head) slabs are evenly spaced
            ok = (out.dim() == 4 and out.stride(3) == 1 and out.stride(2) == out.shape[3]
                  and out.stride(0) == out.stride(1) * out.shape[1])
            if not ok:
                raise RuntimeError("out must be contiguous or a token-range view of a contiguous (B,H,N,D) tensor")
            slab_rows, slab_stride = out.shape[2], out.stride(1)
    if acc_o.shape != part_o.shape or acc_lse.shape != part_lse.shape or acc_lse.shape != acc_o.shape[:-1]:
        raise RuntimeError("shape mismatch between accumulators and partials")
    if out is not None and (out.shape != part_o.shape or out.dtype != part_o.dtype):
        raise RuntimeError("out must match part_o in shape and dtype")
    p = _lib.MergeParams()
    p.acc_o, p.acc_lse = acc_o.data_ptr(), acc_lse.data_ptr()
    p.part_o, p.part_lse = part_o.data_ptr(), part_lse.data_ptr()
    p.out = out.data_ptr() if out is not None else None
    p.rows = acc_lse.numel()
    p.D = acc_o.shape[-1]
    p.dtype = _DTYPES[part_o.dtype]
    p.init = 1 if init else 0
    p.out_rows_per_slab, p.out_slab_stride = slab_rows, slab_stride
    with torch.cuda.device(acc_o.device):
        stream = torch.cuda.current_stream(acc_o.device).cuda_stream
        rc = _lib.lib.miniattn_merge_partials(C.byref(p), C.c_void_p(stream))
    _lib.check(rc, "miniattn_merge_partials")


def selftest_wait(limit_ms: float = 50.0, device: Union[torch.device, str, None] = None) -> int:
    """Run the bounded-wait self-test kernel; returns the status word it produced."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = _lib.lib.miniattn_selftest_wait(C.c_void_p(status.data_ptr()), C.c_uint64(int(limit_ms * 1e6)),
                                             C.c_void_p(stream))
    _lib.check(rc, "miniattn_selftest_wait")
    return int(status.item())
