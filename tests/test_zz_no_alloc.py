"""The allocation-free INT8 pre-pass entry point (miniattn_quant_qk_int8_static).

Some hosts of this library cannot hand it device memory: an inference server that reserved all of
HBM for its KV cache when it started, or a plugin contract that rules out cudaMalloc because an
allocation synchronises the device and may fail at an arbitrary later time.  For them the pre-pass
keeps its only internal scratch (the column sums of K) in a fixed 256 KB array inside the library.

The test drives the new entry point through the C ABI, twice in a row on different inputs (the
array keeps the first call's contents, which must not leak into the second), and requires exactly
the outputs of the existing entry point with a caller-provided scratch buffer.  It also checks that
a problem beyond the built-in limit is refused with a clear message.  The file sorts last so that a
run stopping at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _params(q, k, bufs):
    from miniattn import _lib
    from miniattn.ops import _prepare
    p, _, _ = _prepare(q, k, k, False, None, "bhnd", False, None, "auto", 0, 0)
    p8 = _lib.Int8Params()
    p8.fwd = p
    bufs.fill(p8)
    return p8


def _run(entry, q, k, with_scratch):
    import miniattn
    from miniattn import _lib
    B, Hq, Nq, D = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    bufs = miniattn.Int8QK(B, Hq, Hkv, Nq, Nk, D, DEV)
    for t in (bufs.q8, bufs.k8, bufs.q_scale, bufs.k_scale, bufs.k_mean):
        t.fill_(0)
    p8 = _params(q, k, bufs)
    if not with_scratch:
        p8.k_partial = None
    stream = torch.cuda.current_stream().cuda_stream
    rc = getattr(_lib.lib, entry)(C.byref(p8), C.c_void_p(stream))
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    return [t.clone() for t in (bufs.q8, bufs.k8, bufs.q_scale, bufs.k_scale, bufs.k_mean)]


def test_static_scratch_prepass_matches_the_allocating_entry_point_twice():
    g = torch.Generator().manual_seed(123)
    cases = [
        (torch.float16, (2, 4, 2, 2300, 64)),     # 3 column-sum chunks per head, ragged tail
        (torch.bfloat16, (1, 2, 2, 1024, 128)),   # different shape: stale scratch must not matter
    ]
    for dtype, (B, Hq, Hkv, N, D) in cases:
        q = torch.randn(B, Hq, N, D, generator=g).to(dtype).to(DEV)
        k = (torch.randn(B, Hkv, N, D, generator=g) + 2.0 * torch.randn(1, 1, 1, D, generator=g)).to(dtype).to(DEV)
        want = _run("miniattn_quant_qk_int8", q, k, with_scratch=True)
        got = _run("miniattn_quant_qk_int8_static", q, k, with_scratch=False)
        for name, a, b in zip(("q8", "k8", "q_scale", "k_scale", "k_mean"), got, want):
            assert torch.equal(a, b), f"{name} differs between the two entry points ({dtype})"


def test_static_scratch_limit_is_enforced():
    import miniattn
    from miniattn import _lib
    # B*Hkv*ceil(Nk/1024)*D = 8*32*3*128 = 98304 floats > 65536
    q = torch.zeros(8, 32, 128, 128, dtype=torch.float16, device=DEV)
    k = torch.zeros(8, 32, 2100, 128, dtype=torch.float16, device=DEV)
    bufs = miniattn.Int8QK(8, 32, 32, 128, 2100, 128, DEV)
    p8 = _params(q, k, bufs)
    rc = _lib.lib.miniattn_quant_qk_int8_static(C.byref(p8), None)
    assert rc == -2
    msg = _lib.last_error()
    assert "98304" in msg and "65536" in msg
