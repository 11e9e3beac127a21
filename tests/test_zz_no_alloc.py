"""Bucketing without device allocations.

A worker that owns one pre-carved device pool, or a plugin called from inside another runtime's
step, cannot let this library call cudaMalloc.  `ek_bucket_noalloc` is the entry point for such
callers: no backend handle, no allocator calls, scratch built into the library image.  Here it is
driven through the C ABI with caller-owned device buffers and must reproduce, bit for bit, the
counts / offsets / permutation that the regular routing entry point reports for the same
assignments -- and that the CPU oracle's stable counting sort gives -- on two calls in a row,
since the second call meets the scratch the first one left behind.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import pytest
import torch

from oracle import ek_oracle as O

pytestmark = pytest.mark.gpu


def _bucket_noalloc(lib, ids_dev, E):
    T, k = ids_dev.shape
    counts = torch.full((E,), -7, dtype=torch.int32, device="cuda")
    offsets = torch.full((E + 1,), -7, dtype=torch.int32, device="cuda")
    perm = torch.full((T * k,), -7, dtype=torch.int32, device="cuda")
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    st = lib.ek_bucket_noalloc(ids_dev.data_ptr(), T, k, E, counts.data_ptr(), offsets.data_ptr(), perm.data_ptr(),
                               C.c_void_p(stream), err, 256)
    return st, err.value.decode(), counts.cpu(), offsets.cpu(), perm.cpu()


def test_bucket_noalloc_matches_regular_entry_point_twice_in_a_row():
    import ek_b200
    from ek_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(123)
    E, k = 256, 8
    be = ek_b200.Backend(ek_b200.BackendConfig(hidden=128, intermediate=128, n_experts=E, top_k=k, scoring=1,
                                               n_group=8, topk_group=4, routed_scaling=2.5, max_tokens=2048))
    # second call is smaller than the first, so stale scratch from the first would show
    for T in (1500, 37):
        logits = torch.randn(T, E, generator=g) * 2.0
        want = be.route_from_logits(logits)              # existing entry point
        ids_dev = want["ids"].cuda()
        torch.cuda.synchronize()
        st, msg, counts, offsets, perm = _bucket_noalloc(lib, ids_dev, E)
        assert st == 0, msg
        assert torch.equal(counts, want["counts"])
        assert torch.equal(offsets, want["offsets"])
        assert torch.equal(perm, want["perm"])
        # and, independently of this library, against the CPU restatement of the reference's bucketing
        c, o, p = O.bucket(want["ids"], E)
        assert torch.equal(counts, c) and torch.equal(offsets, o) and torch.equal(perm, p)
    be.close()


def test_bucket_noalloc_limits_and_bad_ids():
    from ek_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    E = 16
    big = torch.zeros(65536 // 8 + 1, 8, dtype=torch.int32, device="cuda")     # one row beyond the built-in scratch
    st, msg, *_ = _bucket_noalloc(lib, big, E)
    assert st == 3 and "exceeds" in msg
    bad = torch.tensor([[0, 1], [2, 99]], dtype=torch.int32, device="cuda")
    st, msg, *_ = _bucket_noalloc(lib, bad, E)
    assert st == 18 and "99" in msg
    # and the scratch is usable again afterwards
    good = torch.tensor([[3, 1], [1, 0], [3, 2]], dtype=torch.int32, device="cuda")
    st, msg, counts, offsets, perm = _bucket_noalloc(lib, good, E)
    assert st == 0, msg
    assert counts[:4].tolist() == [1, 2, 1, 2] and int(counts.sum()) == 6
    assert offsets[:5].tolist() == [0, 1, 3, 4, 6]
    assert perm.tolist() == [3, 1, 2, 5, 0, 4]
