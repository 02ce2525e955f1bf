"""Allocation-free decode attention, called through its exported C symbol.

Some hosts of this library cannot get device memory when they call decode attention: a C/C++ serving loop
without PyTorch's allocator, or an engine process that already gave all free device memory to the KV
pool.  For them the shared object exports ``mb_paged_decode_attention_noalloc``, whose split-KV scratch is
a fixed 16 MiB array inside the library image.  The test loads the symbol with ctypes, runs it twice in a
row on different inputs (the array keeps the first call's contents, which must not leak into the second
result) and compares each output with the regular tensor-scratch entry point; it also checks that an
oversized request is refused without launching anything.  The file name sorts last so that a
stop-at-first-failure run has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 4 * 1024 * 1024


def _lib():
    from miles_b200 import _build
    from miles_b200.ops import _ext

    _ext.load(required=True)  # builds the shared object if needed and loads libtorch first
    lib = ctypes.CDLL(str(_build.TARGET))
    fn = lib.mb_paged_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    lib.mb_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _case(seed, B, lens, Hq=32, Hk=4, ps=64, max_pages=24):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    n_pages = 1 + sum((l + ps - 1) // ps for l in lens)
    kc = torch.randn(n_pages * ps, Hk, 128, device=dev, dtype=torch.bfloat16, generator=g)
    vc = torch.randn(n_pages * ps, Hk, 128, device=dev, dtype=torch.bfloat16, generator=g)
    q = torch.randn(B, Hq, 128, device=dev, dtype=torch.bfloat16, generator=g)
    bt = torch.zeros(B, max_pages, dtype=torch.int32, device=dev)
    nxt = 1
    for b, l in enumerate(lens):
        n = (l + ps - 1) // ps
        bt[b, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
    return q, kc, vc, bt, torch.tensor(lens, dtype=torch.int32, device=dev), ps, max_pages


def test_no_alloc_entry_point_matches_regular_path_twice(ext):
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lens, splits in ((1, [700, 64, 1, 1300], 8), (2, [33, 1500, 257, 90], 5)):
        q, kc, vc, bt, sl, ps, max_pages = _case(seed, len(lens), lens)
        B, Hq, Hk = q.shape[0], q.shape[1], kc.shape[1]
        want = torch.empty_like(q)
        scratch = torch.empty(B * Hq * splits * 130, dtype=torch.float32, device=q.device)
        ext.paged_decode_attention(q, kc, vc, bt, sl, want, scratch, ps, splits, 128 ** -0.5)
        got = torch.full_like(q, float("nan"))
        status = torch.zeros(1, dtype=torch.int32, device=q.device)

        def call():
            return fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), got.data_ptr(), B, Hq, Hk, ps,
                      max_pages, splits, ctypes.c_float(128 ** -0.5), kc.shape[0], status.data_ptr(), ctypes.c_void_p(stream))

        rc = call()  # also the warm-up: the first call on a device looks up the scratch address
        assert rc == 0, lib.mb_noalloc_last_error().decode()
        torch.cuda.synchronize()
        # neither torch's allocator nor the driver may hand out memory during a call: the caching allocator's
        # counter cannot see a raw cudaMalloc, the driver's free-byte count can
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        got.fill_(float("nan"))
        rc = call()
        assert rc == 0, lib.mb_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before and torch.cuda.mem_get_info()[0] == free_before
        assert torch.isfinite(got.float()).all() and status.item() == 0
        assert (got.float() - want.float()).abs().max().item() < 2e-2


def test_no_alloc_entry_point_rejects_oversized_requests(ext):
    lib, fn = _lib()
    q, kc, vc, bt, sl, ps, max_pages = _case(3, 2, [10, 20])
    out = torch.zeros_like(q)
    splits = SCRATCH_FLOATS // (130 * 2 * 32) + 1
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), out.data_ptr(), 2, 32, 4, ps, max_pages,
            splits, ctypes.c_float(0.1), kc.shape[0], None, ctypes.c_void_p(0))
    assert rc == -2 and b"exceed" in lib.mb_noalloc_last_error()
    torch.cuda.synchronize()
    assert out.abs().sum().item() == 0
    assert fn(None, kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), out.data_ptr(), 2, 32, 4, ps, max_pages, 1,
              ctypes.c_float(0.1), kc.shape[0], None, ctypes.c_void_p(0)) == -1


def test_no_alloc_entry_point_does_not_follow_bad_tables(ext):
    """Lengths and page ids come from device memory a C host filled. A length past the block-table row is clamped and
    a page id outside the cache reads as zeros; the kernel records which happened and touches no address outside the
    cache (the call returns normally and the next call works)."""
    lib, fn = _lib()
    q, kc, vc, bt, sl, ps, max_pages = _case(4, 2, [200, 300])
    out = torch.zeros_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=q.device)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), sl.data_ptr(), out.data_ptr(), 2, 32, 4, ps, max_pages,
                4, ctypes.c_float(128 ** -0.5), kc.shape[0], status.data_ptr(), ctypes.c_void_p(stream))
        torch.cuda.synchronize()
        return rc

    good_bt = bt.clone()
    bt[1, 2] = 10 ** 6  # far outside the cache
    assert call() == 0 and status.item() == 9 and torch.isfinite(out.float()).all()
    bt.copy_(good_bt)
    status.zero_()
    sl[0] = max_pages * ps + 5000  # longer than its block-table row
    assert call() == 0 and status.item() == 8 and torch.isfinite(out.float()).all()
    sl[0] = 200
    status.zero_()
    assert call() == 0 and status.item() == 0
