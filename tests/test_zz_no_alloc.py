"""ani_sort_noalloc: the sort for hosts that are not allowed to allocate device memory (its
scratch is a fixed array inside the library).  Collected last on purpose, so that a run which
stops at the first failure has already run every other test.

The entry point must give exactly what ani_sort gives.  It is called twice in a row on
different batches -- the second smaller than the first -- because the scratch array is shared
by all calls and still holds the first call's tile counts when the second one starts.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _sort_with(fn, a_dev, torch):
    n = a_dev.numel()
    scatter = torch.full((n,), -7, dtype=torch.int32, device=a_dev.device)
    gather = torch.full((n,), -7, dtype=torch.int32, device=a_dev.device)
    counts = torch.full((4,), -7, dtype=torch.int32, device=a_dev.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr() if t.numel() else 0)  # noqa: E731
    status = fn(p(a_dev), n, p(scatter), p(gather), p(counts), stream)
    assert status == 0, status
    torch.cuda.synchronize()
    return scatter.cpu().numpy(), gather.cpu().numpy(), counts.cpu().numpy()


_first_call_done = False


def test_noalloc_first_call_inside_a_stream_capture_is_refused():
    """The first call on a device looks up the address of the library's array, which must not happen while
    the stream is being captured: such a call is refused and launches nothing.  (Only meaningful when
    this is the first ani_sort_noalloc call of the process, which it is when the file runs in order.)"""
    global _first_call_done
    import torch
    from khan_b200 import _lib

    lib = _lib.lib()
    a = torch.from_numpy(np.random.default_rng(3).integers(0, 4, 5000).astype(np.int32)).to("cuda:0")
    out = [torch.empty(5000, dtype=torch.int32, device="cuda:0"), torch.empty(5000, dtype=torch.int32, device="cuda:0"),
           torch.empty(4, dtype=torch.int32, device="cuda:0")]
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        g.capture_begin()
        status = lib.ani_sort_noalloc(a.data_ptr(), 5000, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                      ctypes.c_void_p(side.cuda_stream))
        g.capture_end()
    assert status == (0 if _first_call_done else -10)
    _first_call_done = True


def test_noalloc_sort_matches_sort_on_two_calls_in_a_row():
    global _first_call_done
    _first_call_done = True
    import torch
    from khan_b200 import _lib

    assert torch.cuda.is_available()
    lib = _lib.lib()
    rng = np.random.default_rng(2024)
    first = rng.choice(4, size=150_001, p=[0.6, 0.25, 0.1, 0.05]).astype(np.int32)
    second = rng.integers(0, 4, size=9_313).astype(np.int32)
    for batch in (first, second):
        a = torch.from_numpy(batch).to("cuda:0")
        expected = _sort_with(lib.ani_sort, a, torch)
        got = _sort_with(lib.ani_sort_noalloc, a, torch)
        for g, e in zip(got, expected):
            np.testing.assert_array_equal(g, e)   # integer outputs: bit for bit
        # and both agree with a stable argsort done on the host
        order = np.argsort(batch, kind="stable")
        inv = np.empty(batch.size, np.int64)
        inv[order] = np.arange(batch.size)
        np.testing.assert_array_equal(got[1], inv)
        np.testing.assert_array_equal(got[2], np.bincount(batch, minlength=4))


def test_noalloc_sort_rejects_what_does_not_fit():
    from khan_b200 import _lib

    lib = _lib.lib()
    limit = lib.ani_sort_noalloc_max_atoms()
    assert limit == 4_194_304
    # size checks come before any pointer is touched or anything is launched
    assert lib.ani_sort_noalloc(None, limit + 1, None, None, None, None) == -7
    assert "beyond" in lib.ani_status_string(-7).decode()
