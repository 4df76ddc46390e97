"""The peer-memory mean kernel (ani_peer_*) on ONE GPU: the single-rank case, graph capture, and the bounded
wait -- a peer that never arrives makes the call end with ANI_ERR_TIMEOUT in the device status word instead
of hanging, and the context stays usable.  (The several-rank case runs in bench.py, which checks the result
against the library all-reduce.)"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _create(L, rank, world, n):
    p = ctypes.c_void_p()
    assert L.ani_peer_create(rank, world, n, ctypes.byref(p)) == 0
    return p


@pytest.mark.parametrize("two_halves", [0, 1])
def test_single_rank_mean_is_the_identity_and_replays_in_a_graph(two_halves):
    import torch
    from khan_b200 import _lib, ani_mod
    L = _lib.lib()
    n = 296_464
    p = _create(L, 0, 1, n)
    assert L.ani_peer_set_two_halves(p, two_halves) == 0
    x = torch.randn(n, device="cuda")
    want = x.clone()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):       # the staging buffer alternates, the step counter advances on the device
        assert L.ani_peer_mean_f32(p, x.data_ptr(), n, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(x, want)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert L.ani_peer_mean_f32(p, x.data_ptr(), n, s) == 0
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(x, want) and ani_mod.device_status() == 0
    # argument checks: length not a multiple of 4, longer than the capacity, misaligned buffer
    assert L.ani_peer_mean_f32(p, x.data_ptr(), 10, stream) == -2
    assert L.ani_peer_mean_f32(p, x.data_ptr(), n + 4, stream) == -2
    assert L.ani_peer_mean_f32(p, x.data_ptr() + 4, n - 4, stream) == -9
    assert L.ani_peer_destroy(p) == 0


@pytest.mark.parametrize("two_halves", [0, 1])
def test_a_rank_that_never_arrives_ends_the_wait_with_a_status_not_a_hang(two_halves):
    import torch
    import gpu_util
    from khan_b200 import _lib, ani_mod
    L = _lib.lib()
    n = 4096
    me, absent = _create(L, 0, 2, n), _create(L, 1, 2, n)     # rank 1 exists but never calls
    assert L.ani_peer_set_two_halves(me, two_halves) == 0
    assert L.ani_peer_connect_raw(me, 1, L.ani_peer_block(absent)) == 0
    assert L.ani_peer_connect_raw(me, 1, L.ani_peer_block(absent)) == -6   # already connected
    assert L.ani_peer_set_spin_limit(me, 2000) == 0           # a fraction of a millisecond
    assert ani_mod.device_status() == 0
    x = torch.ones(n, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.ani_peer_mean_f32(me, x.data_ptr(), n, stream) == 0
    assert ani_mod.device_status() == -8                       # ANI_ERR_TIMEOUT, and reading clears it
    assert ani_mod.device_status() == 0
    # the call ended like any other (the absent rank's staging buffers hold zeros: its own slice is 1/2,
    # and in the two-halves form the absent rank's slice comes back as the zeros it never replaced) ...
    want = torch.full_like(x, 0.5)
    if two_halves:
        want[n // 2:] = 0.0
    assert torch.equal(x, want)
    # ... and the context is fine: another kernel of the library runs and is right
    a = np.random.default_rng(0).integers(0, 4, 1000).astype(np.int32)
    si, gi, ac = gpu_util.gpu_sort(a)
    assert ac.sum() == 1000
    # an unconnected rank is refused on the host
    lonely = _create(L, 0, 2, n)
    assert L.ani_peer_mean_f32(lonely, x.data_ptr(), n, stream) == -1
    for h in (me, absent, lonely):
        assert L.ani_peer_destroy(h) == 0
