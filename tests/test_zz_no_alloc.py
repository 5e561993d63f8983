"""The allocation-free Hausdorff entry point, called through the C ABI.

Who needs it: host code that may not allocate device memory at call time (a server whose memory
pool already owns the whole GPU, a plug-in whose compute callback is forbidden to allocate, a
real-time loop that cannot absorb an allocator stall).  The regular entry point asks such a
caller for scratch; this one uses a fixed array inside the library instead, so it must give the
same answers -- including on a second call, when the array still holds the first call's keys.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, static, x1, x2):
    from torchpairwise_b200 import _abi
    B, N1, M1, D = x1.shape
    N2, M2 = x2.shape[1], x2.shape[2]
    out = torch.empty(B, N1, N2, device="cuda")
    i1 = torch.empty(B, N1, N2, dtype=torch.int64, device="cuda")
    i2 = torch.empty(B, N1, N2, dtype=torch.int64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    if static:
        st = lib.tpw_hausdorff_forward_static(_abi.F32, x1.data_ptr(), x2.data_ptr(), None, None, out.data_ptr(),
                                              i1.data_ptr(), i2.data_ptr(), B, N1, N2, M1, M2, D, stream)
    else:
        scratch = torch.empty(lib.tpw_hausdorff_scratch_bytes(B, N1, N2, M1), dtype=torch.uint8, device="cuda")
        st = lib.tpw_hausdorff_forward(_abi.F32, x1.data_ptr(), x2.data_ptr(), None, None, out.data_ptr(),
                                       i1.data_ptr(), i2.data_ptr(), scratch.data_ptr(), B, N1, N2, M1, M2, D, stream)
    _abi.check(st, "hausdorff forward")
    torch.cuda.synchronize()
    return out, i1, i2


def test_static_scratch_entry_point_matches_the_regular_one():
    from torchpairwise_b200 import _abi
    lib = _abi.lib
    assert lib.tpw_hausdorff_static_max_pairs() == 65536
    g = torch.Generator().manual_seed(31)
    # first call: 24 set pairs, several CTAs per pair
    a1 = torch.rand(2, 4, 3000, 3, generator=g).cuda()
    b1 = torch.rand(2, 3, 2500, 3, generator=g).cuda()
    # second call right after it: fewer pairs and other data, so stale keys of the first call
    # would show if the array were not cleared
    a2 = torch.rand(1, 3, 700, 3, generator=g).cuda() * 0.01
    b2 = torch.rand(1, 2, 900, 3, generator=g).cuda() * 0.01
    ref1 = _call(lib, False, a1, b1)
    ref2 = _call(lib, False, a2, b2)
    got1 = _call(lib, True, a1, b1)
    free_before, _ = torch.cuda.mem_get_info()
    got2 = _call(lib, True, a2, b2)
    free_after, _ = torch.cuda.mem_get_info()
    for got, ref in ((got1, ref1), (got2, ref2)):
        assert torch.equal(got[0], ref[0])  # same kernels, same arithmetic: identical bits
        assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])
    # the outputs above were allocated by the test before the call; the call itself takes nothing
    assert free_after >= free_before - (1 << 20)
    # a third call repeats the first problem on the now-dirty array
    got3 = _call(lib, True, a1, b1)
    assert torch.equal(got3[0], ref1[0]) and torch.equal(got3[1], ref1[1]) and torch.equal(got3[2], ref1[2])


def test_static_scratch_entry_point_refuses_oversized_problems():
    from torchpairwise_b200 import _abi
    lib = _abi.lib
    x = torch.rand(1, 1, 4, 3, device="cuda")
    # 257 * 256 = 65792 set pairs > 65536: refused on the host, nothing launched, pointers untouched
    st = lib.tpw_hausdorff_forward_static(_abi.F32, x.data_ptr(), x.data_ptr(), None, None, x.data_ptr(),
                                          x.data_ptr(), x.data_ptr(), 1, 257, 256, 4, 4, 3, None)
    assert st == 1
    msg = lib.tpw_last_error().decode()
    assert "65792" in msg and "65536" in msg
    torch.cuda.synchronize()
