"""apus_cuda_dispatch_dev_static — the dispatch for callers that cannot call
the device allocator (a server whose own pool owns all of HBM, or code inside
a no-allocation section): its scratch is an array built into the library.

Checked through the C-ABI against apus_cuda_dispatch_dev on the same device
buffers, twice in a row with different sizes, so the second call runs over
whatever the first left in the shared array.  Collected last on purpose."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(gpu, torch, T, TK, E, seed):
    rng = np.random.default_rng(seed)
    idx = np.stack([rng.choice(E, TK, replace=False) for _ in range(T)]
                   ).astype(np.int32)
    d_idx = torch.from_numpy(idx).cuda()
    outs = []
    for fn in (gpu.dispatch_dev, gpu.dispatch_dev_static):
        counts = torch.full((E,), -1, dtype=torch.int32, device="cuda")
        offsets = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
        perm = torch.full((T * TK,), -1, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        fn(d_idx.data_ptr(), T, TK, E, counts.data_ptr(), offsets.data_ptr(),
           perm.data_ptr(), stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        outs.append((counts.cpu().numpy(), offsets.cpu().numpy(),
                     perm.cpu().numpy()))
    for a, b in zip(*outs):
        assert np.array_equal(a, b)          # integer work: bit-exact
    assert np.array_equal(outs[1][2], np.argsort(idx.ravel(), kind="stable"))


def test_static_scratch_dispatch_matches_twice_in_a_row(gpu):
    import torch
    _case(gpu, torch, 2000, 8, 256, 1)       # three-pass path, uses the array
    _case(gpu, torch, 700, 8, 256, 2)        # smaller: stale entries remain
    _case(gpu, torch, 3, 8, 256, 3)          # single-block path


def test_static_scratch_dispatch_allocates_nothing(gpu):
    """After one call (which looks up the array's address), further calls leave
    the device's free memory exactly where it was: the caller whose pool owns
    the rest of HBM never sees the library take a byte."""
    import torch
    T, TK, E = 2000, 8, 256
    rng = np.random.default_rng(4)
    idx = torch.from_numpy(rng.integers(0, E, (T, TK)).astype(np.int32)).cuda()
    counts = torch.empty((E,), dtype=torch.int32, device="cuda")
    offsets = torch.empty((E + 1,), dtype=torch.int32, device="cuda")
    perm = torch.empty((T * TK,), dtype=torch.int32, device="cuda")
    sp = torch.cuda.current_stream().cuda_stream
    args = (idx.data_ptr(), T, TK, E, counts.data_ptr(), offsets.data_ptr(),
            perm.data_ptr())
    gpu.dispatch_dev_static(*args, stream=sp)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        gpu.dispatch_dev_static(*args, stream=sp)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0


def test_static_scratch_dispatch_refuses_oversize(gpu):
    import torch
    T, TK, E = 40000, 8, 1000                # 1250 units * 1000 > 262144
    d = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(Exception) as ei:
        gpu.dispatch_dev_static(d.data_ptr(), T, TK, E, d.data_ptr(),
                                d.data_ptr(), d.data_ptr())
    assert "exceeds" in str(ei.value)
