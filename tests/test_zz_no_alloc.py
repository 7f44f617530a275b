"""db_colsum_static: the column-sum entry point for callers that cannot allocate.

A host that has given all device memory to its own pool, or that runs where
cudaMalloc is not permitted, still needs the bias gradient (a column sum).  This
variant keeps its partial sums in an array compiled into the library.  It must
agree with db_colsum bit for bit (same kernels, same order), twice in a row,
since every call reuses the same array; sizes beyond the array are refused."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_allocating_entry_point_twice(cuda):
    import torch
    from deepbind_b200 import _lib, SmatException
    from deepbind_b200.smat import bind_stream
    dll = _lib.load()
    bind_stream()
    rng = np.random.default_rng(123)
    for call, (nrow, ncol) in enumerate([(15895, 16), (3001, 130)]):
        A = torch.from_numpy(rng.standard_normal((nrow, ncol)).astype(np.float32)).cuda()
        want = torch.empty(ncol, dtype=torch.float32, device="cuda")
        got = torch.full((ncol,), float("nan"), dtype=torch.float32, device="cuda")
        dll.db_colsum(want.data_ptr(), A.data_ptr(), nrow, ncol)
        dll.db_colsum_static(got.data_ptr(), A.data_ptr(), nrow, ncol)
        torch.cuda.synchronize()
        assert torch.equal(got, want), "call %d differs" % call
        ref = A.double().sum(dim=0)
        assert float((got.double() - ref).abs().max()) <= 1e-5 * float(A.abs().sum(dim=0).max())
    # No device memory is created by the static entry point: after the priming calls above
    # (the address look-up happens in the first one), the driver's count of free bytes is the
    # same before and after further calls, and so is torch's allocator (which the library
    # never goes through).  The buffers are made before the first reading.
    A = torch.from_numpy(rng.standard_normal((9000, 64)).astype(np.float32)).cuda()
    got = torch.empty(64, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0 = torch.cuda.memory_reserved()
    scratch0 = dll.db_scratch_bytes()
    for _ in range(3):
        dll.db_colsum_static(got.data_ptr(), A.data_ptr(), 9000, 64)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "db_colsum_static changed the device's free memory by %d bytes" % (free0 - free1)
    assert torch.cuda.memory_reserved() == reserved0 and dll.db_scratch_bytes() == scratch0
    assert float((got.double() - A.double().sum(dim=0)).abs().max()) <= 1e-5 * float(A.abs().sum(dim=0).max())
    # beyond the built-in array: a clear error, nothing launched
    big = torch.zeros((4, 8), dtype=torch.float32, device="cuda")
    out = torch.zeros(70000, dtype=torch.float32, device="cuda")
    with pytest.raises(SmatException, match="db_colsum_static supports"):
        dll.db_colsum_static(out.data_ptr(), big.data_ptr(), 1025, 70000)
    # an empty input still gives zeros
    dll.db_colsum_static(out.data_ptr(), big.data_ptr(), 0, 8)
    torch.cuda.synchronize()
    assert float(out[:8].abs().max()) == 0.0
