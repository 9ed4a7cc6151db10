"""smoe_count_cumsum_noalloc: the histogram / prefix sum for callers that cannot provide a workspace.

Some hosts of this library own every byte of device memory themselves (memory planned ahead of time, a single
allocator the library has no access to) or sit at a point where an allocation's device-wide synchronisation is
not acceptable; they can pass inputs and outputs only.  For them the library carries its scratch inside itself.
This test calls the entry point through the C ABI, twice in a row on different inputs (the scratch is shared and
keeps the previous call's contents), and requires exactly the results of the workspace-taking entry point.

The file name sorts last on purpose: a run that stops at the first failure has then run every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, _lib, x, E):
    dev = x.device
    stream = torch.cuda.current_stream().cuda_stream
    code = _lib.dtype_code(x.dtype)
    want_c = torch.full((E,), -1, dtype=torch.int32, device=dev)
    want_s = torch.full((E,), -1, dtype=torch.int32, device=dev)
    ws = torch.empty(lib.smoe_count_cumsum_workspace_bytes(E) // 4, dtype=torch.int32, device=dev)
    assert lib.smoe_count_cumsum(x.data_ptr(), code, x.numel(), E, want_c.data_ptr(), want_s.data_ptr(),
                                 ws.data_ptr(), stream) == 0
    got_c = torch.full((E,), -2, dtype=torch.int32, device=dev)
    got_s = torch.full((E,), -2, dtype=torch.int32, device=dev)
    assert lib.smoe_count_cumsum_noalloc(x.data_ptr(), code, x.numel(), E, got_c.data_ptr(), got_s.data_ptr(),
                                         stream) == 0
    torch.cuda.synchronize()
    return (got_c, got_s), (want_c, want_s)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row(built_library):
    from sonicmoe import _lib

    lib = _lib.lib
    assert torch.cuda.is_available()
    limit = lib.smoe_count_cumsum_noalloc_max_experts()
    assert limit == 1024
    g = torch.Generator().manual_seed(0)
    # first call: many bins, long input; second call right after it: fewer bins, different length and dtype,
    # so stale scratch contents from the first call would show
    cases = [(262144, 1024, torch.int32), (5003, 128, torch.int64), (0, 8, torch.int32), (77, limit, torch.int32)]
    for n, E, dt in cases:
        x = torch.randint(0, E, (n,), generator=g, dtype=dt).cuda()
        (got_c, got_s), (want_c, want_s) = _both(lib, _lib, x, E)
        assert torch.equal(got_c, want_c), (n, E)
        assert torch.equal(got_s, want_s), (n, E)
        assert torch.equal(got_c.cpu(), torch.bincount(x.cpu().long(), minlength=E).int())

    # count only (no cumsum requested)
    x = torch.randint(0, 64, (1000,), generator=g, dtype=torch.int32).cuda()
    only = torch.empty(64, dtype=torch.int32, device="cuda")
    assert lib.smoe_count_cumsum_noalloc(x.data_ptr(), _lib.SMOE_I32, 1000, 64, only.data_ptr(), None,
                                         torch.cuda.current_stream().cuda_stream) == 0
    assert torch.equal(only.cpu(), torch.bincount(x.cpu().long(), minlength=64).int())


def test_noalloc_rejects_sizes_beyond_its_scratch(built_library):
    from sonicmoe import _lib

    lib = _lib.lib
    limit = lib.smoe_count_cumsum_noalloc_max_experts()
    x = torch.zeros(16, dtype=torch.int32, device="cuda")
    out = torch.empty(limit + 4, dtype=torch.int32, device="cuda")
    rc = lib.smoe_count_cumsum_noalloc(x.data_ptr(), _lib.SMOE_I32, 16, limit + 4, out.data_ptr(), None, None)
    assert rc == -8  # SMOE_ERR_NOALLOC_LIMIT: nothing launched
    with pytest.raises(_lib.SonicMoEError, match="built-in scratch"):
        _lib.check(rc, "count_cumsum_noalloc")
