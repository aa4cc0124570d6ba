"""The workspace-free scan (`b200c_exclusive_scan_static`) against the regular one.

Some hosts of this library cannot give it a workspace: their GPU memory is planned and handed out
before the first request, or they run under a "no allocation once warmed up" rule because
cudaMalloc/cudaFree stall the whole device.  For them the library keeps the scan's partial sums in
a fixed 64 KiB array of its own.  The test calls that entry point through the C ABI twice in a row
(a large input, then a smaller one, so the second call runs over whatever the first left in the
array) and demands exactly the offsets `b200c_exclusive_scan` produces; it also checks that an
input beyond the fixed capacity is refused instead of overrunning the array.

The file sorts last on purpose: a run that stops at the first failure has then seen every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _scan_static(counts):
    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    m = counts.numel()
    offsets = torch.full((m + 1,), -7, dtype=torch.long, device=counts.device)
    status = lib.b200c_exclusive_scan_static(counts.data_ptr(), m, offsets.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
    return status, offsets


def test_static_scan_matches_workspace_scan_on_consecutive_calls():
    from pytorch_cluster_b200 import _native, cabi

    g = torch.Generator().manual_seed(2024)
    sizes = [3_000_001, 70_001, 1, 2048, 2049]  # consecutive calls share (and overwrite) the one array
    for m in sizes:
        counts = torch.randint(0, 5000, (m,), generator=g, dtype=torch.int32).to(DEV)
        want = cabi.exclusive_scan(counts)
        status, got = _scan_static(counts)
        assert status == _native.B200C_OK, _native.cabi().b200c_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"m={m}: offsets differ from b200c_exclusive_scan"
        # and against plain arithmetic, so that two equal mistakes cannot agree
        ref = torch.zeros(m + 1, dtype=torch.long)
        ref[1:] = torch.cumsum(counts.cpu().long(), 0)
        assert torch.equal(got.cpu(), ref)


def test_static_scan_empty_input():
    from pytorch_cluster_b200 import _native

    status, got = _scan_static(torch.empty(0, dtype=torch.int32, device=DEV))
    assert status == _native.B200C_OK
    assert got.tolist() == [0]


def test_static_scan_refuses_inputs_beyond_its_fixed_scratch():
    from pytorch_cluster_b200 import _native

    lib = _native.cabi()
    too_many = (1 << 24) + 1
    # the size check comes first: no pointer is touched and nothing is launched
    status = lib.b200c_exclusive_scan_static(None, too_many, None, None)
    assert status == 4  # B200C_ERR_WORKSPACE
    msg = lib.b200c_last_error().decode()
    assert "at most" in msg and str(1 << 24) in msg
