"""The allocation-free W4A16 GEMM entry point against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.  The entry point serves callers that cannot allocate device memory at
call time (a server that gave the whole GPU to its own arena, a latency-critical loop); its
split-K scratch is an array inside the library, shared by all calls, so the check is made on
two calls in a row: the second call finds the first call's partial sums in the scratch and
must not be disturbed by them."""
import numpy as np
import pytest
import torch

from oracle import kairos_oracle as ko

RTOL = ATOL = 1e-2


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.gpu
@pytest.mark.parametrize('m,k,n', [(16, 4096, 4096), (48, 1152, 96), (64, 4096, 1024)])
def test_no_alloc_gemm_matches_regular_entry_point(m, k, n):
    from kairos_b200 import ops, runtime
    from kairos_b200._lib import check, lib
    x, w = ko.make_case(m, k, n, seed=70 + m)
    res = ko.from_module(w)
    xd = _dev(x)
    qw, sc, sz = _dev(res['qweight']), _dev(res['scales']), _dev(res['scaled_zeros'])
    assert lib.kairos_gemm_workspace_bytes(m, n, k) > 0, 'case must exercise the split-K scratch'
    y_ref = ops.gemm_forward_cuda_new(xd, qw, sc, sz)            # regular entry point, torch-owned workspace
    oracle = ko.y_w4a16(x, res)
    st = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        y = torch.full((m, n), float('nan'), dtype=torch.float16, device='cuda')
        if call == 1:
            # a different problem in between leaves foreign partial sums in the shared scratch
            other = torch.empty((8, n), dtype=torch.float16, device='cuda')
            check(lib.kairos_w4a16_gemm_noalloc(xd[:8].contiguous().data_ptr(), qw.data_ptr(), sc.data_ptr(),
                                                sz.data_ptr(), None, other.data_ptr(), 8, n, k, st), 'noalloc')
        check(lib.kairos_w4a16_gemm_noalloc(xd.data_ptr(), qw.data_ptr(), sc.data_ptr(), sz.data_ptr(), None,
                                            y.data_ptr(), m, n, k, st), 'noalloc')
        torch.cuda.synchronize()
        yh, rh = y.cpu().numpy(), y_ref.cpu().numpy()
        bad, _ = ko.within_tolerance(yh, rh, RTOL, ATOL)
        assert bad == 0, f'call {call}: {bad} outputs differ from the regular entry point'
        bad, _ = ko.within_tolerance(yh, oracle, RTOL, ATOL)
        assert bad == 0, f'call {call}: {bad} outputs outside tolerance of the oracle'
    assert runtime.device_status() == 0


def test_no_alloc_gemm_rejects_oversize_and_bad_shapes():
    """Validation happens before any CUDA call, so this part runs without a GPU."""
    from kairos_b200._lib import lib
    assert lib.kairos_gemm_workspace_bytes(512, 4096, 4096) > (5 << 20)
    assert lib.kairos_w4a16_gemm_noalloc(16, 16, 16, 16, None, 16, 512, 4096, 4096, None) == -4
    assert b'5 MiB' in lib.kairos_last_error()
    assert lib.kairos_w4a16_gemm_noalloc(16, 16, 16, 16, None, 16, 4, 12, 128, None) == -1     # N % 8
    assert lib.kairos_w4a16_gemm_noalloc(16, 16, 16, 16, None, 16, 0, 64, 128, None) == 0      # M == 0
    for m in (1, 16, 33, 64):
        for n, k in ((4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336), (8192, 28672)):
            assert lib.kairos_gemm_workspace_bytes(m, n, k) <= (5 << 20)
