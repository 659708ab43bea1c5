"""forge_chol_inv_upper_noalloc: the factorisation entry point that allocates nothing.

It serves callers that cannot get device memory at the moment they need to factor a Hessian again — the
layer driver after it has committed all of HBM to its batches, or an application whose memory manager
forbids cudaMalloc — by keeping the workspace in an array inside the library.  The test calls it through
the C ABI twice in a row (the array is shared and keeps the previous call's contents) and compares with
the workspace-taking entry point, which runs the same kernels: the results must be identical.
"""
import pytest
import torch

from helpers import random_spd

pytestmark = pytest.mark.gpu


def _damped(C, seed):
    H = random_spd(C, seed)
    H[range(C), range(C)] += 0.01 * H.diag().mean()
    return torch.flip(H, (0, 1)).contiguous()


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    assert torch.cuda.is_available()
    from forge import _abi, ops
    dev = "cuda"
    max_c = _abi.query("forge_noalloc_max_c")
    assert max_c >= 2048
    warmed_up = False
    for C, seed in ((320, 91), (192, 92)):      # second call is smaller: stale scratch beyond it is ignored
        A = _damped(C, seed)
        U_ref, ud_ref, info_ref = ops.chol_inv_upper(A.clone().to(dev).view(1, C, C), zero_lower=True)
        A_d = A.clone().to(dev)
        U = torch.empty((C, C), dtype=torch.float32, device=dev)
        ud = torch.empty(C, dtype=torch.float32, device=dev)
        info = torch.full((1,), -1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()    # earlier tests may have frees pending on other streams: settle them first
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        _abi.call("forge_chol_inv_upper_noalloc", _abi.ptr(A_d), C, _abi.ptr(U), _abi.ptr(ud), _abi.ptr(info), 1,
                  _abi.stream_ptr())
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # torch's counter only sees torch's own allocator: the driver's view of free device memory must not move either
        # once the first call (which makes the runtime load the array's module) is behind us
        if warmed_up:
            assert torch.cuda.mem_get_info()[0] == free_before
        warmed_up = True
        assert int(info.item()) == 0 and int(info_ref.item()) == 0
        assert torch.equal(U, U_ref[0]) and torch.equal(ud, ud_ref[0])


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    from forge import _abi
    dev = "cuda"
    max_c = _abi.query("forge_noalloc_max_c")
    dummy = torch.zeros(16, dtype=torch.float32, device=dev)
    info = torch.zeros(1, dtype=torch.int32, device=dev)
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        _abi.call("forge_chol_inv_upper_noalloc", _abi.ptr(dummy), max_c + 64, _abi.ptr(dummy), _abi.ptr(dummy),
                  _abi.ptr(info), 1, _abi.stream_ptr())
