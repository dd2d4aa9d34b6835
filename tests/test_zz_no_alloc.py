"""The allocation-free second moment (collected last: a failure here cannot hide another test).

Who needs it: code that takes calibration statistics at a point where it must not allocate on
the device - a forward hook running while another framework's caching allocator owns the GPU, a
process in which a stream capture is under way, a deployment with a fixed memory budget.  The
entry point keeps the kernel's scratch (the per-item output tiles) in a 64 MiB array inside the
library, so the caller passes only the activations, the [K, K] sum and a status word.

Checked here, through the C-ABI, on two calls in a row: same sum as the workspace entry point
within the tolerance of the second-moment tests (the two may split the tokens differently, so
fp32 partial sums are added in a different order), the status word is cleared and stays zero,
device memory in use does not move, and sizes beyond the fixed scratch are refused."""

import pytest
import torch

from tests.helpers import DEV, activations

pytestmark = pytest.mark.gpu


def _norm_err(got, want):
    want = want.double().cpu()
    scale = want.diagonal().clamp_min(1e-30).sqrt()
    return ((got.double().cpu() - want) / (scale[:, None] * scale[None, :])).abs().max().item()


def _noalloc(x, s, status):
    from hi2_b200 import _lib

    _lib.call("hi2_hessian_accumulate_noalloc", _lib.ptr(x), _lib.DTYPES[x.dtype], x.shape[0], x.shape[1],
              _lib.ptr(s), _lib.ptr(status), _lib.stream(x.device))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_two_calls_match_the_workspace_entry_point(dtype):
    from hi2_b200.hessian import HessianStats

    tokens, k = 20000, 1024
    xa = activations(tokens, k, 41, dtype=dtype).to(DEV)
    xb = activations(tokens // 2 + 7, k, 42, dtype=dtype).to(DEV)
    ref = HessianStats(k, DEV)
    s = torch.zeros(k, k, device=DEV)
    status = torch.full((1,), 99, dtype=torch.int32, device=DEV)  # the call must clear it
    torch.cuda.synchronize()
    for i, x in enumerate((xa, xb)):
        ref.update(x)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        used_before = torch.cuda.memory_allocated()
        _noalloc(x, s, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        if i == 1:  # by now nothing lazy is left to load: the call itself must hold no new memory
            assert torch.cuda.mem_get_info()[0] >= free_before - (2 << 20)  # the scratch would be >= 8 MiB
        assert torch.cuda.memory_allocated() == used_before
        assert _norm_err(s, ref.S) < 1e-5, _norm_err(s, ref.S)
        assert torch.equal(s, s.T)
    want = xa.double().T @ xa.double() + xb.double().T @ xb.double()
    assert _norm_err(s, want) < 2e-5


def test_sizes_beyond_the_fixed_scratch_are_refused():
    x = torch.zeros(256, 8192, dtype=torch.bfloat16, device=DEV)
    s = torch.zeros(8192, 8192, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="fixed scratch"):
        _noalloc(x, s, status)
    with pytest.raises(ValueError):
        _noalloc(torch.zeros(64, 512, dtype=torch.bfloat16, device=DEV), torch.zeros(512, 512, device=DEV), status)
    with pytest.raises(ValueError):
        _noalloc(torch.zeros(512, 512, device=DEV), torch.zeros(512, 512, device=DEV), status)


def test_widest_input_of_the_fixed_scratch_and_the_first_one_beyond():
    """K = 5632 fills the 512-tile array (506 upper-triangle tiles): with enough tokens for the
    planner to want several token splits, the split count must be clamped to what the array holds and
    the sum still be right; K = 5648 (the next multiple of 16) is refused."""
    from hi2_b200.hessian import HessianStats

    k, tokens = 5632, 40000
    x = activations(tokens, k, 43, dtype=torch.bfloat16).to(DEV)
    ref = HessianStats(k, DEV)
    ref.update(x)
    s = torch.zeros(k, k, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _noalloc(x, s, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert _norm_err(s, ref.S) < 1e-5 and torch.equal(s, s.T)
    with pytest.raises(RuntimeError, match="fixed scratch"):
        _noalloc(torch.zeros(256, 5648, dtype=torch.bfloat16, device=DEV), torch.zeros(5648, 5648, device=DEV), status)
