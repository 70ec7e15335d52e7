"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

TORCH_DT = {"f16": torch.float16, "bf16": torch.bfloat16}
# required tolerance for 16-bit outputs against the fp32 reference
RTOL, ATOL = 2e-2, 2e-2


def dev(a, dtype=None):
    """numpy -> CUDA tensor (float arrays are cast to the 16-bit storage dtype)."""
    t = torch.from_numpy(np.ascontiguousarray(a))
    if t.dtype == torch.float32 and dtype is not None:
        t = t.to(TORCH_DT[dtype])
    return t.cuda()


def host(t):
    return t.detach().float().cpu().numpy()


def assert_close(got, want, rtol=RTOL, atol=ATOL):
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol)


def assert_lse_close(got, want):
    assert np.array_equal(np.isneginf(got), np.isneginf(want))
    live = ~np.isneginf(want)
    np.testing.assert_allclose(got[live], want[live], rtol=1e-3, atol=2e-3)
