"""GPU: the entry point that allocates nothing must give what the regular one gives.

Some users of this library cannot call cudaMalloc when they reach the spike kernel: their
application owns all device memory through its own pool, or they call from a place where the
CUDA allocator must not be entered.  ``slayer_b200_srm_get_spikes_noalloc`` serves them with
scratch memory that is a fixed array inside the library.  Because that array is shared by all
calls and keeps what the previous call left in it, the check is made on two calls in a row
with different data.  This file sorts last on purpose: a run that stops at the first failure
has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from slayerpytorch_b200 import capi

pytestmark = pytest.mark.gpu


def run(entry, u0, nu, theta, Ts):
    u = u0.clone()
    s = torch.empty_like(u)
    T = u.shape[-1]
    rc = getattr(capi.load(), entry)(
        ctypes.c_void_p(s.data_ptr()), ctypes.c_void_p(u.data_ptr()), ctypes.c_void_p(nu.data_ptr()),
        u.numel() // T, nu.numel(), T, float(theta), float(Ts),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    capi.check(rc, entry)
    torch.cuda.synchronize()
    return s, u


def test_no_alloc_entry_point_matches_regular_one_on_two_calls_in_a_row():
    gen = torch.Generator().manual_seed(77)
    nu = torch.tensor([-0.0, -20.0, -14.7, -8.1, -4.0, -1.8, -0.8, -0.3, -0.1, -0.05, -0.02]).cuda()
    cases = [((4, 37, 1, 3, 300), 8.0), ((2, 700, 1, 1, 64), 12.0)]     # second call: more row blocks, other T
    for shape, scale in cases:
        u0 = (torch.randn(shape, generator=gen) * scale).cuda()
        s_ref, u_ref = run("slayer_b200_srm_get_spikes", u0, nu, 10.0, 1.0)
        s_new, u_new = run("slayer_b200_srm_get_spikes_noalloc", u0, nu, 10.0, 1.0)
        assert s_ref.sum() > 0
        assert torch.equal(s_new, s_ref)                 # bit-exact, as for the regular entry point
        assert torch.equal(u_new, u_ref)
    # the same data again after the array has been used by a larger launch
    s_again, u_again = run("slayer_b200_srm_get_spikes_noalloc", u0, nu, 10.0, 1.0)
    assert torch.equal(s_again, s_ref) and torch.equal(u_again, u_ref)


def test_no_alloc_entry_point_rejects_what_it_has_no_scratch_for():
    lib = capi.load()
    one = ctypes.c_void_p(256)
    null = ctypes.c_void_p(0)
    too_many_rows = 65536 * 32 + 1
    assert lib.slayer_b200_srm_get_spikes_noalloc(one, ctypes.c_void_p(512), one, too_many_rows, 11, 300,
                                                  10.0, 1.0, null) == -3
    assert b"exceed" in lib.slayer_b200_last_error()
    # row length that is not a multiple of four cannot use bulk tensor copies
    assert lib.slayer_b200_srm_get_spikes_noalloc(one, ctypes.c_void_p(512), one, 64, 11, 301, 10.0, 1.0, null) == -3
