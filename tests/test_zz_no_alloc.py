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


def finished(rows, T):
    """What the entry point's own array says about its last launch: (return code, first block
    of 32 rows that was not walked to the end, or -1)."""
    bad = ctypes.c_int64(-7)
    rc = capi.load().slayer_b200_srm_get_spikes_noalloc_status(rows, T, ctypes.byref(bad))
    return rc, bad.value


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
        assert finished(u0.numel() // shape[-1], shape[-1]) == (0, -1)      # every row block ran to its end
    # the same data again after the array has been used by a larger launch
    s_again, u_again = run("slayer_b200_srm_get_spikes_noalloc", u0, nu, 10.0, 1.0)
    assert torch.equal(s_again, s_ref) and torch.equal(u_again, u_ref)


@pytest.mark.parametrize("taps", [2, 34, 110, 257])
def test_no_alloc_entry_point_with_long_refractory_kernels(taps):
    """Refractory kernels of 34 to 257 taps keep their taps in shared memory (other variants of
    the kernel than the 11-tap case above); two calls in a row again."""
    gen = torch.Generator().manual_seed(taps)
    nu = (-torch.rand(taps, generator=gen) * 6).cuda()
    for shape in ((3, 50, 1, 1, 300), (2, 9, 1, 7, 128)):
        u0 = (torch.randn(shape, generator=gen) * 8).cuda()
        s_ref, u_ref = run("slayer_b200_srm_get_spikes", u0, nu, 10.0, 1.0)
        s_new, u_new = run("slayer_b200_srm_get_spikes_noalloc", u0, nu, 10.0, 1.0)
        assert s_ref.sum() > 0
        assert torch.equal(s_new, s_ref) and torch.equal(u_new, u_ref)
        assert finished(u0.numel() // shape[-1], shape[-1]) == (0, -1)


def test_no_alloc_entry_point_at_its_row_limit():
    """Exactly 65536 blocks of 32 rows - every entry of the array - is accepted (rows of four
    steps keep the tensors small); the status reader covers all of them."""
    rows, T = 65536 * 32, 4
    gen = torch.Generator().manual_seed(4)
    nu = torch.tensor([0.0, -20.0, -14.7]).cuda()
    u0 = (torch.randn(rows, 1, 1, 1, T, generator=gen) * 8).cuda()
    s_ref, u_ref = run("slayer_b200_srm_get_spikes", u0, nu, 10.0, 1.0)
    for _ in range(2):
        s_new, u_new = run("slayer_b200_srm_get_spikes_noalloc", u0, nu, 10.0, 1.0)
        assert torch.equal(s_new, s_ref) and torch.equal(u_new, u_ref)
        assert finished(rows, T) == (0, -1)
    # a smaller launch afterwards leaves the tail of the array as the large one set it: the
    # reader is told the size of the launch it is asked about, and a size that was not the last
    # launch's reads as unfinished blocks
    small = (torch.randn(64, 1, 1, 1, 128, generator=gen) * 8).cuda()
    run("slayer_b200_srm_get_spikes_noalloc", small, nu, 10.0, 1.0)
    assert finished(64, 128) == (0, -1)
    rc, bad = finished(96, 128)
    assert rc == -4 and bad == 2


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
