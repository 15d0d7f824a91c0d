"""ctypes view of the C ABI in ``include/slayer_b200.h``.

For callers that hold raw device pointers (``tensor.data_ptr()``, CuPy, cuda-python ...).
Every function of the header is declared here with its argument types; ``SYMBOLS`` is the
list the tests check against the header.  Loading fails loudly when the library is not built.
"""
import ctypes
import os

from . import LIB_DIR

LIB_PATH = os.path.join(LIB_DIR, "libslayer_b200.so")

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_u32 = ctypes.c_uint32
_f = ctypes.c_float
_int = ctypes.c_int

SYMBOLS = {
    "slayer_b200_abi_version": (_int, []),
    "slayer_b200_last_error": (ctypes.c_char_p, []),
    "slayer_b200_conv": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "slayer_b200_corr": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "slayer_b200_corr_spike_grad": (_int, [_p, _p, _p, _p, _i64, _i64, _i64, _f, _f, _f, _f, _p]),
    "slayer_b200_shift_scalar": (_int, [_p, _p, _f, _i64, _i64, _f, _p]),
    "slayer_b200_shift_lut": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "slayer_b200_srm_get_spikes": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _f, _p]),
    "slayer_b200_srm_get_spikes_noalloc": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _f, _p]),
    "slayer_b200_srm_get_spikes_noalloc_status": (_int, [_i64, _i64, ctypes.POINTER(_i64)]),
    "slayer_b200_selftest_bounded_wait": (_int, [_int, _p]),
    "slayer_b200_pack_spikes": (_int, [_p, _p, _i64, _i64, _p]),
    "slayer_b200_unpack_spikes": (_int, [_p, _p, _i64, _i64, _f, _p]),
    "slayer_b200_srm_get_spikes_packed": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "slayer_b200_conv_packed": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _f, _p]),
    "slayer_b200_bin_events": (_int, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64,
                                      ctypes.c_double, _i64, _int, _p]),
    "slayer_b200_bin_events_packed": (_int, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64,
                                             ctypes.c_double, _i64, _p]),
    "slayer_b200_num_spikes_loss": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _f, _f, _p]),
    "slayer_b200_loihi_get_spikes": (_int, [_p, _p, _p, _p, _i64, _i64, _u32, _u32, _u32, _u32, _u32, _p]),
    "slayer_b200_loihi_get_spikes_delayed": (_int, [_p, _p, _p, _p, _i64, _i64, _u32, _u32, _u32, _u32, _u32, _i64, _p]),
    "slayer_b200_spike_grad": (_int, [_p, _p, _p, _i64, _f, _f, _f, _p]),
    "slayer_b200_srm_get_spikes_delayed": (_int, [_p, _p, _p, _p, _p, _f, _i64, _i64, _i64, _i64, _f, _f, _p]),
    "slayer_b200_spike_grad_shift": (_int, [_p, _p, _p, _p, _f, _i64, _i64, _i64, _f, _f, _f, _f, _p]),
    "slayer_b200_delay_grad": (_int, [_p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "slayer_b200_device_status": (_int, [ctypes.POINTER(ctypes.c_int)]),
    "slayer_b200_set_tma": (_int, [_int]),
    "slayer_b200_set_fir_packed": (_int, [_int]),
    "slayer_b200_set_fir_skip_zeros": (_int, [_int]),
    "slayer_b200_set_fir_flow": (_int, [_int]),
    "slayer_b200_set_srm_stages": (_int, [_int]),
}

_lib = None


class SlayerB200Error(RuntimeError):
    pass


def load():
    """dlopen the library and declare every entry point."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise OSError("slayer_b200: %s is not built (run `python -m slayerpytorch_b200.build`); "
                          "there is no CPU fallback" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)         # AttributeError if the symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc, what):
    if rc != 0:
        msg = load().slayer_b200_last_error()
        raise SlayerB200Error("%s failed (%d): %s" % (what, rc, (msg or b"").decode()))


def call(name, *args):
    """Call an entry point by name and raise SlayerB200Error on a non-zero return code."""
    rc = getattr(load(), name)(*args)
    check(rc, name)


def device_status():
    """Read and clear the device-side status word of the current device (synchronises)."""
    value = ctypes.c_int(0)
    check(load().slayer_b200_device_status(ctypes.byref(value)), "slayer_b200_device_status")
    return value.value


def set_fir_packed(mode):
    """Select the conv / corr kernel: 0 / False = scalar, 1 / True = packed (tile size chosen per
    launch), 2 = packed with half-size tiles (two CTAs per SM), 3 = packed with full-size tiles.
    Returns the previous setting."""
    return int(load().slayer_b200_set_fir_packed(int(mode)))


def set_fir_flow(mode):
    """Form of the scalar conv / corr kernel: 1 = no per-tile barrier, 2 = the same with more
    registers and 16-byte accesses for rows off the 16-byte grid (default), 3 = as 2 without the
    latter, 0 = one barrier per tile.  Returns the previous setting."""
    return int(load().slayer_b200_set_fir_flow(int(mode)))


def set_srm_stages(stages):
    """Stages per warp of the SRM spike kernel in large launches (2 .. 8); returns the previous setting."""
    return int(load().slayer_b200_set_srm_stages(int(stages)))


def set_fir_skip_zeros(mode):
    """Zero skipping in conv / corr / conv_packed: 0 / False = never, 1 / True = a probe on the device
    picks the event-driven kernel for mostly-zero inputs (default), 2 = the event-driven kernel for
    every input it can take.  Returns the previous setting."""
    return int(load().slayer_b200_set_fir_skip_zeros(int(mode)))


def set_tma(enable):
    """Enable/disable the bulk-tensor-copy kernels; returns the previous setting."""
    return bool(load().slayer_b200_set_tma(1 if enable else 0))
