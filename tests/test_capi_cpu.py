"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, and rejects
bad arguments before touching the GPU."""
import ctypes
import os
import re

import pytest

from slayerpytorch_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(slayer_b200_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    declared = header_symbols()
    assert declared, "no declarations found in include/*.h"
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(capi.SYMBOLS), declared ^ set(capi.SYMBOLS)
    assert lib.slayer_b200_abi_version() >= 1


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    text = open(os.path.join(ROOT, "include", "slayer_b200.h")).read()
    for m in re.finditer(r"/\*((?:(?!\*/).)*)\*/\s*int (slayer_b200_\w+)\(", text, flags=re.S):
        comment, name = m.group(1), m.group(2)
        if name == "slayer_b200_abi_version":
            continue
        assert re.search(r"src/[\w/]+\.(h|cu|py):\d+", comment) or "no counterpart" in comment, name


def test_argument_validation_needs_no_gpu():
    lib = capi.load()
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)
    # negative sizes
    assert lib.slayer_b200_conv(one, one, one, -1, 4, 2, 1.0, null) == -1
    assert b"negative" in lib.slayer_b200_last_error()
    assert lib.slayer_b200_shift_scalar(one, one, 1.0, 2, -4, 1.0, null) == -1
    # null pointers with non-empty work
    assert lib.slayer_b200_corr(null, one, one, 2, 4, 2, 1.0, null) == -1
    assert b"null" in lib.slayer_b200_last_error()
    assert lib.slayer_b200_srm_get_spikes(null, null, null, 2, 3, 4, 1.0, 1.0, null) == -1
    assert lib.slayer_b200_spike_grad(null, null, null, 8, 1.0, 1.0, 1.0, null) == -1
    # aliasing that the kernels do not support
    assert lib.slayer_b200_conv(one, one, one, 2, 4, 2, 1.0, null) == -1
    assert b"alias" in lib.slayer_b200_last_error()
    # Loihi refractory delay of zero is undefined in the reference and rejected here
    assert lib.slayer_b200_loihi_get_spikes(one, one, one, one, 2, 4, 0, 80, 1, 1, 0, null) == -1
    assert b"refDelay" in lib.slayer_b200_last_error()
    # empty work is a successful no-op
    assert lib.slayer_b200_conv(null, null, null, 0, 4, 2, 1.0, null) == 0
    assert lib.slayer_b200_shift_lut(null, null, null, 0, 5, 4, 1.0, null) == 0
    assert lib.slayer_b200_loihi_get_spikes(null, null, null, null, 0, 4, 0, 80, 1, 1, 1, null) == 0
    assert lib.slayer_b200_last_error() == b""
    with pytest.raises(capi.SlayerB200Error):
        capi.call("slayer_b200_conv", one, one, one, -1, 4, 2, 1.0, null)
