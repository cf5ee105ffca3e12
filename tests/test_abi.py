"""The C-ABI library: it loads, exports every symbol include/ingot_qmm.h declares, and fails cleanly without a GPU."""
import ctypes as C
import os
import re

import pytest
import torch

from ingot_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ingot_qmm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(iq_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(capi.SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = capi.lib()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/ingot_qmm.h but not exported"


def test_modulemap_names_the_header():
    mm = open(os.path.join(ROOT, "include", "module.modulemap")).read()
    assert "module CIngotQMM" in mm and 'header "ingot_qmm.h"' in mm


def test_strerror_and_version():
    lib = capi.lib()
    assert lib.iq_abi_version() == 1
    assert lib.iq_strerror(0) == b"ok"
    assert b"workspace" in lib.iq_strerror(-4)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure path")
def test_context_creation_fails_loudly_without_a_gpu():
    h = C.c_void_p()
    st = capi.lib().iq_ctx_create(0, C.byref(h))
    assert st < 0 and not h.value
    with pytest.raises(capi.IngotError):
        capi.Context(0)


def test_struct_layouts_match_the_header():
    # iq_qlinear: 3 pointers + 6 int32; iq_moe_desc field order as declared
    assert C.sizeof(capi.QLinear) == 3 * 8 + 6 * 4
    assert [f[0] for f in capi.QLinear._fields_] == ["w", "scales", "biases", "n", "k", "bits", "group", "mode", "experts"]
    text = open(os.path.join(ROOT, "include", "ingot_qmm.h")).read()
    body = text[text.index("typedef struct iq_moe_desc {"):text.index("} iq_moe_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = re.findall(r"(\w+);", body)
    assert names == [f[0] for f in capi.MoeDesc._fields_]
