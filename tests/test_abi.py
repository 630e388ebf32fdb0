"""The C-ABI library loads and exports every symbol that include/*.h declare (no GPU work)."""

import ctypes
import re
from pathlib import Path

import pytest

from white_matter_b200 import _native

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "wm_b200.h").read_text()
ALL_HEADERS = "\n".join(p.read_text() for p in sorted((ROOT / "include").glob("*.h")))


def declared_symbols():
    return sorted(set(re.findall(r"^WM_API [\w\s\*]*?\b(wm_\w+)\s*\(", ALL_HEADERS, flags=re.M)))


def test_header_declares_the_operator_roles():
    names = declared_symbols()
    for role in (
        "wm_cyclic_attn_fwd", "wm_cyclic_attn_bwd", "wm_cyclic_attn_doc_fwd", "wm_cyclic_attn_doc_bwd",
        "wm_strict_attn_fwd", "wm_strict_attn_bwd", "wm_strict_packed_fwd", "wm_strict_packed_bwd",
        "wm_strict_decode", "wm_mix_sources_fwd", "wm_mix_sources_bwd",
    ):
        assert role in names


@pytest.mark.parametrize("symbol", declared_symbols())
def test_library_exports(symbol):
    lib = _native.load_library()
    assert getattr(lib, symbol) is not None


def test_abi_version_and_argument_rejection_without_a_device():
    lib = _native.load_library()
    assert lib.wm_abi_version() == 1
    args = _native.AttnArgs()
    # all-zero arguments are rejected before any CUDA call
    assert lib.wm_cyclic_attn_fwd(ctypes.byref(args), None) == -1
    assert b"dtype" in lib.wm_last_error() or b"sizes" in lib.wm_last_error()
    mix = _native.MixArgs()
    assert lib.wm_mix_sources_fwd(ctypes.byref(mix), None) == -1


def test_struct_layout_matches_header_field_order():
    fields = [name for name, _ in _native.AttnArgs._fields_]
    body = HEADER.split("typedef struct wm_attn_args {")[1].split("} wm_attn_args;")[0]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    declared = re.findall(r"(\w+)(?:\[3\])?;", body)
    assert fields == declared
    mix_fields = [name for name, _ in _native.MixArgs._fields_]
    body = HEADER.split("typedef struct wm_mix_args {")[1].split("} wm_mix_args;")[0]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    assert mix_fields == re.findall(r"(\w+);", body)
