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


STRUCTS = {
    "wm_attn_args": _native.AttnArgs,
    "wm_mix_args": _native.MixArgs,
    "wm_qprep_args": _native.QueryPrepArgs,
    "wm_pool_append_args": _native.PoolAppendArgs,
    "wm_pool_mix_args": _native.PoolMixArgs,
    "wm_pool_finish_args": _native.PoolFinishArgs,
    "wm_source_mix": _native.SourceMix,
}
C_TYPES = {"int64_t": ctypes.c_int64, "int32_t": ctypes.c_int32, "size_t": ctypes.c_size_t, "float": ctypes.c_float}


def header_fields(struct):
    """(name, ctypes type) of every member of a struct of the public header, in order."""
    body = HEADER.split(f"typedef struct {struct} {{")[1].split(f"}} {struct};")[0]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for statement in filter(None, (part.strip() for part in body.split(";"))):
        match = re.fullmatch(r"(?:const\s+)?(\w+)\s*(\*?)\s*(.+)", statement, flags=re.S)
        base = match.group(1) + match.group(2)
        for declarator in match.group(3).split(","):
            name, _, extent = declarator.strip().partition("[")
            kind = ctypes.c_void_p if base.endswith("*") else C_TYPES[base]
            fields.append((name.strip(), kind * int(extent.rstrip("]")) if extent else kind))
    return fields


def test_every_struct_of_the_header_is_mirrored():
    assert sorted(re.findall(r"typedef struct (\w+) \{", HEADER)) == sorted(STRUCTS)


@pytest.mark.parametrize("struct", sorted(STRUCTS))
def test_struct_layout_matches_header(struct):
    declared = header_fields(struct)
    mirrored = STRUCTS[struct]._fields_
    assert [name for name, _ in mirrored] == [name for name, _ in declared]
    for (name, have), (_, want) in zip(mirrored, declared):
        assert ctypes.sizeof(have) == ctypes.sizeof(want), name
        assert (have is ctypes.c_float) == (want is ctypes.c_float), name
