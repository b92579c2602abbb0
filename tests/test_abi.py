"""The C-ABI library builds, loads and exports what include/vlgpu.h declares (no GPU calls)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "vlgpu.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vl_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_entry_points():
    names = declared_symbols()
    for must in ("vl_calculate_distances", "vl_search_from_seeds", "vl_queue_insert", "vl_queue_pop", "vl_prune",
                 "vl_beam_search", "vl_seen_add", "vl_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/vlgpu.h but not exported"


def test_binding_table_matches_header(built_lib):
    from vectorlink_gpu import _lib
    assert sorted(_lib.EXPORTS) == [s for s in declared_symbols() if not s.startswith("vl_beam_params")]


def test_struct_mirror_has_the_size_of_the_c_struct(tmp_path, built_lib):
    import subprocess
    from vectorlink_gpu._lib import BeamParams
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "vlgpu.h"\nint main(){printf("%zu", sizeof(vl_beam_params));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)])
    assert int(subprocess.check_output([str(exe)]).decode()) == ctypes.sizeof(BeamParams)


def test_rejected_call_reports_an_error_text(built_lib):
    from vectorlink_gpu import _lib
    lib = _lib.lib()
    assert lib.vl_abi_version() == 4
    rc = lib.vl_sort_pairs(None, None, 1, 8, 0, None)
    assert rc != 0 and b"null" in lib.vl_last_error()


def test_cpu_tensors_are_refused_not_computed_on_the_host(built_lib):
    import torch
    from vectorlink_gpu import _lib
    from vectorlink_gpu.kernels import calculate_distances
    v = torch.zeros(4, 8)
    with pytest.raises(_lib.VlError):
        calculate_distances(v, torch.zeros(4, 2, dtype=torch.int32))


def test_connected_components_rejects_bad_shapes_without_touching_the_gpu(built_lib):
    from vectorlink_gpu import _lib
    lib = _lib.lib()
    assert lib.vl_connected_components(None, None, 1 << 31, 4, 4, ctypes.c_float(0.5), None, None, None) != 0
    assert b"int32" in lib.vl_last_error()
    assert lib.vl_connected_components(None, None, 10, 4, 2, ctypes.c_float(0.5), None, None, None) != 0   # ld < w
    assert lib.vl_connected_components(None, None, 0, 4, 4, ctypes.c_float(0.5), None, None, None) == 0     # no nodes: nothing to do
