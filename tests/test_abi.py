"""The C ABI as a loadable library: every declared entry point is exported, the column table matches
the header, and the host-only helpers work without a GPU. No compute entry point is called here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from pj_testlib import ROOT, abi, pj


def declared_functions(header="petjson.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pj_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native):
    names = declared_functions()
    assert {"pj_create", "pj_destroy", "pj_parse", "pj_parse_shard", "pj_write", "pj_index_records"} <= set(names)
    L = native.lib()
    for n in names:
        assert hasattr(L, n), n
    gen = declared_functions("petjson_gen.h")
    assert {"pj_gen_text", "pj_gen_columns"} <= set(gen)
    for n in gen:
        assert hasattr(native.gen_lib(), n), n
        assert not hasattr(L, n), "the generator is not part of the GPU library"


def test_no_entry_point_takes_a_library_type():
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "petjson.h")).read(), flags=re.S)
    assert "torch" not in text and "cudaStream_t" not in text and "#include <cuda" not in text


def test_column_table_matches_header(native):
    L = native.lib()
    seen = 0
    for cid in range(abi.PJ_MAX_COLS):
        name, elem, owner = C.c_char_p(), C.c_uint32(), C.c_uint32()
        st = L.pj_column_info(cid, C.byref(name), C.byref(elem), C.byref(owner))
        if cid in abi.COL_BY_ID:
            c = abi.COL_BY_ID[cid]
            assert st == 0 and name.value.decode() == c.name and elem.value == np.dtype(c.dtype).itemsize and owner.value == c.owner
            seen += 1
        else:
            assert st == abi.PJ_ERR_ARG
    assert seen == len(abi.COLUMNS)
    header = open(os.path.join(ROOT, "include", "petjson.h")).read()
    for c in abi.COLUMNS:
        m = re.search(r"PJ_COL_%s\s*=\s*(\d+)" % c.name.upper(), header)
        assert m and int(m.group(1)) == c.id, c.name


def test_status_and_kind_names(native):
    L = native.lib()
    assert L.pj_version() == 1
    assert L.pj_status_str(abi.PJ_ERR_CAPACITY) == b"PJ_ERR_CAPACITY"
    for i, n in enumerate(abi.ERROR_KIND_NAMES):
        assert L.pj_error_kind_str(i).decode() == n


def test_columns_sizes_bounds(native):
    probe = abi.pj_columns()
    assert native.lib().pj_columns_sizes(abi.PJ_SCHEMA_PET, 1000, 300000, 0, C.byref(probe)) == 0
    assert probe.col[abi.COL_BY_NAME["rec_start"].id].bytes >= 8000
    assert probe.col[abi.COL_BY_NAME["pet_name_data"].id].bytes >= 300000
    assert probe.col[abi.COL_BY_NAME["pet_tag_id"].id].bytes >= 8 * 150000
    assert probe.col[abi.COL_BY_NAME["ord_id"].id].bytes == 0
    assert native.lib().pj_columns_sizes(9, 1, 1, 0, C.byref(probe)) == abi.PJ_ERR_ARG


def test_create_without_a_gpu_fails_loudly(native):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(native.PetJsonError) as e:
        native.Context()
    assert e.value.status == abi.PJ_ERR_CUDA


def test_product_never_loads_the_checker():
    """Nothing under the package or bench's product path may reference oracle/."""
    pkg = os.path.join(ROOT, "micronaut3-bug_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".c", ".cpp")) and f != "build.py":
                assert "oracle" not in open(os.path.join(dirpath, f), errors="ignore").read(), f
