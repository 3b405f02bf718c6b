"""CPU checks of the boundary: the shared library loads, exports every symbol
the header declares, and rejects bad geometry without touching a GPU."""
import ctypes as C
import os
import re

from conftest import ROOT, load_pkg


def _ensure_built():
    build = load_pkg("build")
    return build.build()


def test_library_exports_every_declared_symbol():
    path = _ensure_built()
    lib = C.CDLL(path)
    header = open(os.path.join(ROOT, "include", "loda_b200.h")).read()
    declared = set(re.findall(r"\b(loda_[a-z0-9_]+)\s*\(", header))
    assert {"loda_append_decode", "loda_select_l1", "loda_select_l2", "loda_gather_attend",
            "loda_decode_step", "loda_build_index", "loda_write_prefill"} <= declared
    for name in declared:
        assert hasattr(lib, name), name
    capi = load_pkg("_capi")
    assert set(capi.EXPORTS) <= declared


def test_geometry_validation_needs_no_gpu():
    _ensure_built()
    capi = load_pkg("_capi")
    lib = capi.lib()
    good = dict(dtype=0, num_q_heads=32, num_kv_heads=8, head_dim=128, head_dim_v=128, sub_dims=32,
                sub_lo0=48, sub_lo1=112, page=16, num_pages=100, max_blocks=2112, max_requests=4,
                max_query_tokens=4, max_visible=1024, k_far=96, k_near=32, level2_topk=1024, sink=4,
                swa=128, near_len=4096, pool_near_len=4096)
    g = capi.Geometry(**good)
    assert lib.loda_workspace_bytes(C.byref(g)) > 0
    for field, bad in (("dtype", 1), ("page", 24), ("sub_dims", 48), ("num_q_heads", 30),
                       ("max_visible", 512), ("swa", 100), ("max_blocks", 70000)):
        g = capi.Geometry(**{**good, field: bad})
        assert lib.loda_workspace_bytes(C.byref(g)) == 0, field
        assert lib.loda_last_error()
    assert b"sm_100a" in lib.loda_version()


def test_struct_layouts_match_the_header():
    capi = load_pkg("_capi")
    header = open(os.path.join(ROOT, "include", "loda_b200.h")).read()
    for cls, cname in ((capi.Geometry, "loda_geometry"), (capi.Layer, "loda_layer"),
                       (capi.Batch, "loda_batch"), (capi.Selection, "loda_selection")):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = re.findall(r"(\w+)\s*;", body)
        assert names == [f[0] for f in cls._fields_], cname
