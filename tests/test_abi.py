"""The drop-in boundary: libnova_b200.so loads without a GPU and exports every function that
include/nova_b200.h and include/nova_b200_testing.h declare; the Python binding declares the same set.  No compute is called."""
import ctypes
import os
import re

from conftest import ROOT


def declared_functions():
    text = "".join(open(os.path.join(ROOT, "include", f)).read() for f in ("nova_b200.h", "nova_b200_testing.h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"typedef struct \{.*?\} \w+;", "", text, flags=re.S)
    names = re.findall(r"\b((?:nova|dev)_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_symbols_exported(nv):
    names = declared_functions()
    assert len(names) > 90
    handle = ctypes.CDLL(nv.LIB_PATH)
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, missing


def test_binding_covers_header(nv):
    assert sorted(nv.SIGNATURES) == declared_functions()


def test_status_strings_and_host_only_calls(nv):
    assert nv.lib.nova_status_string(0) == b"ok"
    assert b"pool" in nv.lib.nova_status_string(nv.ERR_POOL_FULL)
    assert nv.lib.nova_launch_count() >= 0
    sh = nv.KvShape(28, 4, 128, 16, nv.KV_F32, 1)
    assert nv.lib.nova_attn_scratch_floats(ctypes.byref(sh)) == 28 * 32 * 130   # src/model.cpp:148
    assert nv.synth_key(1, 2, 3, 4) != nv.synth_key(1, 2, 3, 5)
    assert nv.lib.nova_launcher_set_kernel(2) == nv.ERR_INVALID and nv.lib.nova_launcher_set_kernel(-1) == nv.ERR_INVALID
    assert nv.lib.nova_launcher_set_kernel(1) == nv.OK and nv.lib.nova_launcher_set_kernel(0) == nv.OK      # a switch, no GPU work


def test_no_product_path_into_oracle():
    """The product must not reach into the checker: no file of the package names oracle/."""
    pkg = os.path.join(ROOT, "conflux-nova_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp", ".h")):
                src = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in src.lower(), os.path.join(dirpath, f)
