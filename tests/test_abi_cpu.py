"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import subprocess

import pytest

from mx230_b200 import _lib, build


def test_library_builds_and_loads(lib_built):
    assert os.path.exists(lib_built)
    L = _lib.lib()
    assert L.mx230_abi_version() == 1


def test_every_declared_symbol_is_exported(lib_built):
    protos = _lib.declared_functions()
    assert len(protos) >= 45, sorted(protos)
    raw = C.CDLL(lib_built)
    missing = [n for n in protos if not hasattr(raw, n)]
    assert not missing, missing
    # and nothing is exported that the header does not declare
    out = subprocess.run(["nm", "-D", "--defined-only", lib_built], capture_output=True, text=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if " T mx230_" in ln}
    extra = {e for e in exported if e.startswith("mx230_") and "launch" not in e
             and e not in protos and not e.startswith("mx230_set_error") and e != "mx230_fail"
             and e != "mx230_make_tmap_bf16"}
    assert not extra, extra


def test_status_strings_and_errors(lib_built):
    L = _lib.lib()
    assert L.mx230_status_string(0) == b"ok"
    assert b"workspace" in L.mx230_status_string(_lib.ERR_WORKSPACE)
    # null out-pointer is rejected before any CUDA call
    assert L.mx230_create(None, 0, 0) == _lib.ERR_INVALID_ARG
    assert b"null" in L.mx230_last_error()
    # four staged bf16 tensors plus the row-norm partials of Q and K (2 x 48 heads x 32 parts floats)
    assert L.mx230_flash_workspace_bytes(48, 4096, 1) == 4 * 48 * 4096 * 64 * 2 + 2 * 48 * 32 * 4
    assert L.mx230_flash_workspace_bytes(0, 4096, 1) == 0


def test_create_without_device_fails_loudly(lib_built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from mx230_b200.common import Handle
    with pytest.raises(_lib.Mx230Error) as e:
        Handle(0, 0)
    assert e.value.code in (_lib.ERR_NO_DEVICE, _lib.ERR_CUDA)


def test_sources_are_sm100a_only():
    assert build.ARCH_FLAGS == ["-gencode", "arch=compute_100a,code=sm_100a"]
    assert len(build.sources()) >= 5


def test_rust_extern_block_matches_the_header():
    """include/mx230_sys.rs is generated from the header; it must be regenerated when a prototype changes."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "include", "gen_rust_extern.py")], capture_output=True,
                         text=True, check=True).stdout
    assert out == open(os.path.join(root, "include", "mx230_sys.rs")).read()
    assert out.count("pub fn mx230_") == len(_lib.declared_functions())


def test_splitkv_comm_rejects_bad_arguments_without_a_device(lib_built):
    L = _lib.lib()
    c = C.c_void_p()
    assert L.mx230_splitkv_comm_create(None, 0, 2, 8, 64, C.byref(c)) == _lib.ERR_INVALID_ARG
    assert L.mx230_splitkv_exchange_merge(None, None, None, None) == _lib.ERR_INVALID_ARG
    assert L.mx230_splitkv_wait_merge(None, None, None) == _lib.ERR_INVALID_ARG
    assert L.mx230_splitkv_comm_disconnect(None) == _lib.ERR_INVALID_ARG
    L.mx230_splitkv_comm_destroy(None)   # a null communicator is ignored


def test_header_is_plain_c_and_links_against_the_library(lib_built, tmp_path):
    """The boundary is a C ABI: the header compiles as pedantic C99 and as C++, and a C program that calls through it
    links against the shared library and runs without a GPU (version and error-string calls only)."""
    import shutil
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cc, cxx = shutil.which("gcc") or shutil.which("cc"), shutil.which("g++") or shutil.which("c++")
    if cc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "abi.c"
    src.write_text('#include <stdio.h>\n#include <string.h>\n#include "mx230_attn.h"\n'
                   'int main(void) {\n'
                   '    mx230_splitkv_comm *c = 0;\n'
                   '    if (mx230_abi_version() != MX230_ABI_VERSION) return 1;\n'
                   '    if (mx230_splitkv_comm_create(0, 0, 2, 8, 64, &c) != MX230_ERR_INVALID_ARG) return 2;\n'
                   '    if (strlen(mx230_last_error()) == 0) return 3;\n'
                   '    if (mx230_gemm_workspace_bytes(512, 1152, 896, 1) != 512u * 896u * 2u) return 4;\n'
                   '    puts(mx230_status_string(MX230_ERR_WORKSPACE));\n'
                   '    return 0;\n}\n')
    inc = os.path.join(root, "include")
    subprocess.run([cc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", inc, "-fsyntax-only", str(src)], check=True)
    if cxx:
        subprocess.run([cxx, "-std=c++11", "-Wall", "-I", inc, "-fsyntax-only", "-x", "c++", str(src)], check=True)
    exe = tmp_path / "abi"
    libdir = os.path.dirname(lib_built)
    subprocess.run([cc, "-std=c99", "-I", inc, str(src), "-o", str(exe), "-L", libdir, "-lmx230_attn",
                    "-Wl,-rpath," + libdir], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, (out.returncode, out.stdout, out.stderr)
    assert out.stdout.strip()
