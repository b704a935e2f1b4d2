"""The C interface: a C11 program built against include/kestrel.h alone drives the host
runtime; every function the header declares is exported by a library, and every function a
library exports is declared in the header; the Python bindings take their types from it."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "kestrel-llm_b200", "include")


def test_a_c11_caller_drives_cache_scheduler_and_packer(tmp_path):
    from kestrel_llm_b200.csrc import build
    gcc = shutil.which("gcc")
    if not gcc:
        pytest.skip("no gcc")
    lib = build.build_host(verbose=False)
    exe = str(tmp_path / "host_api_test")
    r = subprocess.run([gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-I", INCLUDE, os.path.join(ROOT, "tests", "c", "host_api_test.c"),
                        "-o", exe, "-L", os.path.dirname(lib), "-lkestrel_host", "-Wl,-rpath," + os.path.dirname(lib)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and r.stdout.startswith("OK"), r.stdout + r.stderr


def _exported(lib: str):
    nm = shutil.which("nm")
    if not nm:
        pytest.skip("no nm")
    out = subprocess.run([nm, "-D", "--defined-only", lib], capture_output=True, text=True, check=True).stdout
    return {l.split()[-1] for l in out.splitlines() if " T " in l}


def test_header_and_host_library_name_the_same_functions():
    from kestrel_llm_b200.csrc import build, cdecl
    funcs, consts = cdecl.parse()
    host = {n for n in funcs if n.startswith(("kcache_", "ksched_", "kbatch_"))}
    got = {s for s in _exported(build.build_host(verbose=False)) if s.startswith("k")}
    assert got == host, f"only in the library: {sorted(got - host)}; only in the header: {sorted(host - got)}"
    assert consts["KBATCH_LAYOUT_INTS"] > max(v for k, v in consts.items() if k.startswith("KB_"))


def test_header_and_kernel_library_name_the_same_functions():
    from kestrel_llm_b200.csrc import build, cdecl
    funcs, _ = cdecl.parse()
    want = {n for n in funcs if n.startswith(("kestrel_", "kprog_", "krunner_"))}
    got = {s for s in _exported(build.build_cuda(verbose=False)) if s.startswith(("kestrel_", "kprog_", "krunner_"))}
    assert got == want, f"only in the library: {sorted(got - want)}; only in the header: {sorted(want - got)}"


def test_bindings_take_their_types_from_the_header():
    import ctypes
    from kestrel_llm_b200.cache.manager import host_library
    from kestrel_llm_b200.csrc import cdecl
    funcs, _ = cdecl.parse()
    lib = host_library()
    for name, (res, args, names) in funcs.items():
        if name.startswith(("kcache_", "ksched_", "kbatch_")):
            fn = getattr(lib, name)
            assert fn.restype == res and list(fn.argtypes) == args, name
    res, args, names = funcs["kestrel_step_raw"]
    assert names[:3] == ["runner", "n", "ids"] and args[1] is ctypes.c_int and args[8] is ctypes.c_longlong
    # no source file declares an exported function by hand any more
    pat = re.compile(r'extern\s+"C"\s+int\s+k(estrel|cache|sched|batch)_')
    for folder in ("kernels", "host"):
        d = os.path.join(ROOT, "kestrel-llm_b200", "csrc", folder)
        for f in os.listdir(d):
            if f.endswith((".cu", ".cpp", ".cuh", ".h")) and f != "linear_noalloc.h":
                assert not pat.search(open(os.path.join(d, f)).read()), f"{f} declares an entry point outside kestrel.h"
