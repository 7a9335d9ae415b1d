"""CPU checks of the boundary: the shared library loads and exports every C symbol that
include/jllm_b200.h declares and every C++ symbol of the reference's public kernel/pool API
with the reference's own mangling (tests/golden/api_symbols.txt, taken from a build of the
reference's sources)."""
import ctypes
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "genie-ai-runtime_b200", "libjllm_b200.so")


def _exported():
    out = subprocess.run(["nm", "-D", "--defined-only", LIB], capture_output=True, text=True, check=True).stdout
    return {l.split()[-1] for l in out.splitlines() if l.strip()}


def test_library_exists_and_loads():
    assert os.path.exists(LIB), "run `python __graft_entry__.py` (build) first"
    ctypes.CDLL(LIB)


def test_every_declared_c_symbol_is_exported():
    hdr = open(os.path.join(ROOT, "include", "jllm_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b(jllm_b200_\w+)\s*\(", hdr))
    assert len(names) > 60
    missing = sorted(names - _exported())
    assert not missing, missing


def test_reference_cpp_symbols_are_exported():
    want = open(os.path.join(ROOT, "tests", "golden", "api_symbols.txt")).read().split()
    assert len(want) >= 50          # 46 free functions and non-const members + the four const members of KVCachePool
    missing = sorted(set(want) - _exported())
    assert not missing, missing


def test_no_oracle_or_torch_dependency_in_library():
    out = subprocess.run(["ldd", LIB], capture_output=True, text=True).stdout
    assert "oracle" not in out and "torch" not in out
    # the library must not reference the CPU checker's symbols either
    und = subprocess.run(["nm", "-D", "--undefined-only", LIB], capture_output=True, text=True).stdout
    assert "orc_" not in und


def test_pool_object_layout_matches_reference():
    """sizeof/offsets of the pool classes equal the reference's (the engine embeds them by value).
    Compiled against the reference header when the tree is present, else against recorded values."""
    ref_inc = os.path.join(os.environ.get("JLLM_REFERENCE_DIR", "/root/reference"), "include")
    src = r'''
    #include <cstdio>
    #include <cstddef>
    #define private public
    #include "%s"
    int main() { using namespace jllm;
      printf("%%zu %%zu %%zu %%zu %%zu %%zu %%zu\n", sizeof(KVCachePool), offsetof(KVCachePool, gpu_pool_), offsetof(KVCachePool, cpu_pool_),
             offsetof(KVCachePool, kv_scales_), offsetof(KVCachePool, used_tokens_), sizeof(ScratchPool), offsetof(ScratchPool, offset_)); }
    '''
    import tempfile
    def layout(header, incs):
        with tempfile.TemporaryDirectory() as d:
            p = os.path.join(d, "l.cpp")
            open(p, "w").write(src % header)
            exe = os.path.join(d, "l")
            subprocess.check_call(["g++", "-std=c++17", "-w", "-I/usr/local/cuda/include"] + incs + [p, "-o", exe])
            return subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()
    mine = layout("jllm_b200_api.hpp", ["-I" + os.path.join(ROOT, "include")])
    assert mine == ["56", "24", "32", "40", "48", "24", "16"]
    if os.path.isdir(ref_inc):
        assert layout("jllm_memory.h", ["-I" + ref_inc]) == mine
