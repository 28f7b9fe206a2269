"""The C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "embla_cuda_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(embla_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from embla_metal_b200 import build
    lib = ctypes.CDLL(build.build())
    names = _declared()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_version_and_error_strings():
    from embla_metal_b200 import attn
    L = attn.lib()
    assert b"sm_100a" in L.embla_version()
    assert isinstance(L.embla_last_error(), bytes)


def test_bad_arguments_fail_without_a_gpu():
    """Argument checks come before any CUDA call, so they can be exercised on a CPU-only host."""
    from embla_metal_b200 import attn
    L = attn.lib()
    out = ctypes.c_void_p()
    assert L.embla_attn_create(None, ctypes.byref(out)) == attn.BAD_ARG
    cfg = attn.AttnConfig(16, 3, attn.F16, 1, 1024)          # 16 query heads do not divide over 3 kv heads
    assert L.embla_attn_create(ctypes.byref(cfg), ctypes.byref(out)) == attn.BAD_ARG
    assert b"n_kv_heads" in L.embla_last_error()
    cfg = attn.AttnConfig(32, 2, attn.F16, 1, 1024)          # 16 query heads a kv head: over the kernels' 8
    assert L.embla_attn_create(ctypes.byref(cfg), ctypes.byref(out)) == attn.UNSUPPORTED
    assert L.embla_kv_pool_create(0, 4, attn.KV_INT8, attn.SCALE_F16, 8, ctypes.byref(out)) == attn.BAD_ARG
    assert L.embla_kv_pool_create(1, 4, 7, attn.SCALE_F16, 8, ctypes.byref(out)) == attn.BAD_ARG
    assert L.embla_select_keys(None, None, 0, None, 1, 0, None, None) == attn.BAD_ARG


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "embla_metal_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("the oracle", "").replace("CPU oracle", "").replace("oracle's", "").replace(
                    "oracle fixes", ""), f"{f} refers to oracle/"


def test_c_caller_compiles_links_and_runs(tmp_path):
    """A C99 program that includes only the public header, linked against the built library."""
    import subprocess
    from embla_metal_b200 import build
    lib = build.build()
    exe = str(tmp_path / "abi_check")
    src = os.path.join(ROOT, "tests", "c_abi", "abi_check.c")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), src, "-o", exe,
                    lib, "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout + out.stderr
