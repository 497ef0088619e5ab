"""The drop-in boundary without a GPU: every symbol declared in include/*.h is
exported by the built libraries, the pure-function parts behave like the
reference's, and the host bindings mirror the reference's loader rules."""
import ctypes as C
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = {
    "fp8_gemm.h": ("FP8GEMM_API", "libfp8gemm.so"),
    "fa_sm120.h": ("FA_API", "libfa_sm120.so"),
    "fp8_quantize.h": ("FP8QUANT_API", "libfp8quant.so"),
    "fp8_block.h": ("FP8BLOCK_API", "libfp8block.so"),
}


def declared_symbols(header, macro):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(macro + r"\s+[\w\s\*]+?\b(\w+)\s*\(", text)


@pytest.mark.parametrize("header", sorted(HEADERS))
def test_every_declared_symbol_is_exported(built_libs, header):
    macro, libname = HEADERS[header]
    names = declared_symbols(header, macro)
    assert len(names) >= 2
    lib = C.CDLL(os.path.join(built_libs, libname))
    for n in names:
        assert hasattr(lib, n), f"{libname} does not export {n}"


def test_reference_symbol_names_present(built_libs):
    # exactly what backend/cuda/fp8_gemm.go:36-38 and fa_forward.go:100-112 register
    g = C.CDLL(os.path.join(built_libs, "libfp8gemm.so"))
    for n in ("fp8_gemm", "fp8_gemm_original", "fp8_gemm_singlesync"):
        getattr(g, n)
    f = C.CDLL(os.path.join(built_libs, "libfa_sm120.so"))
    for n in ("fa_create", "fa_destroy", "fa_forward", "fa_forward_train", "fa_version", "fa_status_str",
              "fa_last_cuda_error", "fa_dispatch_select", "fa_kernel_name"):
        getattr(f, n)


def test_only_the_abi_is_visible(built_libs):
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(built_libs, "libfa_sm120.so")],
                         capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l}
    assert exported == set(declared_symbols("fa_sm120.h", "FA_API"))


# libs/fa_sm120/test/test_dispatch.c (29 rows) + libs/fa_sm120/go/gofa/gofa_test.go:15-37
DISPATCH_ROWS = [
    (4, 1024, 128, 0, 0, 103), (4, 2048, 128, 0, 0, 103), (4, 4096, 128, 0, 0, 102), (8, 2048, 128, 0, 0, 102),
    (8, 4096, 128, 0, 0, 102), (16, 2048, 128, 0, 0, 102), (16, 4096, 128, 0, 0, 105), (32, 2048, 128, 0, 0, 105),
    (32, 4096, 128, 0, 0, 100), (32, 8192, 128, 0, 0, 100), (64, 4096, 128, 0, 0, 105), (64, 8192, 128, 0, 0, 100),
    (128, 2048, 128, 0, 0, 105), (128, 4096, 128, 0, 0, 100), (128, 8192, 128, 0, 0, 100), (256, 2048, 128, 0, 0, 100),
    (256, 4096, 128, 0, 0, 100), (4, 4096, 128, 1, 1024, 102), (4, 8192, 128, 1, 1024, 104), (8, 8192, 128, 1, 1024, 102),
    (16, 8192, 128, 1, 1024, 101), (32, 8192, 128, 1, 1024, 101), (64, 8192, 128, 1, 1024, 101),
    (4, 1024, 64, 0, 0, 201), (4, 2048, 64, 0, 0, 201), (64, 8192, 64, 0, 0, 200), (16, 4096, 64, 0, 0, 200),
    (64, 8192, 96, 0, 0, -1), (0, 100, 128, 0, 0, -1),
]


def test_dispatch_table(built_libs):
    from goml_b200 import fa_forward as F
    for bh, sl, hd, ca, w, want in DISPATCH_ROWS:
        assert F.FADispatchSelect(bh, sl, hd, ca, w) == want, (bh, sl, hd, ca, w)
    assert F.FAKernelName(100) == "v121r" and F.FAKernelName(201) == "v80b" and F.FAKernelName(-1) == "<none>"
    assert F.FADispatchSelect(4, -5, 128, 0, 0) == -1


def test_reference_dispatch_test_program_passes_unchanged(built_libs, tmp_path):
    import oracle
    src = os.path.join(oracle.reference_root(), "libs/fa_sm120/test/test_dispatch.c")
    if not os.path.exists(src) or not shutil.which("gcc"):
        pytest.skip("reference tree not present")
    exe = tmp_path / "test_dispatch"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(exe), src, "-L", built_libs,
                    "-lfa_sm120", f"-Wl,-rpath,{built_libs}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "29/29 cases pass" in r.stdout


def test_status_strings_and_null_handling(built_libs):
    from goml_b200 import fa_forward as F
    lib = F.FALoad()
    assert F.FAStatusString(0) == "OK"
    assert F.FAStatusString(1) == "invalid argument"
    assert "head_dim" in F.FAStatusString(3)
    assert F.FAStatusString(5) == "CUDA runtime error"
    assert F.FAStatusString(99) == "unknown"
    assert lib.fa_destroy(None) == 0                       # FA_OK on NULL (fa_sm120.h:120)
    assert lib.fa_last_cuda_error(None) == b""              # "" for a NULL context
    assert lib.fa_create(None) == F.FA_ERR_INVALID_ARG
    assert "sm100a" in F.FAVersion()
    assert lib.fa_forward(None, None, None, None, None, 1, 1, 128, 0, 0, 1.0, None) == F.FA_ERR_INVALID_ARG


def test_gemm_argument_errors_without_gpu(built_libs):
    from goml_b200 import fp8_gemm as G
    lib = G._init()
    assert "tcgen05" in G.version()
    assert lib.fp8_gemm(-1, 8, 16, None, None, None, 1, None) == 1      # cudaErrorInvalidValue
    assert lib.fp8_gemm(8, 8, 16, None, None, None, 1, None) == 1       # null pointers
    assert lib.fp8_gemm(0, 8, 16, None, None, None, 1, None) == 0       # empty problem is a no-op
    assert lib.fp8_gemm(8, 8, 24, 16, 16, 16, 1, None) == 1             # K % 16 != 0
    assert lib.fp8_gemm(8, 8, 32, 8, 16, 16, 1, None) == 1              # A not 16-byte aligned
    assert lib.fp8_gemm_scaled(8, 8, 32, 16, 16, 16, 1.0, None, None, 7, None) == 1  # bad out dtype
    with pytest.raises(G.FP8GEMMError, match=r"fp8_gemm: CUDA error 1"):
        G.FP8GEMM(8, 8, 24, 16, 16, 16)


def test_loader_follows_reference_search_order(tmp_path, monkeypatch, built_libs):
    from goml_b200 import loader
    d = tmp_path / "mylibs"
    d.mkdir()
    (d / "libfp8gemm.so").write_bytes(b"")
    monkeypatch.setenv("GOML_LIBS_DIR", str(d))
    assert loader.libs_dir() == str(d)                                   # $GOML_LIBS_DIR wins
    assert loader.resolve_lib("libfp8gemm.so") == str(d / "libfp8gemm.so")
    assert loader.resolve_lib("libnothing_here.so") == "libnothing_here.so"  # bare name for the OS loader
    monkeypatch.delenv("GOML_LIBS_DIR")
    assert loader.resolve_lib("libfp8gemm.so") == os.path.join(built_libs, "libfp8gemm.so")
    with pytest.raises(loader.LibraryNotFound):
        loader.dlopen("libnothing_here.so")


def test_fa_error_message_shape():
    from goml_b200 import fa_forward as F
    e = F.FAError("fa_forward_train", F.FA_ERR_INVALID_ARG, "window must be in [0, seq_len]")
    assert str(e) == "fa_forward_train: invalid argument (window must be in [0, seq_len])"
    assert e.status == 1


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "goml_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, f


def test_build_script_builds_and_honours_target_only(tmp_path):
    # goml_b200/build_cuda.sh is the counterpart of the reference's scripts/build_cuda.sh for these libraries; unlike
    # that script (scripts/build_cuda.sh:67-87 never reads the variable its Makefile:24-32 exports) it honours
    # GOML_TARGET_ONLY, and refuses a target list without sm_100a
    script = os.path.join(ROOT, "goml_b200", "build_cuda.sh")
    if not shutil.which("nvcc"):
        pytest.skip("nvcc not available")
    env = dict(os.environ, LIBS_DIR=str(tmp_path))
    r = subprocess.run(["bash", script, "quant"], env=env, capture_output=True, text=True)
    assert r.returncode == 0 and (tmp_path / "libfp8quant.so").exists(), r.stdout + r.stderr
    assert "arch=compute_100a,code=sm_100a" in r.stdout
    env["GOML_TARGET_ONLY"] = "-gencode arch=compute_89,code=sm_89"
    r = subprocess.run(["bash", script, "quant"], env=env, capture_output=True, text=True)
    assert r.returncode == 2 and "sm_100a-only" in r.stderr
    env["GOML_TARGET_ONLY"] = "-gencode arch=compute_100a,code=sm_100a"
    r = subprocess.run(["bash", script, "nosuchtarget"], env=env, capture_output=True, text=True)
    assert r.returncode == 2


def test_family_name_alias_loads_the_same_library(built_libs):
    # libflash_attention_fp8.so is an alias of libfa_sm120.so for callers that look the attention library up by the
    # libflash_attention*.so family name
    import ctypes
    alias = os.path.join(built_libs, "libflash_attention_fp8.so")
    assert os.path.islink(alias) and os.readlink(alias) == "libfa_sm120.so"
    lib = ctypes.CDLL(alias)
    lib.fa_version.restype = ctypes.c_char_p
    assert b"sm100a" in lib.fa_version()
