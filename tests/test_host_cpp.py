"""The C++ host layer (goml_b200/host/goml_cuda.hpp): the mirror of goml's Go package backend/cuda.
The test program is compiled with g++ and run twice: without a GPU (loader rules, error text,
dispatcher, partitions) and on a GPU (closed-form LSE, GEMM self-check, quantise->attention chain,
head sharding through the device manager)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.fixture(scope="module")
def host_exe(tmp_path_factory, built_libs):
    if not shutil.which("g++"):
        pytest.skip("g++ not available")
    exe = tmp_path_factory.mktemp("host") / "test_host"
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(CUDA, "include"), os.path.join(ROOT, "tests", "host_cpp", "test_host.cpp"),
           "-o", str(exe), "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return str(exe)


def _env(built_libs):
    env = dict(os.environ)
    env["GOML_LIBS_DIR"] = built_libs
    env["LD_LIBRARY_PATH"] = os.path.join(CUDA, "lib64") + ":" + env.get("LD_LIBRARY_PATH", "")
    return env


def test_host_layer_without_gpu(host_exe, built_libs):
    r = subprocess.run([host_exe, "cpu", built_libs], capture_output=True, text=True, env=_env(built_libs))
    assert r.returncode == 0 and "cpu ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_host_layer_on_gpu(host_exe, built_libs, cuda):
    r = subprocess.run([host_exe, "gpu"], capture_output=True, text=True, env=_env(built_libs), timeout=300)
    assert r.returncode == 0 and "gpu ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_decoder_block_through_the_cpp_dispatch(host_exe, built_libs, cuda, tmp_path):
    # goml::cuda::nn::FP8DecoderBlock (the C++ twin of go/nn/fp8_dispatch.go) on inputs written here, against the CPU
    # restatement with the same quantisation points; the bar of tests/test_decoder_block_gpu.py
    import numpy as np
    import oracle as O
    from oracle.decoder_block import decoder_block
    B, S, d, H, Fh = 2, 128, 256, 4, 704
    cfg = "block-cpp"
    w = {n: O.seeded_normal(n, shp, std=0.02, config=cfg) for n, shp in
         dict(wqkv=(3 * d, d), wo=(d, d), wgate_up=(2 * Fh, d), wdown=(d, Fh)).items()}
    g1 = 1.0 + 0.1 * O.seeded_normal("g1", (d,), config=cfg)
    g2 = 1.0 + 0.1 * O.seeded_normal("g2", (d,), config=cfg)
    x = O.seeded_normal("x", (B * S, d), config=cfg)
    for name, a in dict(w, g1=g1, g2=g2, x=x).items():
        np.ascontiguousarray(a, np.float32).tofile(tmp_path / f"{name}.f32")
    r = subprocess.run([host_exe, "block", str(tmp_path), str(B), str(S), str(d), str(H), str(Fh)], capture_output=True, text=True,
                       env=_env(built_libs), timeout=300)
    assert r.returncode == 0 and "block ok" in r.stdout, r.stdout + r.stderr
    got = np.fromfile(tmp_path / "y.f32", np.float32).reshape(B * S, d).astype(np.float64)
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    ref = decoder_block(f32(x), B, S, H, f32(w["wqkv"]), f32(w["wo"]), f32(w["wgate_up"]), f32(w["wdown"]), f32(g1), f32(g2),
                        residual_in_epilogue=True, swiglu_in_epilogue=True)
    assert np.isfinite(got).all()
    maxabs, meanrel = O.error_stats(got, ref)
    assert maxabs <= 2e-2 and meanrel <= 1e-2, (maxabs, meanrel)
    maxabs_d, meanrel_d = O.error_stats(got - x, ref - x)
    assert maxabs_d <= 2e-2 and meanrel_d <= 5e-2, (maxabs_d, meanrel_d)
