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
