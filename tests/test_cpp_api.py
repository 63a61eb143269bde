"""The C++ host API (include/glm53f_kda.hpp, the header-only mirror of the reference's kernel.rs) compiled with g++
against the built library: its host-side checks on the CPU, and the reference's flows on a GPU."""
import importlib
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "glm53f-afd_b200")


def build(tmp_path, source, extra=()):
    importlib.import_module("glm53f-afd_b200").build()
    exe = str(tmp_path / os.path.splitext(source)[0])
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", source), "-o", exe,
           "-L", LIBDIR, "-lglm53f_kda", f"-Wl,-rpath,{LIBDIR}", *extra]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_host_checks_without_a_gpu(tmp_path):
    exe = build(tmp_path, "host_checks.cpp")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "all host checks passed" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_flows_on_the_gpu(tmp_path):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = build(tmp_path, "gpu_flows.cpp", ["-I", os.path.join(cuda, "include"), "-L", os.path.join(cuda, "lib64"), "-lcudart", f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"])
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "all GPU flows passed" in r.stdout, r.stdout + r.stderr
