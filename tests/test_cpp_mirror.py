"""The C++ host mirror (include/vfold_const.hpp): tests/cpp/test_const_mirror.cpp is compiled with g++ against
libvfold.so. Without a GPU its builder / type-inference / error checks run (`--host`); on a GPU box the
folding cases, written after the reference's own gtest cases, run as well."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "vpux_plugin_b200")
BIN = os.path.join(PKG, "build", "test_const_mirror")


def _build():
    from vpux_plugin_b200 import lib
    lib.raw()  # raises when libvfold.so is missing
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    src = os.path.join(ROOT, "tests", "cpp", "test_const_mirror.cpp")
    deps = [src, os.path.join(ROOT, "include", "vfold_const.hpp"), os.path.join(ROOT, "include", "vfold.h")]
    if os.path.exists(BIN) and all(os.path.getmtime(BIN) >= os.path.getmtime(d) for d in deps):
        return BIN
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), src, "-o", BIN,
           "-L", PKG, "-lvfold", "-Wl,-rpath," + PKG, "-Wl,--allow-shlib-undefined"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    return BIN


def _run(args):
    env = dict(os.environ)
    try:  # the CUDA runtime libvfold.so links against ships inside the python environment
        import nvidia.cuda_runtime as cr
        libdir = os.path.join(os.path.dirname(cr.__file__), "lib")
        env["LD_LIBRARY_PATH"] = libdir + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    except ImportError:
        pass
    return subprocess.run([_build()] + args, capture_output=True, text=True, env=env, timeout=300)


def test_cpp_mirror_host_checks():
    r = _run(["--host"])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "host: 0 failed" in r.stdout


@pytest.mark.gpu
def test_cpp_mirror_folds_on_gpu():
    r = _run([])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all: 0 failed" in r.stdout
