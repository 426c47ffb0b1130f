"""Builds and runs the reference's tests written against the C++ host mirror
(xor-net_b200/host/xor_net_attn.hpp) on top of the C ABI."""
import os
import subprocess

import pytest

import xor_net_b200 as xn


def build(repo_root, tmp):
    exe = os.path.join(tmp, "test_reference_suite")
    libdir = os.path.dirname(xn.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(repo_root, "include"),
           "-I", os.path.join(libdir, "host"), os.path.join(repo_root, "tests", "cpp", "test_reference_suite.cpp"),
           "-o", exe, "-L", libdir, "-lxn_attn", f"-Wl,-rpath,{libdir}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_cpp_host_mirror_compiles(repo_root, tmp_path):
    xn.build_library()
    assert os.path.exists(build(repo_root, str(tmp_path)))


@pytest.mark.gpu
def test_reference_suite_through_the_cpp_host_mirror(repo_root, tmp_path):
    exe = build(repo_root, str(tmp_path))
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all reference tests passed" in res.stdout
