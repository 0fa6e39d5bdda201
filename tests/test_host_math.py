"""Compiles the kernels' decode helpers (edge0_b200/csrc/formats.cuh) for the CPU and checks the per-unit integer
dot products and scale decoding against the checker, bit for bit."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_kernel_decode_math_on_host(tmp_path):
    exe = tmp_path / "host_math"
    obj = tmp_path / "moe_oracle.o"
    subprocess.check_call(["gcc", "-std=c11", "-O1", "-ffp-contract=off", "-c", os.path.join(ROOT, "oracle", "moe_oracle.c"), "-o", str(obj)])
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-o", str(exe), os.path.join(ROOT, "tests", "host_math_check.cpp"), str(obj), "-lm"])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
