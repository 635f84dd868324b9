"""The C++ builder mirror (tcacomp_b200/csrc/host/): builds tests/cpp/host_tests.cpp against
libtcab_host.so and runs it. Without a GPU only the builder / classifier half runs (the reference's
pkg/builder_test.go and pkg/oracle_test.go cases); with -m gpu the runner-protocol half launches the
reference's suite kernels through the rungs and the output lines are checked the way
testing/orchestrator.py checks them: canary 0 and MAXDIFF within the suite's tolerance."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUT = os.path.join(ROOT, "tests", "cpp", "_build")

# testing/suite.toml tolerances (max abs diff); the e2e row sum uses internal/e2e/e2e_test.go:15-21
TOL = {"RowSum": 2e-3, "Softmax": 2e-3, "Transpose": 1e-5, "ScaleCopy": 1e-5, "Axpy3": 1e-5, "Layernorm": 1e-5,
       "RowSumE2E": 2e-3, "MatmulScale": 2e-3, "GemmBiasRelu": 2e-2,
       # kernels written as .tca text in host_tests.cpp and taken through the text frontend
       "TcaWeightedFold": 1e-5, "TcaMidAxisMax": 1e-6, "TcaScores": 2e-3}


def build_binary(with_cuda: bool) -> str:
    from tcacomp_b200 import build
    build.build()
    os.makedirs(OUT, exist_ok=True)
    exe = os.path.join(OUT, "host_tests_gpu" if with_cuda else "host_tests")
    src = os.path.join(ROOT, "tests", "cpp", "host_tests.cpp")
    lib = os.path.join(ROOT, "tcacomp_b200")
    deps = [src, os.path.join(lib, "libtcab_host.so"), os.path.join(lib, "libtcab.so")]
    if os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    cmd = ["g++", "-O1", "-std=c++17", "-Wall", "-o", exe, src, "-L" + lib, "-ltcab_host", "-ltcab",
           "-Wl,-rpath," + lib]
    if with_cuda:
        cuda = os.path.dirname(os.path.dirname(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"))
        cmd += ["-DHOST_TESTS_WITH_CUDA", "-I" + os.path.join(cuda, "include"), "-L" + os.path.join(cuda, "lib64"),
                "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    subprocess.run(cmd, check=True)
    return exe


def test_builder_mirror_cpu():
    r = subprocess.run([build_binary(False)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout[-3000:]
    m = re.search(r"(\d+) checks, (\d+) failures", r.stdout)
    assert m and int(m.group(1)) >= 80 and int(m.group(2)) == 0, r.stdout[-3000:]


@pytest.mark.gpu
def test_suite_kernels_through_the_rungs():
    r = subprocess.run([build_binary(True), "--gpu"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1000:]
    blocks = re.split(r"^KERNEL ", r.stdout, flags=re.M)[1:]
    seen = {}
    for blk in blocks:
        name = blk.split()[0]
        f = dict(re.findall(r"^(CANARY|CHECKSUM|REF_CHECKSUM|MAXDIFF) (\S+)$", blk, flags=re.M))
        assert set(f) == {"CANARY", "CHECKSUM", "REF_CHECKSUM", "MAXDIFF"}, blk
        assert int(f["CANARY"]) == 0, name
        assert float(f["MAXDIFF"]) <= TOL[name], (name, f["MAXDIFF"])
        assert abs(float(f["CHECKSUM"]) - float(f["REF_CHECKSUM"])) <= 1e-4 * abs(float(f["REF_CHECKSUM"])), name
        seen[name] = float(f["MAXDIFF"])
    assert set(seen) == set(TOL), seen
    assert "TCA_CONST_EXTENT rejected" in r.stdout
