"""Builds and runs tests/cpp/test_frontend.cc: the C++ KernelCodeGen front end exercised
with the reference's own call sequences (test/test.cc), on CPU (graph, plan, errors) and on
the GPU (plans executed and compared with the CPU oracle)."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CPP = ROOT / "tests" / "cpp"
LIB = ROOT / "kernelcodegen_b200" / "lib"
ORACLE = ROOT / "oracle"


@pytest.fixture(scope="module")
def exe():
    from kernelcodegen_b200 import build as kb
    kb.build_all()
    from oracle import oracle
    oracle.build()
    out = CPP / "build" / "test_frontend"
    out.parent.mkdir(exist_ok=True)
    src = CPP / "test_frontend.cc"
    cmd = ["g++", "-O1", "-std=c++17", "-pthread", "-I", str(ROOT / "include"), str(src), "-o", str(out),
           "-L", str(LIB), "-lkcg_runtime", "-lkcg_kernels", "-L", str(ORACLE), "-lkcg_oracle",
           "-L", "/usr/local/cuda/lib64", "-lcudart",
           f"-Wl,-rpath,{LIB}", f"-Wl,-rpath,{ORACLE}", "-Wl,-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def test_frontend_cpu(exe):
    r = subprocess.run([str(exe), "cpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "frontend cpu tests passed" in r.stdout


@pytest.mark.gpu
def test_frontend_gpu(exe):
    r = subprocess.run([str(exe), "gpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "frontend gpu tests passed" in r.stdout


@pytest.mark.gpu
def test_frontend_sharded_run_two_gpus(exe, tmp_path):
    """Two processes, one per GPU, drive KernelCodeGenerator::run with a ShardSpec and the NCCL
    gather entirely from C++; each compares its gathered result with its own unsharded run."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    id_file = tmp_path / "nccl_id.bin"
    env = dict(__import__("os").environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([str(exe), "shard", str(world), str(r), str(id_file)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, env=env) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"shard rank {r} of {world} passed" in out, out[-3000:]
