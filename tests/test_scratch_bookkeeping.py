"""The context's grow-on-demand scratch bookkeeping, exercised on the host with an allocator that fails."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_grow_buf_failure_paths(tmp_path):
    exe = str(tmp_path / "test_scratch")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-o", exe, os.path.join(ROOT, "tests", "cpp", "test_scratch.cpp")])
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout + out.stderr
