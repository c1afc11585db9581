"""Host-side native code under AddressSanitizer + UndefinedBehaviorSanitizer (CPU-only target).

The reference builds its native host code without sanitizers; device-side memory checking tools
are not available here, so the host C++ (the per-sequence LRU bookkeeping of the sparse KV offload)
gets a sanitizer build with its own driver."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_sparse_kv_offload_host_code_under_asan_ubsan(tmp_path):
    exe = str(tmp_path / "sko_sanitize")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", "-pthread",
           os.path.join(ROOT, "vllm_ascend_b200", "csrc", "sparse_kv_offload.cpp"),
           os.path.join(ROOT, "tests", "native", "sko_sanitize_main.cpp"), "-o", exe]
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find -lasan" in build.stderr or "libasan" in build.stderr):
        pytest.skip("sanitizer runtime libraries are not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    env.pop("LD_PRELOAD", None)
    run = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=300)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert run.stdout.startswith("OK ")
