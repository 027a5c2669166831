"""Host-side native code under AddressSanitizer + UBSan and under ThreadSanitizer: the C++ sources
are rebuilt with the sanitizer flags into a stand-alone stress driver (tests/native/) and run."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCES = [os.path.join(ROOT, "csrc", "serve", "kv_scheduler.cpp"),
           os.path.join(ROOT, "csrc", "runtime", "rrec_reader.cpp"),
           os.path.join(ROOT, "csrc", "runtime", "batch_loader.cpp"),
           os.path.join(ROOT, "csrc", "runtime", "fd_exchange.cpp"),
           os.path.join(ROOT, "tests", "native", "host_sanitize_driver.cpp")]


@pytest.mark.parametrize("flags", ["-fsanitize=address,undefined", "-fsanitize=thread"])
def test_host_native_code_under_sanitizers(flags, tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "driver")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", flags,
                            "-fno-sanitize-recover=all", "-pthread", "-o", exe] + SOURCES,
                           capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find" in build.stderr or "unrecognized" in build.stderr):
        pytest.skip("sanitizer runtime not installed: " + build.stderr[-200:])
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([exe, str(tmp_path / "s.rrec")], capture_output=True, text=True, timeout=300,
                         env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "HOST SANITIZE DRIVER OK" in run.stdout
    assert "ERROR: AddressSanitizer" not in run.stderr and "WARNING: ThreadSanitizer" not in run.stderr
    assert "runtime error" not in run.stderr
