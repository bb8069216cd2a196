"""The C++ runtime under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer (CPU only)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "art_b200", "csrc", "engine")


@pytest.mark.parametrize("flags", ["address,undefined", "thread"])
def test_block_manager_under_sanitizers(tmp_path, flags):
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    exe = tmp_path / "bm_selftest"
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={flags}", "-fno-omit-frame-pointer",
           os.path.join(SRC, "block_manager.cpp"), os.path.join(SRC, "block_manager_selftest.cpp"), "-lpthread", "-o", str(exe)]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    if build.returncode != 0 and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed: " + build.stderr.strip().splitlines()[-1])
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="halt_on_error=1", TSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([str(exe), "4", "3000"], capture_output=True, text=True, timeout=300, env=env)
    print(run.stdout[-500:], run.stderr[-3000:])
    assert run.returncode == 0 and "selftest ok" in run.stdout


@pytest.mark.parametrize("flags", ["address,undefined", "thread"])
def test_token_mask_builder_under_sanitizers(tmp_path, flags):
    if shutil.which("g++") is None:
        pytest.skip("no host compiler")
    exe = tmp_path / "tm_selftest"
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={flags}", "-fno-omit-frame-pointer",
           os.path.join(SRC, "token_mask.cpp"), os.path.join(SRC, "token_mask_selftest.cpp"), "-lpthread", "-o", str(exe)]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    if build.returncode != 0 and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtime not installed: " + build.stderr.strip().splitlines()[-1])
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="halt_on_error=1", TSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([str(exe), "4", "3000"], capture_output=True, text=True, timeout=300, env=env)
    print(run.stdout[-500:], run.stderr[-3000:])
    assert run.returncode == 0 and "selftest ok" in run.stdout
