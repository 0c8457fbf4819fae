"""The host-side cache manager and session table under AddressSanitizer + UBSan (CPU only).

``tests/sanitizer_driver.cpp`` is compiled together with the product's ``manager.cpp`` and
``sessions.cpp`` (``-fsanitize=address,undefined -fno-sanitize-recover=all``) and drives random
histories of create / step / popn / fork / destroy / reset, the work-split builders, and session
acquire / release / speculative rollback; any out-of-bounds access, use after free, leak or
undefined arithmetic ends the run with a non-zero exit code.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "combsengine_b200", "csrc")


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path_factory.mktemp("san") / "sanitizer_driver")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
           "-fno-omit-frame-pointer", os.path.join(ROOT, "tests", "sanitizer_driver.cpp"),
           os.path.join(CSRC, "manager.cpp"), os.path.join(CSRC, "sessions.cpp"), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_manager_and_sessions_are_clean_under_asan_and_ubsan(driver, seed):
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    r = subprocess.run([driver, str(seed)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    assert "sanitizer_driver ok" in r.stdout
