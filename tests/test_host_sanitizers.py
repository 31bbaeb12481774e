"""The C++ host runtime (cache manager, scheduler, step packing) under the
address and undefined-behaviour sanitizers: tests/host_sanitize.cpp drives it
with random traffic (arrivals, aborts, pre-emption, steps launched ahead,
window release) and audits the cache manager after every step."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "lyapunov_engine_b200", "csrc", "host")


@pytest.fixture(scope="module")
def binary(tmp_path_factory):
    compilers = [c for c in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++", shutil.which("clang++")) if c and os.path.exists(c)]
    if not compilers:
        pytest.skip("no C++ compiler")
    out = str(tmp_path_factory.mktemp("sanitize") / "host_sanitize")
    sources = [os.path.join(HOST, f) for f in ("block_manager.cpp", "scheduler.cpp", "step_pack.cpp")]
    said = ""
    for cxx in dict.fromkeys(compilers):        # the first that has the sanitizers' runtime libraries
        cmd = [cxx, "-std=c++20", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
               "-fno-sanitize-recover=all", "-Wall", "-Wextra", "-I", HOST, os.path.join(ROOT, "tests", "host_sanitize.cpp"),
               *sources, "-o", out]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode == 0:
            break
        said = proc.stdout
        missing_runtime = "cannot find" in said and ("asan" in said.lower() or "ubsan" in said.lower())
        assert missing_runtime, said[-3000:]
    else:
        pytest.skip("no compiler here has the sanitizers' runtime libraries: " + said[-300:])
    return out


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_traffic_under_sanitizers(binary, seed):
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    proc = subprocess.run([binary, str(seed), "600"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env,
                          timeout=120)
    assert proc.returncode == 0, proc.stdout[-4000:]
    import re
    counts = dict(zip(("steps", "ahead", "pages", "reused", "preemptions"), map(int, re.findall(r"(\d+) (?:steps|launched|pages|of them|pre-emptions)", proc.stdout))))
    assert counts["steps"] > 100 and counts["ahead"] > 0 and counts["reused"] > 0 and counts["preemptions"] > 0, proc.stdout
