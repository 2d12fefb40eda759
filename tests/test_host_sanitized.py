"""The C++ host library (page pools, cache manager, scheduler, step packing) under AddressSanitizer and
UndefinedBehaviorSanitizer (CPU): the library is built with -fsanitize=address,undefined and the host-side
tests run against it in a child process with the sanitizer's runtime preloaded. Any report fails the run.
The reference records that it runs no such tool (PROGRESS.md:84-90)."""
import os
import shutil
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def test_host_library_under_asan_and_ubsan():
    cxx = runtime = None
    for cand in (os.environ.get("CXX"), "g++", "/usr/bin/g++", "clang++"):      # the first compiler that brings the runtime
        cand = cand and shutil.which(cand)
        if not cand:
            continue
        path = subprocess.run([cand, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
        if os.path.isabs(path) and os.path.exists(path):
            cxx, runtime = cand, path
            break
    if cxx is None:
        pytest.skip("no compiler with an AddressSanitizer runtime")
    # The C++ runtime goes in beside it: the interpreter does not link it, and the sanitizer looks up the
    # functions it intercepts (throwing an exception among them) when the process starts.
    stdcxx = subprocess.run([cxx, "-print-file-name=libstdc++.so.6"], capture_output=True, text=True).stdout.strip()
    if os.path.isabs(stdcxx) and os.path.exists(stdcxx):
        runtime = runtime + " " + stdcxx
    env = dict(os.environ, CXX=cxx, LLMRS_HOST_SANITIZE="1", LD_PRELOAD=runtime,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=97", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    files = [os.path.join(HERE, f) for f in ("test_cache_manager.py", "test_scheduler.py", "test_step_pack.py")]
    run = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider", *files],
                         capture_output=True, text=True, env=env, timeout=1200, cwd=os.path.dirname(HERE))
    text = run.stdout[-3000:] + run.stderr[-3000:]
    assert "AddressSanitizer" not in text and "runtime error" not in text, text
    assert run.returncode == 0, text
    assert " passed" in run.stdout
