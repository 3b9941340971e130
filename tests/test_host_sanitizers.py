"""The host library (cache bookkeeping, host sampler) under the compiler's sanitizers: `host_fuzz.cpp`
drives it with random valid call sequences; any out-of-bounds access, undefined arithmetic or data
race between the sampler's threads ends the run with a report. Skips where the compiler has no
sanitizer runtime. No GPU needed."""
import shutil
import subprocess
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
SOURCES = sorted((HERE.parent / "kapel_b200" / "csrc" / "host").glob("*.cpp"))


@pytest.mark.parametrize("flags", [["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], ["-fsanitize=thread"]],
                         ids=["address+undefined", "thread"])
def test_random_calls_under_sanitizers(flags, tmp_path):
    cxx = shutil.which("g++") or shutil.which("c++") or shutil.which("clang++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    exe = tmp_path / "host_fuzz"
    build = subprocess.run([cxx, "-O1", "-g", "-std=c++17", "-pthread", *flags, str(HERE / "host_fuzz.cpp"), *map(str, SOURCES), "-o", str(exe)],
                           capture_output=True, text=True)
    if build.returncode != 0:
        pytest.skip(f"the compiler cannot build with {flags[0]}: {build.stderr[-300:]}")
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and run.stdout.strip().endswith("ok"), run.stdout[-2000:] + run.stderr[-4000:]
