"""The host-side native code under sanitizers: the stress program (``csrc/selftest/native_stress.cpp``) is built once with the
thread sanitizer (loader workers, slot ring, consumer) and once with the address + undefined-behaviour sanitizers (shard
reader, BPE containers, KV page pool under random operations, GGUF reader on thousands of damaged files) and must exit 0 with nothing reported."""
import shutil
import subprocess
from pathlib import Path

import pytest

CSRC = Path(__file__).resolve().parent.parent / "openagents_b200" / "csrc"
SOURCES = [CSRC / "selftest" / "native_stress.cpp", CSRC / "data" / "token_data.cpp", CSRC / "data" / "bpe.cpp", CSRC / "kv" / "kv_alloc.cpp",
           CSRC / "gguf" / "gguf.cpp", CSRC / "gguf" / "quant.cpp"]


@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_native_stress_is_clean(tmp_path, sanitizer):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = tmp_path / "stress"
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-I", str(CSRC), *map(str, SOURCES), "-o", str(exe),
                            "-pthread", "-fopenmp"],
                           capture_output=True, text=True)
    if build.returncode != 0 and ("cannot find" in build.stderr or "sanitizer" in build.stderr.lower() and "unrecognized" in build.stderr):
        pytest.skip("this toolchain has no " + sanitizer + " sanitizer runtime")
    assert build.returncode == 0, build.stderr[-2000:]
    scratch = tmp_path / "scratch"
    scratch.mkdir()
    run = subprocess.run([str(exe), str(scratch)], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "0 failed checks" in run.stdout and "WARNING: ThreadSanitizer" not in run.stderr and "ERROR: AddressSanitizer" not in run.stderr
    assert "runtime error" not in run.stderr                  # what the undefined-behaviour sanitizer prints
