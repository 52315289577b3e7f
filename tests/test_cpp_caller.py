"""The C++ mirror of the reference's Rust API (include/sg_gpu.hpp) compiles against the C ABI and,
on a GPU, replays the reference's attn_decode_sliding test through it."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "parity_decode_sliding.bin")


def _build():
    from oracle import sg_oracle
    from super_gemma_b200 import build

    build.build()
    sg_oracle.build()
    pkg, orc = os.path.join(ROOT, "super_gemma_b200"), os.path.join(ROOT, "oracle")
    cmd = ["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "parity_decode_sliding.cpp"),
           "-o", EXE, f"-L{pkg}", "-l:libsgattn.so", f"-L{orc}", "-l:libsgoracle.so", f"-Wl,-rpath,{pkg}", f"-Wl,-rpath,{orc}"]
    subprocess.run(cmd, check=True)


def test_cpp_caller_builds_and_skips_without_a_gpu():
    import torch

    _build()
    if torch.cuda.is_available():
        pytest.skip("a device is present: covered by the gpu test")
    r = subprocess.run([EXE], capture_output=True, text=True)
    assert r.returncode == 77, r.stdout + r.stderr  # NoDevice surfaces as the reference's 'skip'


@pytest.mark.gpu
def test_cpp_caller_replays_the_reference_decode_test():
    _build()
    r = subprocess.run([EXE], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def test_cpp_page_cache_mirror():
    from super_gemma_b200 import build

    build.build()
    pkg = os.path.join(ROOT, "super_gemma_b200")
    exe = os.path.join(ROOT, "tests", "cpp", "page_cache.bin")
    subprocess.run(["g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "page_cache.cpp"), "-o", exe,
                    f"-L{pkg}", "-l:libsgattn.so", f"-Wl,-rpath,{pkg}"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and "page cache ok" in r.stdout, r.stdout + r.stderr
