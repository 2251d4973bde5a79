"""A compiled C consumer of the boundary: tests/c_abi/fixture.c includes include/q4_gpu.h as C99, is built
with -Wall -Wextra -Werror -pedantic and linked against libq4gpu.so -- the way the reference binds its device code
(plain linking, reference Makefile:21-25) -- and replays the reference's own fixture for this path
(src/q4_test.c:134-238).  Without a GPU the build and link are checked; with one the program runs."""
import os
import subprocess

import pytest

import q4gpu

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "c_abi", "fixture.c")
INC = os.path.dirname(q4gpu.HEADER_PATH)
LIBDIR = os.path.dirname(q4gpu.LIB_PATH)


def build(tmp_path):
    exe = str(tmp_path / "q4_c_fixture")
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-O1", "-I", INC, SRC, "-o", exe,
           "-L", LIBDIR, "-lq4gpu", "-lm", "-Wl,-rpath," + LIBDIR]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, "C consumer does not build:\n" + r.stdout
    return exe


def test_c_consumer_compiles_and_links_as_c99(tmp_path):
    assert os.path.exists(q4gpu.LIB_PATH), "libq4gpu.so not built"
    exe = build(tmp_path)
    assert os.path.exists(exe)
    # the header alone, as strict C99 and as C++
    for lang, std in (("c", "-std=c99"), ("c++", "-std=c++11")):
        r = subprocess.run(["gcc", "-x", lang, std, "-Wall", "-Wextra", "-Werror", "-pedantic", "-fsyntax-only", "-I", INC,
                            "-include", "q4_gpu.h", "-"], input="int main(void) { return 0; }\n",
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        assert r.returncode == 0, r.stdout


@pytest.mark.gpu
def test_c_consumer_replays_the_reference_fixture(tmp_path):
    exe = build(tmp_path)
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0, r.stdout
    assert "0 failure(s)" in r.stdout and "FAIL" not in r.stdout, r.stdout
    for must in ("f32 KV within 1e-3", "f16 KV within 2e-2", "q8_0 KV within 8e-2", "store decode over all rows"):
        assert "ok   " + "reference fixture, " + must in r.stdout or "ok   " + must in r.stdout, r.stdout
