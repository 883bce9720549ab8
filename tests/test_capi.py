"""The C API (include/gemmars_b200.h).  Without a GPU: the library builds, a C program links
against it, starts an interpreter of its own and gets the error conventions right (NULL or -1
with a message per thread, no crash on NULL), and the same holds when the library is loaded
into a process that is Python already.  With a GPU: a C program loads a model folder, generates,
steps, holds a conversation, and its tokens are those of the plain implementation."""
import ctypes
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def capi():
    from gemmars_b200.capi import build
    return build.library()


@pytest.fixture(scope="module")
def smoke_program(capi, tmp_path_factory):
    out = str(tmp_path_factory.mktemp("capi") / "capi_smoke")
    d = os.path.dirname(capi)
    subprocess.run(["gcc", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "capi_smoke.c"), "-L", d, "-lgemmars_b200", f"-Wl,-rpath,{d}", "-o", out],
                   check=True, capture_output=True, text=True)
    return out


def test_a_c_program_gets_errors_as_return_values(smoke_program):
    env = dict(os.environ, GEMMARS_B200_HOME=ROOT)
    p = subprocess.run([smoke_program, "--errors"], capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0, (p.returncode, p.stdout, p.stderr[-2000:])
    assert "not a model folder" in p.stdout and "unknown option 'no_such_option'" in p.stdout
    assert "version: " in p.stdout


def test_inside_a_python_process(capi, tmp_path):
    lib = ctypes.CDLL(capi)
    lib.gb_last_error.restype = ctypes.c_char_p
    lib.gb_version.restype = ctypes.c_char_p
    lib.gb_engine_load.restype = ctypes.c_void_p
    lib.gb_engine_load.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    assert lib.gb_version().decode().count(".") == 2
    assert lib.gb_engine_load(str(tmp_path / "none").encode(), None) is None
    assert "not a model folder" in lib.gb_last_error().decode()
    assert lib.gb_engine_load(str(tmp_path).encode(), b"dtype=int8") is None
    assert "dtype" in lib.gb_last_error().decode()
    # option strings: pairs separated by ';' or newlines, '#' lines skipped, a pair without '=' refused
    from gemmars_b200.capi import host
    o = host.parse_options("dtype=fp32\n# a comment\nmax_batch=3; cuda_graphs=0")
    assert (o.dtype, o.max_batch, o.cuda_graphs) == ("float32", 3, False)
    with pytest.raises(ValueError, match="not key=value"):
        host.parse_options("dtype")


@pytest.mark.gpu
def test_a_c_program_generates_steps_and_converses(smoke_program, model_folders):
    import numpy as np
    import plain_qwen3 as plain
    from tiny_configs import TINY_A
    folder = model_folders(TINY_A)
    pcfg, w = plain.load_folder(folder)
    env = dict(os.environ, GEMMARS_B200_HOME=ROOT)
    p = subprocess.run([smoke_program, folder, "dtype=float32;max_batch=4"], capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, (p.returncode, p.stdout[-2000:], p.stderr[-3000:])
    lines = dict(l.split(": ", 1) if ": " in l else (l.split(":")[0], "") for l in p.stdout.splitlines() if ":" in l)
    ids = lambda key: [int(x) for x in lines[key].split()]
    p0, p1 = [5, 17, 3, 9, 9], [4]
    gen = lambda prompt, n: plain.generate(pcfg, w, prompt, n)[0]
    assert "B200" in lines["devices"] or "cuda:0" in lines["devices"]
    info = json.loads(lines["info"])
    assert info["vocab_size"] == TINY_A["vocab_size"] and info["dtype"] == "float32" and info["layers"] == 2
    assert ids("generate0") == gen(p0, 6)
    assert ids("generate1") == gen(p1, 3)                       # cancelled by the callback after three tokens
    assert lines["reasons"].split()[:2] == ["1", "2"] and lines["reasons"].split()[-1] == "9"
    stats = json.loads(lines["stats"])
    assert stats["prompt_tokens"] == 6 and stats["generated_tokens"] >= 6
    assert int(lines["step_argmax"]) == plain.argmax(plain.forward(pcfg, w, p0 + [7])[-1].astype(np.float32))
    first = gen(p0, 6)
    assert ids("send0") == first
    assert ids("send1") == gen(p0 + first + p1, 6)              # the token that was not run is fed first
    assert ids("complete") == gen(p1, 6) and lines["code"] == "1"
