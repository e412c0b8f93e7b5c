"""The C API (oracle_engine_b200/capi): the header from C and C++, errors as messages, and, on the GPU,
steps and generation through it against the Python engine that it runs."""
import ctypes
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle_engine_b200.capi import build as capi_build

TESTS = Path(__file__).resolve().parent


class GenParamsC(ctypes.Structure):
    _fields_ = [("n_predict", ctypes.c_int), ("temperature", ctypes.c_float), ("top_p", ctypes.c_float),
                ("top_k", ctypes.c_int), ("repeat_penalty", ctypes.c_float), ("repeat_last_n", ctypes.c_int),
                ("seed", ctypes.c_longlong), ("ignore_eos", ctypes.c_int), ("batch_size", ctypes.c_int),
                ("max_step_tokens", ctypes.c_int)]


ON_TOKEN = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.c_void_p)


@pytest.fixture(scope="module")
def lib():
    so = ctypes.CDLL(str(capi_build.build(verbose=False)))
    so.oe_last_error.restype = ctypes.c_char_p
    so.oe_load.restype = ctypes.c_void_p
    so.oe_load.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_longlong]
    so.oe_free.argtypes = [ctypes.c_void_p]
    for name in ("oe_vocab_size", "oe_max_seq_len", "oe_alloc_slot"):
        getattr(so, name).argtypes = [ctypes.c_void_p]
    so.oe_free_slot.argtypes = [ctypes.c_void_p, ctypes.c_int]
    so.oe_step.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 6
    so.oe_generate.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                               ctypes.POINTER(GenParamsC), ctypes.c_void_p, ctypes.c_void_p, ON_TOKEN, ctypes.c_void_p]
    so.oe_default_params.argtypes = [ctypes.POINTER(GenParamsC)]
    return so


@pytest.fixture(scope="module")
def demo(tmp_path_factory):
    """tests/capi_demo.c compiled as C against the header and the library."""
    capi_build.build(verbose=False)
    exe = tmp_path_factory.mktemp("capi") / "capi_demo"
    cmd = ["gcc", "-std=c99", "-Wall", "-Werror", "-o", str(exe), str(TESTS / "capi_demo.c")] + capi_build.link_flags()
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return str(exe)


def run_demo(exe, model_dir, dtype):
    env = dict(os.environ, OE_PYTHON=sys.executable)
    return subprocess.run([exe, model_dir, dtype], capture_output=True, text=True, env=env, timeout=600)


def ints(values):
    return np.ascontiguousarray(values, dtype=np.int32)


def ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_header_is_c_and_cpp(tmp_path):
    src = tmp_path / "use.c"
    src.write_text('#include "oe.h"\nint main(void) { oe_gen_params p; oe_default_params(&p); return p.top_k == 40 ? 0 : 1; }\n')
    include = f"-I{capi_build.HERE}"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only", include, str(src)], check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", include, str(src)], check=True)


def test_defaults_are_the_reference_s(lib):
    p = GenParamsC()
    lib.oe_default_params(ctypes.byref(p))
    assert (p.n_predict, p.top_k, p.repeat_last_n, p.seed, p.ignore_eos) == (256, 40, 64, 0, 0)
    assert (round(p.temperature, 6), round(p.top_p, 6), round(p.repeat_penalty, 6)) == (0.7, 0.9, 1.15)


def test_failures_come_back_as_messages(lib, tmp_path, model_dirs):
    assert lib.oe_load(str(tmp_path / "nothing").encode(), b"bfloat16", 64) is None
    assert b"config.json" in lib.oe_last_error()
    assert lib.oe_load(model_dirs["A"].encode(), b"float16", 64) is None
    assert b"dtype must be bfloat16 or float32" in lib.oe_last_error()
    assert lib.oe_load(model_dirs["A"].encode(), b"float32", 0) is None
    assert b"max_tokens" in lib.oe_last_error()
    assert lib.oe_alloc_slot(None) == -1 and b"handle is null" in lib.oe_last_error()
    assert lib.oe_step(None, 1, None, None, None, None, None, None) == -1
    lib.oe_free(None)


def test_no_device_is_a_message_not_a_crash(lib, model_dirs):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    assert lib.oe_load(model_dirs["A"].encode(), b"float32", 64) is None
    assert b"needs a CUDA device" in lib.oe_last_error()


@pytest.mark.gpu
def test_weight_errors_reach_the_c_caller(lib, tmp_path, model_dirs):
    """The loader's one error (missing, unexpected, wrong shapes) is the message a C program reads."""
    import json
    import shutil
    d = tmp_path / "broken"
    shutil.copytree(model_dirs["A"], d)
    raw = json.loads((d / "config.json").read_text())
    raw["intermediate_size"] += 8
    (d / "config.json").write_text(json.dumps(raw))
    assert lib.oe_load(str(d).encode(), b"float32", 64) is None
    msg = lib.oe_last_error().decode()
    assert "shape" in msg and "mlp" in msg, msg


def test_c_program_reports_a_missing_folder(demo, tmp_path):
    """A C program with an interpreter of its own (no Python process around it): the library starts one,
    finds the package beside itself and hands the loader's message back."""
    got = run_demo(demo, str(tmp_path / "nothing"), "bfloat16")
    assert got.returncode == 1, got.stderr
    assert "oe_load" in got.stderr and "config.json" in got.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_and_generation_through_the_c_api_equal_the_engine_s(lib, model_dirs, dtype):
    from oracle_engine_b200 import GenParams, SequenceStep
    from oracle_engine_b200.engine.engine import Engine
    folder = model_dirs["B"]
    eng = Engine.from_pretrained(folder, dtype=dtype, max_tokens=1024)
    h = lib.oe_load(folder.encode(), dtype.encode(), 1024)
    assert h, lib.oe_last_error()
    vocab = lib.oe_vocab_size(h)
    assert vocab == eng.spec.vocab_size and lib.oe_max_seq_len(h) == eng.max_seq_len
    # a batch of two prompts of unequal length, then one token each; logits bit for bit the engine's
    prompts = [[5, 17, 3, 9, 200, 41, 77], [8, 4]]
    slots_c = [lib.oe_alloc_slot(h) for _ in prompts]
    slots_p = [eng.alloc() for _ in prompts]
    assert min(slots_c) >= 0
    out = np.empty((3, vocab), dtype=np.float32)
    rows = lib.oe_step(h, 2, ptr(ints(slots_c)), ptr(ints(prompts[0] + prompts[1])), ptr(ints([7, 2])),
                       ptr(ints([0, 6, 1])), ptr(ints([2, 1])), ptr(out))
    assert rows == 3, lib.oe_last_error()
    ref = eng.step([SequenceStep(slots_p[0], prompts[0], [0, 6]), SequenceStep(slots_p[1], prompts[1], [1])])
    assert np.array_equal(out, ref.float().cpu().numpy())
    out1 = np.empty((2, vocab), dtype=np.float32)
    assert lib.oe_step(h, 2, ptr(ints(slots_c)), ptr(ints([11, 12])), ptr(ints([1, 1])), ptr(ints([0, 0])),
                       ptr(ints([1, 1])), ptr(out1)) == 2, lib.oe_last_error()
    ref1 = eng.step([SequenceStep(slots_p[0], [11], [0]), SequenceStep(slots_p[1], [12], [0])])
    assert np.array_equal(out1, ref1.float().cpu().numpy())
    # a refused step changes nothing: the same step afterwards gives what the engine gives
    assert lib.oe_step(h, 1, ptr(ints(slots_c[:1])), ptr(ints([vocab])), ptr(ints([1])), ptr(ints([0])),
                       ptr(ints([1])), ptr(out1)) == -1
    assert b"outside the vocabulary" in lib.oe_last_error()
    for s in slots_c:
        assert lib.oe_free_slot(h, s) == 0
    assert lib.oe_free_slot(h, slots_c[0]) == -1          # freed twice: an error, not a crash
    # generation: sampled, seeded, in two batches; tokens and the callback's order
    p = GenParamsC()
    lib.oe_default_params(ctypes.byref(p))
    p.n_predict, p.seed, p.batch_size, p.ignore_eos = 9, 4, 2, 1
    reqs = [[5, 17, 3], [8, 4, 100, 7, 7, 2], [300]]
    heard = []
    cb = ON_TOKEN(lambda i, tok, user: heard.append((i, tok)))
    got, lens = np.zeros(3 * 9, dtype=np.int32), np.zeros(3, dtype=np.int32)
    assert lib.oe_generate(h, 3, ptr(ints(sum(reqs, []))), ptr(ints([len(r) for r in reqs])), ctypes.byref(p),
                           ptr(got), ptr(lens), cb, None) == 0, lib.oe_last_error()
    want = eng.generate(reqs, GenParams(n_predict=9, temperature=float(np.float32(0.7)), top_p=float(np.float32(0.9)),
                                        repeat_penalty=float(np.float32(1.15)), seed=4, ignore_eos=True), batch_size=2)
    assert [got[i * 9:i * 9 + lens[i]].tolist() for i in range(3)] == want
    assert sorted(heard) == sorted((i, t) for i, new in enumerate(want) for t in new)
    lib.oe_free(h)


@pytest.mark.gpu
def test_c_program_steps_and_generates(demo, model_dirs):
    """The demo as a process of its own (embedded interpreter) against the engine in this process."""
    from oracle_engine_b200 import GenParams, SequenceStep
    from oracle_engine_b200.engine.engine import Engine
    folder = model_dirs["B"]
    got = run_demo(demo, folder, "float32")
    assert got.returncode == 0, got.stderr
    lines = dict((ln.split(" ", 1)[0] + (" " + ln.split(" ")[1] if ln.startswith(("argmax", "generated")) else ""), ln)
                 for ln in got.stdout.splitlines())
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=512)
    slot = eng.alloc()
    ref = eng.step([SequenceStep(slot, [5, 17, 3, 9, 200], [0, 4])]).argmax(-1).tolist()
    eng.free(slot)
    assert lines["vocab"] == f"vocab {eng.spec.vocab_size}"
    assert [int(lines[f"argmax {r}"].split()[2]) for r in range(2)] == ref
    assert "outside its 1 tokens" in lines["refused"]
    want = eng.generate([[5, 17, 3, 9, 200], [4, 8]], GenParams.greedy(6, ignore_eos=True))
    assert [[int(t) for t in lines[f"generated {i}"].split()[2:]] for i in range(2)] == want
    assert lines["heard"] == "heard 12"
