"""What the C API calls.  Every function takes plain values: an Engine, numbers, strings, and
the addresses of the caller's arrays, which are read and written here through ctypes.  An
exception raised here becomes the C function's error return and the text of gb_last_error().

Reference: the bodies of src/capi.rs:148-163 (load), 198-228 (set), 230-261 (run with a token
callback), 283-330 (info and stats as JSON); here over gemmars_b200.Engine and token ids.
"""
from __future__ import annotations

import ctypes
import json
from typing import List

REASON_CODES = {"stop": 0, "length": 1, "cancelled": 2}     # include/gemmars_b200.h: GB_STOP, GB_LENGTH, GB_CANCELLED
TOKEN_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int32, ctypes.c_int)


class StepItemC(ctypes.Structure):
    """struct GbStepItem."""
    _fields_ = [("slot", ctypes.c_int32), ("tokens", ctypes.POINTER(ctypes.c_int32)), ("n_tokens", ctypes.c_int32),
                ("want", ctypes.POINTER(ctypes.c_int32)), ("n_want", ctypes.c_int32)]


def _ints(address: int, n: int) -> List[int]:
    if n <= 0:
        return []
    if not address:
        raise ValueError("an array of token ids is NULL")
    return list((ctypes.c_int32 * n).from_address(address))


def _put_ints(address: int, values) -> None:
    if address and len(values):
        (ctypes.c_int32 * len(values)).from_address(address)[:] = list(values)


def parse_options(text: str):
    """``key=value`` pairs separated by newlines or ';'; lines that start with '#' are skipped
    (src/capi.rs:109-120)."""
    from ..engine.engine import EngineOptions
    opts = EngineOptions()
    for item in text.replace("\n", ";").split(";"):
        item = item.strip()
        if not item or item.startswith("#"):
            continue
        if "=" not in item:
            raise ValueError(f"option {item!r} is not key=value")
        k, v = item.split("=", 1)
        opts.set(k.strip(), v.strip())
    return opts


def devices() -> str:
    import torch
    if not torch.cuda.is_available():
        return "no CUDA device"
    lines = []
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        lines.append(f"cuda:{i} {p.name}, {p.multi_processor_count} SMs, {p.total_memory / 2**30:.0f} GiB, "
                     f"sm_{p.major}{p.minor}")
    return "\n".join(lines)


def load(model: str, options: str):
    from ..engine.engine import Engine
    return Engine.load(model, parse_options(options))


def free(engine) -> int:
    engine.reset()
    return 0


def set(engine, key: str, value: str) -> int:   # noqa: A001  (the C function's name)
    engine.set(key, value)
    return 0


def open_slot(engine) -> int:
    return engine.runner.open()


def close_slot(engine, slot: int) -> int:
    engine.runner.close(slot)
    return 0


def step(engine, items_addr: int, n_items: int, logits_addr: int, capacity: int) -> int:
    import numpy as np
    import torch
    from .. import kernels
    from ..engine.step import StepItem
    items = []
    for it in (StepItemC * n_items).from_address(items_addr) if n_items else []:
        toks = [it.tokens[i] for i in range(it.n_tokens)]
        want = [it.want[i] for i in range(it.n_want)]
        items.append(StepItem(int(it.slot), toks, want))
    rows = sum(len(it.want) for it in items)
    vocab = engine.runner.vocab_size
    if rows * vocab > capacity:
        raise ValueError(f"logits has room for {capacity} floats, the step writes {rows} x {vocab}")
    if rows and not logits_addr:
        raise ValueError("logits is NULL but logits are wanted")
    out = engine.runner.step(items)
    if out is not None:
        dst = np.ctypeslib.as_array((ctypes.c_float * (rows * vocab)).from_address(logits_addr))
        torch.from_numpy(dst).view(rows, vocab).copy_(out)
        kernels.check_status()
    return rows


def _callback(cb_addr: int, user_addr: int, cancel_addr: int):
    """on_token(index, tokens so far) -> False to end that sequence: the caller's function, and
    the flag that gb_engine_cancel sets."""
    fn = TOKEN_FN(cb_addr) if cb_addr else None
    cancel = ctypes.c_int.from_address(cancel_addr) if cancel_addr else None

    def on_token(index, tokens):
        if cancel is not None and cancel.value:
            return False
        if fn is not None and fn(user_addr or None, index, tokens[-1], len(tokens)) != 0:
            return False
        return True

    return on_token


def generate(engine, prompts_addr: int, lens_addr: int, n: int, out_addr: int, out_stride: int, out_lens_addr: int,
             out_reasons_addr: int, cb_addr: int, user_addr: int, cancel_addr: int) -> int:
    lens = _ints(lens_addr, n)
    pointers = list((ctypes.c_void_p * n).from_address(prompts_addr)) if n else []
    prompts = [_ints(p or 0, m) for p, m in zip(pointers, lens)]
    results = engine.generate(prompts, on_token=_callback(cb_addr, user_addr, cancel_addr))
    for i, r in enumerate(results):
        _put_ints(out_addr + 4 * i * out_stride if out_addr else 0, r.tokens[:max(out_stride, 0)])
    _put_ints(out_lens_addr, [len(r.tokens) for r in results])
    _put_ints(out_reasons_addr, [REASON_CODES[r.reason] for r in results])
    return 0


def _turn(run, tokens_addr, n_tokens, out_addr, capacity, out_len_addr, cb_addr, user_addr, cancel_addr) -> int:
    on_token = _callback(cb_addr, user_addr, cancel_addr)
    result = run(_ints(tokens_addr, n_tokens), lambda toks: on_token(0, toks))
    _put_ints(out_addr, result.tokens[:max(capacity, 0)])
    _put_ints(out_len_addr, [len(result.tokens)])
    return REASON_CODES[result.reason]


def send(engine, *args) -> int:
    return _turn(engine.send, *args)


def complete(engine, *args) -> int:
    return _turn(engine.complete, *args)


def reset(engine) -> int:
    engine.reset()
    return 0


def info_json(engine) -> str:
    return json.dumps(engine.info())


def stats_json(engine) -> str:
    return json.dumps(engine.stats_dict())
