"""The Python entry point: load a model once, then generate.

The names follow the reference's library API where it has them: ``Engine.load(model, options)``
with options as ``key=value`` pairs (src/engine.rs:72-119, 252-329; the C API passes them as
``"k=v;k=v"``, src/capi.rs:109-120), ``set(key, value)`` for the per-turn settings
``max_tokens, temperature, top_k, top_p, seed`` (src/capi.rs:198-228), ``complete`` for a prompt
on its own and ``send`` for the next turn of the one conversation the engine keeps
(src/engine.rs:981-1064), ``reset`` (src/engine.rs:958), ``info`` and ``stats``
(src/engine.rs:405-499).  Prompts and replies are token ids; text goes through a tokenizer.json
when the folder has one.  ``generate`` (batches of prompts) is this engine's own.
"""
from __future__ import annotations

import dataclasses
import os
from typing import List, Optional, Sequence

from .. import kernels
from ..config.base import load_stop_ids
from ..sampling.sampler import BatchSampler, SamplingParams
from .generate import Generated, GenerationLoop, Request
from .model import build_model
from .step import Runner, StepItem


def _parse_bool(key, v):
    if v in ("1", "true", "yes", "on"):
        return True
    if v in ("0", "false", "no", "off", ""):
        return False
    raise ValueError(f"{key}: expected true or false, got {v!r}")


def _parse_opt_int(key, v):
    try:
        n = int(v)
    except ValueError:
        raise ValueError(f"{key}: expected a number, got {v!r}") from None
    return n if n > 0 else None


@dataclasses.dataclass
class EngineOptions:
    """How to load and run a model.  Keys of ``set``: see ``KEYS``."""
    dtype: str = "bfloat16"              # "bfloat16" or "float32" (the true 32-bit path)
    device: str = "cuda:0"               # src/engine.rs:83-85 (here: a CUDA device)
    prefill_chunk: Optional[int] = None  # tokens of one sequence per prefill step (src/engine.rs:86-87)
    max_context: Optional[int] = None    # most tokens of one sequence (src/engine.rs:88-90)
    max_batch: int = 64                  # most sequences generating together
    max_tokens: Optional[int] = None     # tokens the cache holds over all sequences
    cuda_graphs: bool = True             # replay decode steps from captured graphs
    decode_ahead: bool = True            # launch the next decode step before the host has read this step's tokens
    profile: bool = False

    KEYS = ("dtype", "device", "prefill_chunk", "max_context", "max_batch", "max_tokens", "cuda_graphs", "decode_ahead",
            "profile")

    def set(self, key: str, value: str) -> None:
        """Sets an option by name; unknown keys are errors (src/engine.rs:276-329)."""
        if key == "dtype":
            v = {"bf16": "bfloat16", "fp32": "float32", "f32": "float32"}.get(value, value)
            if v not in ("bfloat16", "float32"):
                raise ValueError(f"dtype: unknown precision {value!r} (use bfloat16 or float32)")
            self.dtype = v
        elif key == "device":
            if value not in ("auto", "cuda") and not value.startswith("cuda:"):
                raise ValueError(f"device: unknown device {value!r} (auto|cuda|cuda:N); there is no CPU path")
            self.device = "cuda:0" if value in ("auto", "cuda") else value
        elif key in ("prefill_chunk", "max_context", "max_tokens"):
            setattr(self, key, _parse_opt_int(key, value))
        elif key == "max_batch":
            self.max_batch = _parse_opt_int(key, value) or 1
        elif key in ("cuda_graphs", "decode_ahead", "profile"):
            setattr(self, key, _parse_bool(key, value))
        else:
            raise ValueError(f"unknown option {key!r} (known: {', '.join(self.KEYS)})")

    @classmethod
    def parse(cls, text) -> "EngineOptions":
        """From ``"k=v;k=v"`` (src/capi.rs:109-120), a dict, or an EngineOptions."""
        if isinstance(text, cls):
            return text
        opts = cls()
        if not text:
            return opts
        pairs = text.items() if isinstance(text, dict) else (
            p.split("=", 1) if "=" in p else (p, "true") for p in str(text).split(";") if p.strip())
        for k, v in pairs:
            opts.set(str(k).strip(), str(v).strip())
        return opts


@dataclasses.dataclass
class Stats:
    """Counters of the last call (src/engine.rs:405-435)."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_secs: float = 0.0
    decode_secs: float = 0.0
    decode_steps: int = 0

    def line(self) -> str:  # src/main.rs:486-496
        return ("[prefill {} tok in {:.2f}s = {:.1f} tok/s | decode {} tok in {:.2f}s = {:.1f} tok/s]".format(
            self.prompt_tokens, self.prefill_secs, self.prompt_tokens / max(self.prefill_secs, 1e-9),
            self.generated_tokens, self.decode_secs, self.generated_tokens / max(self.decode_secs, 1e-9)))


class Engine:
    SETTINGS = ("max_tokens", "temperature", "top_k", "top_p", "seed", "stop")

    def __init__(self, model, options: EngineOptions, folder: Optional[str] = None):
        self.model, self.options, self.folder = model, options, folder
        cfg_limit = model.plan.max_positions or None
        self.max_context = min(x for x in (options.max_context, cfg_limit, 1 << 30) if x)
        cache_tokens = options.max_tokens or min(self.max_context, 8192) * min(options.max_batch, 8)
        self.runner = Runner(model, max_tokens=cache_tokens, max_batch=options.max_batch,
                             prefill_chunk=options.prefill_chunk or 2048,
                             use_graphs=options.cuda_graphs and not options.profile)
        self.max_context = min(self.max_context, self.runner.cache.max_seq_len)
        self.stop_ids = list(model.plan.stop_ids)
        if folder is not None:
            self.stop_ids = load_stop_ids(folder, fallback=self.stop_ids) or self.stop_ids
        self.max_new_tokens = 1024
        self.sampling = SamplingParams()
        self.stats = Stats()
        self._conv_slot = None
        self._unfed = None
        self._tokenizer = None

    # ---- loading
    @classmethod
    def load(cls, model: str, options=None) -> "Engine":
        """Loads the model folder ``model`` (config.json + safetensors)."""
        opts = EngineOptions.parse(options)
        if not os.path.isdir(model):
            raise FileNotFoundError(f"{model}: not a model folder (downloads are not supported)")
        return cls(build_model(model, dtype=opts.dtype, device=opts.device), opts, folder=model)

    @classmethod
    def from_config(cls, raw_config: dict, tensors: dict, options=None, consume: bool = False) -> "Engine":
        """An engine over tensors given directly ({checkpoint name: tensor}), e.g. random weights.
        With ``consume`` the tensors are taken out of the dict as they are bound, so that a large
        model and the stacked copies made of it never lie in memory side by side."""
        opts = EngineOptions.parse(options)
        return cls(build_model(raw_config=raw_config, tensors=tensors, dtype=opts.dtype, device=opts.device,
                               consume=consume), opts)

    # ---- settings
    def set(self, key: str, value) -> None:
        """Per-turn settings: max_tokens, temperature, top_k, top_p, seed (src/capi.rs:198-228),
        and stop (comma-separated token ids replacing the checkpoint's)."""
        v = str(value)
        if key == "max_tokens":
            self.max_new_tokens = int(v)
        elif key == "temperature":
            self.sampling = dataclasses.replace(self.sampling, temperature=float(v))
        elif key == "top_k":
            self.sampling = dataclasses.replace(self.sampling, top_k=int(v))
        elif key == "top_p":
            self.sampling = dataclasses.replace(self.sampling, top_p=float(v))
        elif key == "seed":
            self.sampling = dataclasses.replace(self.sampling, seed=int(v))
        elif key == "stop":
            self.stop_ids = [int(x) for x in v.split(",") if x.strip()]
        else:
            raise ValueError(f"unknown setting {key!r} (known: {', '.join(self.SETTINGS)})")
        self.sampling.check()

    # ---- generation
    def _loop(self) -> GenerationLoop:
        r = self.runner

        def step(items):
            return r.step([StepItem(slot, toks, [len(toks) - 1]) for slot, toks in items])

        def make_sampler(params):
            return BatchSampler([p or self.sampling for p in params], r.device)

        # a batch is as large as the free slots allow: the conversation of ``send`` holds one
        return GenerationLoop(r.open, r.close, step, make_sampler,
                              max(1, min(self.options.max_batch, r.cache.slots.free_count)),
                              r.cache.n_pages - r.cache.pages_held(), r.cache.page_size, self.max_context,
                              step_ahead=r.decode_from_device if self.options.decode_ahead else None)

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: Optional[int] = None,
                 sampling: Optional[SamplingParams] = None, stop_ids: Optional[Sequence[int]] = None,
                 on_token=None) -> List[Generated]:
        """Generates for each prompt (token ids), in batches of unequal lengths.  Sequence ``i``
        draws from a generator seeded ``seed + i``."""
        base = sampling or self.sampling
        reqs = [Request(list(p), max_tokens if max_tokens is not None else self.max_new_tokens,
                        tuple(self.stop_ids if stop_ids is None else stop_ids),
                        dataclasses.replace(base, seed=base.seed + i)) for i, p in enumerate(prompts)]
        loop = self._loop()
        results = loop.run(reqs, on_token)
        kernels.check_status()
        self.stats = Stats(sum(len(p) for p in prompts), loop.decode_tokens, loop.prefill_secs, loop.decode_secs,
                           loop.decode_steps)
        return results

    def complete(self, prompt: Sequence[int], on_token=None) -> Generated:
        """One prompt on its own, outside the conversation (src/engine.rs:1025-1035)."""
        cb = (lambda i, toks: on_token(toks)) if on_token else None
        base = self.sampling
        loop = self._loop()
        req = Request(list(prompt), self.max_new_tokens, tuple(self.stop_ids), base)
        return self._timed(loop, [req], cb)[0]

    def _timed(self, loop, reqs, cb):
        res = loop.run(reqs, cb)
        kernels.check_status()
        self.stats = Stats(sum(len(r.prompt) for r in reqs), loop.decode_tokens, loop.prefill_secs,
                           loop.decode_secs, loop.decode_steps)
        return res

    def send(self, tokens: Sequence[int], on_token=None) -> Generated:
        """The next turn of the engine's conversation: appends ``tokens`` to what the cache holds
        and generates a reply; the cache is kept for the turn after (src/engine.rs:981-1064).
        A last token that was generated but not run is fed first (src/generate.rs:105-128).
        A turn that fails after it began forgets the conversation (``reset``)."""
        r = self.runner
        if self._conv_slot is None:
            self._conv_slot = r.open()
        feed = ([self._unfed] if self._unfed is not None else []) + list(tokens)
        if not feed:
            raise ValueError("send: no tokens")
        loop = self._loop()
        cb = (lambda i, toks: on_token(toks)) if on_token else None
        req = Request(feed, self.max_new_tokens, tuple(self.stop_ids), self.sampling)
        try:
            res = loop.run_in_slot(self._conv_slot, r.length(self._conv_slot), req, cb)
            kernels.check_status()
        except ValueError:
            raise                     # refused before anything ran: the conversation is as it was
        except BaseException:
            # a turn that broke off half way leaves a cache that matches no conversation
            self.reset()
            raise
        self._unfed = res.unfed
        self.stats = Stats(len(feed), loop.decode_tokens, loop.prefill_secs, loop.decode_secs, loop.decode_steps)
        return res

    def reset(self) -> None:
        """Forgets the conversation (src/engine.rs:958)."""
        if self._conv_slot is not None:
            self.runner.close(self._conv_slot)
        self._conv_slot, self._unfed = None, None

    # ---- text, when the folder has a tokenizer
    def tokenizer(self):
        if self._tokenizer is None:
            path = os.path.join(self.folder or "", "tokenizer.json")
            if not os.path.exists(path):
                raise FileNotFoundError(f"{path}: no tokenizer in the model folder; pass token ids")
            try:
                from tokenizers import Tokenizer
            except ImportError:
                raise RuntimeError("the 'tokenizers' package is not installed; pass token ids") from None
            self._tokenizer = Tokenizer.from_file(path)
        return self._tokenizer

    # ---- description
    def info(self) -> dict:
        """What was loaded (src/engine.rs:475-499)."""
        cfg = self.model.config
        d = {"architecture": type(cfg).__name__, "dtype": self.model.compute, "layers": len(self.model.plan.layers),
             "hidden_size": self.model.plan.hidden_size, "vocab_size": self.model.plan.vocab_size,
             "max_context": self.max_context, "weight_bytes": self.model.weight_bytes(),
             "cache_pages": self.runner.cache.n_pages, "page_size": self.runner.cache.page_size,
             "stop_ids": list(self.stop_ids)}
        return d

    def profile_start(self) -> None:
        """Starts the per-kernel timing that ``profile_report`` prints (option ``profile``; decode
        steps then run without CUDA graphs so that every launch can be timed)."""
        self._profile_from = self.runner.tokens_run
        kernels.profile_start()

    def profile_report(self) -> str:
        """Time, calls, bytes and bandwidth per category and time per kernel since
        ``profile_start``, per forward token (src/prof.rs:51-83)."""
        return kernels.profile_report(max(1, self.runner.tokens_run - getattr(self, "_profile_from", 0)))

    def stats_dict(self) -> dict:
        return dataclasses.asdict(self.stats)
