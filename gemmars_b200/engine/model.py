"""A model built from a plan: its parts, their weights, and the forward pass over one step.

``DecoderModel`` knows nothing of any architecture: it builds the parts a ``ModelPlan`` names,
asks them which tensors they want, binds those from a checkpoint (or from tensors given
directly), and runs the plan's schedule.  Which model class a folder gets is decided by its
config.json through the architecture registry.

Reference: ``QwenModel::load`` (src/qwen.rs:458-544) and ``forward_impl`` (src/qwen.rs:658-701).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.registry import load_config
from ..csrc import build
from ..parts.base import StepContext, build_block, build_part, compute_dtype
from ..parts.plan import ModelPlan
from ..weights.loader import check_checkpoint, load_checkpoint
from ..weights.safetensors_io import ModelFiles


class DecoderModel:
    def __init__(self, plan: ModelPlan, compute: str, device):
        plan.validate()
        self.plan, self.compute, self.device = plan, compute, torch.device(device)
        self.act_dtype = compute_dtype(compute)
        self.embedding = build_part("embedding", plan.embedding, compute)
        self.blocks = [build_block(ls, compute) for ls in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm, compute)
        self.head = build_part("head", plan.head, compute)
        self.config = None
        self.ignored_tensors = []

    # ---- parts and the tensors they want
    def named_parts(self):
        """(part, its spec) for every part that can hold weights: the model's own and whatever
        each block says it built."""
        yield self.embedding, self.plan.embedding
        for block in self.blocks:
            for part in block.parts().values():
                yield part, part.spec
        yield self.final_norm, self.plan.final_norm
        yield self.head, self.plan.head

    def expected_tensors(self) -> Dict[str, tuple]:
        """{checkpoint tensor name: shape} over all parts."""
        out = {}
        for part, spec in self.named_parts():
            for short, want in part.wants().items():
                name = spec.tensors.get(short)
                if name is None:
                    if want.optional:
                        continue
                    raise ValueError(f"{spec.kind}: the plan names no checkpoint tensor for {short!r}")
                if name in out and tuple(out[name]) != tuple(want.shape):
                    raise ValueError(f"tensor {name} is wanted with shapes {out[name]} and {want.shape}")
                out[name] = tuple(want.shape)
        return out

    def kernel_units(self):
        units = []
        for part, _ in self.named_parts():
            for u in part.kernel_units():
                if u not in units:
                    units.append(u)
        return units

    def bind(self, tensors: Dict[str, torch.Tensor], consume: bool = False) -> None:
        """Gives every part its tensors: matrices in the compute precision, vectors in float32.
        A matrix stored in 32-bit is rounded to bfloat16 for the bfloat16 engine, as the
        reference does for its bf16 matmuls (src/safetensors.rs:707-733).  With ``consume`` a
        tensor leaves ``tensors`` when the last part that wants it has been given it: parts that
        stack matrices (q/k/v, gate/up) make copies, and the originals are then freed part by
        part instead of all at the end."""
        uses = {}
        for part, spec in self.named_parts():
            for short in part.wants():
                name = spec.tensors.get(short)
                if name is not None:
                    uses[name] = uses.get(name, 0) + 1
        converted = {}

        def get(name, role):
            want = torch.float32 if role == "vector" else self.act_dtype
            key = (name, want)
            t = converted.get(key)
            if t is None:
                t = tensors[name]
                if t.device != self.device:
                    t = t.to(self.device)
                if t.dtype != want:
                    t = t.to(want)
                if uses[name] > 1:
                    converted[key] = t          # tied tensors: the same device tensor for every user
            uses[name] -= 1
            if uses[name] == 0:
                for k in [k for k in converted if k[0] == name]:
                    del converted[k]
                if consume:
                    del tensors[name]
            return t

        for part, spec in self.named_parts():
            mine = {}
            for short, want in part.wants().items():
                name = spec.tensors.get(short)
                if name is not None and name in tensors:
                    mine[short] = get(name, want.role)
            part.load(mine)
            del mine

    # ---- cache needs of the schedule
    def cache_needs(self):
        """[(schedule position, [needs])] for entries that keep something of their own."""
        needs = []
        for i, e in enumerate(self.plan.schedule):
            if e.cache_of is not None:
                continue
            mine = self.blocks[e.layer].cache_needs()
            if mine:
                needs.append((i, list(mine)))
        return needs

    # ---- the step
    def forward(self, ctx: StepContext, tokens: torch.Tensor) -> torch.Tensor:
        """Runs the step's packed tokens through the schedule; returns the float32 residual
        stream [T, H] before the final norm."""
        # what the parts keep for the length of a step (a table of angles shared by the layers) is
        # made anew by every run: a context that is run again, eagerly and then under capture,
        # must launch the kernels that fill it again
        ctx.extras.clear()
        x = torch.empty((tokens.numel(), self.plan.hidden_size), dtype=torch.float32, device=self.device)
        self.embedding.forward(ctx, tokens, x)
        carry = None          # what a block's last product left for the next block's first norm
        schedule = self.plan.schedule
        for i, e in enumerate(schedule):
            owner = i if e.cache_of is None else e.cache_of
            block = self.blocks[e.layer]
            ctx.extras["entry"] = i
            if getattr(block, "chains_norms", False):
                after = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
                next_norm = after.first_norm() if getattr(after, "chains_norms", False) else None
                carry = block.forward(ctx, x, ctx.cache.views(owner), writes_cache=e.cache_of is None, h_in=carry,
                                      next_norm=next_norm)
            else:
                block.forward(ctx, x, ctx.cache.views(owner), writes_cache=e.cache_of is None)
                carry = None
        return x

    def logits(self, ctx: StepContext, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] at the packed-token rows ``rows`` (int32)."""
        h = self.final_norm.forward(ctx, x, rows_index=rows)
        return self.head.forward(ctx, h)

    def weight_bytes(self) -> int:
        """Bytes of weights a decode step reads: what each part says of itself, every run of the
        schedule counted (a layer that runs twice is read twice)."""
        runs = {}
        for e in self.plan.schedule:
            runs[e.layer] = runs.get(e.layer, 0) + 1
        total = self.embedding.weight_bytes() + self.final_norm.weight_bytes() + self.head.weight_bytes()
        for i, block in enumerate(self.blocks):
            total += runs.get(i, 0) * sum(part.weight_bytes() for part in block.parts().values())
        return total

    @property
    def capture_depends_on_length(self) -> bool:
        return any(part.capture_depends_on_length for part, _ in self.named_parts())


def build_model(folder: Optional[str] = None, *, raw_config: Optional[dict] = None,
                tensors: Optional[Dict[str, torch.Tensor]] = None, dtype: str = "bfloat16",
                device="cuda:0", compile_kernels: bool = True, consume: bool = False) -> DecoderModel:
    """The model of a folder (config.json + safetensors), or of ``raw_config`` with ``tensors``
    given directly ({checkpoint name: tensor}, e.g. random weights made on the device)."""
    from .. import models  # noqa: F401  (registers the architectures)
    from ..config.registry import resolve_architecture

    if folder is not None:
        arch, cfg = load_config(folder)
        files = ModelFiles(folder)
        names = files.names()
    else:
        arch = resolve_architecture(raw_config)
        cfg = arch.config_class.from_dict(raw_config)
        files, names = None, set(tensors)
    plan = arch.build_plan(cfg, names)
    model = DecoderModel(plan, dtype, device)
    model.config = cfg
    ignored = getattr(plan, "ignored_tensors", [])
    expected = model.expected_tensors()
    if compile_kernels:
        build.ensure(model.kernel_units())
    if files is not None:
        loaded = load_checkpoint(files, expected, ignored, device=model.device)
    else:
        check_checkpoint({n: tuple(t.shape) for n, t in tensors.items()}, expected, ignored, where="(given tensors)")
        loaded = tensors
    model.bind(loaded, consume=consume or files is not None)
    return model
