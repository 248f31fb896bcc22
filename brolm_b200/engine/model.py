"""The generic decoder: a layout of parts, built, loaded and run.

Nothing here names an architecture.  ``DecoderModel`` builds the parts a
``ModelLayout`` lists, loads their tensors by checkpoint name, and runs one
pass over the packed tokens of a step: embedding, the schedule of blocks, the
final norm at the wanted rows, the output matrix and the soft-cap
(order of operations as wlejon/brolm src/gemma2.cpp:326-415).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..cache import Cache
from ..config import ModelConfig, architecture_of, load_config
from ..parts import ModelLayout, Part, PartSpec, linear, part_class
from ..weights import Expected, WeightsError, load_from_folder, load_from_tensors, random_tensors, write_model_folder

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}


def as_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        if d not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {d}")
        return d
    try:
        return DTYPES[d]
    except KeyError:
        raise ValueError(f"unknown dtype '{d}' (bfloat16 or float32)") from None


class DecoderModel:
    def __init__(self, config: ModelConfig, dtype="bfloat16", device="cuda:0",
                 layout: Optional[ModelLayout] = None):
        self.config = config
        self.dtype = as_dtype(dtype)
        self.device = torch.device(device)
        self.layout = layout if layout is not None else architecture_of(config.to_dict()).layout(config)
        self._shared: dict[str, Part] = {}
        self._tensor_names: list[tuple[Part, dict]] = []
        self.blocks: list = []
        for bs in self.layout.blocks:
            # the arrangement is a registered part too: the layout names it, nothing here knows it
            built = {name: self._build(spec) for name, spec in bs.part_specs().items()}
            self.blocks.append(part_class("block", bs.kind)(**built))
        self.final_norm = self._build(self.layout.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.loaded = False
        self.generation = 0          # goes up whenever the tensors a captured step points at are replaced
        self.last_hidden: Optional[torch.Tensor] = None    # the final norm's rows of the last pass

    # construction ---------------------------------------------------------
    def _build(self, spec: PartSpec) -> Part:
        args = {}
        for k, v in spec.args.items():
            if isinstance(v, PartSpec):          # a part inside a part (the position encoding of a mixer)
                key = repr((v.kind, v.name, sorted(v.args.items())))
                if not v.tensors and key in self._shared:
                    v = self._shared[key]
                else:
                    built = self._build(v)
                    if not v.tensors:
                        self._shared[key] = built
                    v = built
            args[k] = v
        part = PartSpec(spec.kind, spec.name, args, spec.tensors).build()
        self._tensor_names.append((part, spec.tensors))
        return part

    def expected_tensors(self) -> dict[str, Expected]:
        """Checkpoint name -> shape and role, for the whole model."""
        out: dict[str, Expected] = {}
        emb = self.layout.embedding
        out[emb.tensor] = Expected((emb.vocab, emb.hidden), "table")
        for part, names in self._tensor_names:
            specs = part.param_specs()
            for local, spec in specs.items():
                if local not in names:
                    raise WeightsError(f"layout gives no checkpoint name for tensor '{local}' of a {part.kind}")
                out[names[local]] = Expected(tuple(spec.shape), spec.role)
        head = self.layout.head
        if head.tensor not in out:
            out[head.tensor] = Expected((emb.vocab, emb.hidden), "matrix", optional=head.tied_to is not None)
        return out

    # weights --------------------------------------------------------------
    def load_weights(self, source) -> "DecoderModel":
        """``source``: a model folder, or a dict of tensors by checkpoint name."""
        expected = self.expected_tensors()
        if isinstance(source, dict):
            tensors = load_from_tensors(source, expected, self.dtype, self.device, self.layout.optional_prefix)
        else:
            tensors = load_from_folder(str(source), expected, self.dtype, self.device, self.layout.optional_prefix)
        self._bind(tensors)
        return self

    def init_random(self, seed: int = 0, weight_std: Optional[float] = None, norm_std: Optional[float] = None,
                    on_device: bool = False) -> "DecoderModel":
        """Fill the model with seeded random weights without a folder in between: the values
        ``write_random_model`` writes for the same seed, made on the host or (``on_device``) on the
        model's device, which is what a model of gigabytes wants."""
        expected = self.expected_tensors()
        gen = random_tensors(expected, seed, weight_std if weight_std is not None else self.layout.weight_std,
                             norm_std if norm_std is not None else self.layout.norm_std,
                             dtype=self.dtype, device=self.device if on_device else "cpu")
        self._bind({n: t.to(self.device) for n, t in gen})
        return self

    def _bind(self, tensors: dict[str, torch.Tensor]) -> None:
        emb, head = self.layout.embedding, self.layout.head
        self.embedding = tensors[emb.tensor]
        if head.tensor in tensors:
            self.head = tensors[head.tensor]
        elif head.tied_to is not None:
            self.head = tensors[head.tied_to]          # the same storage, not a copy
        else:
            raise WeightsError(f"weights: {head.tensor} is missing and the output matrix is not tied",
                               missing=[head.tensor])
        for part, names in self._tensor_names:
            part.bind({local: tensors[ck] for local, ck in names.items() if local in part.param_specs()})
        self.loaded = True
        self.generation += 1

    # cache ----------------------------------------------------------------
    def cache_specs(self) -> list:
        specs = []
        for call in self.layout.schedule:
            specs.append(self.blocks[call.block].cache_spec() if call.cache_of is None else None)
        return specs

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None, max_seq_len: Optional[int] = None) -> Cache:
        cache = Cache(self.cache_specs(), max_tokens, self.dtype, self.device, max_slots=max_slots)
        positions = min(max_seq_len or cache.max_tokens, cache.max_tokens)
        for part, _ in self._tensor_names:
            part.prepare(positions, self.device)
        cache.max_positions = positions
        return cache

    # the pass -------------------------------------------------------------
    def forward(self, ctx, tokens: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Run the packed ``tokens`` of a step; logits (len(rows), vocab), float32."""
        if not self.loaded:
            raise RuntimeError("forward: weights not loaded")
        lay = self.layout
        h = torch.empty((ctx.n_tokens, lay.embedding.hidden), dtype=torch.float32, device=self.device)
        kernels.embed_scale(tokens, self.embedding, lay.embedding.scale, h)
        sched = lay.schedule
        first = self.blocks[sched[0].block].entry_norm
        x = first.apply(h, ctx.dtype) if first is not None else None
        for i, call in enumerate(sched):
            blk = self.blocks[call.block]
            src = i if call.cache_of is None else call.cache_of
            entry = ctx.cache.entries[src]
            nxt = self.blocks[sched[i + 1].block].entry_norm if i + 1 < len(sched) else None
            x = blk.forward(h, x, ctx, entry, call.cache_of is None, nxt)
        head_in = torch.float32 if self.head.dtype == torch.float32 else self.dtype
        if rows.numel() == 0:
            self.last_hidden = torch.empty((0, lay.embedding.hidden), dtype=head_in, device=self.device)
            return torch.empty((0, lay.embedding.vocab), dtype=torch.float32, device=self.device)
        xf = self.final_norm.apply(h, head_in, rows=rows)
        self.last_hidden = xf            # wlejon/brolm's hidden_out (include/brolm/gemma2.h:121-125)
        cap = float(lay.head.softcap or 0.0)
        if kernels.gemm_stream_ok(xf, self.head):
            # the largest stream of weights of a decode step: the TMA ring into tcgen05, soft-cap in the epilogue
            logits = torch.empty((xf.shape[0], self.head.shape[0]), dtype=torch.float32, device=self.device)
            kernels.gemm_stream(xf, self.head, logits, "softcap" if cap > 0 else "store", cap=cap)
            return logits
        logits = linear(xf, self.head, out_dtype=torch.float32)
        if cap > 0:
            kernels.softcap(logits, logits, cap)
        return logits


def load_model(folder: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Folder with config.json and safetensors -> a loaded model of the class config.json names."""
    from .. import models  # noqa: F401  (registers the architectures)
    config = load_config(folder)
    return DecoderModel(config, dtype, device).load_weights(folder)


def write_random_model(config: ModelConfig, folder: str, seed: int = 0, weight_std: Optional[float] = None,
                       norm_std: Optional[float] = None, dtype=torch.bfloat16, device="cpu") -> None:
    """Random-weights mode: write config.json and model.safetensors for ``config``.  The values are a
    function of (seed, tensor name, index) alone; ``device`` only says where they are computed."""
    from .. import models  # noqa: F401
    probe = DecoderModel(config, "float32", "cpu")
    lay = probe.layout
    write_model_folder(folder, config.to_dict(), probe.expected_tensors(), seed,
                       weight_std if weight_std is not None else lay.weight_std,
                       norm_std if norm_std is not None else lay.norm_std, dtype, device)
