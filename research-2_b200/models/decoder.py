"""A decoder put together from parts, and the order in which its layers run.

`ModelSpec` is data: which parts each layer has (LayerSpec), and a schedule, the list of layer
executions of one forward pass. A schedule entry names the layer to run and the cache member
it uses; an entry may name a layer that ran before (the layer runs again with the same
weights and a cache member of its own), or set `writes_cache=False` and name another entry's
member (the layer then reads keys and values that the owning layer wrote earlier in the same
pass). `DecoderModel` builds the parts from a spec and a name -> tensor dict and runs them; it
holds no knowledge of any architecture.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..cache.arena import MemberSpec
from ..parts import LayerSpec, PartSpec, Runtime, build_part, registry
from ..parts.embedding import Head, TokenEmbedding
from ..kernels.ops import resident_decode_rows as ops_resident_rows
from ..parts.resident import ResidentLayers


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int
    cache: int | None = None  # cache member id; None for a mixer without a per-token cache
    writes_cache: bool = True
    state: int | None = None  # state member id; None for a mixer without per-request state


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden: int
    max_seq_len: int
    eos_token: int | None
    embedding: str  # checkpoint name of the token table [V, D]
    head: str  # checkpoint name of the head table [V, D] (the embedding's when tied)
    positions: PartSpec | None
    layers: tuple[LayerSpec, ...]
    final_norm: PartSpec
    schedule: tuple[ScheduleEntry, ...] = field(default=())


def default_schedule(layers, mixers) -> tuple[ScheduleEntry, ...]:
    """Every layer once, in order, each with a cache member / state member of its own."""
    out, n_cache, n_state = [], 0, 0
    for i, _ in enumerate(layers):
        cache = state = None
        if getattr(mixers[i], "cache_spec", None) is not None:
            cache, n_cache = n_cache, n_cache + 1
        if getattr(mixers[i], "state_spec", None) is not None:
            state, n_state = n_state, n_state + 1
        out.append(ScheduleEntry(i, cache, True, state))
    return tuple(out)


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: dict[str, torch.Tensor], rt: Runtime, config=None):
        self.spec, self.rt, self.config = spec, rt, config
        self.vocab_size, self.hidden, self.max_seq_len = spec.vocab_size, spec.hidden, spec.max_seq_len
        self.eos_token = spec.eos_token
        self.embedding = TokenEmbedding(tensors[spec.embedding], rt)
        self.positions = build_part("positions", spec.positions, tensors, rt) if spec.positions else None
        self.blocks = []
        for layer in spec.layers:
            mixer = build_part("mixer", layer.mixer, tensors, rt)
            if self.positions is not None and hasattr(mixer, "rotary") and getattr(self.positions, "rotates", False):
                mixer.rotary = self.positions
            block_cls = registry("block")[layer.block]
            self.blocks.append(block_cls(
                build_part("norm", layer.norm_1, tensors, rt), mixer,
                build_part("norm", layer.norm_2, tensors, rt),
                build_part("feed_forward", layer.feed_forward, tensors, rt), rt.dtype))
        mixers = [b.mixer for b in self.blocks]
        self.schedule = spec.schedule or default_schedule(spec.layers, mixers)
        head_table = self.embedding.table if spec.head == spec.embedding else tensors[spec.head].to(rt.device, rt.dtype)
        self.head = Head(build_part("norm", spec.final_norm, tensors, rt), head_table, rt.dtype)
        self.cache_members, self.state_members = self._members(mixers)
        self._resident = None   # the one-kernel form of a decode step's layers, built at its first use
        self._resident_tried = False

    def _members(self, mixers) -> tuple[list[MemberSpec], list]:
        cache: dict[int, MemberSpec] = {}
        state: dict[int, object] = {}
        for entry in self.schedule:
            mixer = mixers[entry.layer]
            need = getattr(mixer, "cache_spec", None)
            if entry.cache is not None:
                if need is None:
                    raise ValueError(f"schedule: layer {entry.layer} has no per-token cache but names member {entry.cache}")
                if entry.writes_cache:
                    if entry.cache in cache:
                        raise ValueError(f"schedule: cache member {entry.cache} has two writers")
                    cache[entry.cache] = need
            elif need is not None:
                raise ValueError(f"schedule: layer {entry.layer} needs a cache member")
            if entry.state is not None:
                if entry.state in state:
                    raise ValueError(f"schedule: state member {entry.state} is used twice")
                state[entry.state] = mixer.state_spec
        for entry in self.schedule:  # readers come after their member's writer and fit its shape
            if entry.cache is not None and not entry.writes_cache:
                need = mixers[entry.layer].cache_spec
                have = cache.get(entry.cache)
                if have is None or (have.n_kv_heads, have.head_dim) != (need.n_kv_heads, need.head_dim):
                    raise ValueError(f"schedule: layer {entry.layer} reads cache member {entry.cache}, which "
                                     f"no earlier entry writes in a shape that fits")
        if sorted(cache) != list(range(len(cache))) or sorted(state) != list(range(len(state))):
            raise ValueError("schedule: cache and state member ids must count up from 0 without gaps")
        return [cache[i] for i in range(len(cache))], [state[i] for i in range(len(state))]

    def forward(self, ctx, cache_members, state_tensors) -> torch.Tensor:
        """The residual stream through the schedule, then logits at ctx.logit_rows: [W, V] float32."""
        table = self.positions.additive_table() if self.positions is not None else None
        x = self.embedding.forward(ctx, table)
        if ctx.decode_only and ctx.n_tokens <= ops_resident_rows():
            if not self._resident_tried:
                self._resident_tried = True
                self._resident = ResidentLayers.build(self.blocks, self.schedule, self.rt)
            if self._resident is not None and self._resident.forward(x, ctx, cache_members) is not None:
                return self.head.forward(x, ctx.logit_rows)
        for entry in self.schedule:
            cache = cache_members[entry.cache] if entry.cache is not None else None
            state = state_tensors[entry.state] if entry.state is not None else None
            x = self.blocks[entry.layer].forward(x, ctx, cache, state, entry.writes_cache)
        return self.head.forward(x, ctx.logit_rows)

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights that one step reads (each used tensor once)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.embedding.table if self.head.table.data_ptr() != self.embedding.table.data_ptr() else None)
        add(self.head.table)
        for obj in [self.head.norm] + [p for b in self.blocks for p in (b.norm_1, b.mixer, b.norm_2, b.feed_forward)]:
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor):
                    add(v)
        return total
