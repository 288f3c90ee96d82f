"""A decode step's layers as one resident kernel, where the layers are of the kind it is written for.

`ResidentLayers.build` looks at a model's schedule and returns a runner if EVERY entry is a
pre-norm block of paged attention (no rotation of queries and keys), a dense feed-forward and
LayerNorms, in bfloat16, with sizes that the kernel takes (csrc/kernels/decode_resident.cu);
otherwise None, and the model walks its parts one by one as always. Parts say what they are by
duck typing: a block offers `resident_layer()`, which asks its mixer for `resident_attention()`,
its feed-forward for `resident_mlp()` and its norms for `layer_norm_params()`; a part that has
no such method (every part that a test or another architecture defines) simply keeps the whole
model on the general path. The runner holds a second copy of the four matrices of each layer
in the kernel's operand order (`ops.pack_weight_tiles`) and the scratch that the kernel's
phases hand each other; both are allocated once, so a step that runs as a CUDA graph finds
them in place.
"""

from __future__ import annotations

import ctypes as C

import torch

from ..kernels import ops


class ResidentLayers:
    MAX_ROWS = 64

    def __init__(self, layers: list[dict], schedule, device):
        first = layers[schedule[0].layer]
        self.device = device
        self.head_dim, self.n_heads, self.n_kv_heads = first["head_dim"], first["n_heads"], first["n_kv_heads"]
        self.width, self.inner = first["width"], first["inner"]
        self.schedule = schedule
        self.layers = layers
        lib = ops.decode_resident_library(self.head_dim)
        self.max_rows = min(self.MAX_ROWS, int(lib.r2_decode_resident_max_rows()))
        self.packed = {}
        for i, layer in enumerate(layers):
            if any(e.layer == i for e in schedule):
                self.packed[i] = {name: ops.pack_weight_tiles(layer[name]) for name in ("w_qkv", "w_out", "w_fc", "w_pr")}
        rows, qkv_width = self.max_rows, (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        bf16 = dict(dtype=torch.bfloat16, device=device)
        self.qkv = torch.zeros(rows, qkv_width, **bf16)
        self.mixed = torch.zeros(rows, self.n_heads * self.head_dim, **bf16)
        self.hidden = torch.zeros(rows, self.inner, **bf16)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)   # the grid barrier's, zero between launches
        self._tables: dict[int, torch.Tensor] = {}   # layer tables by the cache they point into
        self.stamps = None   # profiling: an int64 tensor of 1 + 10 * layers values that CTA 0 fills with the nanosecond clock

    @classmethod
    def build(cls, blocks, schedule, rt) -> "ResidentLayers | None":
        if rt.dtype != torch.bfloat16 or not schedule:
            return None
        layers = []
        for block in blocks:
            describe = getattr(block, "resident_layer", None)
            layers.append(describe() if describe is not None else None)
        used = [layers[e.layer] for e in schedule]
        if any(layer is None for layer in used):
            return None
        if any(e.cache is None or not e.writes_cache or e.state is not None for e in schedule):
            return None
        first = used[0]
        same = ("head_dim", "n_heads", "n_kv_heads", "width", "inner")
        if any(layer[k] != first[k] for layer in used for k in same):
            return None
        if first["head_dim"] > 128 or first["n_heads"] // first["n_kv_heads"] > 8 or first["width"] % 16 or first["inner"] % 16:
            return None
        return cls(layers, schedule, rt.device)

    def _table(self, cache_members) -> torch.Tensor:
        key = cache_members[self.schedule[0].cache].k.data_ptr()
        table = self._tables.get(key)
        if table is None:
            rows = (ops.ResidentLayerC * len(self.schedule))()
            for i, entry in enumerate(self.schedule):
                layer, packed, member = self.layers[entry.layer], self.packed[entry.layer], cache_members[entry.cache]
                if member.group >= ops.RESIDENT_MAX_GROUPS:
                    return None
                r = rows[i]
                for name in ("w_qkv", "w_out", "w_fc", "w_pr"):
                    setattr(r, name, packed[name].data_ptr())
                for name in ("b_qkv", "b_out", "b_fc", "b_pr", "ln1_g", "ln1_b", "ln2_g", "ln2_b"):
                    setattr(r, name, layer[name].data_ptr())
                r.k_cache, r.v_cache, r.page_stride = member.k.data_ptr(), member.v.data_ptr(), member.page_stride
                r.group, r.page_size, r.n_pages, r.window = member.group, member.page_size, member.n_pages, layer["window"]
                r.scale, r.eps1, r.eps2, r.act = layer["scale"], layer["eps1"], layer["eps2"], ops.ACTIVATIONS[layer["act"]]
            raw = torch.frombuffer(bytearray(bytes(rows)), dtype=torch.uint8)
            table = self._tables[key] = raw.to(self.device)
        return table

    def forward(self, x: torch.Tensor, ctx, cache_members) -> torch.Tensor | None:
        """x [T, D] float32 through every layer, in place; None where the kernel does not take the
        batch (the caller then walks the parts)."""
        n = x.shape[0]
        most = min(self.max_rows, ops.resident_decode_rows())
        if self.width > 1024 and n > 8:
            # measured at width 1,600 (GPT-2 1.5B): 3.39 against 3.12 ms a step at 12 rows, 3.56 against 3.24 at 16; at
            # width 1,024 the resident kernel is still the faster one there (1.16 against 1.24 ms at 16 rows)
            most = min(most, 8)
        if not (ctx.decode_only and 0 < n <= most and x.is_contiguous()):
            return None
        if len(ctx.block_tables) > ops.RESIDENT_MAX_GROUPS:
            return None
        table = self._table(cache_members)
        if table is None:
            return None
        sizes = {cache_members[e.cache].page_size for e in self.schedule}
        size = next(iter(sizes))
        shift = size.bit_length() - 1 if len(sizes) == 1 and size & (size - 1) == 0 else -1
        if len(sizes) > 1 and any(s & (s - 1) for s in sizes):
            return None  # the kernel takes one way of splitting a position into page and offset
        shape = ops.ResidentShapeC(len(self.schedule), self.width, self.inner, self.n_heads, self.n_kv_heads, n)
        b = ops.ResidentBuffersC()
        b.x, b.qkv, b.mixed, b.hidden = x.data_ptr(), self.qkv.data_ptr(), self.mixed.data_ptr(), self.hidden.data_ptr()
        b.barrier = self.counters.data_ptr()
        b.error_flag = ops.error_word(self.device).data_ptr()
        b.positions, b.seq_lens = ctx.positions.data_ptr(), ctx.seq_lens.data_ptr()
        for g, (tables, slots) in enumerate(zip(ctx.block_tables, ctx.slot_mapping)):
            b.block_tables[g], b.slot_mapping[g], b.table_width[g] = tables.data_ptr(), slots.data_ptr(), tables.shape[1]
        b.stamps = self.stamps.data_ptr() if self.stamps is not None else None
        if not ops.decode_resident(self.head_dim, table, shape, b, shift, self.device):
            return None
        return x
