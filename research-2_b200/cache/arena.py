"""The memory that the cache manager's indices point into.

Per cache group one tensor [num_pages + 1, page_elems]: page 0 is the null page (real memory,
never handed out). A page holds, for each member layer of the group, K then V for `page_size`
tokens, each laid out [kv_head][offset][head_dim], so a (page, head) tile is contiguous. One
block table per request and group therefore serves all the group's layers (the reference packs
all layers of a group into one page row too: kelpie-models/kelpie_models/sdk/kv.py:1-34,
118-143). Per-request state of fixed size lives beside it: one tensor [max_requests, *shape]
per state-holding mixer, indexed by the request's state slot.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .manager import GroupSpec


@dataclass(frozen=True)
class MemberSpec:
    """What one layer's cache needs: a group (by window) and the size of a token's K or V."""

    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass
class CacheMember:
    """One layer's K and V inside its group's pages (pointers + strides for the kernels)."""

    group: int
    k: torch.Tensor  # 1-D views into the group's tensor; only their data_ptr is used
    v: torch.Tensor
    page_stride: int  # elements between consecutive pages
    page_size: int
    n_pages: int  # including the null page
    n_kv_heads: int
    head_dim: int
    window: int


def derive_groups(members: list[MemberSpec], page_size: int, num_pages: int) -> tuple[list[GroupSpec], list[int]]:
    """Members with the same lifetime (here: the same window) share a group
    (kelpie-models/kelpie_models/sdk/groups.py:268-294). -> (groups, group index per member)."""
    keys: list[int] = []
    index: list[int] = []
    for m in members:
        if m.window not in keys:
            keys.append(m.window)
        index.append(keys.index(m.window))
    if not keys:  # a model without any per-token cache still gets one (empty) group
        keys.append(0)
    return [GroupSpec(page_size, w, num_pages) for w in keys], index


class KVArena:
    def __init__(self, members: list[MemberSpec], groups: list[GroupSpec], member_group: list[int],
                 dtype: torch.dtype, device: torch.device | str):
        self.groups = groups
        self.dtype = dtype
        sizes = [0] * len(groups)
        offsets = []
        for m, g in zip(members, member_group):
            elems = m.n_kv_heads * groups[g].page_size * m.head_dim
            offsets.append((sizes[g], sizes[g] + elems))
            sizes[g] += 2 * elems
        self.tensors = [
            torch.zeros(groups[g].num_pages + 1, max(sizes[g], 1), dtype=dtype, device=device)
            for g in range(len(groups))
        ]
        self.members: list[CacheMember] = []
        for (k_off, v_off), m, g in zip(offsets, members, member_group):
            flat = self.tensors[g].view(-1)
            self.members.append(CacheMember(
                group=g, k=flat[k_off:], v=flat[v_off:], page_stride=sizes[g], page_size=groups[g].page_size,
                n_pages=groups[g].num_pages + 1, n_kv_heads=m.n_kv_heads, head_dim=m.head_dim, window=m.window,
            ))

    def fill_(self, value: float) -> None:
        """Tests fill the pool with a loud value so that a read of a slot never written shows."""
        for t in self.tensors:
            t.fill_(value)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)
