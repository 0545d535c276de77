"""Device side of the cache: page tensors of every group and state arenas.

Group ``g`` owns two tensors ``[runs_in_group, pages, kv_heads, page_size,
head_dim]`` (keys, values) in the storage dtype: the keys of one kv head in one
page are contiguous, so a kernel that serves one kv head reads whole runs of
memory.  Token ``p`` of a request lies in page ``block_table[p // page_size]``
at offset ``p % page_size`` of every run of the group (its *slot* is
``page * page_size + offset``).  A run that declares fixed-size state owns an arena
``[state_slots, *shape]``; a request's row is zeroed when the request starts.
The reference keeps one pair of tensors ``[layers, blocks * block_size,
kv_heads, head_dim]`` (tinyvllm/paged_kv.py:53-65).
"""

from __future__ import annotations

import torch

from ..parts.base import KVNeed, StateNeed
from .manager import CacheGroup


def group_runs(needs: list, cache_from: list) -> tuple[list[CacheGroup], dict[int, tuple[int, int]]]:
    """Groups of equal KV need, and for every run that attends over a cache the
    (group, index inside the group) of the cache it reads."""
    groups: list[CacheGroup] = []
    members: list[list[int]] = []
    where: dict[int, tuple[int, int]] = {}
    for run, need in enumerate(needs):
        if not isinstance(need, KVNeed) or cache_from[run] is not None:
            continue
        for g, group in enumerate(groups):
            if (group.num_kv_heads, group.head_dim, group.window) == (
                    need.num_kv_heads, need.head_dim, need.window):
                members[g].append(run)
                where[run] = (g, len(members[g]) - 1)
                break
        else:
            groups.append(CacheGroup((), need.num_kv_heads, need.head_dim, need.window))
            members.append([run])
            where[run] = (len(groups) - 1, 0)
    groups = [CacheGroup(tuple(m), g.num_kv_heads, g.head_dim, g.window)
              for g, m in zip(groups, members)]
    for run, source in enumerate(cache_from):
        if source is None:
            continue
        need, theirs = needs[run], needs[source]
        if not isinstance(need, KVNeed) or not isinstance(theirs, KVNeed) or (
                need.num_kv_heads, need.head_dim) != (theirs.num_kv_heads, theirs.head_dim):
            raise ValueError(f"run {run} cannot read the cache of run {source}: shapes differ")
        if need.window != theirs.window:
            raise ValueError(f"run {run} and run {source} must agree on the window")
        where[run] = where[source]
    return groups, where


def bytes_per_page(group: CacheGroup, page_size: int, itemsize: int) -> int:
    return 2 * len(group.runs) * page_size * group.num_kv_heads * group.head_dim * itemsize


class CacheStorage:
    def __init__(self, groups, where, needs, *, page_size: int, pages_per_group,
                 num_state_slots: int, dtype: torch.dtype, device) -> None:
        self.groups = tuple(groups)
        self.where = dict(where)
        self.page_size = page_size
        self.dtype = dtype
        self.device = device
        if isinstance(pages_per_group, int):
            pages_per_group = [pages_per_group] * len(self.groups)
        self.pages_per_group = tuple(pages_per_group)
        self.keys, self.values = [], []
        for group, pages in zip(self.groups, self.pages_per_group):
            shape = (len(group.runs), pages, group.num_kv_heads, page_size, group.head_dim)
            self.keys.append(torch.zeros(shape, dtype=dtype, device=device))
            self.values.append(torch.zeros(shape, dtype=dtype, device=device))
        self.state: dict[int, torch.Tensor] = {}
        for run, need in enumerate(needs):
            if isinstance(need, StateNeed):
                self.state[run] = torch.zeros(
                    (num_state_slots,) + tuple(need.shape), dtype=need.dtype, device=device)

    def group_of(self, run: int) -> int:
        return self.where[run][0]

    def kv_of(self, run: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Keys and values ``[pages, kv_heads, page_size, head_dim]`` of one run."""
        group, index = self.where[run]
        return self.keys[group][index], self.values[group][index]

    def state_of(self, run: int) -> torch.Tensor:
        return self.state[run]

    def clear_state(self, slots) -> None:
        """Zero the state rows of requests that start in this step."""
        if not self.state or not slots:
            return
        index = torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
        for arena in self.state.values():
            arena.index_fill_(0, index, 0)
