"""The cache manager: keys and values in pages with a block table per request, and slots for fixed-size state.

Layers whose mixers keep the same thing form a *group* (all keys of every position; the keys of a window; nothing).
Each group has its own pool of pages and its own block tables, so a group with a window gives pages back as soon as
the window has passed them while a full group keeps them until the request ends.  What a mixer keeps per position is
its own business: a need lists the tensors (heads, width) one position holds -- keys and values of equal shape for
attention, one latent vector for a mixer that keeps such, keys and values of different widths -- and the group gets one
pool per listed tensor, (layers, pages, heads, page_size, width), so one head of one page is contiguous.  A page of a
group holds `page_size` positions of every layer of the group.  Position p of a request lives in page
table[row, p // page_size], slot p % page_size; an entry is -1 before it is given and again after a window has passed
it.

Per-request state of fixed size (a recurrent mixer's state) lives in `state` tensors indexed by the request's state
slot; a slot is zeroed when a request takes it.  The Llama architecture has no such state: its slot count is still
managed, so a mixer that declares a state finds its place.

The reference keeps one whole context per slot (src/mashbox/runtime/kvcache.py:5-9, 64-74) and moves fixed-size state by
slot (src/mashbox/runtime/engine.py:329-351); pages, per-group tables and give-back are this engine's own.
Everything here is host bookkeeping plus the device tensors; no kernel is launched from this file.
"""
from dataclasses import dataclass
from typing import Optional

import numpy as np

from ..errors import CacheError
from .pages import Pool


@dataclass(frozen=True)
class CacheNeed:
    """What one mixer keeps per position: kind "full" (every position) or "window" (the last `window` positions), and
    `tensors`, one (heads, width) per tensor a position holds, each stored in a pool of its own."""
    kind: str
    tensors: tuple
    window: Optional[int] = None

    @classmethod
    def keys_and_values(cls, kv_heads, head_dim, window=None):
        """what attention keeps: a key and a value of (kv_heads, head_dim) per position"""
        shape = (int(kv_heads), int(head_dim))
        return cls("window" if window else "full", (shape, shape), int(window) if window else None)


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state one mixer keeps per request: a tensor of `shape` and dtype name per state slot."""
    shape: tuple
    dtype: str = "float32"


class Group:
    def __init__(self, need, cache_ids, num_pages, max_requests, max_blocks):
        self.need, self.cache_ids = need, list(cache_ids)
        self.index_of = {c: i for i, c in enumerate(self.cache_ids)}
        self.pool = Pool(num_pages, "page")
        self.table = np.full((max_requests, max_blocks), -1, np.int32)
        self.pools = None                   # device tensors, one per tensor of the need: (layers, pages, heads, page_size, width)
        self.device_table = None            # device copy of `table`
        self.pending = []                   # (flat index, value) table changes not yet on the device


class Request:
    def __init__(self, row, state_slot, n_groups):
        self.row, self.state_slot = row, state_slot
        self.length = 0                     # positions committed
        self.reserved = 0                   # positions covered by pages (>= length)
        self.first_block = [0] * n_groups   # blocks below it were given back (window groups)


class CacheManager:
    def __init__(self, needs, states, page_size, num_pages, max_requests, max_context, dtype=None, device=None):
        """needs: {cache id: CacheNeed or None}; states: {cache id: StateNeed}; dtype/device None: no tensors are
        made (host bookkeeping only, as the CPU tests use it)."""
        self.page_size, self.num_pages, self.max_requests = int(page_size), int(num_pages), int(max_requests)
        self.max_context = int(max_context) if max_context else self.num_pages * self.page_size
        self.max_blocks = max(1, -(-self.max_context // self.page_size))
        self.device, self.dtype = device, dtype
        by_need = {}
        for cid, need in needs.items():
            if need is None:
                continue
            if need.kind not in ("full", "window") or (need.kind == "window" and not need.window) or not need.tensors \
                    or any(len(t) != 2 or min(t) < 1 for t in need.tensors):
                raise CacheError(f"cache need {need} is not understood")
            by_need.setdefault(need, []).append(cid)
        self.groups = [Group(need, cids, self.num_pages, self.max_requests, self.max_blocks)
                       for need, cids in by_need.items()]
        self.group_of = {cid: gi for gi, g in enumerate(self.groups) for cid in g.cache_ids}
        self.rows = Pool(self.max_requests, "request row")
        self.state_slots = Pool(self.max_requests, "state slot")
        self.state_needs = dict(states)
        self.state = {}
        self.requests = {}
        # Beside the pages, rows and state slots that requests are given there is one more of each on the device,
        # outside the bookkeeping: a sequence of one token at position 0 that reads and writes only the spare page.
        # The step function fills decode batches up with such sequences (their results are dropped), so that batches
        # of nearby sizes share one captured graph.
        self.pool_pages = self.num_pages + 1
        self.spare_row = self.spare_state_slot = self.max_requests
        if device is not None:
            import torch
            for g in self.groups:
                g.pools = [torch.zeros((len(g.cache_ids), self.pool_pages, heads, self.page_size, width), dtype=dtype,
                                       device=device) for heads, width in g.need.tensors]
                g.device_table = torch.full((self.max_requests + 1, self.max_blocks), -1, dtype=torch.int32, device=device)
                g.device_table[self.spare_row, 0] = self.num_pages
            for cid, s in self.state_needs.items():
                self.state[cid] = torch.zeros((self.max_requests + 1,) + tuple(s.shape), dtype=getattr(torch, s.dtype),
                                              device=device)

    # -------------------------------------------------------------------------------------------- requests
    def admit(self, rid):
        if rid in self.requests:
            raise CacheError(f"request {rid!r} is already live")
        row = self.rows.take()
        try:
            slot = self.state_slots.take()
        except CacheError:
            self.rows.give(row)
            raise
        self.requests[rid] = Request(row, slot, len(self.groups))
        for t in self.state.values():
            t[slot].zero_()
        return self.requests[rid]

    def can_admit(self):
        return self.rows.n_free > 0 and self.state_slots.n_free > 0

    def get(self, rid):
        try:
            return self.requests[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def length(self, rid):
        return self.get(rid).length

    def _first_needed(self, g, length):
        """first block a query at position >= length can still read in group g"""
        if g.need.kind != "window":
            return 0
        return max(0, length - g.need.window + 1) // self.page_size

    def pages_needed(self, rid, n_new):
        """pages each group must still give so that n_new more positions fit -> list per group"""
        r = self.get(rid)
        end = r.length + n_new
        have = -(-r.reserved // self.page_size)
        want = -(-end // self.page_size)
        return [max(0, want - max(have, r.first_block[gi])) if want > have else 0 for gi in range(len(self.groups))]

    def can_extend(self, rid, n_new):
        r = self.get(rid)
        if r.length + n_new > self.max_context:
            return False
        return all(n <= g.pool.n_free for n, g in zip(self.pages_needed(rid, n_new), self.groups))

    def extend(self, rid, n_new):
        """Gives the request pages for positions length .. length + n_new - 1 in every group, all or nothing."""
        r = self.get(rid)
        end = r.length + n_new
        if end > self.max_context:
            raise CacheError(f"request {rid!r} would hold {end} tokens, over the context of {self.max_context}")
        if not self.can_extend(rid, n_new):
            raise CacheError("no free page")
        have = -(-r.reserved // self.page_size)
        want = -(-end // self.page_size)
        for gi, g in enumerate(self.groups):
            for b in range(max(have, r.first_block[gi]), want):
                pg = g.pool.take()
                g.table[r.row, b] = pg
                g.pending.append((r.row * self.max_blocks + b, pg))
        r.reserved = max(r.reserved, end)

    def commit(self, rid, n_new):
        """n_new positions were written: the request grows, and window groups give back the pages passed for good."""
        r = self.get(rid)
        if r.length + n_new > r.reserved:
            raise CacheError(f"request {rid!r} commits positions it holds no pages for")
        r.length += n_new
        for gi, g in enumerate(self.groups):
            first = min(self._first_needed(g, r.length), -(-r.reserved // self.page_size))
            for b in range(r.first_block[gi], first):
                pg = int(g.table[r.row, b])
                if pg >= 0:
                    g.pool.give(pg)
                    g.table[r.row, b] = -1
                    g.pending.append((r.row * self.max_blocks + b, -1))
            r.first_block[gi] = max(r.first_block[gi], first)

    def release(self, rid):
        """The request ends (finished, cancelled or preempted): every page, its row and its state slot come back."""
        r = self.get(rid)
        for g in self.groups:
            row = g.table[r.row]
            for b in np.nonzero(row >= 0)[0]:
                g.pool.give(int(row[b]))
                g.pending.append((r.row * self.max_blocks + int(b), -1))
            row[:] = -1
        self.rows.give(r.row)
        self.state_slots.give(r.state_slot)
        del self.requests[rid]

    # -------------------------------------------------------------------------------------------- device side
    def flush_tables(self):
        """Sends the table entries changed since the last call to the device copies (one small scatter per group)."""
        if self.device is None:
            for g in self.groups:
                g.pending.clear()
            return
        import torch
        for g in self.groups:
            if not g.pending:
                continue
            last = dict(g.pending)                      # a later change of the same entry wins
            idx = torch.tensor(list(last.keys()), dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
            val = torch.tensor(list(last.values()), dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            g.device_table.view(-1).index_copy_(0, idx, val)
            g.pending.clear()

    def layer_cache(self, cache_id):
        """-> (group, pool of each tensor of the need ...) of one cache id: a pool is (pages, heads, page_size, width);
        attention gets (group, k pool, v pool)"""
        g = self.groups[self.group_of[cache_id]]
        i = g.index_of[cache_id]
        return (g,) + tuple(pool[i] for pool in g.pools)

    def pages_to_hold(self, tokens, portion):
        """-> per group, the most pages a request of `tokens` tokens holds at any time when it is fed in portions of at
        most `portion` tokens: every page of a full group; of a window group only those the window and one portion
        reach (what lies behind the window is given back at every commit)"""
        whole = -(-int(tokens) // self.page_size)
        out = []
        for g in self.groups:
            if g.need.kind == "window":
                out.append(min(whole, -(-(g.need.window - 1 + int(portion)) // self.page_size) + 1))
            else:
                out.append(whole)
        return out

    def pages_held(self, rid):
        """-> per group, the pages the request holds now"""
        r = self.get(rid)
        return [int((g.table[r.row] >= 0).sum()) for g in self.groups]

    # -------------------------------------------------------------------------------------------- checks
    def free_pages(self):
        return [g.pool.n_free for g in self.groups]

    def check(self):
        """Invariants: no page lost, held twice or free while in a table; rows and state slots likewise."""
        for g in self.groups:
            g.pool.check()
            in_tables = g.table[g.table >= 0]
            if len(np.unique(in_tables)) != len(in_tables):
                raise CacheError("a page is in two places of the block tables")
            held = {i for i in range(g.pool.n) if g.pool.held[i]}
            if held != set(int(x) for x in in_tables):
                raise CacheError("the pages held and the pages in the block tables differ")
        self.rows.check()
        self.state_slots.check()
        live_rows = sorted(r.row for r in self.requests.values())
        if live_rows != [i for i in range(self.rows.n) if self.rows.held[i]]:
            raise CacheError("request rows held and live requests differ")
