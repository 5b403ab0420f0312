"""Prefix reuse across requests: full KV pages keyed by the tokens that produced them (the engine-side counterpart of
vLLM's automatic prefix caching, which the reference leaves on outside IsoExec runs, and of its boundary-state store for
recurrent layers, ISO/ops/gdn/gdn_cpr_state.py:63-215).

A page holds the keys and values of 128 consecutive positions. The K/V rows of a position depend only on the tokens up to
it (and on the weights), not on the batch or the chunk they were computed in, so a page filled by one request can be
read by any later request whose first ``128 * (k + 1)`` tokens are the same: the later request starts its prefill behind
the matched pages and produces the same bits as if it had computed them (the same argument that lets the samples of one
prompt share its pages). The cache is keyed by a digest CHAIN, ``key_k = H(key_{k-1}, tokens of page k)``, so a key
stands for the whole prefix; an entry also keeps its page's tokens and its parent key, and a match compares both, so
that a digest collision can never hand out foreign keys and values.

The cache holds one reference on every page it lists (``PageAllocator.share``), so a cached page survives the request
that filled it. A page whose only holder is the cache is evictable; eviction is least-recently-used, leaves before roots
(a match touches its chain from the leaf to the root). Everything is dropped at a weight sync and at sleep
(``LLMEngine.reset_prefix_cache``): keys and values computed under old weights must not be read under new ones.

Models with recurrent (GatedDeltaNet) layers also need the recurrent state AT the boundary where the reuse ends; those
states live in a byte-budgeted store keyed by the same chain keys (``BoundaryStates``), and a match on such a model ends
at the deepest page boundary for which a state is stored.
"""

from __future__ import annotations

import hashlib
from array import array
from collections import OrderedDict

from ..ops.functional import PAGE

_ROOT = b"\x00" * 16


def chain_keys(tokens: list[int], n_pages: int) -> list[bytes]:
    """``key_0 .. key_{n_pages-1}`` of the first ``n_pages`` full pages of ``tokens``."""
    out, prev = [], _ROOT
    for k in range(n_pages):
        prev = hashlib.blake2b(prev + array("q", tokens[k * PAGE:(k + 1) * PAGE]).tobytes(), digest_size=16).digest()
        out.append(prev)
    return out


class PrefixCache:
    def __init__(self, allocator, boundary: "BoundaryStates | None" = None):
        self.alloc = allocator
        self.boundary = boundary                  # set for models with recurrent layers
        self.table: OrderedDict[bytes, tuple[int, bytes, tuple]] = OrderedDict()     # key -> (page, parent key, page tokens)
        self.hits = self.misses = self.hit_tokens = self.stored = self.evicted = 0

    def __len__(self) -> int:
        return len(self.table)

    def match(self, tokens: list[int]) -> tuple[list[int], bytes | None]:
        """The longest cached prefix of ``tokens`` that leaves at least one token to compute (the last token's logits are
        always needed): (its pages, the chain key of its end or None when nothing matched). The pages are SHARED with the
        caller (one reference each is taken here)."""
        limit = (len(tokens) - 1) // PAGE
        keys = chain_keys(tokens, limit)
        n, prev = 0, _ROOT
        for k, key in enumerate(keys):
            e = self.table.get(key)
            if e is None or e[1] != prev or e[2] != tuple(tokens[k * PAGE:(k + 1) * PAGE]):
                break
            n, prev = k + 1, key
        if self.boundary is not None:             # recurrent layers: the reuse must end where a boundary state is stored
            while n > 0 and keys[n - 1] not in self.boundary:
                n -= 1
        if n == 0:
            self.misses += 1
            return [], None
        for key in reversed(keys[:n]):            # leaf first, so that the root ends up most recently used
            self.table.move_to_end(key)
        pages = [self.table[key][0] for key in keys[:n]]
        self.alloc.share(pages)
        self.hits += 1
        self.hit_tokens += n * PAGE
        return pages, keys[n - 1]

    def insert(self, tokens: list[int], pages: list[int], computed: int) -> int:
        """List the full pages among the first ``computed`` positions of a sequence (``pages`` are the sequence's pages in
        order). A prefix that is cached already under another page keeps the older page. Returns the new entries."""
        n = min(computed // PAGE, len(pages))
        new, prev = 0, _ROOT
        for k, key in enumerate(chain_keys(tokens, n)):
            e = self.table.get(key)
            if e is None:
                self.alloc.share([pages[k]])
                self.table[key] = (pages[k], prev, tuple(tokens[k * PAGE:(k + 1) * PAGE]))
                new += 1
            elif e[1] != prev or e[2] != tuple(tokens[k * PAGE:(k + 1) * PAGE]):
                break                             # a digest collision: this chain is not cached beyond here
            prev = key
        self.stored += new
        return new

    def evictable(self) -> int:
        return sum(1 for page, _p, _t in self.table.values() if self.alloc.refs[page] == 1)

    def evict(self, n: int) -> int:
        """Give back up to ``n`` pages that only the cache holds, least recently used first. Returns how many."""
        done = 0
        for key in list(self.table):
            if done >= n:
                break
            page = self.table[key][0]
            if self.alloc.refs[page] == 1:
                del self.table[key]
                self.alloc.release([page])
                if self.boundary is not None:
                    self.boundary.drop(key)
                done += 1
        self.evicted += done
        return done

    def clear(self) -> None:
        for page, _p, _t in self.table.values():
            self.alloc.release([page])
        self.table.clear()
        if self.boundary is not None:
            self.boundary.clear()

    def stats(self) -> dict:
        out = {"entries": len(self.table), "hits": self.hits, "misses": self.misses, "hit_tokens": self.hit_tokens,
               "stored": self.stored, "evicted": self.evicted}
        if self.boundary is not None:
            out["boundary"] = self.boundary.stats()
        return out


class BoundaryStates:
    """Recurrent state at page boundaries, keyed by the chain key of the prefix that ends there: per GatedDeltaNet layer
    the conv tail and the fp32 state, cloned from a sequence's row at a moment when its open chunk is empty (a page
    boundary is a chunk boundary). Least-recently-used within a byte budget; one state larger than the budget is refused
    once with a message instead of thrashing."""

    def __init__(self, budget_bytes: int):
        self.budget = int(budget_bytes)
        self.d: OrderedDict[bytes, tuple[dict, int]] = OrderedDict()
        self.bytes = 0
        self.stores = self.evictions = self.oversize = 0

    def __contains__(self, key: bytes) -> bool:
        return key in self.d

    def put(self, key: bytes, state: dict) -> bool:
        """``state``: {layer: (conv tail, fp32 state)}, already cloned. True iff a new entry was stored."""
        if key in self.d:
            self.d.move_to_end(key)
            return False
        n = sum(c.numel() * c.element_size() + s.numel() * s.element_size() for c, s in state.values())
        if n > self.budget:
            if not self.oversize:
                print(f"[prefix cache] one boundary state is {n / 2**20:.1f} MiB, the whole budget {self.budget / 2**20:.1f} MiB: "
                      f"no state can be stored and no prefix of this model will be reused; raise prefix_cache_state_mb", flush=True)
            self.oversize += 1
            return False
        while self.bytes + n > self.budget and self.d:
            _k, (_st, m) = self.d.popitem(last=False)
            self.bytes -= m
            self.evictions += 1
        self.d[key] = (state, n)
        self.bytes += n
        self.stores += 1
        return True

    def get(self, key: bytes) -> dict:
        self.d.move_to_end(key)
        return self.d[key][0]

    def drop(self, key: bytes) -> None:
        e = self.d.pop(key, None)
        if e is not None:
            self.bytes -= e[1]

    def clear(self) -> None:
        self.d.clear()
        self.bytes = 0

    def stats(self) -> dict:
        return {"entries": len(self.d), "MiB": round(self.bytes / 2**20, 1), "stores": self.stores, "evictions": self.evictions,
                "oversize_refusals": self.oversize}
