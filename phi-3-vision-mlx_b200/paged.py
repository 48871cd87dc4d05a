"""Page pool shared by all live sequences: the cache manager of the continuous-batching engine (engine.py).

The Phi-3 path sizes one rectangular slab per batch (model.KVCacheB200: every row owns pages_per_seq pages for the whole call).
A serving engine cannot: requests arrive and leave at different times and lengths. Here a fixed number of 64-token pages is
allocated once, a sequence takes a slot (one row of the block table) when it is admitted and pages from a free list as its
tokens arrive, and gives both back when it ends, so pages and slots are used again by later requests.

Per layer there is one K pool [page][kv heads][64][key size] and one V pool [page][kv heads][64][value size]; the sizes may
differ between layers (`layout` = [(kv_heads, key size, value size), ...]; a layer without a cache of its own gives zeros). Pools are zero-initialised and only ever hold finite
numbers, so a masked slot can never poison a weighted sum. The block table lives on the device; the host keeps a mirror and
uploads the rows that changed before a step.

Recurrent state. A model whose layers carry a state from token to token (a token shift, a matrix memory, the last token) names the fp32 numbers
each of its state buffers needs per sequence (`state_layout` = [numbers per slot, ...]); the pool allocates them once as
[slots][numbers] and a sequence's state lives in the row of its slot. Nothing is cleared when a slot changes hands: the kernels
start a sequence whose first token has position 0 from the zero state whatever the row holds.
"""
import torch

PAGE = 64


class PoolExhausted(RuntimeError):
    pass


class PagePool:
    def __init__(self, layout, max_tokens, n_slots, dtype, device, state_layout=()):
        self.layout, self.dtype, self.dev = list(layout), dtype, torch.device(device)
        self.state_layout = [int(n) for n in state_layout]
        self.n_pages = max(1, -(-int(max_tokens) // PAGE))
        self.n_slots = int(n_slots)
        self.k = [torch.zeros((self.n_pages, g, PAGE, d), dtype=dtype, device=self.dev) for g, d, _ in self.layout]
        self.v = [torch.zeros((self.n_pages, g, PAGE, dv), dtype=dtype, device=self.dev) for g, _, dv in self.layout]
        self.bt_host = torch.zeros((self.n_slots, self.n_pages), dtype=torch.int32)
        self.block_table = torch.zeros((self.n_slots, self.n_pages), dtype=torch.int32, device=self.dev)
        self.state = [torch.zeros((self.n_slots, n), dtype=torch.float32, device=self.dev) for n in self.state_layout]
        self.free_pages = list(range(self.n_pages - 1, -1, -1))      # pop() hands out page 0 first
        self.free_slots = list(range(self.n_slots - 1, -1, -1))
        self.pages = {}                                              # slot -> page ids in sequence order
        self.length = {}                                             # slot -> tokens held
        self._dirty = set()

    # ---- slots
    def admit(self):
        if not self.free_slots:
            raise PoolExhausted(f'all {self.n_slots} sequence slots are in use')
        s = self.free_slots.pop()
        self.pages[s], self.length[s] = [], 0
        return s

    def release(self, slot):
        """give the sequence's pages and its slot back; nothing is cleared (the next owner overwrites what it reads)"""
        self.free_pages.extend(reversed(self.pages.pop(slot)))
        del self.length[slot]
        self.free_slots.append(slot)

    # ---- pages
    def pages_needed(self, slot, n_new):
        return max(0, -(-(self.length[slot] + n_new) // PAGE) - len(self.pages[slot]))

    def can_extend(self, slot, n_new):
        return self.pages_needed(slot, n_new) <= len(self.free_pages)

    def extend(self, slot, n_new):
        """make room for n_new more tokens of `slot`; returns the position of the first of them"""
        need = self.pages_needed(slot, n_new)
        if need > len(self.free_pages):
            raise PoolExhausted(f'page pool exhausted: {need} pages wanted, {len(self.free_pages)} of {self.n_pages} free')
        pg = self.pages[slot]
        for _ in range(need):
            p = self.free_pages.pop()
            self.bt_host[slot, len(pg)] = p
            pg.append(p)
        if need:
            self._dirty.add(slot)
        start = self.length[slot]
        self.length[slot] = start + n_new
        return start

    def sync(self):
        """upload the block-table rows that changed since the last step"""
        for s in sorted(self._dirty):
            n = len(self.pages[s]) if s in self.pages else 0
            if n:
                self.block_table[s, :n].copy_(self.bt_host[s, :n], non_blocking=True)
        self._dirty.clear()

    @property
    def tokens_free(self):
        return len(self.free_pages) * PAGE
