"""Executable specification of the paged KV bookkeeping (block pool, tables, slot mappings,
refcounts, copy-on-write, prefix sharing), written independently of the C++ manager in plain
Python.  Test infrastructure: the C++ manager must reproduce its state bit for bit."""
from collections import deque

MASK = (1 << 64) - 1


def splitmix64(state):
    state = (state + 0x9E3779B97F4A7C15) & MASK
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return state, z ^ (z >> 31)


class SpecPool:
    def __init__(self, num_blocks, block_size=16, seed=0, shuffle=True, min_prefix_length=4):
        order = list(range(num_blocks))
        if shuffle:
            st = seed
            for i in range(num_blocks - 1, 0, -1):
                st, r = splitmix64(st)
                j = r % (i + 1)
                order[i], order[j] = order[j], order[i]
        self.free = deque(order)
        self.ref = [0] * num_blocks
        self.bs = block_size
        self.seqs = {}
        self.next_id = 0
        self.cow_events = 0
        self.copies = []
        self.spans = {}      # token tuple -> block list held by the prefix store
        self.min_prefix = min_prefix_length

    def _change(self, b, d):
        self.ref[b] += d
        assert self.ref[b] >= 0
        if self.ref[b] == 0:
            self.free.append(b)

    def _take(self):
        b = self.free.popleft()
        self._change(b, +1)
        return b

    def add_sequence(self):
        i = self.next_id
        self.next_id += 1
        self.seqs[i] = [[], 0]
        return i

    def append(self, seq, n):
        blocks, length = self.seqs[seq]
        partial = length % self.bs != 0
        cow = n > 0 and partial and self.ref[blocks[-1]] > 1
        fresh = -(-(length + n) // self.bs) - len(blocks)
        if fresh + (1 if cow else 0) > len(self.free):
            return None
        if cow:
            old = blocks[-1]
            mine = self._take()
            self.copies.append((old, mine))
            self._change(old, -1)
            blocks[-1] = mine
            self.cow_events += 1
        for _ in range(fresh):
            blocks.append(self._take())
        slots = [blocks[(length + i) // self.bs] * self.bs + (length + i) % self.bs for i in range(n)]
        self.seqs[seq][1] = length + n
        return slots

    def free_sequence(self, seq):
        for b in self.seqs.pop(seq)[0]:
            self._change(b, -1)

    def match_prefix(self, seq, tokens):
        """Longest stored span that is a prefix of tokens (the tree's last terminal on the path)."""
        best = None
        for key in self.spans:
            if len(key) <= len(tokens) and tuple(tokens[:len(key)]) == key:
                if best is None or len(key) > len(best):
                    best = key
        if best is None or len(best) < self.min_prefix or len(best) == 0:
            return 0
        need = -(-len(best) // self.bs)
        blocks = self.spans[best][:need]
        for b in blocks:
            self._change(b, +1)
        self.seqs[seq] = [list(blocks), len(best)]
        return len(best)

    def insert_prefix(self, seq, tokens):
        n = len(tokens)
        blocks = self.seqs[seq][0][:-(-n // self.bs)]
        for b in blocks:
            self._change(b, +1)
        key = tuple(tokens)
        if key in self.spans:
            for b in self.spans[key]:
                self._change(b, -1)
        self.spans[key] = list(blocks)

    def table_row(self, seq, width):
        b = self.seqs[seq][0]
        return b + [-1] * (width - len(b))
