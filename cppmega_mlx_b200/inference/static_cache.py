"""Fixed-capacity decode cache whose write position lives on the device.

``HybridKVCache`` grows its buffers and keeps positions as Python integers, so every decode step launches kernels with new
arguments.  ``StaticDecodeCache`` holds ``[B, capacity, …]`` buffers per attention layer and one device-side position *per
sequence*; a one-token step writes row ``pos[b]`` of sequence ``b`` and attends over ``lengths = pos + 1`` keys, so the *same*
kernel arguments serve every step and the whole step can be captured once in a CUDA graph and replayed
(``inference/graph_decode.py``).  Because the positions are per sequence, the rows of one batch may be at different points of
different requests (``inference/serving_engine.py`` admits and retires requests slot by slot between replays); ``active``
marks which rows advance.  The reference has no counterpart: its caches are the growing kind
(``cppmega_mlx/inference/engine.py:52-138``) and its step is traced by ``mx.compile``.
"""
from __future__ import annotations

import torch


class StaticDecodeCache:
    static = True

    def __init__(self, num_layers: int, batch: int, capacity: int, device):
        self.num_layers, self.batch, self.capacity = num_layers, batch, capacity
        self.pos = torch.zeros(batch, dtype=torch.int64, device=device)   # per sequence: next row to write == tokens stored
        self.active = torch.ones(batch, dtype=torch.int64, device=device)  # 1 = this row advances at the end of a step
        self._rows = torch.arange(batch, device=device)
        self._len32 = torch.ones(batch, dtype=torch.int32, device=device)   # pos + 1 per sequence, kept in step with pos
        self._rope: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}      # per-step memo of rope rows at ``pos``
        self.a: list[torch.Tensor | None] = [None] * num_layers           # keys or the MLA latent
        self.b: list[torch.Tensor | None] = [None] * num_layers           # values or the indexer keys

    # -- HybridKVCache-compatible surface used by the layers ------------------------------------
    def position(self, layer_idx: int) -> torch.Tensor:
        return self.pos

    @property
    def offset(self) -> torch.Tensor:
        return self.pos

    def lengths(self) -> torch.Tensor:
        """[B] int32: keys visible to the token being decoded (its own row included). One fixed tensor, updated by ``advance``."""
        return self._len32

    def rope(self, rot_dim: int, theta: float, scaling=None) -> tuple[torch.Tensor, torch.Tensor]:
        """cos/sin rows [B, rot_dim/2] at each sequence's position, computed once per step however many layers ask. The layers
        apply them by treating the batch as the sequence axis of a single row (a one-token step has nothing else there)."""
        from ..ops.rope import rope_tables_at
        key = (rot_dim, theta, scaling)
        hit = self._rope.get(key)
        if hit is None:
            hit = rope_tables_at(self.pos, rot_dim, theta, scaling, capacity=self.capacity)
            self._rope[key] = hit
        return hit

    def _buf(self, store: list, layer_idx: int, x: torch.Tensor) -> torch.Tensor:
        buf = store[layer_idx]
        if buf is None:
            buf = torch.zeros((self.batch, self.capacity, *x.shape[2:]), dtype=x.dtype, device=x.device)
            store[layer_idx] = buf
        return buf

    def write_a(self, layer_idx: int, x: torch.Tensor) -> torch.Tensor:
        """Store ``x`` [B,1,…] at the current position; returns the whole ``[B, capacity, …]`` buffer."""
        buf = self._buf(self.a, layer_idx, x)
        buf[self._rows, self.pos] = x[:, 0].to(buf.dtype)
        return buf

    def write_b(self, layer_idx: int, x: torch.Tensor) -> torch.Tensor:
        buf = self._buf(self.b, layer_idx, x)
        buf[self._rows, self.pos] = x[:, 0].to(buf.dtype)
        return buf

    # -- how the layers address the stored rows (overridden by the paged cache) -------------------
    def attention_rows(self, buf: torch.Tensor, kv_heads: int, dim: int) -> torch.Tensor:
        """``buf`` as the ``[B | pages, rows, kv_heads, dim]`` view ``decode_attention`` reads."""
        return buf.view(buf.shape[0], buf.shape[1], kv_heads, dim)

    def table(self) -> torch.Tensor | None:
        """Page table for ``decode_attention`` (``None``: rows of sequence ``b`` are ``buf[b]``)."""
        return None

    def dense_rows(self, buf: torch.Tensor) -> torch.Tensor:
        """``[B, capacity, …]`` rows in logical order (the indexer scores all of them)."""
        return buf

    def advance(self, n: int = 1) -> None:
        self.pos += self.active * n
        self._len32 += (self.active * n).to(torch.int32)
        self._rope.clear()

    # -- hand-over from a prefill done with the growing cache -----------------------------------
    def load_slot(self, slot: int, kv, tokens_seen: int) -> None:
        """Put a single-sequence ``HybridKVCache`` (after its prefill) into row ``slot`` and set that row's position."""
        n = tokens_seen
        if n >= self.capacity:
            raise ValueError(f"prefill of {n} tokens leaves no room in a static cache of {self.capacity}")
        for i in range(self.num_layers):
            src_a = kv.a[i].fetch(n)
            if self.a[i] is None:
                self.a[i] = torch.zeros((self.batch, self.capacity, *src_a.shape[2:]), dtype=src_a.dtype, device=src_a.device)
            self.a[i][slot, :n] = src_a[0]
            if kv.has_b[i]:
                src_b = kv.b[i].fetch(n)
                if self.b[i] is None:
                    self.b[i] = torch.zeros((self.batch, self.capacity, *src_b.shape[2:]), dtype=src_b.dtype, device=src_b.device)
                self.b[i][slot, :n] = src_b[0]
        self.pos[slot] = n
        self._len32[slot] = n + 1
        self._rope.clear()

    def load_from(self, kv, tokens_seen: int | None = None) -> None:
        """Copy the contents of a ``HybridKVCache`` (after prefill) and take over its position (``tokens_seen`` when the
        model has no attention layer to read it from)."""
        n = kv.offset if tokens_seen is None else tokens_seen
        if n > self.capacity:
            raise ValueError(f"prefill of {n} tokens exceeds the static capacity {self.capacity}")
        for i in range(self.num_layers):
            if kv.lengths[i] != n:
                raise ValueError("all attention layers must be at the same position")
            src_a = kv.a[i].fetch(n)
            self.a[i] = torch.zeros((self.batch, self.capacity, *src_a.shape[2:]), dtype=src_a.dtype, device=src_a.device)
            self.a[i][:, :n] = src_a
            if kv.has_b[i]:
                src_b = kv.b[i].fetch(n)
                self.b[i] = torch.zeros((self.batch, self.capacity, *src_b.shape[2:]), dtype=src_b.dtype, device=src_b.device)
                self.b[i][:, :n] = src_b
        self.pos.fill_(n)
        self._len32.fill_(n + 1)
        self._rope.clear()

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.a + self.b if t is not None)


class PagedDecodeCache(StaticDecodeCache):
    """The same device-position cache over *pages*: per layer one pool ``[num_pages, page_size, …]`` shared by all sequences and
    a device page table ``[B, max_pages]`` mapping each sequence's logical pages to pool pages.  A step writes row
    ``(table[b, pos // page_size], pos % page_size)`` and attention reads through the table (``ops/decode_attention.py``), so
    no sequence reserves more memory than the pages it has been given.  Which pages those are is the caller's business
    (``ServingEngine`` takes them from the scheduler's ``PagedKVBlockManager``); ``set_pages`` publishes them to the device."""

    def __init__(self, num_layers: int, batch: int, *, num_pages: int, page_size: int, max_pages_per_seq: int, device):
        super().__init__(num_layers, batch, max_pages_per_seq * page_size, device)
        self.num_pages, self.page_size, self.max_pages = num_pages, page_size, max_pages_per_seq
        self._table = torch.zeros(batch, max_pages_per_seq, dtype=torch.int32, device=device)
        self._published: list[int] = [0] * batch           # how many table entries of each row are valid

    def _buf(self, store: list, layer_idx: int, x: torch.Tensor) -> torch.Tensor:
        buf = store[layer_idx]
        if buf is None:
            buf = torch.zeros((self.num_pages, self.page_size, *x.shape[2:]), dtype=x.dtype, device=x.device)
            store[layer_idx] = buf
        return buf

    def _write(self, store: list, layer_idx: int, x: torch.Tensor) -> torch.Tensor:
        buf = self._buf(store, layer_idx, x)
        page = self._table[self._rows, self.pos // self.page_size].long()
        buf[page, self.pos % self.page_size] = x[:, 0].to(buf.dtype)
        return buf

    def write_a(self, layer_idx: int, x: torch.Tensor) -> torch.Tensor:
        return self._write(self.a, layer_idx, x)

    def write_b(self, layer_idx: int, x: torch.Tensor) -> torch.Tensor:
        return self._write(self.b, layer_idx, x)

    def table(self) -> torch.Tensor:
        return self._table

    def dense_rows(self, buf: torch.Tensor) -> torch.Tensor:
        g = buf[self._table.long()]                        # [B, max_pages, page_size, …]
        return g.reshape(self.batch, self.capacity, *buf.shape[2:])

    def set_pages(self, slot: int, pages: list[int]) -> None:
        """Publish ``pages`` (pool page ids, in logical order) as row ``slot`` of the table; only new entries are written."""
        if len(pages) > self.max_pages:
            raise ValueError(f"{len(pages)} pages exceed the per-sequence limit {self.max_pages}")
        have = self._published[slot]
        if len(pages) < have or have == 0:
            have = 0
        if len(pages) > have:
            self._table[slot, have:len(pages)] = torch.tensor(pages[have:], dtype=torch.int32, device=self._table.device)
        self._published[slot] = len(pages)

    def clear_pages(self, slot: int, fill: int = 0) -> None:
        """Forget ``slot``'s pages; its table row points at page ``fill`` (a scratch page for rows that idle along)."""
        self._published[slot] = 0
        self._table[slot].fill_(fill)

    def load_slot(self, slot: int, kv, tokens_seen: int) -> None:
        """Scatter a single-sequence ``HybridKVCache`` (after its prefill) into the pages already published for ``slot``."""
        n = tokens_seen
        if n >= self.capacity or (n + self.page_size) // self.page_size > self._published[slot]:
            raise ValueError(f"slot {slot} has {self._published[slot]} pages, {n + 1} tokens need more")
        idx = torch.arange(n, device=self.pos.device)
        pages = self._table[slot, idx // self.page_size].long()
        for i in range(self.num_layers):
            src_a = kv.a[i].fetch(n)
            self._buf(self.a, i, src_a)[pages, idx % self.page_size] = src_a[0]
            if kv.has_b[i]:
                src_b = kv.b[i].fetch(n)
                self._buf(self.b, i, src_b)[pages, idx % self.page_size] = src_b[0]
        self.pos[slot] = n
        self._len32[slot] = n + 1
        self._rope.clear()

    def load_from(self, kv, tokens_seen: int | None = None) -> None:
        raise NotImplementedError("a paged cache is filled slot by slot (load_slot)")
