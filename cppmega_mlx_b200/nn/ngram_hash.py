"""N-gram hash embedding: each of ``len(orders)·num_heads`` tables hashes the last ``order`` token ids
with an XOR of odd multipliers plus a bias, modulo a prime table size, into one unified embedding
table; the concatenated lookups are projected (zero-init) to the hidden size.
Parity: ``cppmega_mlx/nn/ngram_hash.py:8-34`` (prime sizes), ``:139-157`` (hash), ``:37-167`` (module)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .basic import Embedding, Linear

_PRIMES = (499_801, 499_819, 499_853, 499_879, 499_883, 499_897, 499_903, 499_927, 499_943, 499_957, 499_969,
           499_973, 499_979, 500_009, 500_029, 500_041)


def pick_primes(count: int, target_size: int) -> tuple[int, ...]:
    cand = [p for p in _PRIMES if abs(p - target_size) / target_size < 0.5]
    if len(cand) >= count:
        return tuple(cand[:count])
    return tuple(target_size + i for i in range(count))


class NgramHashEmbedding(nn.Module):
    def __init__(self, *, hidden_size: int, orders: tuple[int, ...] = (2, 3), num_heads: int = 8,
                 table_size: int = 500_000, embed_dim: int = 16, dropout: float = 0.0, seed: int | None = None):
        super().__init__()
        if hidden_size <= 0 or num_heads <= 0 or table_size <= 0 or embed_dim <= 0:
            raise ValueError("hidden_size, num_heads, table_size and embed_dim must be positive")
        if not orders or any(o <= 0 for o in orders):
            raise ValueError("orders must be a non-empty tuple of positive ints")
        if not 0.0 <= dropout < 1.0:
            raise ValueError("dropout must be in [0, 1)")
        self.hidden_size, self.orders, self.num_heads = hidden_size, tuple(int(o) for o in orders), int(num_heads)
        self.num_tables = len(self.orders) * self.num_heads
        self.embed_dim, self.max_order = int(embed_dim), max(self.orders)
        self.table_sizes = pick_primes(self.num_tables, table_size)
        offs, total = [], 0
        for sz in self.table_sizes:
            offs.append(total)
            total += sz
        gen = torch.Generator().manual_seed(seed if seed is not None else torch.seed() % (2 ** 31))
        self.register_buffer("table_offsets", torch.tensor(offs, dtype=torch.int64))
        self.register_buffer("table_sizes_t", torch.tensor(self.table_sizes, dtype=torch.int64))
        self.register_buffer("hash_mults", torch.randint(1, 2 ** 31, (self.num_tables, self.max_order), generator=gen) | 1)
        self.register_buffer("hash_bias", torch.randint(0, 2 ** 31, (self.num_tables,), generator=gen))
        order_list = [o for o in self.orders for _ in range(self.num_heads)]
        self.register_buffer("order_for_table", torch.tensor(order_list, dtype=torch.int64))
        mask = torch.zeros(self.max_order, self.num_tables, dtype=torch.int64)
        for t, o in enumerate(order_list):
            mask[:o, t] = 1
        self.register_buffer("order_mask", mask)
        self.unified_table = Embedding(total, self.embed_dim)
        self.out_proj = Linear(self.num_tables * self.embed_dim, hidden_size, zero_init=True)
        self.dropout = nn.Dropout(dropout)

    def _hash_all(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Unified-table row ids, [B, tables, S]."""
        if token_ids.dim() != 2:
            raise ValueError("token_ids must be shaped (B,S)")
        ids = token_ids.long()
        b, s = ids.shape
        shifted = [ids]
        for p in range(1, self.max_order):
            shifted.append(torch.zeros_like(ids) if p >= s else torch.cat([ids.new_zeros(b, p), ids[:, :-p]], dim=1))
        sh = torch.stack(shifted, 0)  # [P,B,S]
        prod = self.hash_mults.t()[:, :, None, None] * sh[:, None] * self.order_mask[:, :, None, None]  # [P,T,B,S]
        hashed = prod[0]
        for p in range(1, self.max_order):
            hashed = hashed ^ prod[p]
        hashed = hashed ^ self.hash_bias[:, None, None]
        hashed = torch.remainder(hashed, self.table_sizes_t[:, None, None]) + self.table_offsets[:, None, None]
        return hashed.permute(1, 0, 2)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        idx = self._hash_all(token_ids)
        b, t, s = idx.shape
        emb = self.unified_table(idx).permute(0, 2, 1, 3).reshape(b, s, t * self.embed_dim)
        return self.dropout(self.out_proj(emb))


CppMegaNgramHashEmbedding = NgramHashEmbedding
