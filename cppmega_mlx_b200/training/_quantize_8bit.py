"""Block-wise 8-bit codecs for optimizer state: uint8 codes plus one fp32 absmax per 256 values.

``symmetric_int8_v1``: ``q = clamp(round(v / absmax · 127), ±127) + 128``
(``cppmega_mlx/training/_quantize_8bit.py:99-108``).
``dynamic_int8_v1``: nearest entry of the 256-value signed "dynamic" code book of bitsandbytes
(``create_dynamic_map(signed=True, max_exponent_bits=7, total_bits=8)``: seven decades, decade ``i``
holding ``2^i`` midpoints of a linear split of [0.1, 1], plus 0 and 1) found by an 8-step binary search
and a nearest-neighbour fix-up (``:267-332`` table, ``:362-380`` search).  The code book is generated
here from that rule rather than stored.
"""
from __future__ import annotations

import functools

import torch

BLOCK_SIZE = 256
DEFAULT_BLOCK_SIZE = BLOCK_SIZE
QUANT_RANGE = 127
QUANT_BIAS = 128
QUANT_SCHEMES = ("symmetric_int8_v1", "dynamic_int8_v1")


@functools.lru_cache(maxsize=None)
def _dynamic_values() -> tuple[float, ...]:
    bits, exp_bits = 7, 7
    vals: list[float] = []
    for i in range(exp_bits):
        n = 2 ** (i + bits - exp_bits) + 1
        edges = torch.linspace(0.1, 1.0, n, dtype=torch.float32)
        mids = ((edges[:-1] + edges[1:]) / 2.0)
        scale = 10.0 ** (-(exp_bits - 1) + i)
        m = (mids * scale).tolist()
        vals += m + [-x for x in m]
    vals += [0.0, 1.0]
    assert len(vals) == 256
    return tuple(sorted(vals))


_lut_cache: dict[str, torch.Tensor] = {}


def create_dynamic_map(device=None) -> torch.Tensor:
    key = str(device)
    t = _lut_cache.get(key)
    if t is None:
        t = _lut_cache[key] = torch.tensor(_dynamic_values(), dtype=torch.float32, device=device)
    return t


def _blocks(flat: torch.Tensor, block: int):
    n = flat.numel()
    nb = (n + block - 1) // block
    pad = nb * block - n
    x = torch.nn.functional.pad(flat, (0, pad)) if pad else flat
    return x.view(nb, block), n


def _check_scheme(scheme: str) -> None:
    if scheme not in QUANT_SCHEMES:
        raise ValueError(f"unknown quantization scheme {scheme!r}; expected one of {QUANT_SCHEMES}")


def quantize_symmetric_values(values: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    denom = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = torch.round(values / denom * QUANT_RANGE).clamp_(-QUANT_RANGE, QUANT_RANGE)
    return (q.to(torch.int32) + QUANT_BIAS).to(torch.uint8)


def dequantize_symmetric_values(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return (q.to(torch.int32) - QUANT_BIAS).float() * (1.0 / QUANT_RANGE) * scale


def quantize_dynamic_values(values: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    lut = create_dynamic_map(values.device)
    denom = torch.where(scale > 0, scale, torch.ones_like(scale))
    x = (values / denom).clamp_(-1.0, 1.0)
    lo = torch.zeros_like(x, dtype=torch.int64)
    hi = torch.full_like(lo, 255)
    for _ in range(8):
        mid = (lo + hi) // 2
        right = lut[mid] < x
        lo = torch.where(right, mid + 1, lo)
        hi = torch.where(right, hi, mid)
    prev = (lo - 1).clamp(min=0)
    use_prev = (lo > 0) & ((lut[prev] - x).abs() < (lut[lo] - x).abs())
    return torch.where(use_prev, prev, lo).to(torch.uint8)


def dequantize_dynamic_values(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return create_dynamic_map(q.device)[q.long()] * scale


def quantize_blockwise(fp: torch.Tensor, block_size: int = BLOCK_SIZE, *, scheme: str = "symmetric_int8_v1"):
    """→ (codes uint8 [n], absmax fp32 [ceil(n/block)])."""
    _check_scheme(scheme)
    x, n = _blocks(fp.reshape(-1).float(), block_size)
    absmax = x.abs().amax(dim=1)
    fn = quantize_symmetric_values if scheme == "symmetric_int8_v1" else quantize_dynamic_values
    q = fn(x, absmax[:, None]).reshape(-1)[:n]
    return q.contiguous(), absmax.contiguous()


def dequantize_blockwise(q: torch.Tensor, absmax: torch.Tensor, numel: int | None = None, block_size: int = BLOCK_SIZE,
                         *, scheme: str = "symmetric_int8_v1") -> torch.Tensor:
    _check_scheme(scheme)
    n = q.numel() if numel is None else numel
    x, _ = _blocks(q.reshape(-1), block_size)
    fn = dequantize_symmetric_values if scheme == "symmetric_int8_v1" else dequantize_dynamic_values
    return fn(x, absmax[:, None].float()).reshape(-1)[:n]


quantize_dynamic_blockwise = functools.partial(quantize_blockwise, scheme="symmetric_int8_v1")
quantize_dynamic_lut_blockwise = functools.partial(quantize_blockwise, scheme="dynamic_int8_v1")
