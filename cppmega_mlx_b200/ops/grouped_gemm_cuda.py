"""Grouped (per-expert) GEMM on the tcgen05 kernel, without a host synchronisation.

Tokens routed to experts are scattered into a *padded, expert-sorted* buffer whose expert segments start on 128-row boundaries,
so every 128-row GEMM tile belongs to exactly one expert.  The buffer has a static size (``assignments + E·127`` rounded up to
128), the per-tile expert table and the per-expert row ranges are computed on the device, and the three products of a linear
layer map onto the batched kernel in ``csrc/gemm_bf16.cu``:

* forward   ``Y = X · W[e]ᵀ``      : A = X (2-D), B = W stacked ``[E, out, in]``, tile table picks the expert slice;
* dgrad     ``dX = dY · W[e]``     : same with B read MN-major;
* wgrad     ``dW[e] = dY[e]ᵀ X[e]``: batched over experts, both operands MN-major views of the whole buffers with the
  contraction clipped to the expert's row range (padding rows are zero, an empty range yields zeros).

The reference has no grouped kernel: it evaluates every expert on every token (``cppmega_mlx/nn/moe.py:166-228``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _backend as B
from . import gemm as G

TILE = 128


@dataclass
class GroupedLayout:
    num_experts: int
    rows: int                    # padded buffer rows (static)
    slot: torch.Tensor           # [A] int64: row of each (sorted) assignment in the padded buffer
    order: torch.Tensor          # [A] int64: assignment indices sorted by expert (stable)
    tile_group: torch.Tensor     # [rows/128] int32
    k_ranges: torch.Tensor       # [E, 2] int32
    counts: torch.Tensor         # [E] int64
    valid_rows: torch.Tensor | None = None   # [rows] bool, set by producers that do not clear their buffers
    used_rows: torch.Tensor | None = None    # int32 device scalar: rows of the padded buffer that belong to some expert segment;
                                             # the GEMMs skip every 128-row tile beyond it (rows there are neither read nor written)


def padded_rows(num_assignments: int, num_experts: int) -> int:
    return (num_assignments + num_experts * (TILE - 1) + TILE - 1) // TILE * TILE


def build_layout(expert_ids: torch.Tensor, num_experts: int) -> GroupedLayout:
    """``expert_ids`` [A] (any int dtype, on the GPU). Pure device-side tensor ops: no ``.item()``, no host sync."""
    A = expert_ids.numel()
    rows = padded_rows(A, num_experts)
    e = expert_ids.reshape(-1).long()
    order = torch.argsort(e, stable=True)
    counts = torch.bincount(e, minlength=num_experts)
    pad_counts = (counts + TILE - 1) // TILE * TILE
    pad_end = torch.cumsum(pad_counts, 0)
    pad_off = pad_end - pad_counts
    off = torch.cumsum(counts, 0) - counts
    se = e[order]
    slot = pad_off[se] + (torch.arange(A, device=e.device) - off[se])
    tile_start = torch.arange(rows // TILE, device=e.device) * TILE
    tile_group = torch.searchsorted(pad_end, tile_start, right=True).clamp_(max=num_experts - 1).int()
    k_ranges = torch.stack([pad_off, pad_end], 1).int().contiguous()
    return GroupedLayout(num_experts, rows, slot, order, tile_group, k_ranges, counts, used_rows=pad_end[-1:].int())


def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (B.on_gpu(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 3 and w.is_contiguous()
            and x.shape[-1] % 8 == 0 and w.shape[1] % 8 == 0 and w.shape[2] == x.shape[-1])


def _fwd(x, w, L: GroupedLayout, b_mn: bool, flags: int = 0):
    """b_mn False: Y[rows,out] = X·W[e]ᵀ (W [E,out,in]).  b_mn True: Y[rows,in] = X·W[e] (X has `out` columns).
    ``flags``: an element-wise epilogue of the GEMM (``gemm.EPI_RELU2``)."""
    E, out_f, in_f = w.shape
    N = in_f if b_mn else out_f
    K = out_f if b_mn else in_f
    y = torch.empty(L.rows, N, dtype=torch.bfloat16, device=x.device)
    G.gemm_batched(x, w, y, M=L.rows, N=N, K=K, a_mn=False, b_mn=b_mn, lda=x.stride(0), ldb=in_f, ldc=N, nb=(1, 1, 1),
                   sA=(0, 0, 0), sB=(out_f * in_f, 0, 0), sC=(0, 0, 0), tile_group=L.tile_group, b_groups=E, m_limit=L.used_rows, flags=flags)
    return y


def _wgrad(gy, x, L: GroupedLayout, shape):
    E, out_f, in_f = shape
    gw = torch.empty(E, out_f, in_f, dtype=torch.bfloat16, device=x.device)
    G.gemm_batched(gy, x, gw, M=out_f, N=in_f, K=L.rows, a_mn=True, b_mn=True, lda=gy.stride(0), ldb=x.stride(0), ldc=in_f,
                   nb=(E, 1, 1), sA=(0, 0, 0), sB=(0, 0, 0), sC=(out_f * in_f, 0, 0), a_div2=E, b_div2=E, k_ranges=L.k_ranges)
    return gw


class _GroupedLinearPadded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, L, act):
        ctx.L, ctx.act = L, act
        y = _fwd(x, w, L, False, G.EPI_RELU2 if act == "relu2" else 0)
        if act == "relu2":
            ctx.save_for_backward(x, w, y)      # relu(z) = sqrt(y): the pre-activation is not kept
        else:
            ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, gy):
        L = ctx.L
        if ctx.act == "relu2":
            x, w, y = ctx.saved_tensors
            rows = int(y.shape[0])
            # rows beyond the used part of the buffer were never written by the forward product
            gz = gy.float() * (2.0 * y.float().sqrt())
            if L.used_rows is not None:
                gz = torch.where(torch.arange(rows, device=y.device)[:, None] < L.used_rows, gz, 0.0)
            gy = gz.to(torch.bfloat16)
        else:
            x, w = ctx.saved_tensors
            gy = gy.contiguous()
        gx = _fwd(gy, w, L, True) if ctx.needs_input_grad[0] else None
        gw = _wgrad(gy, x, L, w.shape) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None


def grouped_linear_padded(x: torch.Tensor, w: torch.Tensor, layout: GroupedLayout, act: str | None = None) -> torch.Tensor:
    """x [layout.rows, in] (padding rows zero) × w [E, out, in] → [layout.rows, out]; differentiable.  ``act="relu2"`` applies
    relu(·)² in the GEMM epilogue."""
    if act not in (None, "relu2"):
        raise ValueError(f"unsupported fused activation {act!r}")
    return _GroupedLinearPadded.apply(x.contiguous(), w, layout, act)


def scatter_to_padded(flat: torch.Tensor, tok: torch.Tensor, layout: GroupedLayout) -> torch.Tensor:
    """Rows ``flat[tok]`` placed at ``layout.slot``; everything else zero. Differentiable (index ops)."""
    xp = flat.new_zeros(layout.rows, flat.shape[1])
    return xp.index_copy(0, layout.slot, flat.index_select(0, tok))
