import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,n,k", [(64, 1000, 32), (300, 4096, 2048), (17, 8192, 2048), (5, 100, 128)])
def test_topk_select_matches_reference(rows, n, k):
    from cppmega_mlx_b200 import ops
    torch.manual_seed(rows)
    sc = torch.randn(rows, n, device="cuda")
    sc[0, :50] = 1.5  # ties
    starts = torch.randint(0, n // 4, (rows,), device="cuda", dtype=torch.int32)
    ends = (starts + torch.randint(1, n, (rows,), device="cuda", dtype=torch.int32)).clamp(max=n)
    got = ops.topk_select(sc, k, starts, ends)
    ref = ops.topk_select_reference(sc, k, starts, ends)
    assert got.shape == ref.shape
    for r in range(rows):
        g = got[r][got[r] >= 0]
        e = ref[r][ref[r] >= 0]
        assert g.numel() == e.numel() and g.unique().numel() == g.numel()
        assert ((g >= starts[r]) & (g < ends[r])).all()
        # same multiset of selected scores (ties may pick different indices)
        assert torch.allclose(sc[r][g.long()].sort().values, sc[r][e.long()].sort().values)
