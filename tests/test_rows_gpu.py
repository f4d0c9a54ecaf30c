"""Embedding lookup / gradient and pack / unpack row kernels against their PyTorch statements."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,V,H,lo,hi", [(1000, 512, 256, 0, 512), (4096, 2048, 1024, 512, 1024), (7, 64, 8, 0, 64)])
def test_embedding_matches_torch(T, V, H, lo, hi):
    from lm_engine_b200.ops.embedding import embedding

    torch.manual_seed(0)
    ids = torch.randint(0, V, (2, T // 2 if T > 7 else 7), device="cuda")
    ids[0, :3] = ids[0, 0]            # a run of equal ids
    W = torch.randn(hi - lo, H, device="cuda").to(torch.bfloat16).requires_grad_(True)
    out = embedding(ids, W, lo, hi)
    dy = torch.randn_like(out)
    out.backward(dy)
    Wr = W.detach().float().requires_grad_(True)
    inside = (ids >= lo) & (ids < hi)
    ref = F.embedding((ids - lo).masked_fill(~inside, 0), Wr) * inside.unsqueeze(-1)
    ref.backward(dy.float())
    torch.testing.assert_close(out.float(), ref, rtol=0, atol=0)
    torch.testing.assert_close(W.grad.float(), Wr.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype,row", [(torch.bfloat16, (64,)), (torch.float32, (3, 4)), (torch.bfloat16, (2, 8, 16))])
def test_pack_unpack_match_index_path(dtype, row):
    from lm_engine_b200.ops import packing

    torch.manual_seed(0)
    B, S = 5, 37
    lens = torch.tensor([37, 1, 0, 20, 9], device="cuda")
    cu = F.pad(lens.cumsum(0), (1, 0)).to(torch.int32)
    x = torch.randn(B, S, *row, device="cuda").to(dtype).requires_grad_(True)
    packed = packing.pack_sequence(x, cu)
    g = torch.randn_like(packed)
    packed.backward(g)
    idx = packing._flat_index(cu, S, None)
    ref = x.detach().reshape(B * S, *row).index_select(0, idx)
    torch.testing.assert_close(packed, ref, rtol=0, atol=0)
    gref = torch.zeros(B * S, *row, dtype=dtype, device="cuda").index_copy(0, idx, g).view_as(x)
    torch.testing.assert_close(x.grad, gref, rtol=0, atol=0)
    p2 = packed.detach().requires_grad_(True)
    un = packing.unpack_sequence(p2, cu, (B, S, *row))
    un_ref = torch.zeros(B * S, *row, dtype=dtype, device="cuda").index_copy(0, idx, packed.detach()).view_as(x)
    torch.testing.assert_close(un, un_ref, rtol=0, atol=0)
    un.backward(x.detach())
    torch.testing.assert_close(p2.grad, ref, rtol=0, atol=0)
