import torch


def test_pack_unpack_roundtrip_and_gradient():
    from lm_engine_b200.ops.packing import (compute_cu_seqlens_and_max_seqlen_from_attention_mask, pack_sequence,
                                            unpack_sequence)

    torch.manual_seed(0)
    B, S, H = 4, 9, 5
    lens = [9, 3, 0, 6]
    mask = torch.zeros(B, S, dtype=torch.long)
    for b, n in enumerate(lens):
        if n:
            mask[b, S - n:] = 1
    cu, mx = compute_cu_seqlens_and_max_seqlen_from_attention_mask(mask)
    assert cu.tolist() == [0, 9, 12, 12, 18] and mx == 9
    x = torch.randn(B, S, H, requires_grad=True)
    p = pack_sequence(x, cu)
    want = torch.cat([x[b, S - n:] for b, n in enumerate(lens)])
    assert torch.equal(p, want)
    u = unpack_sequence(p, cu, (B, S, H))
    assert torch.equal(u, x * mask[..., None])
    u.sum().backward()
    assert torch.equal(x.grad, mask[..., None].expand(B, S, H).float())
    ids = torch.arange(B * S).view(B, S)
    a, b2 = pack_sequence([ids, x.detach()], cu, total_tokens=18)
    assert a.tolist() == [i for b, n in enumerate(lens) for i in range(b * S + S - n, b * S + S)]
