"""Block-scaled e4m3 numerics (1 x 128 activation scales, 128 x 128 weight scales): quantisers, the K-block-wise
oracle of the product, the advantage over one scale per tensor on data with outliers, and a small model trained with
the block-scaled linears next to the same model in fp32."""

import torch


def test_quantisers_round_trip_within_e4m3_precision():
    from lm_engine_b200.ops import fp8_block as fb

    torch.manual_seed(0)
    x = torch.randn(64, 512) * torch.logspace(-3, 2, 64)[:, None]          # rows of very different magnitude
    q, s = fb.quantize_rows(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (64, 4)
    back = fb.dequantize_rows(q, s)
    assert float(((back - x).abs() / (x.abs().amax(-1, keepdim=True))).max()) < 2 ** -4   # 3 mantissa bits, per block
    w = torch.randn(256, 384)
    qw, sw = fb.quantize_tiles(w)
    assert sw.shape == (2, 3)
    assert float((fb.dequantize_tiles(qw, sw) - w).abs().max() / w.abs().max()) < 2 ** -4
    # the largest element of every block maps onto the largest e4m3 value
    assert float(q.float().reshape(64, 4, 128).abs().amax(-1).min()) == fb.E4M3_MAX


def test_block_wise_oracle_equals_the_product_of_the_dequantised_operands():
    from lm_engine_b200.ops import fp8_block as fb

    torch.manual_seed(1)
    x, w = torch.randn(96, 384), torch.randn(256, 384) * 0.1
    (xq, sx), (wq, sw) = fb.quantize_rows(x), fb.quantize_tiles(w)
    y = fb.block_scaled_matmul_reference(xq, sx, wq, sw)
    want = fb.dequantize_rows(xq, sx).double() @ fb.dequantize_tiles(wq, sw).double().t()
    torch.testing.assert_close(y.double(), want, rtol=1e-5, atol=1e-5)
    # and it is close to the exact product
    exact = x @ w.t()
    assert float((y - exact).norm() / exact.norm()) < 0.05


def test_block_scales_beat_one_scale_per_tensor_on_outliers():
    from lm_engine_b200.ops import fp8_block as fb

    torch.manual_seed(2)
    x = torch.randn(128, 512)
    x[:, 7] *= 3e4                                                         # one outlier feature sets a tensor-wide scale
    w = torch.randn(256, 512) * 0.05
    w[:, 7] = 0                                                            # ... without carrying the result itself
    exact = x @ w.t()
    block = fb.fake_quant_rows(x) @ fb.fake_quant_tiles(w).t()
    scale = fb.E4M3_MAX / x.abs().max()
    tensorwise = ((x * scale).to(torch.float8_e4m3fn).float() / scale) @ fb.fake_quant_tiles(w).t()
    err_block = float((block - exact).norm() / exact.norm())
    err_tensor = float((tensorwise - exact).norm() / exact.norm())
    assert err_block < 0.5 * err_tensor, (err_block, err_tensor)


def test_linear_gradients_are_close_to_the_exact_ones():
    from lm_engine_b200.ops import fp8_block as fb

    torch.manual_seed(3)
    x = torch.randn(4, 50, 256, requires_grad=True)                        # 200 tokens: a partial last token block
    w = (torch.randn(384, 256) * 0.05).requires_grad_(True)
    b = torch.zeros(384, requires_grad=True)
    xr, wr, br = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    y = fb.linear_block_scaled(x, w, b)
    yr = torch.nn.functional.linear(xr, wr, br)
    g = torch.randn_like(yr)
    y.backward(g)
    yr.backward(g)

    def rel(a, c):
        return float((a - c).norm() / c.norm())

    assert rel(y, yr) < 0.06 and rel(x.grad, xr.grad) < 0.06 and rel(w.grad, wr.grad) < 0.06
    torch.testing.assert_close(b.grad, br.grad)


def test_small_model_trains_as_in_fp32():
    """120 AdamW steps of a 2-layer model on a repeating batch: the block-scaled run follows the fp32 run."""
    from lm_engine_b200.fp8 import convert_to_fp8_training
    from lm_engine_b200.models import build_model, config_from_dict, dense_config

    def run(block: bool):
        torch.manual_seed(0)
        cfg = dense_config(vocab_size=256, hidden_size=128, num_layers=2, num_attention_heads=2, num_key_value_heads=2,
                           intermediate_size=256, head_dim=64, max_position_embeddings=64)
        model = build_model(config_from_dict(cfg.to_dict()))
        if block:
            assert convert_to_fp8_training(model, scaling="block") > 0
            assert any(getattr(p, "fp8", None) == "block" for p in model.parameters())
        opt = torch.optim.AdamW(model.parameters(), lr=2e-3, weight_decay=0.0)
        data = torch.randint(0, 256, (4, 65), generator=torch.Generator().manual_seed(5))
        losses = []
        for _ in range(120):
            out = model(input_ids=data[:, :-1])
            loss = torch.nn.functional.cross_entropy(out.logits.float().reshape(-1, 256), data[:, 1:].reshape(-1))
            opt.zero_grad()
            loss.backward()
            opt.step()
            losses.append(float(loss))
        return losses

    ref, blk = run(False), run(True)
    assert ref[-1] < 0.5 * ref[0]                                           # the task is learnable
    assert abs(blk[-1] - ref[-1]) < 0.15 * ref[0]
    assert max(abs(a - b) for a, b in zip(ref[:20], blk[:20])) < 0.1 * ref[0]
