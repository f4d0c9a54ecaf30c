"""FP8 linear path: quantiser and scaled GEMM against PyTorch fp32 statements of the same arithmetic."""

import pytest
import torch


def test_quantize_reference_roundtrip_cpu():
    from lm_engine_b200.ops import fp8

    torch.manual_seed(0)
    x = torch.randn(64, 48) * 3
    for fmt, tol in ((fp8.E4M3, 0.07), (fp8.E5M2, 0.13)):
        q = fp8.quantize(x, fmt, transposed=True)
        back = q.dequantize()
        assert ((back - x).abs() <= tol * x.abs() + 1e-2 * x.abs().max()).all()
        torch.testing.assert_close(q.dequantize(transposed=True), back.t())


def test_linear_fp8_cpu_matches_emulation():
    """The CPU statement of the fp8 linear (used as the oracle on the GPU) is close to the fp32 linear."""
    from lm_engine_b200.ops import fp8

    torch.manual_seed(1)
    x, w = torch.randn(32, 64), torch.randn(48, 64) * 0.1
    xq, wq = fp8.quantize(x, fp8.E4M3), fp8.quantize(w, fp8.E4M3)
    y = fp8.gemm_fp8(xq.q, fp8.E4M3, xq.scale_inv, wq.q, fp8.E4M3, wq.scale_inv, out_dtype=torch.float32)
    ref = x @ w.t()
    assert (y - ref).norm() / ref.norm() < 0.05


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("R,C", [(256, 512), (1040, 208), (64, 16)])
def test_quantize_kernel_matches_reference(fmt, R, C):
    from lm_engine_b200.ops import fp8

    torch.manual_seed(2)
    x = (torch.randn(R, C, device="cuda") * 2.5).to(torch.bfloat16)
    got = fp8.quantize(x, fmt, rowwise=True, transposed=True)
    want = fp8.quantize_reference(x, fmt, rowwise=True, transposed=True)
    torch.testing.assert_close(got.scale_inv, want.scale_inv, rtol=1e-6, atol=0)
    # identical scale -> identical codes except for round-to-nearest ties in the fp32 product (at most one ulp)
    a, b = got.dequantize(), want.dequantize()
    assert (a - b).abs().max() <= 0.13 * b.abs().max() / 8
    assert (got.q != want.q).float().mean() < 1e-3
    assert torch.equal(got.qt, got.q.t().contiguous())


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (384, 128, 208), (8192, 1024, 4096), (130, 264, 144)])
@pytest.mark.parametrize("fmts", [(0, 0), (1, 0)])
def test_gemm_fp8_matches_dequantized_matmul(M, N, K, fmts):
    from lm_engine_b200.ops import _lib, fp8

    torch.manual_seed(3)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    aq, bq = fp8.quantize(a, fmts[0]), fp8.quantize(b, fmts[1])
    got = fp8.gemm_fp8(aq.q, fmts[0], aq.scale_inv, bq.q, fmts[1], bq.scale_inv, out_dtype=torch.float32)
    want = aq.dequantize() @ bq.dequantize().t()
    torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-3 * want.abs().max().item())
    assert _lib.read_status()[0] == 0


@pytest.mark.gpu
def test_linear_fp8_forward_backward_close_to_bf16():
    from lm_engine_b200 import ops

    torch.manual_seed(4)
    T, K, N = 512, 256, 384
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    w8 = w.detach().clone().requires_grad_(True)
    w8.fp8 = True
    x8 = x.detach().clone().requires_grad_(True)
    dy = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    y = ops.linear(x, w)
    y8 = ops.linear(x8, w8)
    y.backward(dy)
    y8.backward(dy)

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm()).item()

    assert rel(y8, y) < 0.06 and rel(x8.grad, x.grad) < 0.08 and rel(w8.grad, w.grad) < 0.08


@pytest.mark.gpu
def test_linear_swiglu_fp8_and_main_grad_accumulation():
    from lm_engine_b200 import ops

    torch.manual_seed(5)
    T, K, N = 256, 128, 512
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, K, device="cuda") * 0.08).to(torch.bfloat16).requires_grad_(True)
    w.fp8 = True
    w.main_grad = torch.full((N, K), 7.0, device="cuda", dtype=torch.bfloat16)
    w.main_grad_stale = True
    ref_w = w.detach().clone().requires_grad_(True)
    ref_x = x.detach().clone().requires_grad_(True)
    dy = torch.randn(T, N // 2, device="cuda").to(torch.bfloat16)
    ops.linear_swiglu(x, w).backward(dy)
    first = w.main_grad.clone()
    ops.linear_swiglu(ref_x, ref_w).backward(dy)
    assert ((first.float() - ref_w.grad.float()).norm() / ref_w.grad.float().norm()) < 0.1   # overwrote the 7s
    ops.linear_swiglu(x.detach().requires_grad_(True), w).backward(dy)
    torch.testing.assert_close(w.main_grad.float(), 2 * first.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_fp8_training_tracks_bf16():
    """Same model / data / optimizer in bf16 and with the block linears on the 8-bit path: the loss curves of a few
    steps stay close and every converted layer really ran 8-bit GEMMs."""
    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.enums import GradientCheckpointingMethod
    from lm_engine_b200.fp8 import convert_to_fp8_training
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.models import dense_config
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer

    def run(use_fp8):
        cfg = dense_config(vocab_size=2048, hidden_size=256, num_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, intermediate_size=1024, head_dim=64, max_position_embeddings=256)
        w = ModelWrapperForPretraining(pretrained_config=cfg.to_dict(), micro_batch_size=2, sequence_length=256,
                                       efficient_initialization=True, dtype="bf16")
        eng = shard_model(w, stage=3, dtype=torch.bfloat16, communication_dtype=None,
                          gradient_checkpointing_method=GradientCheckpointingMethod.block, seed=3)
        n = convert_to_fp8_training(w.model) if use_fp8 else 0
        opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                   "eps": 1e-10}, None, False, 1.0)
        g = torch.Generator(device="cuda").manual_seed(0)
        data = torch.randint(0, 2048, (2, 257), device="cuda", generator=g)
        losses = []
        for _ in range(6):
            opt.zero_grad()
            out = w(data, lm_loss_multiplier=1 / 512)
            out["loss"].backward()
            opt.step()
            losses.append(float(out["loss"]))
        return losses, n

    bf, _ = run(False)
    f8, n = run(True)
    assert n == 8   # qkv, out-proj, fc1, fc2 of two blocks
    assert f8[-1] < f8[0] - 0.5
    for a, b in zip(bf, f8):
        assert abs(a - b) < 0.08 * abs(a), (bf, f8)
    assert _lib.read_status()[0] == 0
