"""The sharded engine end to end on one GPU: bf16 training step against an fp32 PyTorch model with the same weights."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(dtype, cpu_offload=False, step_in_backward=False, max_grad_norm=1.0):
    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.enums import GradientCheckpointingMethod
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.models import dense_config
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer

    cfg = dense_config(vocab_size=2048, hidden_size=256, num_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=1024, head_dim=64, max_position_embeddings=256)
    w = ModelWrapperForPretraining(pretrained_config=cfg.to_dict(), micro_batch_size=2, sequence_length=256,
                                   efficient_initialization=True, dtype="bf16")
    eng = shard_model(w, stage=3, dtype=dtype, communication_dtype=None,
                      gradient_checkpointing_method=GradientCheckpointingMethod.block, seed=3,
                      cpu_offload=cpu_offload)
    opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10},
                           None, False, max_grad_norm, step_in_backward=step_in_backward)
    return cfg, w, eng, opt


def test_smoke_entry():
    import __graft_entry__ as g

    g.smoke()


def test_bf16_gradients_match_fp32_reference():
    """Per-parameter gradients of one bf16 step (through checkpointing, fused epilogues and main_grad accumulation)
    against autograd on an fp32 copy of the model."""
    from lm_engine_b200.models import build_model
    from lm_engine_b200.ops import _lib

    cfg, w, eng, opt = _setup(torch.bfloat16)
    ref = build_model(cfg).cuda().float()
    ref.load_state_dict(eng.full_state_dict())
    g = torch.Generator(device="cuda").manual_seed(0)
    fixed = torch.randint(0, 2048, (2, 257), device="cuda", generator=g)
    opt.zero_grad()
    out = w(fixed, lm_loss_multiplier=1 / 512)
    out["loss"].backward()
    eng.finish_backward()
    grads = eng.full_state_dict("grad")
    logits = ref(fixed[:, :-1]).logits
    rl = torch.nn.functional.cross_entropy(logits.float().view(-1, 2048), fixed[:, 1:].reshape(-1))
    rl.backward()
    assert abs(float(out["loss"]) - float(rl)) < 2e-2
    bad = []
    for n, p in ref.named_parameters():
        err = ((grads[n].float() - p.grad).norm() / (p.grad.norm() + 1e-12)).item()
        if err > 5e-2:
            bad.append((n, err))
    assert not bad, bad
    assert _lib.read_status()[0] == 0


def test_bf16_training_tracks_fp32_reference():
    from lm_engine_b200.models import build_model
    from lm_engine_b200.ops import _lib

    cfg, w, eng, opt = _setup(torch.bfloat16)
    ref = build_model(cfg).cuda().float()
    ref.load_state_dict(eng.full_state_dict())
    nodecay = [p for n, p in ref.named_parameters() if "ln_" in n]
    decay = [p for n, p in ref.named_parameters() if "ln_" not in n]
    ropt = torch.optim.AdamW([{"params": decay}, {"params": nodecay, "weight_decay": 0.0}], lr=1e-3,
                             betas=(0.9, 0.95), eps=1e-10, weight_decay=0.1)
    g = torch.Generator(device="cuda").manual_seed(0)
    fixed = torch.randint(0, 2048, (2, 257), device="cuda", generator=g)
    losses, ref_losses, norms, ref_norms = [], [], [], []
    for _ in range(8):
        opt.zero_grad()
        out = w(fixed, lm_loss_multiplier=1 / 512)
        out["loss"].backward()
        norms.append(float(opt.step()))
        losses.append(float(out["loss"]))
        ropt.zero_grad()
        logits = ref(fixed[:, :-1]).logits
        rl = torch.nn.functional.cross_entropy(logits.float().view(-1, 2048), fixed[:, 1:].reshape(-1))
        rl.backward()
        ref_norms.append(float(torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)))
        ropt.step()
        ref_losses.append(float(rl))
    assert _lib.read_status()[0] == 0
    assert abs(norms[0] - ref_norms[0]) / ref_norms[0] < 0.02, (norms, ref_norms)
    # same batch every step: the loss must fall, and the bf16 engine must follow the fp32 trajectory
    assert losses[-1] < losses[0] - 0.5, losses
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 0.05 * max(1.0, b), (losses, ref_losses)


def _run_steps(n, **kw):
    cfg, w, eng, opt = _setup(torch.bfloat16, **kw)
    g = torch.Generator(device="cuda").manual_seed(0)
    fixed = torch.randint(0, 2048, (2, 257), device="cuda", generator=g)
    losses = []
    for _ in range(n):
        opt.zero_grad()
        out = w(fixed, lm_loss_multiplier=1 / 512)
        out["loss"].backward()
        opt.step()
        losses.append(float(out["loss"]))
    return losses, eng


def test_cpu_offloaded_optimizer_state_follows_the_device_step():
    """`cpu_offload`: master weights and AdamW moments in pinned host memory, updated there; the trajectory is the
    device one up to the rounding of the host arithmetic."""
    base, _ = _run_steps(5)
    off, eng = _run_steps(5, cpu_offload=True)
    assert all(u.master.device.type == "cpu" and u.master.is_pinned() for u in eng.all_units)
    for a, b in zip(off, base):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (off, base)


def test_optimizer_in_backward_on_the_reduction_stream():
    """Stepping each unit behind its gradient reduction (no clipping) equals the step after the backward pass."""
    base, _ = _run_steps(5, max_grad_norm=None)
    hooked, _ = _run_steps(5, max_grad_norm=None, step_in_backward=True)
    for a, b in zip(hooked, base):
        assert abs(a - b) < 1e-3 * max(1.0, abs(b)), (hooked, base)
