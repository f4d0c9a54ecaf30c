"""Tensor / sequence / context / expert parallel training on gloo ranks against one process that sees the whole
batch: the per-step loss and the global gradient norm must agree for several optimizer steps (a wrong gradient
anywhere shows up in the next step's loss and norm)."""

import numpy as np
import pytest
import torch

from .dist_utils import run_distributed

VOCAB, SEQ = 256, 32


def _config(kind: str) -> dict:
    from lm_engine_b200.models import dense_config

    d = dense_config(vocab_size=VOCAB, hidden_size=64, num_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     intermediate_size=128, max_position_embeddings=SEQ).to_dict()
    if kind == "moe":
        d["mlp_blocks"] = [{"mlp_type": "MoE", "intermediate_size": 32, "num_experts": 4, "num_experts_per_tok": 2,
                            "activation_function": "swiglu", "shared_intermediate_size": 64, "add_bias": False}
                           for _ in range(2)]
        d["router_aux_loss_coef"] = 0.01
    if kind == "hybrid":     # recurrent mixers whose state (and convolution window) crosses the sequence shards
        d["sequence_mixer_blocks"] = [
            dict(sequence_mixer_type="mamba2", state_size=8, intermediate_size=128, num_heads=4, conv_kernel_size=4,
                 activation_function="silu", num_groups=1, chunk_size=8, normalization_function="rmsnorm"),
            dict(sequence_mixer_type="m2rnn", k_head_dim=4, v_head_dim=8, num_q_heads=2, num_k_heads=2, num_v_heads=4,
                 num_f_heads=4, num_g_heads=4, num_weight_heads=4, use_residual=True, kernel_size=4,
                 activation_function="silu", add_bias=False, gradient_clipping=None,
                 normalization_function="rmsnorm")]
        d["position_embedding_type"] = "nope"
    if kind == "bias":
        for b in d["sequence_mixer_blocks"] + d["mlp_blocks"]:
            b["add_bias"] = True
        d["normalization_function"] = "layernorm"
    return d


def _train(rank, world, kind, topo, weights_dir, steps, total_mbs, sequence_parallel=False, padding_free=False):
    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager(zero_stage=3, **topo)
    dl_world = ProcessGroupManager.get_data_loading_world_size()
    dl_rank = ProcessGroupManager.get_data_loading_rank()
    mbs = total_mbs // dl_world
    w = ModelWrapperForPretraining(model_name=weights_dir, micro_batch_size=mbs, sequence_length=SEQ,
                                   sequence_parallel=sequence_parallel, use_padding_free_transformer=padding_free)
    eng = shard_model(w, stage=3, dtype=torch.float32, communication_dtype=None, seed=1)
    opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 2e-3, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10},
                           None, False, 1.0)
    g = torch.Generator().manual_seed(17)
    data = torch.randint(0, VOCAB, (steps, total_mbs, SEQ + 1), generator=g)
    losses, norms = [], []
    for s in range(steps):
        opt.zero_grad()
        batch = data[s, dl_rank * mbs:(dl_rank + 1) * mbs]
        first_tp = ProcessGroupManager.is_tensor_parallel_first_rank()
        out = w(batch if first_tp else None, lm_loss_multiplier=1 / (mbs * SEQ / topo.get("context_parallel_world_size", 1)))
        out["loss"].backward()
        norms.append(float(opt.step()))
        losses.append(float(out["lm_loss"].detach()))
    return losses, norms, dl_world


def _reference(kind, tmp_path, steps, total_mbs):
    from lm_engine_b200.models import build_model, config_from_dict
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.utils import SafeTensorsWeightsManager

    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=3)
    torch.manual_seed(5)
    cfg = config_from_dict(_config(kind))
    model = build_model(cfg)
    d = str(tmp_path / "weights")
    cfg.save_pretrained(d)
    SafeTensorsWeightsManager.save_state_dict(model.state_dict(), d)
    out = _train(0, 1, kind, {}, d, steps, total_mbs)
    ProcessGroupManager.destroy_process_groups()
    return d, out


CASES = [
    ("dense", {"tensor_parallel_world_size": 2}, False),
    ("dense", {"tensor_parallel_world_size": 2}, True),
    ("bias", {"tensor_parallel_world_size": 2}, True),
    ("dense", {"context_parallel_world_size": 2, "context_parallel_attention": "ring"}, False),
    ("dense", {"context_parallel_world_size": 2, "context_parallel_attention": "ulysses"}, False),
    ("dense", {"context_parallel_world_size": 2, "context_parallel_attention": "ulysses",
               "context_parallel_load_balancing_method": "headtail"}, False),
    ("hybrid", {"context_parallel_world_size": 2}, False),
    ("moe", {"expert_parallel_world_size": 2}, False),
    ("moe", {"tensor_parallel_world_size": 2}, False),
]


@pytest.mark.parametrize("kind,topo,sp", CASES, ids=["tp2", "tp2-sp", "tp2-sp-bias", "cp2-ring", "cp2-ulysses", "cp2-ulysses-headtail", "cp2-hybrid", "ep2", "moe-tp2"])
def test_parallel_training_matches_single_process(kind, topo, sp, tmp_path):
    steps, total_mbs = 3, 2
    d, (ref_loss, ref_norm, _) = _reference(kind, tmp_path, steps, total_mbs)
    outs = run_distributed(_train, 2, kind, topo, d, steps, total_mbs, sp)
    dl_world = outs[0][2]
    # ranks of different data-parallel groups see different micro-batches: average their mean losses
    if dl_world == 1 and "context_parallel_world_size" not in topo:
        loss = outs[0][0]
    else:   # data-parallel ranks see different micro-batches, context-parallel ranks different tokens
        loss = [sum(o[0][s] for o in outs) / len(outs) for s in range(steps)]
    np.testing.assert_allclose(loss, ref_loss, rtol=2e-4)
    for o in outs:
        np.testing.assert_allclose(o[1], ref_norm, rtol=2e-3)


def _ulysses_rank(rank, world, method):
    from lm_engine_b200.ops import attention
    from lm_engine_b200.parallel.context_parallel import shard_indices
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.parallel.ulysses import ulysses_attention

    ProcessGroupManager(context_parallel_world_size=world, context_parallel_load_balancing_method=method)
    g = torch.Generator().manual_seed(3)
    B, S, Hq, Hkv, D = 2, 32, 8, 2, 16          # 2 K/V heads over 4 ranks: each K/V head is replicated twice
    q, k, v, do = (torch.randn(B, S, h, D, generator=g, dtype=torch.float64) for h in (Hq, Hkv, Hkv, Hq))
    full = [t.clone().requires_grad_() for t in (q, k, v)]
    ref = attention(*full, causal=True)
    ref.backward(do)
    idx = shard_indices(S, world, rank, method)
    loc = [t[:, idx].clone().requires_grad_() for t in (q, k, v)]
    out = ulysses_attention(*loc, causal=True)
    out.backward(do[:, idx])
    torch.testing.assert_close(out, ref[:, idx].detach(), rtol=1e-9, atol=1e-9)
    for a, b in zip(loc, full):
        torch.testing.assert_close(a.grad, b.grad[:, idx], rtol=1e-9, atol=1e-9)
    return True


@pytest.mark.parametrize("method", [None, "headtail"])
def test_ulysses_attention_replicated_kv_heads(method):
    assert all(run_distributed(_ulysses_rank, 4, method))


@pytest.mark.parametrize("kind,topo,sp", [("dense", {"tensor_parallel_world_size": 2}, True), ("hybrid", {}, False)],
                         ids=["tp2-sp", "dp2-hybrid"])
def test_padding_free_training_matches_the_batched_layout(kind, topo, sp, tmp_path):
    """Packed tokens [mbs * S] + cu_seqlens on two ranks against the [mbs, S] layout in one process."""
    steps, total_mbs = 3, 2
    d, (ref_loss, ref_norm, _) = _reference(kind, tmp_path, steps, total_mbs)
    outs = run_distributed(_train, 2, kind, topo, d, steps, total_mbs, sp, True)
    loss = outs[0][0] if outs[0][2] == 1 else [sum(o[0][s] for o in outs) / len(outs) for s in range(steps)]
    np.testing.assert_allclose(loss, ref_loss, rtol=2e-4)
    for o in outs:
        np.testing.assert_allclose(o[1], ref_norm, rtol=2e-3)


CASES_4_RANKS = [
    ("dense", {"tensor_parallel_world_size": 2}, True),                                      # TP2 + SP x ZeRO-3 over 2
    ("dense", {"context_parallel_world_size": 2, "context_parallel_attention": "ring"}, False),      # CP2 x ZeRO-3 over 2
    ("dense", {"tensor_parallel_world_size": 2, "context_parallel_world_size": 2}, False),   # TP2 x CP2
    ("moe", {"expert_parallel_world_size": 2}, False),                                       # EP2, experts replicated x2
    ("hybrid", {"context_parallel_world_size": 2}, False),                                   # recurrent CP2 x ZeRO-3 over 2
]


@pytest.mark.parametrize("kind,topo,sp", CASES_4_RANKS,
                         ids=["tp2-sp-x-dp2", "cp2-ring-x-dp2", "tp2-x-cp2", "ep2-x-dp2", "cp2-hybrid-x-dp2"])
def test_composed_meshes_on_four_ranks_match_single_process(kind, topo, sp, tmp_path):
    """Two parallel dimensions at once on 4 gloo ranks (the reference tests TP x PP x ZeRO combinations the same
    way, tests/dcp/dcp_test.py): loss and gradient norm of every step against one process."""
    steps, total_mbs = 3, 4          # expert parallelism alone leaves 4 data-parallel ranks: one sample each
    d, (ref_loss, ref_norm, _) = _reference(kind, tmp_path, steps, total_mbs)
    outs = run_distributed(_train, 4, kind, topo, d, steps, total_mbs, sp, timeout=600)
    loss = [sum(o[0][s] for o in outs) / len(outs) for s in range(steps)]
    np.testing.assert_allclose(loss, ref_loss, rtol=3e-4)
    for o in outs:
        np.testing.assert_allclose(o[1], ref_norm, rtol=3e-3)
