"""Small CPU unit tests: LR schedules, parameter groups, GLU packing, weight (de)interleaving, engine group layout."""

import math

import pytest
import torch


def test_lr_schedules_boundaries():
    from lm_engine_b200.enums import LRDecaySchedule
    from lm_engine_b200.optimization.lr_scheduler import lr_factor

    kw = dict(num_warmup_steps=10, num_constant_steps=5, num_decay_steps=20, num_training_steps=100,
              lr_decay_factor=0.1)
    for style in (LRDecaySchedule.cosine, LRDecaySchedule.linear):
        assert lr_factor(0, style=style, **kw) == 0
        assert lr_factor(5, style=style, **kw) == pytest.approx(0.5)
        assert lr_factor(10, style=style, **kw) == 1 and lr_factor(15, style=style, **kw) == 1
        assert lr_factor(35, style=style, **kw) == pytest.approx(0.1)
        assert lr_factor(80, style=style, **kw) == pytest.approx(0.1)
    assert lr_factor(25, style=LRDecaySchedule.cosine, **kw) == pytest.approx(0.55)
    assert lr_factor(25, style=LRDecaySchedule.linear, **kw) == pytest.approx(0.55)
    e = math.e
    want = 0.9 * e / (e - 1) * math.exp(-1) + (0.1 * e - 1) / (e - 1)
    assert lr_factor(35, style=LRDecaySchedule.exponential, **kw) == pytest.approx(want)
    assert lr_factor(35, style=LRDecaySchedule.exponential, **kw) == pytest.approx(0.1)
    ckw = dict(kw, num_decay_steps=0)
    assert lr_factor(50, style=LRDecaySchedule.constant, **ckw) == 1


def test_scheduler_matches_lambda_lr_semantics():
    from lm_engine_b200.enums import LRDecaySchedule
    from lm_engine_b200.optimization.lr_scheduler import LRScheduler

    class Opt:
        param_groups = [{"lr": 2.0}, {"lr": 0.5}]

    s = LRScheduler(Opt(), style=LRDecaySchedule.cosine, num_warmup_steps=4, num_constant_steps=0,
                    num_decay_steps=None, num_training_steps=20, lr_decay_factor=0.1)
    assert s.get_last_lr() == [0.0, 0.0]          # construction performs the step-0 update
    s.step()
    assert s.get_last_lr() == [0.5, 0.125]
    sd = s.state_dict()
    for _ in range(5):
        s.step()
    s.load_state_dict(sd)
    assert s.last_epoch == 1


def test_param_groups_follow_markers():
    from lm_engine_b200.enums import ParamsGroupMethod
    from lm_engine_b200.models import build_model, dense_config
    from lm_engine_b200.optimization.params_group import get_param_groups

    cfg = dense_config(vocab_size=64, hidden_size=32, num_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       intermediate_size=64, max_position_embeddings=32, m_width=2.0)
    for b in cfg.sequence_mixer_blocks + cfg.mlp_blocks:
        b.add_bias = True
    model = build_model(cfg)
    plain = get_param_groups(model, {"lr": 1e-3}, None).get_param_names()
    assert set(plain) == {"normal", "no_weight_decay"}
    assert all(n.endswith("bias") or ".ln_" in n or "ln_f" in n for n in plain["no_weight_decay"])
    assert "transformer.wte.weight" in plain["normal"] and "lm_head.weight" in plain["normal"]
    mup = get_param_groups(model, {"lr": 1e-3}, ParamsGroupMethod.mup, m_width=2.0)
    names = mup.get_param_names()
    assert set(names) == {"normal", "no_weight_decay", "mup"}
    assert "transformer.h.0.mlp_block.c_fc.weight" in names["mup"]
    assert "transformer.wte.weight" in names["normal"]
    tg = {g["params"][0].shape: g for g in mup.to_torch_compatible_params_groups()}
    lrs = sorted(g.get("lr", 1e-3) for g in mup.to_torch_compatible_params_groups())
    assert lrs[0] == pytest.approx(5e-4)
    total = sum(len(v) for v in names.values())
    assert total == len(list(model.named_parameters()))


def test_glu_packing_and_weight_interleaving_are_inverse():
    from lm_engine_b200.models.layers.attention import (interleave_query_key_value_tensor_for_attention,
                                                        split_query_key_value_tensor_for_attention)
    from lm_engine_b200.models.layers.mlp import interleave_up_gate, split_up_gate
    from lm_engine_b200.ops import swiglu_packed

    torch.manual_seed(0)
    up, gate = torch.randn(6, 5), torch.randn(6, 5)
    packed = interleave_up_gate(up, gate)
    u2, g2 = split_up_gate(packed)
    assert torch.equal(u2, up) and torch.equal(g2, gate)
    x = torch.randn(3, 5)
    y = swiglu_packed(x @ packed.t())
    torch.testing.assert_close(y, (x @ up.t()) * torch.nn.functional.silu(x @ gate.t()))
    Hq, Hkv, D = 8, 2, 4
    q, k, v = torch.randn(Hq * D, 7), torch.randn(Hkv * D, 7), torch.randn(Hkv * D, 7)
    qkv = interleave_query_key_value_tensor_for_attention(q, k, v, Hq, Hkv, D)
    q2, k2, v2 = split_query_key_value_tensor_for_attention(qkv, Hq, Hkv, D)
    assert torch.equal(q2, q) and torch.equal(k2, k) and torch.equal(v2, v)
    # group g of the fused layout = its 4 query heads, then its key head, then its value head
    assert torch.equal(qkv[: 4 * D], q[: 4 * D]) and torch.equal(qkv[4 * D:5 * D], k[:D])


def test_moe_group_layout_is_a_padded_partition():
    from lm_engine_b200.ops.moe import GroupLayout

    counts = torch.tensor([130, 0, 1, 128])
    ids = torch.repeat_interleave(torch.arange(4), counts)
    lay = GroupLayout(ids, counts)
    assert lay.k0.tolist() == [0, 256, 256, 384] and lay.kb.tolist() == [4, 0, 2, 2]
    assert lay.tile_group.tolist()[:4] == [0, 0, 2, 3] and set(lay.tile_group.tolist()[4:]) <= {-1}
    assert lay.dest.unique().numel() == ids.numel()
    x = torch.arange(ids.numel(), dtype=torch.float32)[:, None].repeat(1, 2)
    assert torch.equal(lay.gather(lay.scatter(x)), x)
    assert lay.capacity % 128 == 0 and lay.capacity >= 512


def test_sweep_generation_and_collection(tmp_path):
    import json
    import os

    import yaml

    from lm_engine_b200.sweep import collect, generate_trials, materialise

    sweep = {"method": "grid", "parameters": {"optimizer_args.class_args.lr": {"values": [1e-4, 1e-3]},
                                              "training_parameters.micro_batch_size": {"values": [1, 2, 4]}}}
    trials = generate_trials(sweep, None)
    assert len(trials) == 6
    base = {"optimizer_args": {"class_args": {"lr": 1.0, "eps": 1e-8}}, "training_parameters": {"micro_batch_size": 8},
            "save_args": {"save_path": "x", "save_interval": 5}}
    paths = materialise(base, trials, str(tmp_path))
    cfg = yaml.safe_load(open(paths[4]))
    assert cfg["optimizer_args"]["class_args"] == {"lr": 1e-3, "eps": 1e-8}
    assert cfg["training_parameters"]["micro_batch_size"] == 2 and cfg["save_args"]["save_interval"] == 5
    assert cfg["save_args"]["save_path"].endswith(os.path.join("trial-4", "checkpoints"))
    rnd = generate_trials({"method": "bayes", "parameters": {"a.b": {"distribution": "log_uniform_values",
                                                                     "min": 1e-5, "max": 1e-2}}}, 16, seed=1)
    assert all(1e-5 <= t["a.b"] <= 1e-2 for t in rnd) and len({t["a.b"] for t in rnd}) == 16
    for i, v in ((0, 3.0), (3, 1.5)):
        with open(tmp_path / f"trial-{i}" / "metrics.jsonl", "w") as f:
            f.write(json.dumps({"context": "train", "step": 1, "lm_loss": 9.0}) + "\n")
            f.write(json.dumps({"context": "train", "step": 2, "lm_loss": v}) + "\n")
    ranked = collect(str(tmp_path), "train/lm_loss")
    assert [r[0] for r in ranked] == [3, 0] and ranked[0][1] == 1.5
