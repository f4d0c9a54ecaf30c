"""Every shipped example config parses through its argument class, and the tiny one trains end to end."""

import glob
import os

import pytest
import yaml

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")


def _load(path):
    with open(path) as f:
        return yaml.safe_load(f)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(ROOT, "**", "*.yml"), recursive=True)))
def test_config_parses(path):
    from lm_engine_b200.arguments import DistillationArgs, TrainingArgs, UnshardingArgs
    from lm_engine_b200.models import config_from_dict

    cfg = _load(path)
    if "parameters" in cfg and "method" in cfg:          # sweep description
        from lm_engine_b200.sweep import generate_trials

        assert len(generate_trials(cfg, 4)) == 4
        return
    if "unsharded_path" in cfg:
        UnshardingArgs(**cfg)
        return
    cls = DistillationArgs if "teacher_args" in cfg else TrainingArgs
    args = cls(**cfg)
    pc = args.model_args.pretrained_config
    if pc is not None:
        c = config_from_dict(pc)
        assert len(c.sequence_mixer_blocks) == c.num_layers == len(c.mlp_blocks)


def test_tiny_config_trains(tmp_path, monkeypatch):
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.train import main

    cfg = _load(os.path.join(ROOT, "pretraining", "tiny-synthetic.yml"))
    cfg["save_args"]["save_path"] = str(tmp_path / "ckpt")
    cfg["training_parameters"]["num_training_steps"] = 4
    cfg["save_args"]["save_interval"] = 4
    p = tmp_path / "c.yml"
    p.write_text(yaml.safe_dump(cfg))
    ProcessGroupManager.destroy_process_groups()
    monkeypatch.setattr("sys.argv", ["train", "--config", str(p)])
    main(TrainingArgs)
    ProcessGroupManager.destroy_process_groups()
    assert os.path.isfile(tmp_path / "ckpt" / "latest_checkpointed_iteration.json")


_REF_CONFIGS = os.path.join(os.path.dirname(ROOT), "baseline", "_ref", "configs")


@pytest.mark.skipif(not os.path.isdir(_REF_CONFIGS), reason="no copy of the reference project's configs/ under baseline/_ref")
def test_every_reference_config_parses():
    """The YAML schema is the public surface shared with the reference project: each of its own example configs
    (training, finetuning, distillation, unsharding, sweeps, research models) has to load through this repository's
    argument classes, and every model description in them has to build a config object."""
    from lm_engine_b200.arguments import DistillationArgs, TrainingArgs, UnshardingArgs
    from lm_engine_b200.models import config_from_dict

    paths = sorted(glob.glob(os.path.join(_REF_CONFIGS, "**", "*.yml"), recursive=True))
    assert len(paths) >= 40
    parsed = models = 0
    for path in paths:
        cfg = _load(path)
        if not isinstance(cfg, dict):
            continue
        if "parameters" in cfg and "method" in cfg:            # W&B sweep description
            continue
        if "unsharded_path" in cfg:
            UnshardingArgs(**cfg)
            parsed += 1
            continue
        if "model_args" not in cfg:
            continue
        args = (DistillationArgs if "teacher_args" in cfg else TrainingArgs)(**cfg)
        parsed += 1
        pc = args.model_args.pretrained_config
        if pc is not None:
            c = config_from_dict(pc)
            assert len(c.sequence_mixer_blocks) == c.num_layers == len(c.mlp_blocks), path
            models += 1
    assert parsed >= 40 and models >= 38, (parsed, models)
