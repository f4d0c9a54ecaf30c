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
