"""The benchmark's model table: every entry is a valid model config and a valid training config, and the
parallelism options produce the distributed arguments they name."""

import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@pytest.mark.parametrize("name", ["llama3-8b", "llama-1b", "tiny", "moe-64e", "moe-ep8", "dense-20b", "hybrid-mamba2",
                                  "hybrid-m2rnn", "hybrid-2p7b"])
def test_every_bench_model_builds_on_the_meta_device(name):
    import bench
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.models import build_model, config_from_dict

    assert set(bench.MODELS) >= {name}
    cfg = bench.model_config(name, 4096)
    with torch.device("meta"):
        model = build_model(config_from_dict(cfg))
    params = sum(p.numel() for p in model.parameters())
    expected = {"llama3-8b": 8.0e9, "dense-20b": 20.3e9, "hybrid-2p7b": 2.75e9, "moe-ep8": 10.1e9}
    if name in expected:
        assert abs(params - expected[name]) < 0.03 * expected[name], params
    TrainingArgs(**bench.training_config(name, 4096, 2, 3, ["fused_linear_cross_entropy"], None))


def test_parallelism_options_reach_the_distributed_arguments():
    import bench
    from lm_engine_b200.arguments import TrainingArgs

    cfg = bench.training_config("dense-20b", 8192, 1, 3, [], None)
    cfg["distributed_args"].update(tensor_parallel_world_size=4, sequence_parallel=True,
                                   use_async_tensor_parallel=True, context_parallel_world_size=2,
                                   context_parallel_attention="ring")
    cfg["training_parameters"]["gradient_accumulation_steps"] = 8
    a = TrainingArgs(**cfg)
    d = a.distributed_args
    assert (d.tensor_parallel_world_size, d.sequence_parallel, d.use_async_tensor_parallel) == (4, True, True)
    assert d.context_parallel_world_size == 2 and d.context_parallel_attention == "ring"
    assert a.training_parameters.gradient_accumulation_steps == 8
