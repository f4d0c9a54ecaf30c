"""Failure detection without touching a GPU: heartbeat / watchdog logic, a rank that dies before a collective (the
others get an error from the process-group timeout instead of hanging), and damaged checkpoints."""

import json
import os
import time

import pytest
import torch

from .dist_utils import run_distributed


def test_heartbeat_detects_stalled_self_and_missing_peers(tmp_path):
    from lm_engine_b200.utils.watchdog import Heartbeat

    fired = []
    hb = Heartbeat(str(tmp_path), rank=0, world_size=3, stall_seconds=0.3, poll_seconds=0.05,
                   on_stall=lambda h: fired.append(h.step))
    peer = Heartbeat(str(tmp_path), rank=1, world_size=3, stall_seconds=0.3)
    hb.beat(1, [0, 0, 0, 0])
    peer.beat(1)
    own, stale = hb.check()
    assert not own and stale == [2]           # rank 2 never wrote a heartbeat
    hb.start()
    time.sleep(0.6)                            # nobody beats: own rank stalls, rank 1 goes stale too
    hb.stop()
    assert fired and fired[0] == 1
    assert hb.stalled_peers == [1, 2]
    rec = json.load(open(tmp_path / "heartbeat-0.json"))
    assert rec["step"] == 1 and rec["device_status"] == [0, 0, 0, 0]


def _rank_that_dies(rank, world):
    import datetime

    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)                         # a healthy step first
    if rank == 1:
        return "left"                          # leaves between steps, with nothing in flight
    try:
        dist.all_reduce(t)                     # the survivor must get an error, not hang
    except Exception as e:  # noqa: BLE001
        return f"error: {type(e).__name__}"
    return "completed"


def test_surviving_rank_gets_an_error_when_a_peer_leaves():
    t0 = time.time()
    out = run_distributed(_rank_that_dies, 2, timeout=120)
    assert out[1] == "left"
    assert out[0].startswith("error"), out
    assert time.time() - t0 < 90


def _tiny_training(tmp_path):
    import yaml

    from lm_engine_b200.arguments import TrainingArgs

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "pretraining")
    cfg = yaml.safe_load(open(os.path.join(root, "tiny-synthetic.yml")))
    cfg["save_args"] = {"save_path": str(tmp_path / "ckpt"), "save_interval": 2}
    cfg["training_parameters"]["num_training_steps"] = 2
    return cfg, TrainingArgs


def test_damaged_checkpoints_fail_loudly(tmp_path, monkeypatch):
    import yaml

    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.train import main

    cfg, TrainingArgs = _tiny_training(tmp_path)
    p = tmp_path / "a.yml"
    p.write_text(yaml.safe_dump(cfg))
    ProcessGroupManager.destroy_process_groups()
    monkeypatch.setattr("sys.argv", ["train", "--config", str(p)])
    main(TrainingArgs)
    ProcessGroupManager.destroy_process_groups()
    ckpt = tmp_path / "ckpt"
    assert json.load(open(ckpt / "latest_checkpointed_iteration.json"))["latest_checkpointed_iteration"] == 2
    assert not [d for d in os.listdir(ckpt) if d.startswith("tmp") or d.endswith(".tmp")]   # atomic publish

    cfg["load_args"] = {"load_path": str(ckpt)}
    cfg["training_parameters"]["num_training_steps"] = 3
    cfg["save_args"]["save_interval"] = 100
    # (a) the pointer file is corrupt
    (ckpt / "latest_checkpointed_iteration.json").write_text("{not json")
    p.write_text(yaml.safe_dump(cfg))
    with pytest.raises(Exception):
        main(TrainingArgs)
    ProcessGroupManager.destroy_process_groups()
    # (b) the pointer is fine again but a shard of the model is truncated
    (ckpt / "latest_checkpointed_iteration.json").write_text(json.dumps({"latest_checkpointed_iteration": 2}))
    shards = [os.path.join(dp, f) for dp, _, fs in os.walk(ckpt / "global_step2") for f in fs if f.endswith(".distcp")]
    assert shards
    with open(shards[0], "r+b") as f:
        f.truncate(max(os.path.getsize(shards[0]) // 2, 1))
    with pytest.raises(BaseException):   # torch's CheckpointException derives from BaseException
        main(TrainingArgs)
    ProcessGroupManager.destroy_process_groups()


def test_expired_device_wait_stops_training():
    """The training loop looks at the kernel library's status block once per step; a non-zero first word (a bounded
    wait ran out: the step used rows that never arrived) must raise instead of training on."""
    from lm_engine_b200.train_utils import DeviceWaitExpired, check_device_status

    assert check_device_status(3, [0, 0, 0, 0, 0, 0, 0, 0]) == [0, 0, 0, 0, 0, 0, 0, 0]
    with pytest.raises(DeviceWaitExpired) as e:
        check_device_status(7, [2, 861, 0, 5, 0, 0, 0, 0])      # peer flag wait of source rank 1
    assert "step 7" in str(e.value) and "861" in str(e.value)


def test_train_loop_reads_status_every_step(monkeypatch, tmp_path):
    """With a faked status reader that reports an expired wait on the second step, `train` stops on that step and
    the heartbeat file of the first step carries the status words."""
    import json

    import lm_engine_b200.train as train_mod
    from lm_engine_b200.train_utils import DeviceWaitExpired

    calls = {"n": 0}

    def fake_check(step, status=None):
        calls["n"] += 1
        st = [0] * 8 if calls["n"] < 2 else [2, 861, 0, 1, 0, 0, 0, 0]
        if st[0]:
            raise DeviceWaitExpired(f"step {step}")
        return st

    monkeypatch.setattr(train_mod, "check_device_status", fake_check)
    monkeypatch.setattr(train_mod, "train_step_without_pipeline_parallel",
                        lambda *a, **k: train_mod.MetricsTrackingDict({"loss": 1.0}))

    class _NS:
        def __init__(self, **kw):
            self.__dict__.update(kw)

    args = _NS(training_parameters=_NS(gradient_accumulation_steps=1, micro_batch_size=1, global_batch_size=1,
                                       num_training_steps=5, gradient_clipping=1.0, eval_during_training=False,
                                       eval_interval=None),
               distributed_args=_NS(gradient_checkpointing_method=None, gradient_checkpointing_args={},
                                    sync_every_gradient_accumulation_step=False),
               datasets=[_NS(class_args={})], logging_args=_NS(log_interval=100, cost_per_accelerator_per_hour=None,
                                                             torch_profiler_trace_path=None),
               save_args=_NS(save_path=str(tmp_path / "ckpt"), save_interval=10**9),
               tuning_args=_NS(tuning_method=None))

    class _Models(list):
        def train(self):
            return self

    monkeypatch.setenv("LME_HEARTBEAT_DIR", str(tmp_path / "hb"))
    with pytest.raises(DeviceWaitExpired):
        train_mod.train(args, _Models([_NS(config=None)]), None, None, None, None, None, None, None)
    assert calls["n"] == 2
    rec = json.load(open(tmp_path / "hb" / "heartbeat-0.json"))
    assert rec["step"] == 2 and rec["device_status"] == [0] * 8


def test_watchdog_abort_requires_nvls_off():
    from lm_engine_b200.utils.watchdog import abort_is_safe

    assert not abort_is_safe({})                                             # NCCL decides by itself: may bind NVLS
    assert not abort_is_safe({"NCCL_NVLS_ENABLE": "1"})
    assert abort_is_safe({"NCCL_NVLS_ENABLE": "0"})
    assert not abort_is_safe({"NCCL_NVLS_ENABLE": "0", "LME_REDUCE_SCATTER": "nvls"})
