"""Training-loop helpers: metric reduction, console line, and the model FLOP count used for TFLOPs / MFU.

The FLOP count restates the accounting of lm_engine/train_utils.py:67-204 so that throughput figures of both
engines are comparable: a linear layer costs ``2mkn`` forward and twice that backward (+ one forward when its block
is checkpointed); attention ``2 b s w h`` forward (w = window or s, i.e. the causal half) and 2.5x that backward;
GLU MLPs x1.5; MoE x top-k; the LM head is a linear layer.  Models containing mixers without an entry return 0.
"""

from __future__ import annotations

import json
import logging
import os

import torch
import torch.distributed as dist

from .enums import GradientCheckpointingMethod
from .logging_utils import MetricsTrackingDict, log_metrics
from .models.config import CommonConfig
from .models.layers.activations import is_glu
from .parallel.manager import ProcessGroupManager


def all_reduce_metrics_tracker(metrics: MetricsTrackingDict) -> MetricsTrackingDict:
    """Mean over data-parallel ranks of every metric, with one collective."""
    keys = sorted(metrics.keys())
    if not keys:
        return metrics
    vals = [metrics[k] if isinstance(metrics[k], torch.Tensor) else torch.tensor(float(metrics[k])) for k in keys]
    dev = next((v.device for v in vals if isinstance(v, torch.Tensor) and v.is_cuda), torch.device("cpu"))
    t = torch.stack([v.detach().float().reshape(()).to(dev) for v in vals])
    group = ProcessGroupManager.get_data_parallel_group()
    if group is not None:
        dist.all_reduce(t, group=group)
        t = t / ProcessGroupManager.get_data_parallel_world_size()
    out = t.tolist()
    return MetricsTrackingDict({k: v for k, v in zip(keys, out)})


class DeviceWaitExpired(RuntimeError):
    """A bounded device-side wait of the kernel library ran out: data that a kernel expected never arrived."""


def read_device_status() -> list[int] | None:
    """The kernel library's status block (``None`` without a GPU).  Word 0 != 0: a wait on a peer's flag or on an
    mbarrier expired and the kernel went on without the data it waited for."""
    if not torch.cuda.is_available():
        return None
    from .ops import _lib

    return _lib.read_status(clear=False)


def check_device_status(step: int, status: list[int] | None = None) -> list[int] | None:
    """Called once per optimizer step, right after the metrics were read back (the device is idle then).  Raises when
    a device-side wait expired during the step: its results were computed from rows that never arrived, so the job
    must not go on training on them (the launcher restarts from the last checkpoint)."""
    status = read_device_status() if status is None else status
    if status is not None and status[0] != 0:
        raise DeviceWaitExpired(
            f"step {step}: device status {status[:4]} (code {status[0]}: 1 = mbarrier wait, 2 = peer flag wait, "
            f"3 = bounds; detail {status[1]}, block {status[2]}, count {status[3]}): a bounded wait expired or, with "
            f"code 3 and detail 1200 + rank, the expert-parallel landing slab of that rank overflowed (raise "
            f"LME_EP_CAPACITY_FACTOR); the step's results are not valid")
    return status


_METRICS_FILE: str | None = None


def set_metrics_file(path: str | None) -> None:
    global _METRICS_FILE
    _METRICS_FILE = path


def track_metrics(global_step: int, experiments_tracker, metrics: MetricsTrackingDict | dict, context: str) -> None:
    d = metrics.get_dict() if isinstance(metrics, MetricsTrackingDict) else metrics
    d = {k: (v.item() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    if experiments_tracker is not None:
        experiments_tracker.track(d, step=global_step, context=context)
    # local record next to the checkpoints (set by the training entry point, ``LME_METRICS_FILE`` overrides): one JSON object
    # per logged step, written by the tracking rank; the sweep tool ranks trials from it
    path = os.environ.get("LME_METRICS_FILE", _METRICS_FILE)
    if path and ProcessGroupManager.is_tracking_rank() and os.path.isdir(os.path.dirname(path)):
        with open(path, "a") as f:
            f.write(json.dumps({"context": context, "step": global_step, **{k: v for k, v in d.items()
                                                                            if isinstance(v, (int, float))}}) + "\n")
    parts = [f"step = {global_step}"]
    for k in sorted(d):
        v = d[k]
        if isinstance(v, float):
            parts.append(f"{context}-{k} = {v:.4e}" if k == "learning_rate" else f"{context}-{k} = {v:.4f}")
        else:
            parts.append(f"{context}-{k} = {v}")
    log_metrics(logging.INFO, ", ".join(parts))


def _linear_flops(m: float, k: float, n: float, checkpointed: bool = False) -> float:
    fwd = 2 * m * k * n
    return 3 * fwd + (fwd if checkpointed else 0)


def _attention_flops(b: int, s: int, h: int, window: int | None) -> float:
    fwd = 2 * b * s * (s if window is None else window) * h
    return fwd * 3.5


def get_model_tflops(config: CommonConfig, batch_size: int, sequence_length: int,
                     gradient_checkpointing_method: GradientCheckpointingMethod | None,
                     gradient_checkpointing_args: dict) -> float:
    """TFLOPs of one forward + backward pass over ``batch_size x sequence_length`` tokens."""
    b, s, h, v = batch_size, sequence_length, config.hidden_size, config.vocab_size
    n_ckpt = (gradient_checkpointing_args.get("num_blocks", config.num_layers)
              if gradient_checkpointing_method == GradientCheckpointingMethod.block else 0)
    total = 0.0
    for i in range(config.num_layers):
        blk = config.sequence_mixer_blocks[i]
        ck = i < n_ckpt
        kind = blk.sequence_mixer_type
        if kind == "softmax_attention":
            f = _linear_flops(b * s, h, h * (1 + 2 * blk.num_key_value_heads / blk.num_attention_heads), ck)
            f += _linear_flops(b * s, h, h, ck)
            f += _attention_flops(b, s, h, blk.sliding_window)
        elif kind == "mamba2":
            f = 2 * (4 * b * s * h * blk.intermediate_size + 4 * b * s * blk.intermediate_size * blk.state_size)
        elif kind == "rnn":
            nh = max(blk.num_input_heads, blk.num_weight_heads)
            d = blk.state_head_dim
            f = _linear_flops(b * s, h, (blk.num_input_heads + nh) * d) + _linear_flops(b * s, d * nh, h)
            f += s * nh * (_linear_flops(b, d, d) + b * d)
        elif kind == "gru":
            nh = max(blk.num_input_heads, blk.num_forget_input_heads, blk.num_reset_input_heads,
                     blk.num_weight_heads, blk.num_forget_weight_heads, blk.num_reset_weight_heads)
            d = blk.state_head_dim
            n_in = blk.num_input_heads + blk.num_forget_input_heads + blk.num_reset_input_heads + nh
            f = _linear_flops(b * s, h, n_in * d) + _linear_flops(b * s, d * nh, h)
            f += 3 * s * nh * (_linear_flops(b, d, d) + b * d)
        else:
            return 0.0
        total += f
        mlp = config.mlp_blocks[i]
        m = 2 * _linear_flops(b * s, h, mlp.intermediate_size, ck)
        if mlp.mlp_type == "MoE":
            m *= mlp.num_experts_per_tok
        if is_glu(mlp.activation_function):
            m *= 1.5
        total += m
    total += _linear_flops(b * s, h, v)
    return total / 1e12


def measured_peaks() -> dict:
    """bf16 GEMM throughput / copy bandwidth measured on this machine's GPUs when recorded next to the package,
    else an earlier measurement on the same GPU model."""
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def mfu(tflops_per_step: float, step_time_s: float, world_size: int, sustained: bool = True) -> float:
    pk = measured_peaks()
    peak = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    return tflops_per_step / step_time_s / world_size / peak
