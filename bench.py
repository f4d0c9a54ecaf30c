"""Headline benchmark: pretraining throughput of a Llama-3-8B-shaped dense model (bf16 compute, fp32 master weights
and AdamW state, ZeRO-3, block gradient checkpointing on every layer, seq 4096, micro batch 2 per GPU).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 10 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same config

Prints ONE JSON line on rank 0.  ``value`` is whole-job tokens/s measured on the device (CUDA events around K steps
whose inputs are already resident), max over ranks; ``e2e`` is the same metric through the public training-step API
with the per-step pinned-host -> device copy of the token batch and a device -> host read of the loss inside the
timed region.  Data: synthetic uniform-random token ids; weights: seeded random init.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    # name: (vocab, layers, hidden, heads, kv_heads, head_dim, intermediate, rope_theta)
    "llama3-8b": (128256, 32, 4096, 32, 8, 128, 14336, 500000),
    "llama-1b": (32000, 16, 2048, 16, 8, 128, 5632, 10000),
    "tiny": (2048, 4, 256, 4, 2, 64, 1024, 10000),
    # fine-grained mixture of experts (see MOE): dense dims as above, the MLP of every block is routed
    "moe-64e": (32000, 16, 2048, 16, 4, 128, 1024, 10000),
    # the mixture-of-experts target config: 24 layers, 64 SwiGLU-1024 experts, top-8, aux 0.01, micro batch 4 per GPU,
    # experts split over all N GPUs (expert parallel = N) with ZeRO-3 for the rest
    "moe-ep8": (50304, 24, 2048, 16, 4, 128, 1024, 10000),
    # ~20B dense model of the tensor-parallel target config (run with --tp 4 --seq 8192 --mbs 1 --ga 8 on 8 GPUs)
    "dense-20b": (128256, 48, 6144, 48, 8, 128, 16384, 500000),
    # hybrid: three Mamba-2 (SSD) layers per softmax-attention layer (see HYBRID), no positional embedding
    "hybrid-mamba2": (32000, 16, 2048, 16, 4, 128, 8192, 10000),
    # the long-context hybrid target config (~2.7B): 48 layers, hidden 2560, every 6th layer attention (20 / 4 heads,
    # RoPE theta 1e6), the others Mamba-2 (expand 2, head dim 64, state 128, chunk 256); run with --cp 4 --seq 32768
    "hybrid-2p7b": (50304, 48, 2560, 20, 4, 128, 2048, 1000000),
    # hybrid: three matrix-state RNN layers per softmax-attention layer (see M2RNN_HYBRID)
    "hybrid-m2rnn": (32000, 16, 2048, 16, 4, 128, 8192, 10000),
}
# name: (experts, experts per token, shared expert intermediate size or None, router aux-loss coefficient)
MOE = {"moe-64e": (64, 8, None, 0.01), "moe-ep8": (64, 8, None, 0.01)}
# name: (attention every n-th layer, state size, SSM heads, conv kernel, chunk size)
HYBRID = {"hybrid-mamba2": (4, 128, 64, 4, 256), "hybrid-2p7b": (6, 128, 80, 4, 256)}
# name: (attention every n-th layer, k head dim, v head dim, heads, conv kernel): one q / k head shared by all value
# heads, the layout of the published M2RNN hybrids
M2RNN_HYBRID = {"hybrid-m2rnn": (4, 64, 16, 64, 4)}


LAYERS_OVERRIDE: int | None = None   # --layers: same per-layer shapes with fewer layers (profiling captures only)


def model_config(name: str, seq: int) -> dict:
    v, L, h, nh, nkv, hd, inter, theta = MODELS[name]
    if LAYERS_OVERRIDE is not None:
        L = LAYERS_OVERRIDE
    return {
        "model_type": "gpt_base", "vocab_size": v, "max_position_embeddings": seq, "hidden_size": h,
        "num_layers": L, "normalization_function": "rmsnorm", "layer_norm_epsilon": 1e-5,
        "initializer_range": 0.02, "bos_token_id": 0, "eos_token_id": 1, "pad_token_id": 2,
        "position_embedding_type": ("nope" if (name in HYBRID or name in M2RNN_HYBRID) and name != "hybrid-2p7b"
                                    else "rope"), "rope_theta": theta, "rope_scaling": None, "m_emb": None,
        "m_width": None, "m_residual": None, "init_method": "normal", "embedding_init_method": "normal",
        "use_depth_scaled_init": False, "tie_word_embeddings": False,
        "sequence_mixer_blocks": [_mixer_block(name, i, h, nh, nkv, hd) for i in range(L)],
        "mlp_blocks": [_mlp_block(name, inter) for _ in range(L)],
        "router_aux_loss_coef": MOE[name][3] if name in MOE else 0.001,
        **({"rope_dim": hd} if name == "hybrid-2p7b" else {}),
    }


def _mixer_block(name: str, i: int, h: int, nh: int, nkv: int, hd: int) -> dict:
    if name in HYBRID and (i + 1) % HYBRID[name][0] != 0:
        _, state, heads, conv, chunk = HYBRID[name]
        return {"sequence_mixer_type": "mamba2", "state_size": state, "intermediate_size": 2 * h, "num_heads": heads,
                "conv_kernel_size": conv, "add_bias": False, "use_conv_bias": True, "num_groups": 1,
                "chunk_size": chunk, "activation_function": "silu", "normalization_function": "rmsnorm"}
    if name in M2RNN_HYBRID and (i + 1) % M2RNN_HYBRID[name][0] != 0:
        _, kd, vd, heads, conv = M2RNN_HYBRID[name]
        return {"sequence_mixer_type": "m2rnn", "k_head_dim": kd, "v_head_dim": vd, "num_q_heads": 1,
                "num_k_heads": 1, "num_v_heads": heads, "num_f_heads": heads, "num_g_heads": heads,
                "num_weight_heads": heads, "kernel_size": conv, "add_bias": False, "use_residual": True,
                "activation_function": "silu", "gradient_clipping": 1.0, "normalization_function": "rmsnorm"}
    return {"sequence_mixer_type": "softmax_attention", "num_attention_heads": nh, "num_key_value_heads": nkv,
            "head_dim": hd}


def _mlp_block(name: str, inter: int) -> dict:
    if name not in MOE:
        return {"mlp_type": "MLP", "intermediate_size": inter, "activation_function": "swiglu"}
    experts, topk, shared, _ = MOE[name]
    return {"mlp_type": "MoE", "intermediate_size": inter, "activation_function": "swiglu", "num_experts": experts,
            "num_experts_per_tok": topk, "shared_intermediate_size": shared, "add_bias": False,
            "shared_expert_gating": False, "normalized_topk": True, "dropout": 0}


def training_config(model: str, seq: int, mbs: int, steps: int, kernels: list[str], tokenizer: str | None) -> dict:
    cfg = {
        "random_args": {"seed": 42},
        "model_args": {"pretrained_config": model_config(model, seq), "efficient_initialization": True},
        "tuning_args": {"tuning_method": "pretraining"},
        "optimizer_args": {"class_name": "TorchAdamW",
                           "class_args": {"lr": 3e-4, "weight_decay": 0.1, "betas": [0.9, 0.95], "eps": 1e-10}},
        "lr_scheduler_args": {"num_warmup_steps": 5, "lr_decay_style": "cosine"},
        "datasets": [{"class_name": "SyntheticDataset", "data_name": "synthetic",
                      "class_args": {"sequence_length": seq, "seed": 1234}}],
        "save_args": {"save_path": os.path.join(tempfile.gettempdir(), "lme_bench_ckpt"), "save_interval": 10**9},
        "training_parameters": {"num_training_steps": max(steps, 10**6), "micro_batch_size": mbs,
                                "gradient_accumulation_steps": 1, "eval_during_training": False,
                                "gradient_clipping": 1.0},
        "mixed_precision_args": {"dtype": "bf16"},
        "distributed_args": {"stage": 3, "fsdp_algorithm": 2, "gradient_checkpointing_method": "block"},
        "kernel_args": {"kernels": kernels},
        "logging_args": {"log_interval": 10**9},
    }
    if tokenizer is not None:
        cfg["tokenizer_args"] = {"tokenizer_name": tokenizer}
    return cfg


# ---------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.path = os.path.join(tempfile.gettempdir(), f"lme_clocks_{os.getpid()}.csv")
        self.gpu_index = gpu_index
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "power_w_median": statistics.median(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------- our engine
def run_ours(a) -> dict:
    import torch
    import torch.distributed as dist

    from lm_engine_b200.accelerator import Accelerator
    from lm_engine_b200.arguments import TrainingArgs
    from lm_engine_b200.data.synthetic import SyntheticBatchIterator
    from lm_engine_b200.distributed import wrap_model_container_for_distributed_training
    from lm_engine_b200.kernels import enable_kernels
    from lm_engine_b200.model_wrapper import get_model_container
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.optimization import get_optimizer_container, get_scheduler_container
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.train import train_step_without_pipeline_parallel
    from lm_engine_b200.train_utils import get_model_tflops, measured_peaks
    from lm_engine_b200.utils import disable_generation_cache

    cfg = training_config(a.model, a.seq, a.mbs, a.steps, ["fused_linear_cross_entropy"], None)
    cfg["mixed_precision_args"] = {"dtype": getattr(a, "dtype", "bf16")}
    env_world = int(os.environ.get("WORLD_SIZE", "1"))
    ep = env_world if a.model == "moe-ep8" and MOE[a.model][0] % env_world == 0 else 1
    cfg["distributed_args"]["expert_parallel_world_size"] = ep
    tp, ga = a.tp, a.ga
    if tp > 1:
        cfg["distributed_args"].update(tensor_parallel_world_size=tp, sequence_parallel=True,
                                       use_async_tensor_parallel=True)
    cp = a.cp
    if cp > 1:
        cfg["distributed_args"]["context_parallel_world_size"] = cp
        cfg["distributed_args"]["context_parallel_attention"] = a.cp_attention
    cfg["training_parameters"]["gradient_accumulation_steps"] = ga
    args = TrainingArgs(**cfg)
    d = args.distributed_args
    ProcessGroupManager(zero_stage=d.stage, expert_parallel_world_size=ep, tensor_parallel_world_size=tp,
                        use_async_tensor_parallel=tp > 1, context_parallel_world_size=cp,
                        context_parallel_load_balancing_method=d.context_parallel_load_balancing_method,
                        context_parallel_attention=d.context_parallel_attention)
    world = ProcessGroupManager.get_world_size()
    rank = ProcessGroupManager.get_global_rank()
    args.training_parameters.reset_training_parameters(ProcessGroupManager.get_data_loading_world_size())
    Accelerator.set_seed(args.random_args.seed)
    models = get_model_container(args)
    models, _ = wrap_model_container_for_distributed_training(args, models)
    opts = get_optimizer_container(args.optimizer_args.class_name, args.optimizer_args.class_args, models, None,
                                   max_grad_norm=1.0)
    ls = args.lr_scheduler_args
    scheds = get_scheduler_container(models, opts, ls.num_warmup_steps, 0, None, 10**6, ls.lr_decay_style,
                                     ls.lr_decay_factor, {})
    models.train()
    device = Accelerator.get_current_device()
    vocab = args.model_args.pretrained_config["vocab_size"]
    host_iter = SyntheticBatchIterator(vocab, a.seq, a.mbs, rank=ProcessGroupManager.get_data_loading_rank(),
                                       world=ProcessGroupManager.get_data_loading_world_size(), seed=1234)

    def step(loader):
        # metrics are averaged over the data-parallel ranks and read back every step, as in the reference's step
        return train_step_without_pipeline_parallel(models, opts, scheds, loader, ga, 1.0, reduce_metrics=True)

    def barrier():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    with disable_generation_cache(), enable_kernels(args.kernel_args.kernels):
        # ---- warm-up
        for _ in range(a.warmup):
            m = step(host_iter)
        first_loss = float(m["loss"]) if a.warmup else None
        # ---- phase 1: device-timed, inputs resident on the device
        resident = [{"text": next(host_iter)["text"].to(device)} for _ in range(a.steps * ga)]
        it = iter(resident)
        sampler = ClockSampler(torch.cuda.current_device())
        barrier()
        launches0 = _lib.launch_count
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            m = step(it)
        e1.record()
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        launches = _lib.launch_count - launches0
        dev_ms = e0.elapsed_time(e1)
        # ---- phase 2: end to end (pinned host batch -> device each step, loss read back each step)
        h2d = ga * a.mbs * (a.seq + 1) * 8
        barrier()
        t0 = time.perf_counter()
        losses = []
        for _ in range(a.steps):
            m = step(host_iter)
            losses.append(float(m["loss"]))        # device -> host read of the step's result
        barrier()
        e2e_s = time.perf_counter() - t0
    t = torch.tensor([dev_ms, e2e_s * 1e3], device=device, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    dp_world = ProcessGroupManager.get_data_loading_world_size()      # tensor-parallel ranks share their batches
    tokens = dp_world * ga * a.mbs * a.seq * a.steps
    value = tokens / (dev_ms * 1e-3)
    e2e_value = tokens / (e2e_ms * 1e-3)
    tfl = get_model_tflops(models[0].config, dp_world * ga * a.mbs, a.seq, d.gradient_checkpointing_method,
                           d.gradient_checkpointing_args)
    peaks = measured_peaks()
    status = _lib.read_status(clear=False)
    out = {
        "metric": "tokens/sec (whole job), pretraining step fwd+bwd+clip+AdamW", "value": value,
        "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": dev_ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": getattr(a, "dtype", "bf16"), "data": "synthetic uniform-random token ids, seeded random-init weights",
        "config": {"model": a.model if a.layers is None else f"{a.model}-{a.layers}layers",
                   "global_batch": dp_world * ga * a.mbs, "seq_len": a.seq,
                   "parallelism": f"fsdp2-zero3-dp{dp_world}" + (f"-ep{ep}" if ep > 1 else "")
                   + (f"-tp{tp}-sp-asynctp" if tp > 1 else "") + (f"-cp{cp}-{a.cp_attention}" if cp > 1 else ""),
                   "gradient_accumulation_steps": ga, "micro_batch_per_gpu": a.mbs, "gradient_checkpointing": "block",
                   "optimizer": "AdamW fp32 master+state", "l2": "working set per step >> 126 MB L2, no flush"},
        "tokens_per_sec_per_gpu": value / world,
        "model_tflops_per_gpu": tfl / (dev_ms * 1e-3 / a.steps) / world,
        "mfu_of_measured_sustained_peak": tfl / (dev_ms * 1e-3 / a.steps) / world / peaks["bf16_tflops_sustained"],
        "peaks_source": peaks["source"],
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / a.steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "loss_first": first_loss, "loss_last": losses[-1] if losses else None,
        "device_status": status[:4],
        "impl": "lm_engine_b200",
    }
    if world > 1 and tp == 1 and cp == 1:
        out["multi_gpu_check"] = multi_gpu_check(world, rank, device)
    ProcessGroupManager.destroy_process_groups()
    return out if rank == 0 else None


def multi_gpu_check(world: int, rank: int, device) -> dict:
    """Outside the timed region: one step of a small dense model (2 blocks, hidden 1024) sharded over all ranks
    (ZeRO-3: parameter gathers, the gradient reduce-scatter, the sharded norm) against the same global batch computed
    by every rank alone on replicated weights.  Both start from the same seeded weights; the mean loss and the global
    gradient norm of the two have to agree to bf16 accuracy."""
    import torch
    import torch.distributed as dist

    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.enums import GradientCheckpointingMethod
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.models import dense_config
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer

    seq = 1024
    cfg = dense_config(vocab_size=8192, hidden_size=1024, num_layers=2, num_attention_heads=8, num_key_value_heads=4,
                       intermediate_size=4096, head_dim=128, max_position_embeddings=seq).to_dict()
    tokens = torch.randint(0, 8192, (world, seq + 1), generator=torch.Generator().manual_seed(77)).to(device)
    res = {}
    for name, stage, batch in (("sharded", 3, tokens[rank:rank + 1]), ("replicated", 0, tokens)):
        w = ModelWrapperForPretraining(pretrained_config=cfg, micro_batch_size=batch.size(0), sequence_length=seq,
                                       efficient_initialization=True, dtype="bf16")
        eng = shard_model(w, stage=stage, dtype=torch.bfloat16, communication_dtype=None,
                          gradient_checkpointing_method=GradientCheckpointingMethod.block, seed=7)
        opt = ShardedOptimizer(eng, "TorchAdamW", {"lr": 1e-4, "weight_decay": 0.0, "betas": [0.9, 0.95],
                                                   "eps": 1e-10}, None, False, 1.0)
        opt.zero_grad()
        loss = w(batch, lm_loss_multiplier=1 / (batch.size(0) * seq))["loss"]
        loss.backward()
        norm = opt.step()
        t = torch.stack([loss.detach().float().reshape(()), norm.float().reshape(())])
        if stage == 3:
            dist.all_reduce(t[:1])
            t[0] /= world
        res[name] = t.tolist()
        del w, eng, opt
    return {"loss_sharded": res["sharded"][0], "loss_replicated": res["replicated"][0],
            "grad_norm_sharded": res["sharded"][1], "grad_norm_replicated": res["replicated"][1],
            "loss_abs_diff": abs(res["sharded"][0] - res["replicated"][0]),
            "grad_norm_rel_diff": abs(res["sharded"][1] - res["replicated"][1]) / max(res["replicated"][1], 1e-12)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODELS))
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--mbs", type=int, default=None, help="micro batch per GPU (default 2; 4 for the MoE models)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel group size (with sequence parallel)")
    ap.add_argument("--ga", type=int, default=1, help="gradient accumulation steps")
    ap.add_argument("--cp", type=int, default=1, help="context-parallel group size (the sequence is split over it)")
    ap.add_argument("--cp-attention", default="auto", choices=["auto", "ulysses", "gathered", "ring"],
                    help="context-parallel attention algorithm")
    ap.add_argument("--layers", type=int, default=None,
                    help="override the layer count (profiling captures on a small case; not a benchmark result)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"],
                    help="compute dtype of this repo's arm (the headline number is bf16; fp8 is an extra measurement)")
    a = ap.parse_args()
    global LAYERS_OVERRIDE
    LAYERS_OVERRIDE = a.layers
    if a.mbs is None:
        a.mbs = 4 if a.model in MOE else 2
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if a.gpus != world:
        if world == 1 and a.gpus > 1:
            # convenience: re-launch under torchrun
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", "29512", os.path.abspath(__file__)] + sys.argv[1:]
            sys.exit(subprocess.call(cmd))
    if world == 1 and a.impl == "reference":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("LOCAL_RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
    if a.impl == "reference":
        from baseline.reference_bench import run_reference

        out = run_reference(a, training_config, ClockSampler)
    else:
        out = run_ours(a)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
