"""Reference arm of ``bench.py``: runs the unmodified open-lm-engine/lm-engine package found under ``baseline/_ref``
through its own public API (``TrainingArgs`` -> ``ProcessGroupManager`` -> ``get_model_container`` ->
``wrap_model_container_for_distributed_training`` -> ``get_optimizer_container`` / ``get_scheduler_container`` ->
``train_step_without_pipeline_parallel``) on the same model / batch / sequence / ZeRO-3 / block-checkpointing
configuration, with its stock kernels (``flash_attention_2``; everything else ATen / cuBLAS / NCCL).

Nothing of this repository's engine is imported on that path; only the timing harness (CUDA events, clock sampling,
synthetic token batches) is shared.  The reference needs a tokenizer directory, so a minimal word-level tokenizer is
written to a temporary directory (the model's vocabulary size comes from the config, not from the tokenizer).
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import time
from contextlib import nullcontext

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}


def _make_tokenizer_dir() -> str:
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    path = os.path.join(tempfile.gettempdir(), f"lme_ref_tok_{os.getuid()}")
    done = os.path.join(path, "tokenizer.json")
    if os.path.exists(done):
        return path
    if int(os.environ.get("LOCAL_RANK", "0")) != 0:
        # one rank per node writes the files (published by an atomic rename); the others wait for them
        for _ in range(600):
            if os.path.exists(done):
                return path
            time.sleep(0.1)
        raise RuntimeError("tokenizer files were not written by local rank 0")
    # special-token ids must equal the model config's bos / eos / pad ids (0 / 1 / 2): the reference asserts it
    vocab = {"<bos>": 0, "<eos>": 1, "<pad>": 2, "<unk>": 3, "a": 4, "b": 5}
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="<eos>", pad_token="<pad>",
                                   bos_token="<bos>")
    tmp = tempfile.mkdtemp(prefix="lme_ref_tok_build_")
    fast.save_pretrained(tmp)
    try:
        os.replace(tmp, path)
    except OSError:          # another launcher got there first
        if not os.path.exists(done):
            raise
    return path


class _Batches:
    """Seeded uniform-random ``[mbs, seq + 1]`` int64 batches, pinned on the host or pre-staged on the device."""

    def __init__(self, vocab: int, seq: int, mbs: int, rank: int, world: int, device=None) -> None:
        import torch

        self.torch, self.vocab, self.seq, self.mbs, self.rank, self.world = torch, vocab, seq, mbs, rank, world
        self.cursor, self.device = 0, device

    def __iter__(self):
        return self

    def __next__(self):
        torch = self.torch
        g = torch.Generator().manual_seed(1234 * 1_000_003 + self.cursor + self.rank * self.mbs)
        t = torch.randint(0, self.vocab, (self.mbs, self.seq + 1), generator=g).pin_memory()
        self.cursor += self.mbs * self.world
        return {"text": t if self.device is None else t.to(self.device)}


def run_reference(a, training_config, ClockSampler) -> dict | None:
    if not os.path.isdir(os.path.join(_REF, "lm_engine")):
        return _unavailable("baseline/_ref/lm_engine is missing (offline install did not succeed)")
    sys.path.insert(0, _REF)
    try:
        import torch
        import torch.distributed as dist

        from lm_engine.arguments import TrainingArgs
        from lm_engine.distributed import wrap_model_container_for_distributed_training
        from lm_engine.enums import TuningMethod
        from lm_engine.kernels import enable_kernels
        from lm_engine.model_wrapper import get_model_container
        from lm_engine.optimization import get_optimizer_container, get_scheduler_container
        from lm_engine.parallel.manager import ProcessGroupManager
        from lm_engine.train import train_step_without_pipeline_parallel
        from lm_engine.accelerator import Accelerator
        from lm_engine.utils import disable_generation_cache
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference import failed: {type(e).__name__}: {e}")

    try:
        tok_dir = _make_tokenizer_dir()
        # The reference's stock path with no kernel flag (attention through scaled_dot_product_attention) is its
        # fastest configuration on B200 with the packages of this image: 818 ms per Llama-3-8B step on one GPU
        # against 881 ms with `flash_attention_2` (what its YAMLs enable, flash-attn 2.8) and 866 ms with the QuACK
        # flags added; LME_REF_KERNELS selects the others.
        kernels = [k for k in os.environ.get("LME_REF_KERNELS", "").split(",") if k]
        cfg = training_config(a.model, a.seq, a.mbs, a.steps, kernels, tok_dir)
        cfg["distributed_args"].pop("expert_parallel_world_size", None)
        # With this torch version the reference's default (non-reentrant) block checkpointing raises CheckpointError:
        # FSDP-2 casts the rotary cos/sin inputs of a block to bf16 in forward but skips that cast when the block is
        # recomputed, and the non-reentrant checkpoint compares tensor metadata.  The reference's own
        # `use_reentrant` knob selects the checkpoint implementation without that comparison.
        cfg["distributed_args"]["gradient_checkpointing_args"] = {
            "use_reentrant": os.environ.get("LME_REF_REENTRANT", "1") == "1"}
        tp, ga = getattr(a, "tp", 1), getattr(a, "ga", 1)
        if tp > 1:      # the reference's async TP is an inductor pass (needs torch.compile): plain TP + SP here
            cfg["distributed_args"].update(tensor_parallel_world_size=tp, sequence_parallel=True)
        cfg["training_parameters"]["gradient_accumulation_steps"] = ga
        args = TrainingArgs(**cfg)
        d = args.distributed_args
        ProcessGroupManager(zero_stage=d.stage, tensor_parallel_world_size=tp)
        world = ProcessGroupManager.get_world_size()
        rank = ProcessGroupManager.get_global_rank()
        args.training_parameters.reset_training_parameters(
            data_loading_world_size=ProcessGroupManager.get_data_loading_world_size())
        Accelerator.set_seed(args.random_args.seed)
        models = get_model_container(args, efficient_initialization=True, keep_in_fp32=True)
        models, _ = wrap_model_container_for_distributed_training(args, models)
        opts = get_optimizer_container(
            optimizer_class_name=args.optimizer_args.class_name, optimizer_class_args=args.optimizer_args.class_args,
            model_container=models, params_group_method=None, use_optimizer_with_backward_hook=False)
        ls = args.lr_scheduler_args
        scheds = get_scheduler_container(
            model_container=models, optimizer_container=opts, num_warmup_steps=ls.num_warmup_steps,
            num_constant_steps=0, num_decay_steps=None, num_training_steps=10**6, lr_decay_style=ls.lr_decay_style,
            lr_decay_factor=ls.lr_decay_factor, extra_lr_scheduler_args={}, use_optimizer_with_backward_hook=False)
        models.train()
        device = torch.device("cuda", torch.cuda.current_device())
        vocab = args.model_args.pretrained_config["vocab_size"]
        dl_rank = ProcessGroupManager.get_data_loading_rank()
        dl_world = ProcessGroupManager.get_data_loading_world_size()
        host_iter = _Batches(vocab, a.seq, a.mbs, dl_rank, dl_world)

        def step(loader):
            return train_step_without_pipeline_parallel(
                model_container=models, optimizer_container=opts, lr_scheduler_container=scheds,
                train_dataloader=loader, gradient_clipping=1.0, forward_context=nullcontext,
                backward_context=nullcontext, sync_every_gradient_accumulation_step=False,
                micro_batch_size=a.mbs, gradient_accumulation_steps=ga, sequence_length=a.seq,
                tuning_method=TuningMethod.pretraining)

        def barrier():
            dist.barrier()
            torch.cuda.synchronize()

        # the reference's own train() runs its loop inside these two context managers
        with disable_generation_cache(), enable_kernels(args.kernel_args.kernels):
            for _ in range(a.warmup):
                m = step(host_iter)
            first_loss = float(m["loss"]) if a.warmup else None
            resident = _Batches(vocab, a.seq, a.mbs, dl_rank, dl_world, device=device)
            resident.cursor = host_iter.cursor
            staged = iter([next(resident) for _ in range(a.steps * ga)])
            host_iter.cursor = resident.cursor        # the end-to-end phase reads batches the model has not seen
            sampler = ClockSampler(torch.cuda.current_device())
            barrier()
            if rank == 0:
                sampler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.steps):
                m = step(staged)
            e1.record()
            barrier()
            clocks = sampler.stop() if rank == 0 else None
            dev_ms = e0.elapsed_time(e1)
            barrier()
            t0 = time.perf_counter()
            losses = []
            for _ in range(a.steps):
                m = step(host_iter)
                losses.append(float(m["loss"]))
            barrier()
            e2e_s = time.perf_counter() - t0
        t = torch.tensor([dev_ms, e2e_s * 1e3], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
        tokens = dl_world * ga * a.mbs * a.seq * a.steps
        out = {
            "impl": "reference", "metric": "tokens/sec (whole job), pretraining step fwd+bwd+clip+AdamW",
            "value": tokens / (dev_ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": dev_ms / a.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random token ids, seeded random-init weights",
            "config": {"model": a.model, "global_batch": dl_world * ga * a.mbs, "seq_len": a.seq,
                       "parallelism": f"fsdp2-zero3-dp{dl_world}" + (f"-tp{tp}-sp" if tp > 1 else ""),
                       "gradient_accumulation_steps": ga, "micro_batch_per_gpu": a.mbs,
                       "gradient_checkpointing": "block", "kernels": kernels,
                       "l2": "working set per step >> 126 MB L2, no flush"},
            "tokens_per_sec_per_gpu": tokens / (dev_ms * 1e-3) / world, "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms / a.steps,
                    "h2d_bytes_per_step": a.mbs * (a.seq + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "loss_first": first_loss, "loss_last": losses[-1] if losses else None,
        }
        try:
            ProcessGroupManager.destroy_process_groups()
        except Exception:  # noqa: BLE001
            pass
        return out if rank == 0 else None
    except Exception as e:  # noqa: BLE001
        import traceback

        tb = traceback.format_exc().strip().splitlines()
        return _unavailable(f"reference run failed: {type(e).__name__}: {e} | {tb[-3] if len(tb) > 2 else ''}")


if __name__ == "__main__":
    print(json.dumps(_unavailable("run through bench.py --impl reference")))
