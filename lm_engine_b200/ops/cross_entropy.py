"""Cross entropy over bf16 logits with fp32 statistics; the gradient overwrites the logits in place.

Replaces ``F.cross_entropy(logits.float(), labels, reduction="sum")`` (lm_engine/loss.py:90-99) and, with a process
group, torch's ``loss_parallel`` (lm_engine/train.py:385-386): each tensor-parallel rank passes its vocabulary slice,
the three per-row statistics (max, sum-exp, target logit) are combined across ranks, and every rank rewrites its own
slice with ``(softmax - onehot) * upstream``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _lib


class _CrossEntropySum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index, vocab_start, group):
        V = logits.size(-1)
        x = logits.reshape(-1, V)
        if x.stride(1) != 1:
            x = x.contiguous()
        lab = labels.reshape(-1).to(torch.int64).contiguous()
        T = x.size(0)
        stats = torch.empty((3, T), dtype=torch.float32, device=x.device)
        lib = _lib.cuda_lib()
        _lib.check(lib.lme_ce_stats(x.data_ptr(), x.stride(0), lab.data_ptr(), stats[0].data_ptr(),
                                    stats[1].data_ptr(), stats[2].data_ptr(), T, V, vocab_start, _lib.stream_ptr()),
                   "lme_ce_stats")
        _lib.count_launch()
        row_max, row_sum, tgt = stats[0], stats[1], stats[2]
        if group is not None and dist.get_world_size(group) > 1:
            gmax = row_max.clone()
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            row_sum = row_sum * torch.exp(row_max - gmax)
            packed = torch.stack((row_sum, tgt))
            dist.all_reduce(packed, group=group)
            row_sum, tgt, row_max = packed[0], packed[1], gmax
        lse = row_max + torch.log(row_sum)
        valid = lab != ignore_index
        loss = torch.where(valid, lse - tgt, torch.zeros_like(lse)).sum()
        ctx.save_for_backward(x, lab, lse)
        ctx.meta = (V, vocab_start, ignore_index, logits.shape)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x, lab, lse = ctx.saved_tensors
        V, v0, ignore_index, shape = ctx.meta
        # the upstream scalar stays on the device: no host synchronisation between forward and backward
        scale_dev = dloss.reshape(1).float().contiguous()
        _lib.check(_lib.cuda_lib().lme_ce_grad(x.data_ptr(), x.stride(0), lab.data_ptr(), lse.data_ptr(), x.size(0),
                                               V, v0, 1.0, scale_dev.data_ptr(), ignore_index, _lib.stream_ptr()),
                   "lme_ce_grad")
        _lib.count_launch()
        return x.view(shape), None, None, None, None


def cross_entropy_sum(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, vocab_start: int = 0,
                      group=None) -> torch.Tensor:
    """Sum over tokens of the CE loss (fp32 scalar).  On CUDA bf16 the backward reuses the logits' storage, so the
    caller must not read the logits after ``backward``."""
    if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.size(-1) % 8 == 0:
        return _CrossEntropySum.apply(logits, labels, ignore_index, vocab_start, group)
    if group is not None and dist.get_world_size(group) > 1:
        return _vocab_parallel_reference(logits, labels, ignore_index, vocab_start, group)
    return F.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), labels.reshape(-1), reduction="sum",
                           ignore_index=ignore_index)


class _AllReduceSumFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def _vocab_parallel_reference(logits, labels, ignore_index, vocab_start, group):
    """Differentiable PyTorch statement of the vocab-parallel loss (CPU / gloo path and oracle)."""
    V = logits.size(-1)
    x = logits.reshape(-1, V).float()
    lab = labels.reshape(-1)
    gmax = x.max(-1).values.detach().clone()
    dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    sumexp = _AllReduceSumFn.apply(torch.exp(x - gmax[:, None]).sum(-1), group)
    local = lab - vocab_start
    inside = (local >= 0) & (local < V)
    tgt = torch.where(inside, x.gather(1, local.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(gmax))
    tgt = _AllReduceSumFn.apply(tgt, group)
    loss = gmax + torch.log(sumexp) - tgt
    return torch.where(lab != ignore_index, loss, torch.zeros_like(loss)).sum()
