"""Sparse mixture-of-experts MLP: softmax/top-k router (either order), per-expert SwiGLU/MLP on tokens grouped by
expert, optional shared expert (with sigmoid gate), switch + z auxiliary loss
(lm_engine/modeling_utils/mlp_blocks/moe/module.py:38-355, experts.py:59-236, lm_engine/loss.py:104-127).

Parallel layouts:

* tensor parallel: expert weights split on the intermediate dimension, tokens replicated over the TP group
  (the reference's layout);
* expert parallel (extension): experts split over the ``ep`` group, tokens travel to their experts' owners by
  all-to-all and come back weighted by the router probabilities.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...ops.moe import all_to_all_rows, expert_histogram, grouped_linear
from ...parallel import tp_comm
from ...parallel.manager import ProcessGroupManager
from ...parameter import (
    mark_parameter_as_initialized,
    mark_parameter_as_mup_learning_rate,
    mark_parameter_as_no_weight_decay,
    mark_tp_shard,
)
from ...utils import divide_if_divisible
from ..aux_loss import add_aux_loss
from ..config import MoEArgs
from .activations import GLUActivation, get_activation_function, is_glu, sigmoid
from .dropout import Dropout
from .init_utils import std_for_linear
from .linear import ColumnParallelLinear, ParameterizedLinear, ReplicatedLinear, RowParallelLinear


class Experts(nn.Module):
    """``weight [E_local, out_local, in_local]`` (+ ``bias [E_local, out_local]``)."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool, std: float | None,
                 tp_dim: int | None) -> None:
        super().__init__()
        tp = ProcessGroupManager.get_tensor_parallel_world_size()
        ep = ProcessGroupManager.get_expert_parallel_world_size()
        self.global_num_experts = num_experts
        self.num_experts = divide_if_divisible(num_experts, ep, "num_experts must be divisible by the EP world size")
        self.std = std
        if tp_dim == 1:
            out_features = divide_if_divisible(out_features, tp)
        elif tp_dim == 2:
            in_features = divide_if_divisible(in_features, tp)
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(self.num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(self.num_experts, out_features)) if add_bias else None
        if tp > 1:
            assert not add_bias
            mark_tp_shard(self.weight, tp_dim)
        if ep > 1:
            self.weight.ep_shard_dim = 0
            if self.bias is not None:
                self.bias.ep_shard_dim = 0
        mark_parameter_as_no_weight_decay(self.bias)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        if self.weight.is_meta:
            return
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()
        mark_parameter_as_initialized(self.weight)
        mark_parameter_as_initialized(self.bias)

    def forward(self, x: torch.Tensor, counts: list[int]) -> torch.Tensor:
        return grouped_linear(x, self.weight, counts, self.bias)

    def extra_repr(self) -> str:
        return f"num_experts={self.num_experts}, in_features={self.in_features}, out_features={self.out_features}"


class MoE(nn.Module):
    def __init__(self, hidden_size: int, config: MoEArgs, init_method: str, initializer_range: float,
                 m_width: float | None, num_layers: int, use_depth_scaled_init: bool,
                 use_padding_free_transformer: bool = False, sequence_parallel: bool = False) -> None:
        super().__init__()
        self.hidden_size, self.num_experts, self.top_k = hidden_size, config.num_experts, config.num_experts_per_tok
        self.intermediate_size = config.intermediate_size
        self.shared_intermediate_size = config.shared_intermediate_size
        self.normalized_topk = config.normalized_topk
        self.use_padding_free_transformer = use_padding_free_transformer
        self.sequence_parallel = sequence_parallel
        self.tp_world_size = ProcessGroupManager.get_tensor_parallel_world_size()
        self.ep_world_size = ProcessGroupManager.get_expert_parallel_world_size()
        self.is_glu = is_glu(config.activation_function)
        I = config.intermediate_size
        up_std = std_for_linear(initializer_range, init_method, m_width, hidden_size, num_layers, False)
        down_std = std_for_linear(initializer_range, init_method, m_width, I, num_layers, use_depth_scaled_init)
        self.gate = ReplicatedLinear(hidden_size, self.num_experts, bias=False, std=up_std)
        if config.shared_expert_gating:
            assert self.shared_intermediate_size is not None
            self.shared_expert_gate = ParameterizedLinear(hidden_size, 1, bias=False, std=up_std)
        else:
            self.shared_expert_gate = None
        self.c_fc = Experts(self.num_experts, hidden_size, 2 * I if self.is_glu else I, config.add_bias, up_std, 1)
        if self.shared_intermediate_size is not None:
            SI = self.shared_intermediate_size
            self.c_fc_shared = ColumnParallelLinear(hidden_size, 2 * SI if self.is_glu else SI, bias=config.add_bias,
                                                    std=up_std)
        self.act = get_activation_function(config.activation_function)
        self.c_proj = Experts(self.num_experts, I, hidden_size, config.add_bias, down_std, 2)
        if self.shared_intermediate_size is not None:
            self.c_proj_shared = RowParallelLinear(
                self.shared_intermediate_size, hidden_size, bias=config.add_bias,
                std=std_for_linear(initializer_range, init_method, m_width, self.shared_intermediate_size,
                                   num_layers, use_depth_scaled_init))
            # the shared expert's partial sums are reduced together with the routed experts' below
            self.c_proj_shared.tp_world_size_for_reduce = self.c_proj_shared.tp_world_size
        self.dropout = Dropout(config.dropout)
        for p in (self.gate.weight, self.c_fc.weight, self.c_proj.weight):
            mark_parameter_as_mup_learning_rate(p)
        if self.shared_intermediate_size is not None:
            mark_parameter_as_mup_learning_rate(self.c_fc_shared.weight)
            mark_parameter_as_mup_learning_rate(self.c_proj_shared.weight)

    # ------------------------------------------------------------------ routing
    def _topk(self, x: torch.Tensor):
        if self.top_k == 1:
            return x.max(dim=-1, keepdim=True)
        return x.topk(self.top_k, dim=-1)

    def _route(self, x: torch.Tensor):
        logits = self.gate(x)
        from ...ops.moe import topk_softmax, topk_softmax_eligible

        if topk_softmax_eligible(logits, self.top_k):
            w, sel = topk_softmax(logits, self.top_k, self.normalized_topk)
            return logits, w, sel
        if self.normalized_topk:
            w, sel = self._topk(logits)
            w = F.softmax(w.float(), dim=-1).type_as(x)
        else:
            w = F.softmax(logits.float(), dim=-1).type_as(x)
            w, sel = self._topk(w)
        return logits, w, sel

    # ------------------------------------------------------------------ experts
    def _experts(self, x: torch.Tensor, weights: torch.Tensor, selected: torch.Tensor):
        T = x.size(0)
        if (self.ep_world_size == 1 and self._grouped_kernels(x) and x.size(1) % 8 == 0
                and self.num_experts <= 1024 and selected.numel() > 0):
            # Device-only path: padded per-expert layout from a counting sort of the selection (three small kernels),
            # one scatter kernel, two grouped tcgen05 GEMMs over all experts (SwiGLU fused into the first), one
            # gather-reduce kernel for the weighted combine.  No per-expert launches, no atomics, no host
            # synchronisation on the routing result.
            from ...ops.moe import GroupLayout, combine_tokens, dispatch_tokens

            layout = GroupLayout.from_selection(selected, self.num_experts)
            y_pad = self._grouped_mlp_padded(dispatch_tokens(x, layout), layout)
            return combine_tokens(y_pad, weights.to(x.dtype), layout), layout.freq
        if self.ep_world_size > 1 and self._grouped_kernels(x) and not self.use_padding_free_transformer:
            # Expert parallel on peer memory: rows are pushed into / pulled from the owners' symmetric slabs by
            # kernels, the counts stay on the devices, the experts run as two grouped GEMMs on the landed rows.
            from ...parallel import expert_exchange

            group = ProcessGroupManager.get_expert_parallel_group()
            if expert_exchange.eligible(x, selected, self.num_experts, group):
                return expert_exchange.expert_parallel_mlp(x, weights, selected, self.num_experts, group,
                                                           self._grouped_mlp_padded)
        with torch.no_grad():
            sorted_experts, order = selected.flatten().sort()
            freq = expert_histogram(sorted_experts, self.num_experts)
        token = order // self.top_k
        gates = weights.flatten()[order]
        xs = x[token]
        if self.ep_world_size > 1:
            ys = self._expert_parallel(xs, freq)
        else:
            counts = freq.tolist()
            ys = self.c_proj(self.act(self.c_fc(xs, counts)), counts)
        ys = ys * gates.unsqueeze(-1)
        out = torch.zeros((T, self.hidden_size), dtype=ys.dtype, device=ys.device).index_add(0, token, ys)
        return out, freq

    def _grouped_kernels(self, xs: torch.Tensor) -> bool:
        from ...ops.moe import grouped_kernels_eligible

        return (self.c_fc.bias is None and self.c_proj.bias is None
                and grouped_kernels_eligible(xs, self.c_fc.weight, self.c_proj.weight))

    def _grouped_mlp_padded(self, x_pad: torch.Tensor, layout) -> torch.Tensor:
        from ...ops.moe import grouped_linear_padded

        fuse = isinstance(self.act, GLUActivation) and self.act.is_swiglu
        h = grouped_linear_padded(x_pad, self.c_fc.weight, layout, swiglu=fuse,
                                  dgrad_out=getattr(layout, "input_grad_buffer", None))
        if not fuse:
            h = self.act(h)
        return grouped_linear_padded(h, self.c_proj.weight, layout, out=getattr(layout, "output_buffer", None))

    def _grouped_mlp(self, xs: torch.Tensor, sorted_experts: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
        """Rows already sorted by expert (expert-parallel receive side)."""
        from ...ops.moe import GroupLayout

        layout = GroupLayout(sorted_experts, freq)
        return layout.gather(self._grouped_mlp_padded(layout.scatter(xs), layout))

    def _expert_parallel(self, xs: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
        """Tokens (sorted by global expert id) -> owners of the experts -> local grouped MLP -> back."""
        group = ProcessGroupManager.get_expert_parallel_group()
        ep, local_e = self.ep_world_size, self.c_fc.num_experts
        # counts[r, e]: tokens rank r sends to (global) expert e
        all_freq = [torch.empty_like(freq) for _ in range(ep)]
        dist.all_gather(all_freq, freq, group=group)
        counts = torch.stack(all_freq).tolist()
        me = dist.get_rank(group)
        send = [sum(counts[me][j * local_e:(j + 1) * local_e]) for j in range(ep)]
        recv = [sum(counts[src][me * local_e:(me + 1) * local_e]) for src in range(ep)]
        got = all_to_all_rows(xs, send, recv, group)
        # received rows are ordered (source rank, local expert); regroup by local expert
        seg = [counts[src][me * local_e + e] for src in range(ep) for e in range(local_e)]
        pieces = list(got.split(seg, dim=0))
        by_expert = [pieces[src * local_e + e] for e in range(local_e) for src in range(ep)]
        per_expert = [sum(counts[src][me * local_e + e] for src in range(ep)) for e in range(local_e)]
        h = torch.cat(by_expert, dim=0) if by_expert else got
        if self._grouped_kernels(h) and h.size(0) > 0:
            counts_t = torch.tensor(per_expert, device=h.device)
            ids = torch.repeat_interleave(torch.arange(local_e, device=h.device), counts_t, output_size=h.size(0))
            h = self._grouped_mlp(h, ids, counts_t)
        else:
            h = self.c_proj(self.act(self.c_fc(h, per_expert)), per_expert)
        # back to (source rank, local expert) order and home
        seg2 = [counts[src][me * local_e + e] for e in range(local_e) for src in range(ep)]
        back = list(h.split(seg2, dim=0))
        by_src = [back[e * ep + src] for src in range(ep) for e in range(local_e)]
        h = torch.cat(by_src, dim=0) if by_src else h
        return all_to_all_rows(h, recv, send, group)

    def _shared(self, x: torch.Tensor) -> torch.Tensor:
        g = self.shared_expert_gate(x) if self.shared_expert_gate is not None else None
        # tokens are already replicated over TP here: run the shards locally, reduce with the routed output
        h = ops.linear(x, self.c_fc_shared.weight, self.c_fc_shared.bias)
        h = ops.linear(self.act(h), self.c_proj_shared.weight, None)
        if self.c_proj_shared.bias is not None:
            h = h + self.c_proj_shared.bias / self.tp_world_size
        return h if g is None else h * sigmoid(g)

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x = x.reshape(-1, self.hidden_size)
        sdim = 0
        if self.tp_world_size > 1:
            x = (tp_comm.gather_from_sequence_parallel(x, sdim) if self.sequence_parallel
                 else tp_comm.copy_to_tensor_parallel(x))
        logits, weights, selected = self._route(x)
        out, freq = self._experts(x, weights, selected)
        if self.shared_intermediate_size is not None:
            out = out + self._shared(x)
        if self.tp_world_size > 1:
            out = (tp_comm.scatter_to_sequence_parallel(out, sdim) if self.sequence_parallel
                   else tp_comm.reduce_from_tensor_parallel(out))
        out = out.reshape(*shape[:-1], self.hidden_size)
        out = self.dropout(out)
        add_aux_loss(self._switch_loss(logits, freq) if self.training else 0)
        return out

    def _switch_loss(self, logits: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
        """``E * sum_e p_e f_e + 0.1 * mean(logsumexp(logits)^2)`` with L1-normalised summed probabilities ``p`` and
        (data-parallel summed) token counts ``f``."""
        logits = logits.reshape(-1, logits.size(-1))
        probs = torch.softmax(logits, dim=-1)
        acc = probs.sum(0)
        f = freq.float()
        dp = ProcessGroupManager.get_data_parallel_group()
        if dp is not None:
            f = f.clone()
            dist.all_reduce(f, group=dp)
        switch = logits.size(1) * (F.normalize(acc, p=1, dim=0) * F.normalize(f, p=1, dim=0)).sum()
        z = (torch.logsumexp(logits, dim=-1) ** 2).mean()
        return (switch + 0.1 * z).type_as(logits)

    def get_num_active_parameters(self) -> int:
        n = sum(p.numel() for p in self.parameters())
        for mod in (self.c_fc, self.c_proj):
            for p in mod.parameters():
                n -= p.numel()
                n += p.numel() * self.top_k // self.global_experts(mod)
        return n

    @staticmethod
    def global_experts(mod: Experts) -> int:
        return mod.num_experts
