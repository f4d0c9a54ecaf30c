"""Pipeline parallelism: schedule timetables (pure Python) and 2-rank gloo runs against a single process that
accumulates the same micro-batches."""

import numpy as np
import pytest
import torch

from .dist_utils import run_distributed

VOCAB, SEQ = 256, 16


@pytest.mark.parametrize("schedule,pp,stages,M", [
    ("GPipe", 2, 2, 4), ("GPipe", 4, 8, 3), ("1F1B", 2, 2, 4), ("1F1B", 4, 4, 8), ("1F1B", 4, 4, 2),
    ("Interleaved1F1B", 2, 4, 4), ("Interleaved1F1B", 4, 8, 8), ("Interleaved1F1B", 2, 4, 3),
    ("FlexibleInterleaved1F1B", 4, 12, 6), ("LoopedBFS", 2, 4, 4), ("InterleavedZeroBubble", 2, 4, 4)])
def test_timetable_is_complete_and_ordered(schedule, pp, stages, M):
    from lm_engine_b200.parallel.pipeline_parallel import B, F, Action, build_timetable, rank_orders

    orders = rank_orders(schedule, pp, stages, M)
    table = build_timetable(orders, stages)
    when = {}
    for t, tick in enumerate(table):
        for r, a in enumerate(tick):
            if a is not None:
                assert a.stage % pp == r and a not in when
                when[a] = t
    assert len(when) == 2 * stages * M
    for s in range(stages):
        for m in range(M):
            if s > 0:
                assert when[Action(F, s, m)] > when[Action(F, s - 1, m)]
                assert when[Action(B, s - 1, m)] > when[Action(B, s, m)]
            assert when[Action(B, s, m)] > when[Action(F, s, m)]


def test_1f1b_holds_fewer_activations_than_gpipe():
    from lm_engine_b200.parallel.pipeline_parallel import F, build_timetable, bubble_fraction, rank_orders

    def peak(schedule):
        table = build_timetable(rank_orders(schedule, 4, 4, 8), 4)
        live = best = 0
        for tick in table:
            a = tick[0]
            if a is not None:
                live += 1 if a.kind == F else -1
                best = max(best, live)
        return best, bubble_fraction(table)

    (p1, b1), (pg, bg) = peak("1F1B"), peak("GPipe")
    assert p1 == 4 and pg == 8
    assert 0 < bg < 0.5 and 0 < b1 < 0.5
    # interleaving shrinks the bubble
    t = build_timetable(rank_orders("Interleaved1F1B", 4, 8, 8), 8)
    assert bubble_fraction(t) < b1


def _cfg(moe=False):
    from lm_engine_b200.models import dense_config

    c = dense_config(vocab_size=VOCAB, hidden_size=32, num_layers=4, num_attention_heads=4, num_key_value_heads=2,
                     intermediate_size=64, max_position_embeddings=SEQ)
    return c


def _run(rank, world, pp, stages, schedule, M, mbs, steps, topo=None):
    from lm_engine_b200.arguments import TrainingArgs  # noqa: F401
    from lm_engine_b200.containers import ModelContainer
    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.parallel.pipeline_parallel import PipelineSchedule

    ProcessGroupManager(zero_stage=3, pipeline_parallel_world_size=pp, **(topo or {}))
    pr = ProcessGroupManager.get_pipeline_parallel_rank()
    ids = ProcessGroupManager.topology().pipeline_stage_ids(pr, stages)
    ws = [ModelWrapperForPretraining(pretrained_config=_cfg().to_dict(), micro_batch_size=mbs, sequence_length=SEQ,
                                     efficient_initialization=True, num_pipeline_stages=stages, pipeline_stage_id=i)
          for i in ids]
    mc = ModelContainer(ws)
    opts = []
    for w in ws:
        e = shard_model(w, stage=3, dtype=torch.float32, communication_dtype=None, seed=3)
        opts.append(ShardedOptimizer(e, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                       "eps": 1e-10}, None, False, 1.0))
    g = torch.Generator().manual_seed(9)
    data = torch.randint(0, VOCAB, (steps, M * mbs, SEQ + 1), generator=g)
    losses, norms = [], []
    if stages > 1:
        sched = PipelineSchedule(mc, schedule, stages, M, mbs, SEQ, torch.float32, False)
    for s in range(steps):
        for o in opts:
            o.zero_grad()
        if stages > 1:
            totals = sched.step(data[s])
            total = sum(w.engine.local_sumsq().clone() for w in ws)
            import torch.distributed as dist

            dist.all_reduce(total, group=ProcessGroupManager.get_pipeline_parallel_group())
            for o in opts:
                n = o.step(total_sumsq=total)
            losses.append(float(totals["loss"]) if totals is not None else None)
        else:
            acc = 0.0
            for mb in data[s].chunk(M):
                out = ws[0](mb, lm_loss_multiplier=1 / (mbs * SEQ))
                (out["loss"] / M).backward()
                acc += float(out["loss"].detach()) / M
            n = opts[0].step()
            losses.append(acc)
        norms.append(float(n))
    params = {}
    for w in ws:
        params.update({k: v.cpu().numpy().copy() for k, v in w.engine.full_state_dict().items()})
    return losses, norms, params


@pytest.mark.parametrize("stages,schedule,M", [(2, "1F1B", 4), (2, "GPipe", 3), (4, "Interleaved1F1B", 4)])
def test_two_pipeline_ranks_match_single_process(stages, schedule, M):
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager.destroy_process_groups()
    ref_losses, ref_norms, ref_params = _run(0, 1, 1, 1, None, M, 2, 2)
    ProcessGroupManager.destroy_process_groups()
    outs = run_distributed(_run, 2, 2, stages, schedule, M, 2, 2)
    last = outs[(stages - 1) % 2]
    np.testing.assert_allclose(last[0], ref_losses, rtol=1e-5)
    for o in outs:
        np.testing.assert_allclose(o[1], ref_norms, rtol=1e-4)
    merged = {}
    for o in outs:
        merged.update(o[2])
    assert set(merged) == set(ref_params)
    for k in ref_params:
        np.testing.assert_allclose(merged[k], ref_params[k], rtol=1e-4, atol=1e-6, err_msg=k)


@pytest.mark.parametrize("topo", [{"tensor_parallel_world_size": 2}, {"context_parallel_world_size": 2},
                                  {"context_parallel_world_size": 2, "context_parallel_attention": "ring"}, {}],
                         ids=["pp2-x-tp2", "pp2-x-cp2-ulysses", "pp2-x-cp2-ring", "pp2-x-dp2"])
def test_pipeline_composes_with_a_second_dimension_on_four_ranks(topo, tmp_path):
    """Two pipeline stages x (tensor | context | data) parallel 2 on 4 gloo ranks, 1F1B with 4 micro-batches, against
    one process: losses, gradient norms and the updated weights."""
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    from lm_engine_b200.models import build_model
    from lm_engine_b200.utils import SafeTensorsWeightsManager

    M, mbs, steps = 4, 2, 2
    dp = 1 if topo else 2
    # the same saved weights for every topology (a tensor-parallel rank would otherwise draw its own shard)
    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=3)
    torch.manual_seed(5)
    cfg = _cfg()
    weights = str(tmp_path / "weights")
    cfg.save_pretrained(weights)
    SafeTensorsWeightsManager.save_state_dict(build_model(cfg).state_dict(), weights)
    ProcessGroupManager.destroy_process_groups()
    ref_losses, ref_norms, ref_params = _run_composed(0, 1, 1, 1, None, M, mbs * dp, steps, {}, 1, weights)
    ProcessGroupManager.destroy_process_groups()
    outs = run_distributed(_run_composed, 4, 2, 2, "1F1B", M, mbs, steps, topo, dp, weights, timeout=600)
    last = [o for o in outs if o[0][0] is not None]
    assert last
    loss = [sum(o[0][s] for o in last) / len(last) for s in range(steps)]
    np.testing.assert_allclose(loss, ref_losses, rtol=2e-4)
    for o in outs:
        np.testing.assert_allclose(o[1], ref_norms, rtol=2e-3)
    if "tensor_parallel_world_size" in topo:
        return      # the engines hold tensor-parallel shards; the second step's loss and norm cover the update
    merged = {}
    for o in outs:
        merged.update(o[2])
    assert set(merged) == set(ref_params)
    for k in ref_params:
        np.testing.assert_allclose(merged[k], ref_params[k], rtol=2e-3, atol=2e-5, err_msg=k)


def _run_composed(rank, world, pp, stages, schedule, M, mbs, steps, topo, dp, weights):
    """`_run` on a pp x (tp | cp | dp) mesh from saved weights: data-parallel replicas take their slice of every
    micro-batch."""
    from lm_engine_b200.containers import ModelContainer
    from lm_engine_b200.distributed import shard_model
    from lm_engine_b200.model_wrapper import ModelWrapperForPretraining
    from lm_engine_b200.optimization.optimizer import ShardedOptimizer
    from lm_engine_b200.parallel.manager import ProcessGroupManager
    from lm_engine_b200.parallel.pipeline_parallel import PipelineSchedule

    import torch.distributed as dist

    ProcessGroupManager(zero_stage=3, pipeline_parallel_world_size=pp, **topo)
    pr = ProcessGroupManager.get_pipeline_parallel_rank()
    ids = ProcessGroupManager.topology().pipeline_stage_ids(pr, stages)
    ws = [ModelWrapperForPretraining(model_name=weights, micro_batch_size=mbs, sequence_length=SEQ,
                                     num_pipeline_stages=stages, pipeline_stage_id=i)
          for i in ids]
    mc = ModelContainer(ws)
    opts = []
    for w in ws:
        e = shard_model(w, stage=3, dtype=torch.float32, communication_dtype=None, seed=3)
        opts.append(ShardedOptimizer(e, "TorchAdamW", {"lr": 1e-3, "weight_decay": 0.1, "betas": [0.9, 0.95],
                                                       "eps": 1e-10}, None, False, 1.0))
    g = torch.Generator().manual_seed(9)
    data = torch.randint(0, VOCAB, (steps, M * mbs * dp, SEQ + 1), generator=g)
    dl_rank = ProcessGroupManager.get_data_loading_rank()
    sched = PipelineSchedule(mc, schedule, stages, M, mbs, SEQ, torch.float32, False) if stages > 1 else None
    losses, norms = [], []
    for s in range(steps):
        for o in opts:
            o.zero_grad()
        # micro-batch m of the single-process run is rows [m * mbs * dp, (m + 1) * mbs * dp): this replica's share
        mine = data[s].view(M, dp, mbs, SEQ + 1)[:, dl_rank].reshape(M * mbs, SEQ + 1)
        if sched is None:
            acc = 0.0
            for mb in mine.chunk(M):
                out = ws[0](mb, lm_loss_multiplier=1 / (mbs * SEQ))
                (out["loss"] / M).backward()
                acc += float(out["loss"].detach()) / M
            n = opts[0].step()
            losses.append(acc)
            norms.append(float(n))
            continue
        totals = sched.step(mine)
        total = sum(w.engine.local_sumsq().clone() for w in ws)
        dist.all_reduce(total, group=ProcessGroupManager.get_pipeline_parallel_group())
        for o in opts:
            n = o.step(total_sumsq=total)
        losses.append(float(totals["loss"]) if totals is not None else None)
        norms.append(float(n))
    params = {}
    for w in ws:
        params.update({k: v.cpu().numpy().copy() for k, v in w.engine.full_state_dict().items()})
    return losses, norms, params
