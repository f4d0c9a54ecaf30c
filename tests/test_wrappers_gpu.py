"""Finetuning wrapper on the GPU in bf16: a packed (padding-free) batch gives the summed loss of its documents run
one by one - through the library varlen attention by default and through the tcgen05 attention kernels under the
switch - and gradients reach every parameter."""

import pytest
import torch

pytestmark = pytest.mark.gpu

VOCAB = 256


def _cfg(head_dim):
    from lm_engine_b200.models import dense_config

    return dense_config(vocab_size=VOCAB, hidden_size=4 * head_dim, num_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, intermediate_size=256, head_dim=head_dim,
                        max_position_embeddings=256).to_dict()


@pytest.mark.parametrize("own,head_dim", [(False, 64), (True, 128)])
def test_packed_finetuning_batch_equals_documents_one_by_one(own, head_dim, monkeypatch):
    from lm_engine_b200.model_wrapper.finetuning import ModelWrapperForFinetuning
    from lm_engine_b200.ops import _lib
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    if own:
        monkeypatch.setenv("LME_ATTENTION", "own")
    else:
        monkeypatch.delenv("LME_ATTENTION", raising=False)
    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=0)
    torch.manual_seed(1)
    cfg = _cfg(head_dim)
    packed = ModelWrapperForFinetuning(pretrained_config=cfg, use_padding_free_transformer=True, dtype="bf16")
    plain = ModelWrapperForFinetuning(pretrained_config=cfg, dtype="bf16")
    packed, plain = packed.cuda(), plain.cuda()
    plain.model.load_state_dict(packed.model.state_dict())
    lens = [70, 129, 33]
    ids = torch.randint(0, VOCAB, (sum(lens),), device="cuda")
    cu = torch.tensor([0, 70, 199, 232], dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).cuda()
    out = packed({"input_ids": ids, "labels": ids.clone(), "cu_seqlens": cu, "max_seqlen": torch.tensor(129),
                  "position_ids": pos})
    total = 0
    for a, b in zip([0, 70, 199], [70, 199, 232]):
        d = ids[a:b][None]
        total = total + plain({"input_ids": d, "attention_mask": torch.ones_like(d), "labels": d.clone()})["loss"]
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    torch.testing.assert_close(out["loss"].float(), total.float(), rtol=2e-2, atol=2e-2)
    out["loss"].backward()
    assert all(p.grad is not None and torch.isfinite(p.grad.float()).all() for p in packed.model.parameters())
