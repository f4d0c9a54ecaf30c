"""Finetuning and distillation wrappers against plain PyTorch formulas on the same logits."""

import torch
import torch.nn.functional as F

VOCAB, SEQ = 128, 16


def _cfg(hidden=32):
    from lm_engine_b200.models import dense_config

    return dense_config(vocab_size=VOCAB, hidden_size=hidden, num_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, intermediate_size=64, max_position_embeddings=SEQ)


def _pgm():
    from lm_engine_b200.parallel.manager import ProcessGroupManager

    ProcessGroupManager.destroy_process_groups()
    ProcessGroupManager(zero_stage=0)


def test_finetuning_loss_shifts_and_masks():
    from lm_engine_b200.model_wrapper.finetuning import ModelWrapperForFinetuning

    _pgm()
    torch.manual_seed(0)
    w = ModelWrapperForFinetuning(pretrained_config=_cfg().to_dict())
    ids = torch.randint(0, VOCAB, (2, SEQ))
    labels = ids.clone()
    labels[0, :5] = -100
    mask = torch.ones_like(ids)
    mask[1, :3] = 0  # left padding
    labels[1, :3] = -100
    n = int((labels[:, 1:] != -100).sum())
    out = w({"input_ids": ids, "attention_mask": mask, "labels": labels}, lm_loss_multiplier=1 / n)
    from lm_engine_b200.models import AttentionMaskInfo

    logits = w.model(input_ids=ids, attention_mask_info=AttentionMaskInfo(attention_mask=mask)).logits.float()
    want = F.cross_entropy(logits[:, :-1].reshape(-1, VOCAB), labels[:, 1:].reshape(-1), ignore_index=-100)
    torch.testing.assert_close(out["loss"], want, rtol=1e-5, atol=1e-5)
    out["loss"].backward()
    assert all(p.grad is not None for p in w.model.parameters())


def test_finetuning_packed_batch_does_not_cross_documents():
    from lm_engine_b200.model_wrapper.finetuning import ModelWrapperForFinetuning

    _pgm()
    torch.manual_seed(1)
    w = ModelWrapperForFinetuning(pretrained_config=_cfg().to_dict(), use_padding_free_transformer=True)
    lens = [7, 9]
    ids = torch.randint(0, VOCAB, (sum(lens),))
    cu = torch.tensor([0, 7, 16], dtype=torch.int32)
    pos = torch.cat([torch.arange(l) for l in lens])
    out = w({"input_ids": ids, "labels": ids.clone(), "cu_seqlens": cu, "max_seqlen": torch.tensor(9),
             "position_ids": pos})
    # each document alone, padded-free, gives the same summed loss
    w2 = ModelWrapperForFinetuning(pretrained_config=_cfg().to_dict())
    w2.model.load_state_dict(w.model.state_dict())
    total = 0
    for a, b in ((0, 7), (7, 16)):
        d = ids[a:b][None]
        total = total + w2({"input_ids": d, "attention_mask": torch.ones_like(d), "labels": d.clone()})["loss"]
    torch.testing.assert_close(out["loss"], total, rtol=1e-4, atol=1e-4)


def test_distillation_loss_terms():
    from lm_engine_b200.enums import KLDivergenceMethod
    from lm_engine_b200.model_wrapper.distillation import ModelWrapperForDistillation

    _pgm()
    torch.manual_seed(2)
    tokens = torch.randint(0, VOCAB, (2, SEQ + 1))
    for method in (KLDivergenceMethod.forward, KLDivergenceMethod.backward):
        w = ModelWrapperForDistillation(
            pretrained_config=_cfg().to_dict(), micro_batch_size=2, sequence_length=SEQ,
            teacher_pretrained_config=_cfg(hidden=48).to_dict(), teacher_model_dtype="fp32",
            kl_divergence_method=method, kl_divergence_weight=0.5)
        assert w.has_teacher_model()
        assert not any(k.startswith("teacher") for k in w.state_dict())
        w.train()
        assert not w.teacher_model.training
        out = w(tokens, lm_loss_multiplier=1 / (2 * SEQ))
        s = w.model(input_ids=tokens[:, :-1]).logits.float()
        t = w.teacher_model(input_ids=tokens[:, :-1]).logits.float()
        lm = F.cross_entropy(s.reshape(-1, VOCAB), tokens[:, 1:].reshape(-1))
        sl, tl = F.log_softmax(s, -1).view(-1, VOCAB), F.log_softmax(t, -1).view(-1, VOCAB)
        if method == KLDivergenceMethod.forward:
            kl = (sl.exp() * (sl - tl)).sum(-1).mean()
        else:
            kl = (tl.exp() * (tl - sl)).sum(-1).mean()
        torch.testing.assert_close(out["lm_loss"], lm, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(out["kl_divergence"], kl, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(out["loss"], lm + 0.5 * kl, rtol=1e-4, atol=1e-5)
        out["loss"].backward()
        assert all(p.grad is None for p in w.teacher_model.parameters())
