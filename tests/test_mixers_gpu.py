"""Small models of every mixer / block family on the GPU in bf16 (the CUDA kernels inside the layers)
against the same weights in fp32 on the CPU (PyTorch statements): logits and parameter gradients."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

ATTN = dict(sequence_mixer_type="softmax_attention", num_attention_heads=4, num_key_value_heads=2)
MIXERS = {
    "rnn": dict(sequence_mixer_type="rnn", state_head_dim=16, num_input_heads=2, num_weight_heads=4, add_bias=False,
                normalization_function="rmsnorm", gradient_clipping=1.0, kernel_size=None,
                activation_function="tanh"),
    "gru": dict(sequence_mixer_type="gru", state_head_dim=16, num_input_heads=4, num_forget_input_heads=2,
                num_reset_input_heads=1, num_weight_heads=2, num_forget_weight_heads=4, num_reset_weight_heads=1,
                add_bias=True, normalization_function="rmsnorm", gradient_clipping=None, kernel_size=4,
                activation_function="silu"),
    "m2rnn": dict(sequence_mixer_type="m2rnn", k_head_dim=16, v_head_dim=16, num_q_heads=1, num_k_heads=1,
                  num_v_heads=4, num_f_heads=4, num_g_heads=4, num_weight_heads=2, use_residual=True, kernel_size=4,
                  activation_function="silu", add_bias=False, gradient_clipping=1.0,
                  normalization_function="rmsnorm"),
    "mamba2": dict(sequence_mixer_type="mamba2", state_size=16, intermediate_size=128, num_heads=4,
                   conv_kernel_size=4, activation_function="silu", num_groups=1, chunk_size=16,
                   normalization_function="rmsnorm"),
}


def _config(mixer, model_type="gpt_base", mlp=None, **extra):
    d = _base(mixer, model_type, mlp)
    d.update(extra)
    return d


def _base(mixer, model_type, mlp):
    mlp = mlp or dict(mlp_type="MLP", intermediate_size=128, activation_function="swiglu")
    return dict(model_type=model_type, vocab_size=256, max_position_embeddings=128, hidden_size=64, num_layers=2,
                normalization_function="rmsnorm", layer_norm_epsilon=1e-5, initializer_range=0.05, bos_token_id=0,
                eos_token_id=1, pad_token_id=2, position_embedding_type="nope", rope_theta=10000, rope_scaling=None,
                m_emb=None, m_width=None, m_residual=None, init_method="normal", embedding_init_method="normal",
                use_depth_scaled_init=False, tie_word_embeddings=False, sequence_mixer_blocks=[mixer, dict(ATTN)],
                mlp_blocks=[dict(mlp) for _ in range(2)])


GDN = dict(sequence_mixer_type="gated_deltanet", k_head_dim=16, v_head_dim=32, num_k_heads=2, num_v_heads=4,
           use_gate=True, attention_multiplier=None, allow_neg_eigval=True, kernel_size=4)
MOE = dict(mlp_type="MoE", intermediate_size=64, num_experts=4, num_experts_per_tok=2, activation_function="swiglu",
           shared_intermediate_size=64, add_bias=False)
LINATT = dict(sequence_mixer_type="linear_attention", k_head_dim=16, v_head_dim=16, num_q_heads=2, num_k_heads=2,
              num_v_heads=4, num_g_heads=4, kernel_size=4, activation_function="silu", add_bias=False,
              normalization_function="rmsnorm", attention_multiplier=None)
OTHER = {
    "gated_deltanet": dict(mixer=GDN),
    "linear_attention": dict(mixer=LINATT),
    "moe": dict(mixer=dict(ATTN), mlp=MOE, router_aux_loss_coef=0.01),
    "rope": dict(mixer=dict(ATTN), position_embedding_type="rope", rope_dim=16),
    "palm": dict(mixer=dict(ATTN), model_type="palm", position_embedding_type="rope", rope_dim=16),
    "ladder_residual": dict(mixer=dict(ATTN), model_type="ladder_residual", position_embedding_type="rope",
                            rope_dim=16),
    "crosslayer": dict(mixer=dict(ATTN), model_type="gpt_crosslayer", sharing_pattern=[0, 0],
                       position_embedding_type="rope", rope_dim=16),
    "layernorm_bias": dict(mixer=dict(ATTN, add_bias=True), normalization_function="layernorm",
                           mlp=dict(mlp_type="MLP", intermediate_size=128, activation_function="gelu_pytorch_tanh",
                                    add_bias=True)),
}


@pytest.mark.parametrize("family", sorted(MIXERS) + sorted(OTHER))
def test_model_family_on_gpu_matches_cpu_fp32(family):
    from lm_engine_b200.models import build_model, config_from_dict
    from lm_engine_b200.ops import _lib

    torch.manual_seed(0)
    cfg = _config(MIXERS[family]) if family in MIXERS else _config(**OTHER[family])
    cpu = build_model(config_from_dict(cfg))
    # weights that survive the bf16 cast exactly, so that both models start from the same point
    with torch.no_grad():
        for p in cpu.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    gpu = copy.deepcopy(cpu).to(device="cuda", dtype=torch.bfloat16)
    x = torch.randint(0, 256, (2, 96), generator=torch.Generator().manual_seed(1))
    launches = _lib.launch_count
    out_g = gpu(x.cuda()).logits
    out_c = cpu(x).logits
    out_g.float().pow(2).mean().backward()
    out_c.pow(2).mean().backward()
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    assert _lib.launch_count > launches                       # the layers ran on the kernels
    err = float((out_g.float().cpu() - out_c).norm() / out_c.norm())
    assert err < 3e-2, err
    bad = []
    for (n, pg), (_, pc) in zip(gpu.named_parameters(), cpu.named_parameters()):
        ref = pc.grad
        e = float((pg.grad.float().cpu() - ref).norm() / (ref.norm() + 1e-8))
        if e > 8e-2 and float(ref.norm()) > 1e-6:
            bad.append((n, round(e, 3)))
    assert not bad, bad


CACHED = ["rnn", "gru", "m2rnn", "mamba2", "gated_deltanet", "linear_attention", "rope"]


@pytest.mark.parametrize("family", CACHED)
def test_prefill_and_decode_with_the_cache_match_the_full_forward(family):
    """On the GPU in bf16: prefilling 64 tokens and decoding the next 8 one at a time (the kernels' carried states:
    scans with an initial state, conv state, KV cache) gives the logits of one forward over all 72 tokens."""
    from lm_engine_b200.models import build_model, config_from_dict
    from lm_engine_b200.models.context import GenerationCache
    from lm_engine_b200.ops import _lib

    torch.manual_seed(0)
    cfg = _config(MIXERS[family]) if family in MIXERS else _config(**OTHER[family])
    model = build_model(config_from_dict(cfg)).to(device="cuda", dtype=torch.bfloat16).eval()
    x = torch.randint(0, 256, (2, 72), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        full = model(x).logits.float()
        out = model(x[:, :64], cache_params=GenerationCache())
        steps = [out.logits[:, -1].float()]
        for t in range(64, 71):
            out = model(x[:, t:t + 1], cache_params=out.cache_params)
            steps.append(out.logits[:, -1].float())
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    got = torch.stack(steps, dim=1)                       # logits that predict tokens 64 .. 71
    want = full[:, 63:71]
    err = float((got - want).norm() / want.norm())
    assert err < 3e-2, err



@pytest.mark.parametrize("family", CACHED)
def test_left_padded_prefill_matches_the_unpadded_sample(family):
    """A left-padded row of a batch (attention mask, prefill with a cache) gives the logits of the same tokens run
    alone: padding reaches neither the attention nor the recurrent states / convolution windows."""
    from lm_engine_b200.models import build_model, config_from_dict
    from lm_engine_b200.models.context import AttentionMaskInfo, GenerationCache
    from lm_engine_b200.ops import _lib

    torch.manual_seed(0)
    cfg = _config(MIXERS[family]) if family in MIXERS else _config(**OTHER[family])
    model = build_model(config_from_dict(cfg)).to(device="cuda", dtype=torch.bfloat16).eval()
    g = torch.Generator().manual_seed(3)
    short, long = torch.randint(3, 256, (1, 40), generator=g).cuda(), torch.randint(3, 256, (1, 64), generator=g).cuda()
    batch = torch.cat((torch.cat((torch.full((1, 24), 2, device="cuda"), short), 1), long))
    mask = torch.ones_like(batch)
    mask[0, :24] = 0
    with torch.no_grad():
        alone = model(short, cache_params=GenerationCache()).logits.float()
        both = model(batch, cache_params=GenerationCache(),
                     attention_mask_info=AttentionMaskInfo(attention_mask=mask)).logits.float()
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    err = float((both[0, 24:] - alone[0]).norm() / alone[0].norm())
    assert err < 3e-2, err


@pytest.mark.parametrize("family", ["rnn", "gru", "m2rnn", "mamba2", "gated_deltanet", "linear_attention"])
def test_packed_tokens_match_each_sequence_alone(family):
    """Padding-free input (packed tokens + cu_seqlens) through the recurrent mixers on the GPU: the row-copy kernels
    move the scan inputs into a left-padded batch and back; logits and weight gradients equal those of the
    sequences run one at a time."""
    from lm_engine_b200.models import build_model, config_from_dict
    from lm_engine_b200.models.context import AttentionMaskInfo, PositionInfo
    from lm_engine_b200.ops import _lib

    torch.manual_seed(0)
    cfg = config_from_dict(_config(MIXERS[family]) if family in MIXERS else _config(**OTHER[family]))
    packed = build_model(cfg, use_padding_free_transformer=True).to(device="cuda", dtype=torch.bfloat16)
    plain = build_model(cfg).to(device="cuda", dtype=torch.bfloat16)
    plain.load_state_dict(packed.state_dict())
    lens = [40, 64, 24]
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(3, 256, (sum(lens),), generator=g).cuda()
    cu = torch.tensor([0, 40, 104, 128], dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).cuda()
    out = packed(ids, attention_mask_info=AttentionMaskInfo(cu_seqlens=cu, max_seqlen=max(lens)),
                 position_info=PositionInfo(position_ids=pos)).logits.float()
    alone = torch.cat([plain(ids[a:b][None]).logits[0] for a, b in zip(cu[:-1].tolist(), cu[1:].tolist())]).float()
    err = float((out - alone).norm() / alone.norm())
    assert err < 3e-2, err
    out.pow(2).mean().backward()
    alone.pow(2).mean().backward()
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    for (n, a), (_, b) in zip(packed.named_parameters(), plain.named_parameters()):
        ga, gb = a.grad.float(), b.grad.float()
        assert float((ga - gb).norm() / (gb.norm() + 1e-6)) < 6e-2, n
