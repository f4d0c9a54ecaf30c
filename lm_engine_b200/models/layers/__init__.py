"""Neural building blocks (counterparts of lm_engine/modeling_utils/**)."""

from .activations import get_activation_function, is_glu
from .attention import (
    SoftmaxAttention,
    interleave_query_key_value_tensor_for_attention,
    split_query_key_value_tensor_for_attention,
)
from .dropout import Dropout
from .embedding import LMHead, ParameterizedEmbedding, get_tensor_parallel_vocab_info
from .linear import ColumnParallelLinear, LowRankLinear, ParameterizedLinear, ReplicatedLinear, RowParallelLinear
from .mlp import MLP, interleave_up_gate, split_up_gate
from .norm import LayerNorm, PNorm, RMSNorm, get_normalization_function
from .rope import RoPE, YaRNScaledRoPE, apply_rotary_pos_emb
