"""Operators: hand-written sm_100a kernels behind autograd functions, each with a PyTorch reference statement that
is both the CPU path and the numerical oracle of the tests."""

from .activation import swiglu_backward, swiglu_packed, swiglu_packed_reference
from .cross_entropy import cross_entropy_sum
from .gemm import bmm, bmm_reference, gemm, gemm_reference, linear, linear_swiglu
from .norm import rmsnorm, rmsnorm_reference
from .optimizer import adamw_reference, adamw_step, clip_coef_, sumsq_
from .rope import apply_rope_reference, qkv_split_rope, qkv_split_rope_reference
from .attention import attention, attention_reference
from .packing import compute_cu_seqlens_and_max_seqlen_from_attention_mask, pack_sequence, unpack_sequence
