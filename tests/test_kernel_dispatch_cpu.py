"""Host-side logic around the CUDA kernels that needs no GPU: position runs of context-parallel shards, which
attention blocks the kernels may serve, replay segment sizes of the M2RNN scan, and the eligibility predicates that
keep CPU tensors on the PyTorch statements."""

import pytest
import torch


@pytest.mark.parametrize("method", [None, "headtail"])
@pytest.mark.parametrize("cp", [1, 2, 4])
def test_shard_runs_cover_the_shard_positions(method, cp):
    from lm_engine_b200.parallel.context_parallel import shard_indices
    from lm_engine_b200.parallel.ring_attention import shard_runs

    S = 64 * cp
    seen = []
    for r in range(cp):
        runs = shard_runs(S, cp, r, method)
        pos = torch.cat([torch.arange(a, a + n) for a, n in runs])
        assert torch.equal(pos, shard_indices(S, cp, r, method))
        assert len(runs) == (2 if method == "headtail" else 1)
        seen.append(pos)
    assert torch.equal(torch.cat(seen).sort().values, torch.arange(S))


def test_run_relations():
    from lm_engine_b200.parallel.ring_attention import _relation

    assert _relation((128, 128), (0, 128), True) == "full"        # keys strictly before the queries
    assert _relation((128, 128), (128, 128), True) == "causal"    # the same run
    assert _relation((0, 128), (128, 128), True) == "skip"        # keys after the queries
    assert _relation((64, 128), (0, 128), True) is None           # partial overlap: not kernel-shaped
    assert _relation((0, 128), (128, 128), False) == "full"


def test_ulysses_head_split_rules():
    from lm_engine_b200.parallel.ulysses import ulysses_eligible

    assert ulysses_eligible(32, 8, 4) and ulysses_eligible(32, 8, 8)
    assert ulysses_eligible(8, 2, 4)            # K/V heads replicated twice
    assert not ulysses_eligible(6, 2, 4)        # query heads do not split
    assert not ulysses_eligible(8, 1, 3)


def test_m2rnn_segments_are_chunk_multiples_and_bounded():
    from lm_engine_b200.ops import m2rnn

    seg = m2rnn.segment_length(2, 132, 64, 16, 4096)
    assert seg % 8 == 0 and 8 <= seg <= 4096
    assert 2 * 132 * 64 * 16 * 2 * seg <= m2rnn.RECORD_BYTES
    assert m2rnn.segment_length(1, 1, 16, 16, 10) == 16     # short sequences: one segment, rounded up to a chunk


def test_cpu_tensors_stay_on_the_pytorch_statements():
    from lm_engine_b200.ops import attention_cuda, m2rnn, rnn
    from lm_engine_b200.ops.recurrence import gru, m2rnn as m2rnn_op, rnn as rnn_op

    q = torch.randn(1, 128, 2, 128, dtype=torch.bfloat16)
    assert not attention_cuda.shapes_supported(q, q, q)
    assert not attention_cuda.supports(q, q, q, causal=True, sliding_window=64, attention_mask=None, cu_seqlens=None,
                                       dropout_p=0.0)
    x = torch.randn(1, 5, 2, 16, dtype=torch.bfloat16)
    W = torch.randn(2, 16, 16, dtype=torch.bfloat16)
    assert not rnn.rnn_kernel_eligible(x) and not rnn.rnn_kernel_eligible(x, x, x, gru=True)
    assert not m2rnn.m2rnn_kernel_eligible(x, x, x, x[..., 0], W)
    # the dispatchers fall through to the scans and keep their contract
    y, h = rnn_op(x.float(), W.float())
    assert y.shape == (1, 5, 2, 16) and h.shape == (1, 2, 16)
    y, h = gru(x.float(), x.float(), x.float(), W.float(), W.float(), W.float())
    assert y.shape == (1, 5, 2, 16)
    f = torch.sigmoid(torch.randn(1, 5, 2))
    y, h = m2rnn_op(x.float(), x.float(), x.float(), f, W.float())
    assert y.shape == (1, 5, 2, 16) and h.shape == (1, 2, 16, 16)


def test_embedding_and_packing_fall_back_on_cpu():
    from lm_engine_b200.ops.embedding import embedding
    from lm_engine_b200.ops.packing import pack_sequence, unpack_sequence

    W = torch.randn(10, 8)
    ids = torch.tensor([[1, 12, 3]])
    out = embedding(ids, W, vocab_start=0, vocab_end=10)
    assert torch.equal(out[0, 0], W[1]) and torch.equal(out[0, 1], torch.zeros(8)) and torch.equal(out[0, 2], W[3])
    x = torch.arange(24.).view(2, 3, 4)
    cu = torch.tensor([0, 2, 5])
    packed = pack_sequence(x, cu)
    assert packed.shape == (5, 4) and torch.equal(packed[:2], x[0, 1:])
    assert torch.equal(unpack_sequence(packed, cu, (2, 3, 4))[0, 0], torch.zeros(4))


def test_argument_structs_match_the_c_header(tmp_path):
    """The ctypes mirrors of the scan kernels' argument structs have the size and field offsets the C header gives
    them (compiled with the host compiler; no GPU or nvcc involved)."""
    import ctypes
    import os
    import shutil
    import subprocess

    from lm_engine_b200.ops import m2rnn, rnn

    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        pytest.skip("no host C++ compiler")
    header = os.path.join(os.path.dirname(m2rnn.__file__), "..", "csrc", "lme_api.h")
    src = tmp_path / "probe.cpp"
    src.write_text('#include <cstdio>\n#include <cstddef>\n#include "%s"\n' % os.path.abspath(header) + '''
int main() {
    printf("%zu %zu %zu %zu %zu\\n", sizeof(LmeM2rnnArgs), offsetof(LmeM2rnnArgs, h0), offsetof(LmeM2rnnArgs, hprev),
           offsetof(LmeM2rnnArgs, clip), offsetof(LmeM2rnnArgs, dW_part));
    printf("%zu %zu %zu %zu\\n", sizeof(LmeRnnArgs), offsetof(LmeRnnArgs, h0), offsetof(LmeRnnArgs, hr),
           offsetof(LmeRnnArgs, clip));
    return 0;
}
''')
    exe = tmp_path / "probe"
    subprocess.run([cxx, "-std=c++17", str(src), "-o", str(exe)], check=True)
    lines = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    a, b = m2rnn._Args, rnn._Args
    assert [int(v) for v in lines[0].split()] == [ctypes.sizeof(a), a.h0.offset, a.hprev.offset, a.clip.offset,
                                                  a.dW_part.offset]
    assert [int(v) for v in lines[1].split()] == [ctypes.sizeof(b), b.h0.offset, b.hr.offset, b.clip.offset]


def test_ctypes_signatures_have_the_arity_of_the_header():
    """Every entry point bound in ops/_lib.py is declared in csrc/lme_api.h with the same number of parameters."""
    import os
    import re

    from lm_engine_b200.ops import _lib

    header = open(os.path.join(os.path.dirname(_lib.__file__), "..", "csrc", "lme_api.h")).read()
    header = re.sub(r"//[^\n]*", "", header)
    declared = {}
    for m in re.finditer(r"\bint\s+(lme_\w+)\s*\(([^;{]*?)\)\s*;", header, flags=re.S):
        params = m.group(2).strip()
        declared[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    source = open(_lib.__file__).read()
    bound = {}
    for m in re.finditer(r'"(lme_\w+)":\s*\[([^\]]*)\]', source):
        bound[m.group(1)] = len([a for a in m.group(2).split(",") if a.strip()])
    assert len(bound) > 30
    missing = sorted(set(bound) - set(declared))
    assert not missing, missing
    wrong = {k: (bound[k], declared[k]) for k in bound if bound[k] != declared[k]}
    assert not wrong, wrong
