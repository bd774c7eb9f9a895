"""LSE merge of partials on the GPU against the oracle's restatement of the
reference merge; the Q8_1 epilogue against the oracle's block quantiser."""
import numpy as np
import pytest
import torch

import oracle
from tinycoder_inference_b200 import ops
from tests.util import assert_close, dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seqLen,nH,chunks,hd", [(1, 28, 148, 128), (1, 14, 64, 64), (3, 40, 8, 128), (1, 24, 512, 256),
                                                (2, 5, 1, 32), (1, 28, 7, 128)])
def test_merge_matches_reference_rule(seqLen, nH, chunks, hd):
    rng = np.random.default_rng(chunks + hd)
    acc = rng.standard_normal((seqLen, nH, chunks, hd), dtype=np.float32) * 5
    m = rng.standard_normal((seqLen, nH, chunks), dtype=np.float32) * 3
    l = rng.uniform(0.5, 40.0, (seqLen, nH, chunks)).astype(np.float32)
    # inactive chunks: l == 0 with the initial running max, and junk accumulators that must not be read into the sum
    dead = rng.uniform(size=l.shape) < 0.3
    dead[..., 0] = False
    l[dead] = 0.0
    m[dead] = -1e30
    acc[dead] = 1e30
    want = oracle.combine_partials(acc, m, l, seqLen, nH, chunks, hd)
    out = torch.empty((seqLen, nH, hd), device="cuda")
    q81 = torch.zeros(seqLen * nH * (hd // 32) * 40, dtype=torch.uint8, device="cuda")
    ops.merge_partials(dev(acc), dev(m), dev(l), out, seqLen, nH, chunks, hd, q81=q81)
    torch.cuda.synchronize()
    assert_close(host(out), want, rtol=1e-5, atol=1e-6, what="merge")
    # the Q8_1 blocks are a byte format: exact on the values the merge produced
    assert np.array_equal(host(q81), oracle.q8_1_blocks(host(out)))


def test_all_chunks_empty_gives_zero():
    acc = torch.full((1, 4, 3, 128), 7.0, device="cuda")
    m = torch.full((1, 4, 3), -1e30, device="cuda")
    l = torch.zeros((1, 4, 3), device="cuda")
    out = torch.full((1, 4, 128), 5.0, device="cuda")
    ops.merge_partials(acc, m, l, out, 1, 4, 3, 128)
    assert float(out.abs().sum()) == 0.0


def test_sigmoid_gate():
    seqLen, nH, hd = 3, 16, 256
    rng = np.random.default_rng(1)
    o = rng.standard_normal((seqLen, nH, hd), dtype=np.float32)
    g = rng.standard_normal((seqLen, nH, 2 * hd), dtype=np.float32) * 4
    want = oracle.sigmoid_gate(o, g, seqLen, nH, hd)
    od = dev(o)
    ops.sigmoid_gate(od, dev(g), seqLen, nH, hd)
    assert_close(host(od), want, rtol=1e-5, atol=1e-6, what="sigmoid gate")
