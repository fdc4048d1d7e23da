"""Empty inputs through the C ABI on the GPU: zero rows are a valid call for every operator (the reference's modules accept an empty
batch: a stream with no read rows reaches Scorer._forward, spinf_serve/scorer.py:243-246), and nothing is launched or written."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_zero_rows_everywhere(dev):
    from spinf_serve_b200 import attention as A
    from spinf_serve_b200 import ops

    K, N = 256, 512
    x = torch.empty((0, K), dtype=torch.bfloat16, device=dev)
    w8 = torch.zeros((N, K), dtype=torch.float8_e4m3fn, device=dev)
    ws = torch.ones(N, dtype=torch.float32, device=dev)
    x8, xs = ops.fp8_rowwise_quant(x)
    assert x8.shape == (0, K) and xs.shape == (0, 1)
    assert ops.fp8_rowwise_gemm(x8, xs, w8, ws).shape == (0, N)
    g8, gs, _ = ops.fp8_gemm_glu(x8, xs, w8, ws, "gelu_tanh")
    assert g8.shape == (0, N // 2) and gs.shape[0] == 0
    t8, ts = ops.fp8_tensor_quant(x)
    assert t8.shape == (0, K) and float(ts) == float(torch.tensor(1e-12) / 448.0)
    assert ops.fp8_tensor_gemm(t8, ts, w8, ws[:1].reshape(())).shape == (0, N)
    i8, i_s = ops.int8_rowwise_quant(x)
    assert ops.int8_rowwise_gemm(i8, i_s, torch.zeros((N, K), dtype=torch.int8, device=dev), ws).shape == (0, N)
    assert ops.bf16_gemm(x, torch.zeros((N, K), dtype=torch.bfloat16, device=dev)).shape == (0, N)
    q4 = ops.w4_repack(torch.zeros((N, K // 2), dtype=torch.uint8, device=dev))
    s4 = torch.ones((N, K // 128), dtype=torch.float16, device=dev)
    assert ops.w4_gemm(x, q4, s4, 128).shape == (0, N)
    assert ops.w4_gemm_glu(x, q4, s4, 128, "silu").shape == (0, N // 2)
    assert ops.fused_norm(x, w2=torch.ones(K, dtype=torch.bfloat16, device=dev), want_norm=True)["norm"].shape == (0, K)
    # an empty stream: no blocks, no tiles, no output rows
    z = np.zeros(0, np.int32)
    m = A.stream_masks(z, z, z, 1024, dev)["full_attention"]
    q = torch.empty((0, 4, 128), dtype=torch.bfloat16, device=dev)
    kv = torch.empty((0, 2, 128), dtype=torch.bfloat16, device=dev)
    assert A.tree_attention(q, kv, kv, m, 1.0).shape == (0, 4, 128)
    torch.cuda.synchronize(dev)


def test_abs_max_of_nothing_writes_zero_through_the_c_abi(dev):
    """*out = max |x| over n elements holds for n = 0 too: a caller that feeds it to spinf_fp8_tensor_quant(from_amax = 1) must not
    read what the buffer held before"""
    from spinf_serve_b200 import _lib

    out = torch.full((1,), 123.0, dtype=torch.float32, device=dev)
    assert _lib.lib().spinf_abs_max(None, 0, _lib.ptr(out), _lib.stream_ptr()) == 0
    torch.cuda.synchronize(dev)
    assert float(out) == 0.0
    assert _lib.lib().spinf_abs_max(None, 0, None, _lib.stream_ptr()) == -1


def test_scorer_with_nothing_to_score(dev):
    from spinf_serve_b200.gemma_stack import GemmaConfig, GemmaStack, GemmaWeights
    from spinf_serve_b200.scorer import EngineConfig, Scorer

    cfg = GemmaConfig(layers=1, hidden=256, heads=2, kv_heads=1, head_dim=128, ffn=512, vocab=512, window=64, pattern=2)
    sc = Scorer(GemmaStack(GemmaWeights.random(cfg, 0, dev)), EngineConfig(token_budget=1024, max_tokens=4096), dev)
    assert sc.score_grouped([]) == {} and sc.stats.forwards == 0
