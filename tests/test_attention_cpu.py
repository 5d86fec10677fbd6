"""The PyTorch attention restatement against SDPA and hand-built masks (CPU)."""
import math

import torch

from steptronoss_b200.ops.attention import attention_reference


def test_single_segment_causal_matches_sdpa():
    torch.manual_seed(0)
    q, k, v = torch.randn(50, 4, 16), torch.randn(50, 2, 16), torch.randn(50, 2, 16)
    out = attention_reference(q, k, v, causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1)[None], k.transpose(0, 1)[None].repeat_interleave(2, 1),
        v.transpose(0, 1)[None].repeat_interleave(2, 1), is_causal=True)[0].transpose(0, 1)
    assert torch.allclose(out, ref, atol=1e-5)


def test_packed_segments_do_not_attend_across_documents():
    torch.manual_seed(1)
    q, k, v = torch.randn(30, 2, 8), torch.randn(30, 2, 8), torch.randn(30, 2, 8)
    cu = torch.tensor([0, 10, 30], dtype=torch.int32)
    out = attention_reference(q, k, v, cu, cu, causal=True)
    a = attention_reference(q[:10], k[:10], v[:10], causal=True)
    b = attention_reference(q[10:], k[10:], v[10:], causal=True)
    assert torch.allclose(out, torch.cat([a, b]), atol=1e-6)


def test_sliding_window_and_offset_queries():
    torch.manual_seed(2)
    q, k, v = torch.randn(4, 1, 8), torch.randn(10, 1, 8), torch.randn(10, 1, 8)
    cq, ck = torch.tensor([0, 4], dtype=torch.int32), torch.tensor([0, 10], dtype=torch.int32)
    out = attention_reference(q, k, v, cq, ck, causal=True, window=3)
    s = (q[:, 0] @ k[:, 0].t()) / math.sqrt(8)
    mask = torch.zeros(4, 10, dtype=torch.bool)
    for i in range(4):
        qi = i + 6
        for j in range(10):
            mask[i, j] = (j <= qi) and (j > qi - 3)
    ref = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, 0]
    assert torch.allclose(out[:, 0], ref, atol=1e-6)
