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


def test_adjacent_pair_rope_rotates_neighbouring_dimensions():
    """With ``rope_use_adjacent_pair`` the attention output equals the plain module's on inputs whose q/k rows were
    de-interleaved beforehand, and the rotation itself is the (2i, 2i+1) pair rotation."""
    import torch

    from steptronoss_b200.ops.fused import qknorm_rope_reference
    from steptronoss_b200.parallel.state import PM

    PM.initialize()

    def build(adjacent):
        from tests.tiny_exp import make_tiny_exp

        exp = make_tiny_exp(gbs=1, seq=16, iters=1, layers=1, hidden=32, heads=2, kv_heads=1, head_dim=16, ffn=64, vocab=64)
        c = exp.model_cfg.attn_cfg
        c.rope_use_adjacent_pair, c.params_dtype = adjacent, torch.float32
        PM.set_mesh(exp.model_cfg.parallel_cfg)
        m = c.build_model(layer_id=0)
        torch.manual_seed(0)
        for p in m.parameters():
            torch.nn.init.normal_(p, std=0.3)
        return m

    plain, adj = build(False), build(True)
    adj.load_state_dict(plain.state_dict())
    T, D = 6, 16
    x = torch.randn(T, 32)
    pos = torch.arange(T, dtype=torch.int32)
    cu = torch.tensor([0, T], dtype=torch.int32)
    out = adj(x, pos, cu, T)
    assert out.shape == (T, 32) and torch.isfinite(out).all() and not torch.allclose(out, plain(x, pos, cu, T))

    # the rotation: de-interleave, half-split rotate == rotate neighbours, then de-interleave
    cos, sin = adj.rope.tables(x.device, T)
    qkv = torch.randn(T, 4 * D)                                      # 2 q heads, 1 k head, 1 v head
    perm = adj.pair_perm
    qk = qkv[:, :3 * D].reshape(T, 3, D).index_select(-1, perm).reshape(T, 3 * D)
    q, k, _ = qknorm_rope_reference(torch.cat([qk, qkv[:, 3 * D:]], 1), None, None, cos, sin, pos, 2, 1, D, D, use_norm=False)
    raw = qkv[:, :2 * D].reshape(T, 2, D)
    c, s = cos[pos.long()].unsqueeze(1), sin[pos.long()].unsqueeze(1)
    want = torch.empty_like(raw)
    want[..., 0::2] = raw[..., 0::2] * c - raw[..., 1::2] * s
    want[..., 1::2] = raw[..., 1::2] * c + raw[..., 0::2] * s
    assert torch.allclose(q, want.index_select(-1, perm), atol=1e-6)


def test_gathered_key_plan_tables_for_context_parallel_pieces():
    """Segment tables of the kernels that address keys by global position: a range starts at the multiple of 128 at
    or before its document, the keys in front of the document are counted as skipped, and the key-block schedule
    walks every range in 128-row steps."""
    import torch

    from steptronoss_b200.ops.attention_native import GatheredKeyPlan
    from steptronoss_b200.parallel.context_parallel import cu_seqlens_to_balanced_cp

    # two documents [0, 700) and [700, 2048) over CP = 2 (chunks of 512): rank 0 holds chunks 0 and 3
    halves = cu_seqlens_to_balanced_cp([0, 700, 2048], 2048, 2, 0)
    assert halves == [[(0, 512, 0)], [(1536, 2048, 700)]]
    plan = GatheredKeyPlan(halves[0] + halves[1], 2, 512, "cpu")
    assert plan.cu_q.tolist() == [0, 512, 1024]
    assert plan.seg_k_begin.tolist() == [0, 640]            # 700 rounded down to a multiple of 128
    assert plan.seg_k_skip.tolist() == [0, 60]
    assert plan.seg_k_len.tolist() == [512, 2048 - 640]
    assert plan.k_blk_seg.tolist() == [0] * 4 + [1] * 11
    assert plan.k_blk_row0.tolist() == [0, 128, 256, 384] + [640 + 128 * i for i in range(11)]
    # rank 1 holds chunks 1 and 2: its first half sees document 0 up to 700 and then document 1 from 700 on
    halves1 = cu_seqlens_to_balanced_cp([0, 700, 2048], 2048, 2, 1)
    assert halves1[0] == [(512, 700, 0), (700, 1024, 700)] and halves1[1] == [(1024, 1536, 700)]
