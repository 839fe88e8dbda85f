"""Attention backend classes (the surface an out-of-tree vLLM platform hands to the engine) on the CPU oracle path."""
import torch

from vllm_kunlun_b200.attention.backends import (GQABackend, MetadataBuilder, MLABackend, SparseMLABackend)
from vllm_kunlun_b200.ops.reference import attention as ra


def _md(builder, q_lens, ctx_lens, bs, nblk):
    B = len(q_lens)
    seq = [c + q for q, c in zip(q_lens, ctx_lens)]
    qsl = torch.zeros(B + 1, dtype=torch.int32)
    qsl[1:] = torch.tensor(q_lens).cumsum(0)
    bt = torch.zeros(B, nblk, dtype=torch.int32)
    pos, slots, nxt = [], [], 1
    for b in range(B):
        n = -(-seq[b] // bs)
        bt[b, :n] = torch.arange(nxt, nxt + n)
        nxt += n
        for p in range(ctx_lens[b], seq[b]):
            pos.append(p)
            slots.append(int(bt[b, p // bs]) * bs + p % bs)
    md = builder.build(torch.tensor(pos), torch.tensor(slots), bt, torch.tensor(seq, dtype=torch.int32), qsl, max(q_lens),
                       max(seq), num_decodes=sum(q <= builder.reorder_batch_threshold for q in q_lens))
    md.seq_lens_cpu, md.query_start_loc_cpu = md.seq_lens, md.query_start_loc
    return md, nxt


def test_builder_orders_decodes_first():
    b = MetadataBuilder(num_spec_tokens=1)
    assert b.reorder_batch([7, 1, 2, 30, 1]) == [1, 2, 4, 0, 3]
    assert b.cudagraph_support == "UNIFORM_BATCH"


def test_gqa_backend_forward_matches_plain_attention():
    torch.manual_seed(0)
    H, Hkv, D, bs = 4, 2, 64, 16
    assert D in GQABackend.get_supported_head_sizes() and GQABackend.get_name() == "B200_GQA"
    md, nblocks = _md(GQABackend.get_builder_cls()(), [5, 9], [0, 0], bs, 4)
    cache = torch.zeros(GQABackend.get_kv_cache_shape(nblocks + 1, bs, Hkv, D))
    T = md.num_tokens
    q, k, v = torch.randn(T, H * D), torch.randn(T, Hkv * D), torch.randn(T, Hkv * D)
    impl = GQABackend.get_impl_cls()(H, D, D ** -0.5, Hkv)
    out = impl.forward(q, k, v, cache, md)
    s = 0
    for n in (5, 9):
        want = ra._attend(q[s:s + n].view(n, H, D), k[s:s + n].view(n, Hkv, D), v[s:s + n].view(n, Hkv, D), D ** -0.5, 0, None,
                          None)
        torch.testing.assert_close(out[s:s + n].reshape(n, H, D), want, atol=1e-5, rtol=1e-5)
        s += n
    md.is_dummy = True
    assert impl.forward(q, k, v, cache, md).abs().sum() == 0  # profile run: nothing is computed


def test_mla_backends_shapes_and_sparse_equals_dense_when_topk_covers_the_context():
    torch.manual_seed(1)
    N, bs = 4, 64
    assert MLABackend.get_kv_cache_shape(10, bs) == (10, bs, 576)
    assert SparseMLABackend.get_kv_cache_shape(10, bs, cache_dtype="fp8_ds_mla") == (10, bs, 656)
    md, nblocks = _md(MLABackend.get_builder_cls()(), [70], [0], bs, 3)
    md.req_id_per_token = torch.zeros(70, dtype=torch.int32)
    cache = torch.zeros(MLABackend.get_kv_cache_shape(nblocks + 1, bs))
    q = torch.randn(70, N, 576) * 0.1
    kv_c, k_pe = torch.randn(70, 512), torch.randn(70, 64)
    dense = MLABackend.get_impl_cls()(N, 0.1).forward(q, kv_c, k_pe, cache, md)
    assert dense.shape == (70, N, 512)
    # every query may look at every earlier token: local indices 0..t, -1 beyond
    idx = torch.arange(128).unsqueeze(0).expand(70, 128).clone()
    idx[idx > torch.arange(70).unsqueeze(1)] = -1
    sparse = SparseMLABackend.get_impl_cls()(N, 0.1, topk_tokens=128).forward(q, None, None, cache, md, idx.int())
    torch.testing.assert_close(sparse, dense, atol=1e-5, rtol=1e-4)
