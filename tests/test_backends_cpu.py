"""MLA / sparse-MLA helpers of the attention backend module on the CPU oracle path (the dense backend and the
class contracts are covered by ``test_vllm_plugin_cpu.py``)."""
import torch

from vllm_kunlun_b200 import ops
from vllm_kunlun_b200.attention.backends import sparse_mla_forward


def test_sparse_mla_equals_dense_when_topk_covers_the_context():
    torch.manual_seed(1)
    N, bs, T = 4, 64, 70
    cache = torch.zeros(4, bs, 576)
    kv_c, k_pe = torch.randn(T, 512), torch.randn(T, 64)
    bt = torch.tensor([[1, 2, 0]], dtype=torch.int32)
    slots = torch.tensor([int(bt[0, p // bs]) * bs + p % bs for p in range(T)])
    ops.concat_and_cache_mla(kv_c, k_pe, cache, slots)
    q = torch.randn(T, N, 576) * 0.1
    seq = torch.tensor([T], dtype=torch.int32)
    qsl = torch.tensor([0, T], dtype=torch.int32)
    dense = ops.mla_attention(q, cache, bt, seq, qsl, 0.1, 512, max_query_len=T, max_seq_len=T)
    assert dense.shape == (T, N, 512)
    # every query may look at every earlier token: request-local indices 0..t, -1 beyond
    idx = torch.arange(128).unsqueeze(0).expand(T, 128).clone()
    idx[idx > torch.arange(T).unsqueeze(1)] = -1
    sparse = sparse_mla_forward(q, cache, idx.int(), torch.zeros(T, dtype=torch.int32), bt, 0.1, bs)
    torch.testing.assert_close(sparse, dense, atol=1e-5, rtol=1e-4)
