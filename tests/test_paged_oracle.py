"""CPU checks of the paged-cache oracle (no GPU): gather_pages against an element-by-element restatement."""
import torch

from oracle import oracle as O


def test_gather_pages_element_by_element():
    g = torch.Generator().manual_seed(3)
    n_pages, Hkv, page, D, B, max_pages = 11, 2, 16, 8, 3, 3
    pool = torch.randn(n_pages, Hkv, page, D, generator=g)
    table = torch.tensor([[4, 9, 2 ** 30], [0, 2 ** 30, 2 ** 30], [7, 1, 10]], dtype=torch.int32)
    lens = torch.tensor([17, 16, 48], dtype=torch.int32)
    got = O.gather_pages(pool, table, lens)
    assert got.shape == (B, Hkv, max_pages * page, D)
    for b in range(B):
        for j in range(max_pages * page):
            if j < ((int(lens[b]) + page - 1) // page) * page:
                want = pool[int(table[b, j // page]), :, j % page]
            else:
                want = torch.zeros(Hkv, D)
            assert torch.equal(got[b, :, j], want), (b, j)


def test_decode_paged_oracle_equals_contiguous_oracle():
    g = torch.Generator().manual_seed(4)
    B, H, Hkv, page, D, max_pages = 2, 4, 2, 16, 16, 4
    pool_k = torch.randn(B * max_pages, Hkv, page, D, generator=g)
    pool_v = torch.randn(B * max_pages, Hkv, page, D, generator=g)
    table = torch.randperm(B * max_pages, generator=g).reshape(B, max_pages).to(torch.int32)
    lens = torch.tensor([50, 64], dtype=torch.int32)
    q = torch.randn(B, H, 1, D, generator=g)
    kc = pool_k[table.long()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, D)
    vc = pool_v[table.long()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, D)
    want = O.decode_oracle(q, kc, vc, lens)
    got = O.decode_paged_oracle(q, pool_k, pool_v, table, lens)
    assert torch.allclose(got, want, atol=1e-6, rtol=0)
