"""Shared-prefix decode attention (``decode_attn_group_kernel`` + the per-row kernel + combine) against
an fp32 restatement and against the plain paged kernel: groups whose rows share their prompt pages,
a group with no shared page, ragged lengths, retired rows (length 0), several prefix splits."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(B, G, Hq, Hkv, D, page, ppr, shared_pages, lens, seed=0):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(seed)
    P = B // G
    n_pages = (P + B) * ppr
    k = torch.randn(n_pages, page, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(n_pages, page, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
    q = torch.randn(B, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    j = torch.arange(ppr, device=dev)[None, :]
    p_of_row = torch.arange(P, device=dev).repeat_interleave(G)
    sp = torch.tensor(shared_pages, device=dev)[p_of_row][:, None]
    shared = p_of_row[:, None] * ppr + j
    private = P * ppr + torch.arange(B, device=dev)[:, None] * ppr + (j - sp).clamp(min=0)
    table = torch.where(j < sp, shared, private).to(torch.int32).contiguous()
    prefix = (torch.tensor(shared_pages, device=dev) * page).to(torch.int32)
    return q, k, v, table, prefix, torch.tensor(lens, device=dev, dtype=torch.int32)


def _reference(q, k, v, table, lens, scale):
    B, Hq, D = q.shape
    Hkv = k.shape[2]
    kc = k[table.long()].reshape(B, -1, Hkv, D).float().repeat_interleave(Hq // Hkv, dim=2)
    vc = v[table.long()].reshape(B, -1, Hkv, D).float().repeat_interleave(Hq // Hkv, dim=2)
    s = torch.einsum("bhd,bshd->bhs", q.float(), kc) * scale
    allowed = torch.arange(kc.shape[1], device=q.device)[None, :] < lens[:, None]
    s = s.masked_fill(~allowed[:, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.where(allowed.any(1)[:, None, None], p, torch.zeros_like(p))
    return torch.einsum("bhs,bshd->bhd", p, vc)


@pytest.mark.parametrize("Hq,Hkv,D,G,splits", [(32, 8, 128, 8, 0), (32, 8, 128, 8, 1), (32, 8, 128, 8, 3), (16, 4, 128, 4, 2),
                                                  (16, 2, 128, 4, 1), (16, 4, 64, 8, 2)])
def test_shared_prefix_decode_attention_matches_reference(Hq, Hkv, D, G, splits):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ferrl_b200.ops import cuda as C
    assert C.prefix_attention_supported(D, Hq // Hkv, G)
    P, page, ppr = 3, 64, 12
    B = P * G
    shared_pages = [5, 0, 2]                                  # the second group has no full prompt page
    lens = []
    for p_ in range(P):
        for r in range(G):
            lens.append(shared_pages[p_] * page + 1 + (37 * r + 11 * p_) % 300)
    lens[G + 1] = 0                                            # a retired row
    lens[2 * G:3 * G] = [0] * G                                # a group whose rows are all retired
    lens[3] = shared_pages[0] * page + 1                       # exactly one private key
    q, k, v, table, prefix, kv_len = _setup(B, G, Hq, Hkv, D, page, ppr, shared_pages, lens)
    scale = D ** -0.5
    out = C.decode_attention(q, k, v, kv_len, scale=scale, block_table=table, prefix_len=prefix, group=G, prefix_splits=splits)
    plain = C.decode_attention(q, k, v, kv_len, scale=scale, block_table=table)
    torch.cuda.synchronize()
    ref = _reference(q, k, v, table, kv_len, scale)
    err = (out.float() - ref).abs()
    assert float(err.max()) < 2e-2, float(err.max())            # bf16 output of values of order one
    assert float((out.float() - plain.float()).abs().max()) < 2e-2
    assert torch.all(out[kv_len == 0] == 0)
    # same inputs, same bits
    again = C.decode_attention(q, k, v, kv_len, scale=scale, block_table=table, prefix_len=prefix, group=G, prefix_splits=splits)
    assert torch.equal(out, again)
