"""Paged attention, KV append and the sampler against their dense / CPU oracles."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _pool(P, Hkv, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(P, 128, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(P, 128, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    return k, v


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 1, 128), (8, 2, 128), (4, 4, 64), (16, 2, 128)])
def test_paged_attention_mixed_prefill_decode(Hq, Hkv, D):
    from easydel_b200.ops import serving as S

    P = 40
    kp, vp = _pool(P, Hkv, D, 1)
    # sequences: decode (1 new token, long context), chunked prefill over a cached prefix, fresh prefill
    q_lens = [1, 1, 200, 77, 1]
    kv_lens = [1000, 129, 456, 77, 5]
    B = len(q_lens)
    perm = torch.randperm(P, generator=torch.Generator().manual_seed(3)).tolist()
    maxp = max((L + 127) // 128 for L in kv_lens)
    table = torch.zeros(B, maxp, dtype=torch.int32)
    nxt = 0
    for b, L in enumerate(kv_lens):
        n = (L + 127) // 128
        table[b, :n] = torch.tensor(perm[nxt:nxt + n], dtype=torch.int32)
        nxt += n
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    T = int(cu[-1])
    q = torch.randn(T, Hq, D, device="cuda").to(torch.bfloat16)
    o = S.paged_attention(q, kp, vp, cu.cuda(), torch.tensor(kv_lens, dtype=torch.int32).cuda(), table.cuda(),
                          max(q_lens))
    ref = S.paged_attention_reference(q.cpu(), kp.cpu(), vp.cpu(), cu, torch.tensor(kv_lens), table)
    assert torch.allclose(o.float().cpu(), ref.float(), atol=2e-2, rtol=2e-2), (o.float().cpu() - ref.float()).abs().max()


def test_kv_append_then_attend_matches_dense():
    from easydel_b200.ops import serving as S, reference as R

    Hq, Hkv, D, L = 8, 2, 128, 300
    kp, vp = torch.zeros(8, 128, Hkv, D, device="cuda", dtype=torch.bfloat16), torch.zeros(
        8, 128, Hkv, D, device="cuda", dtype=torch.bfloat16)
    q = torch.randn(L, Hq, D, device="cuda").to(torch.bfloat16)
    k = torch.randn(L, Hkv, D, device="cuda").to(torch.bfloat16)
    v = torch.randn(L, Hkv, D, device="cuda").to(torch.bfloat16)
    pages = [5, 2, 7]
    slots = torch.tensor([pages[i // 128] * 128 + i % 128 for i in range(L)], dtype=torch.int32, device="cuda")
    slots[10] = -1  # a padded token is skipped
    S.kv_append(k, v, kp, vp, slots)
    flat = kp.view(-1, Hkv, D)
    assert torch.equal(flat[pages[1] * 128 + 5], k[133]) and flat[pages[0] * 128 + 10].abs().sum() == 0
    slots[10] = pages[0] * 128 + 10
    S.kv_append(k, v, kp, vp, slots)
    table = torch.tensor([pages], dtype=torch.int32, device="cuda")
    o = S.paged_attention(q, kp, vp, torch.tensor([0, L], dtype=torch.int32, device="cuda"),
                          torch.tensor([L], dtype=torch.int32, device="cuda"), table, L)
    ref = R.attention(q[None], k[None], v[None], causal=True)[0]
    assert torch.allclose(o.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_sampler_greedy_penalties_and_topk():
    from easydel_b200.ops import serving as S

    R_, V = 9, 5000
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = (torch.randn(R_, V, device="cuda", generator=g) * 3).to(torch.bfloat16)
    tok, lp = S.sample(logits, want_logprob=True)
    assert torch.equal(tok.long().cpu(), logits.float().argmax(-1).cpu())
    ref_lp = torch.log_softmax(logits.float(), -1).gather(-1, tok.long()[:, None]).squeeze(-1)
    assert torch.allclose(lp, ref_lp, atol=2e-3)
    # penalties change the arg-max the same way as the oracle
    counts = torch.zeros(R_, V, dtype=torch.int32, device="cuda")
    S.count_update(counts, tok)
    S.count_update(counts, tok)
    assert int(counts.sum()) == 2 * R_
    pres = torch.full((R_,), 0.5, device="cuda")
    freq = torch.full((R_,), 0.7, device="cuda")
    rep = torch.full((R_,), 1.3, device="cuda")
    tok2, _ = S.sample(logits, presence=pres, frequency=freq, repetition=rep, counts=counts)
    z = S.apply_penalties_reference(logits.cpu(), counts.cpu(), pres.cpu(), freq.cpu(), rep.cpu())
    assert torch.equal(tok2.long().cpu(), z.argmax(-1))
    # stochastic rows: draws stay inside the top-k / top-p set and follow the distribution
    temp = torch.full((R_,), 0.8, device="cuda")
    topk = torch.full((R_,), 5, dtype=torch.int32, device="cuda")
    topp = torch.full((R_,), 0.9, device="cuda")
    seeds = torch.arange(R_, dtype=torch.int64, device="cuda") + 100
    hist = torch.zeros(V)
    top5 = logits.float().topk(5, -1).indices.cpu()
    for step in range(200):
        steps = torch.full((R_,), step, dtype=torch.int32, device="cuda")
        t, _ = S.sample(logits, temperature=temp, top_k=topk, top_p=topp, seeds=seeds, steps=steps)
        t = t.long().cpu()
        assert all(int(t[r]) in top5[r].tolist() for r in range(R_))
        hist[t[0]] += 1
    p = torch.softmax(logits[0].float().cpu()[top5[0]] / 0.8, -1)
    assert hist[top5[0][0]] / 200 > 0.5 * float(p[0])
    # same seed and step -> same draw
    steps = torch.zeros(R_, dtype=torch.int32, device="cuda")
    a, _ = S.sample(logits, temperature=temp, top_k=topk, seeds=seeds, steps=steps)
    b, _ = S.sample(logits, temperature=temp, top_k=topk, seeds=seeds, steps=steps)
    assert torch.equal(a, b)


@pytest.mark.parametrize("splits", [2, 4, 7])
def test_split_kv_decode_matches_unsplit(splits):
    """Long contexts cut into page ranges and merged by log-sum-exp give the same output as one pass."""
    from easydel_b200.ops import serving as S

    torch.manual_seed(0)
    dev = "cuda"
    B, Hq, Hkv, D, P = 3, 8, 2, 128, 64
    k_pages = torch.randn(P, 128, Hkv, D, device=dev, dtype=torch.bfloat16)
    v_pages = torch.randn(P, 128, Hkv, D, device=dev, dtype=torch.bfloat16)
    kv_lens = torch.tensor([2000, 130, 901], dtype=torch.int32, device=dev)
    table = torch.zeros(B, 16, dtype=torch.int32, device=dev)
    perm = torch.randperm(P - 1, device=dev)[:48].to(torch.int32) + 1
    table[:, :16] = perm.view(3, 16)
    q = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    sinks = torch.randn(Hq, device=dev)
    for sk in (None, sinks):
        ref = S.paged_attention_reference(q, k_pages, v_pages, cu, kv_lens, table, causal=True, sinks=sk)
        got = S.paged_attention_splitkv(q, k_pages, v_pages, kv_lens, table, splits, sinks=sk)
        assert (got.float() - ref.float()).abs().max() < 2e-2


def test_attn_combine_matches_reference():
    from easydel_b200.ops import serving as S

    torch.manual_seed(1)
    o = torch.randn(3, 5, 4, 64, device="cuda", dtype=torch.bfloat16)
    lse = torch.randn(3, 4, 5, device="cuda")
    lse[1, :, 2] = float("-inf")
    got, l = S.attn_combine(o, lse, want_lse=True)
    ref, lr = S.attn_combine(o.cpu(), lse.cpu(), want_lse=True)
    assert (got.float().cpu() - ref.float()).abs().max() < 2e-2 and (l.cpu() - lr).abs().max() < 1e-4


def test_greedy_sampler_fast_path_matches_argmax():
    from easydel_b200.ops import serving as S

    torch.manual_seed(2)
    logits = torch.randn(37, 128256, device="cuda", dtype=torch.bfloat16)
    tok, lp = S.sample(logits, want_logprob=True)
    ref = logits.float().argmax(-1)
    assert torch.equal(tok.long(), ref)
    ref_lp = torch.log_softmax(logits.float(), -1).gather(-1, ref[:, None])[:, 0]
    assert (lp - ref_lp).abs().max() < 1e-3


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 1, 128), (32, 8, 128), (4, 4, 64), (16, 1, 128), (12, 4, 64)])
@pytest.mark.parametrize("splits,window", [(1, 0), (3, 0), (1, 200)])
def test_streaming_decode_attention(Hq, Hkv, D, splits, window):
    """The decode kernel (one query token per sequence, 32-key tiles streamed per warp) against the reference, with
    ragged key counts (1 key, a count inside a tile, several pages), key splits and a sliding window."""
    from easydel_b200.ops import serving as S

    P = 48
    kp, vp = _pool(P, Hkv, D, 5)
    kv_lens = [1, 31, 33, 128, 129, 777, 1500, 5]
    B = len(kv_lens)
    perm = torch.randperm(P, generator=torch.Generator().manual_seed(8)).tolist()
    maxp = max((L + 127) // 128 for L in kv_lens)
    table = torch.zeros(B, maxp, dtype=torch.int32)
    nxt = 0
    for b, L in enumerate(kv_lens):
        n = (L + 127) // 128
        table[b, :n] = torch.tensor(perm[nxt:nxt + n], dtype=torch.int32)
        nxt += n
    q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
    sinks = torch.randn(Hq, device="cuda") if window == 0 and splits == 1 else None
    lens = torch.tensor(kv_lens, dtype=torch.int32)
    o = S.decode_attention(q, kp, vp, lens.cuda(), table.cuda(), window=window, sinks=sinks, num_splits=splits)
    ref = S.paged_attention_reference(q.cpu(), kp.cpu(), vp.cpu(), torch.arange(B + 1, dtype=torch.int32), lens, table,
                                      window=window, sinks=None if sinks is None else sinks.cpu())
    err = (o.float().cpu() - ref.float()).abs().max().item()
    assert torch.allclose(o.float().cpu(), ref.float(), atol=2e-2, rtol=2e-2), err


@pytest.mark.parametrize("B,H,ctx,splits", [(5, 16, [1, 31, 128, 700, 2049], 1), (3, 40, [513, 64, 900], 1),
                                            (2, 16, [3000, 33], 4)])
def test_latent_decode_attention_kernel(B, H, ctx, splits):
    """Absorbed-form latent attention for decode steps: 576-wide scores and 512-wide value sums over the same paged
    rows, against fp32 softmax attention over the gathered rows."""
    from easydel_b200.ops import serving as S

    torch.manual_seed(0)
    dev = "cuda"
    pages_per = (max(ctx) + 127) // 128
    P = B * pages_per + 1
    pages = (torch.randn(P, 128, 1, 576, device=dev) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(P - 1, device=dev)[: B * pages_per] + 1
    table = perm.view(B, pages_per).to(torch.int32)
    lens = torch.tensor(ctx, dtype=torch.int32, device=dev)
    q = (torch.randn(B, H, 576, device=dev) * 0.5).to(torch.bfloat16)
    scale = 0.07
    o = S.mla_decode_attention(q, pages, lens, table, scale=scale, num_splits=splits)
    for b in range(B):
        rows = pages[table[b].long()].reshape(-1, 576)[: ctx[b]].float()
        s = (q[b].float() @ rows.t()) * scale
        ref = torch.softmax(s, -1) @ rows[:, :512]
        err = (o[b].float() - ref).abs().max() / ref.abs().max()
        assert err < 2e-2, (b, float(err))
