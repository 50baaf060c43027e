"""Python entry points of the serving kernels (paged attention, KV append, sampling)."""

from __future__ import annotations

import math

import torch

from . import _lib

vp, i32, i64, f32 = _lib.vp, _lib.i32, _lib.i64, _lib.f32
_lib.register("edl_attn_paged_lse", i32, [vp, vp, vp, vp, vp, i64, i64, i64, vp, vp, vp, i32, i32, i32, i64, i64, i32,
                                          i32, i32, _lib.f32, i32, i32, _lib.f32, vp, vp, vp])
_lib.register("edl_attn_combine", i32, [vp, i64, vp, i32, i32, i32, i32, vp, vp, vp, vp])
_lib.register("edl_attn_paged", i32, [vp, vp, vp, vp, i64, i64, i64, vp, vp, vp, i32, i32, i32, i64, i64, i32, i32,
                                      i32, f32, i32, i32, f32, vp, vp, vp])
_lib.register("edl_paged_kv_append", i32, [vp, vp, vp, vp, vp, i32, i32, i64, i64, i64, i64, vp, vp])
_lib.register("edl_sample", i32, [vp, i32, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, vp, vp, vp, vp, vp])
_lib.register("edl_count_update", i32, [vp, i64, vp, vp, i32, i32, vp])
_lib.register("edl_gather_rows", i32, [vp, vp, vp, i32, i32, i64, vp])
_lib.register("edl_attn_decode", i32, [vp, vp, vp, vp, vp, i64, i64, i64, vp, vp, i32, i32, i64, i32, i32, i32, f32,
                                       i32, i32, vp, vp, vp])

_lib.register("edl_attn_mla_decode", i32, [vp, vp, vp, vp, i64, i64, vp, vp, i32, i32, i64, i32, f32, i32, vp, vp])

PAGE_SIZE = 128


def kv_append(k: torch.Tensor, v: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
              slot_mapping: torch.Tensor) -> None:
    """Writes new key/value rows ``[T, Hkv, D]`` into the page pools ``[P, page, Hkv, D]`` at flat slots."""
    T = k.shape[0]
    width = k.shape[-2] * k.shape[-1]
    if k.is_cuda:
        assert k.stride(-1) == 1 and k.stride(-2) == k.shape[-1] and v.stride(-2) == v.shape[-1]
        ld_page = k_pages.stride(1)
        _lib.call("edl_paged_kv_append", k.data_ptr(), v.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                  slot_mapping.data_ptr(), T, width, k.stride(0), v.stride(0), ld_page,
                  k_pages.shape[0] * k_pages.shape[1], _lib.status_word(k.device).data_ptr(), _lib.stream_ptr())
        return
    flat_k = k_pages.view(-1, *k_pages.shape[2:])
    flat_v = v_pages.view(-1, *v_pages.shape[2:])
    ok = slot_mapping >= 0
    idx = slot_mapping[ok].long()
    flat_k[idx] = k[ok].to(flat_k.dtype)
    flat_v[idx] = v[ok].to(flat_v.dtype)


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, cu_q: torch.Tensor,
                    kv_lens: torch.Tensor, page_table: torch.Tensor, max_q: int, *, scale: float | None = None,
                    causal: bool = True, window: int = 0, softcap: float = 0.0, sinks=None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """Mixed prefill/decode attention over a paged KV cache.

    q ``[T, Hq, D]`` (new tokens of all sequences, concatenated), pages ``[P, 128, Hkv, D]``,
    ``cu_q`` int32 ``[B+1]``, ``kv_lens`` int32 ``[B]`` (cached + new keys), ``page_table`` int32 ``[B, maxP]``.
    """
    T, Hq, D = q.shape
    Hkv = k_pages.shape[2]
    B = kv_lens.numel()
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if q.is_cuda:
        assert k_pages.shape[1] == PAGE_SIZE, "the paged kernels use pages of 128 tokens"
        assert q.stride(-1) == 1 and q.stride(-2) == D
        if out is None:
            out = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
        _lib.call("edl_attn_paged", q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                  q.stride(0), k_pages.stride(1), out.stride(0), cu_q.data_ptr(), kv_lens.data_ptr(),
                  page_table.data_ptr(), page_table.stride(0), B, int(max_q), T, k_pages.shape[0], Hq, Hkv, D,
                  float(scale), int(causal), int(window or 0), float(softcap or 0.0), _lib.ptr(sinks),
                  _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
        return out
    return paged_attention_reference(q, k_pages, v_pages, cu_q, kv_lens, page_table, scale=scale, causal=causal,
                                     window=window, softcap=softcap, sinks=sinks)


def decode_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, kv_lens: torch.Tensor,
                     page_table: torch.Tensor, *, scale: float | None = None, window: int = 0, sinks=None,
                     num_splits: int = 1) -> torch.Tensor:
    """Decode-step attention (one query token per sequence) with the streaming kernel of
    ``csrc/attention_decode.cu``. q ``[B, Hq, D]``; pages ``[P, 128, Hkv, D]``; ``num_splits`` cuts every
    sequence's keys into that many parts that run as separate CTAs and are merged by :func:`attn_combine`."""
    B, Hq, D = q.shape
    Hkv = k_pages.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    S_ = max(1, int(num_splits))
    out = torch.empty((S_, B, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((S_, Hq, B), dtype=torch.float32, device=q.device) if S_ > 1 else None
    _lib.call("edl_attn_decode", q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), _lib.ptr(lse),
              q.stride(0), k_pages.stride(1), Hq * D, kv_lens.data_ptr(), page_table.data_ptr(),
              page_table.stride(0), B, k_pages.shape[0], Hq, Hkv, D, float(scale), int(window or 0), S_,
              _lib.ptr(sinks) if S_ == 1 else None, _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
    if S_ == 1:
        return out[0]
    return attn_combine(out, lse, sinks=sinks)


def mla_decode_attention(q: torch.Tensor, pages: torch.Tensor, kv_lens: torch.Tensor, page_table: torch.Tensor, *,
                         scale: float, num_splits: int = 1) -> torch.Tensor:
    """Decode-step latent attention in the absorbed form (``csrc/attention_mla_decode.cu``).

    q ``[B, H, 576]`` = (query folded through the key up-projection (512) | rotated rotary query (64)); pages
    ``[P, 128, 1, 576]`` rows (compressed key/value | rotated rotary key). Returns ``[B, H, 512]``: the
    softmax-weighted sums of the rows' compressed part, to be sent through the value up-projection."""
    B, H, W = q.shape
    assert W == 576 and pages.shape[-1] == 576 and pages.shape[1] == PAGE_SIZE and q.is_contiguous()
    S_ = max(1, int(num_splits))
    out = torch.empty((S_, B, H, 512), dtype=q.dtype, device=q.device)
    lse = torch.empty((S_, H, B), dtype=torch.float32, device=q.device) if S_ > 1 else None
    _lib.call("edl_attn_mla_decode", q.data_ptr(), pages.data_ptr(), out.data_ptr(), _lib.ptr(lse), H * 576, H * 512,
              kv_lens.data_ptr(), page_table.data_ptr(), page_table.stride(0), B, pages.shape[0], H, float(scale), S_,
              _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
    if S_ == 1:
        return out[0]
    return attn_combine(out, lse)


def mla_decode_kernel_supports(q: torch.Tensor, pages: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and pages.dtype == torch.bfloat16 and q.shape[-1] == 576
            and pages.shape[-1] == 576 and pages.shape[1] == PAGE_SIZE and pages.is_contiguous())


def decode_kernel_supports(q: torch.Tensor, k_pages: torch.Tensor, softcap: float) -> bool:
    Hq, D = q.shape[-2], q.shape[-1]
    Hkv = k_pages.shape[2]
    return (q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and Hq % Hkv == 0 and Hq // Hkv <= 16
            and not softcap and k_pages.shape[1] == PAGE_SIZE and q.stride(-1) == 1 and q.stride(-2) == D)


def attn_combine(o_parts: torch.Tensor, lse_parts: torch.Tensor, sinks=None, want_lse: bool = False):
    """Merges ``o_parts [S, R, H, D]`` with ``lse_parts [S, H, R]`` (disjoint key ranges) into ``[R, H, D]``."""
    S_, R_, H, D = o_parts.shape
    if o_parts.is_cuda:
        o_parts = o_parts.contiguous()      # strides of size-1 dimensions are arbitrary: pass the dense pitch
        out = torch.empty(R_, H, D, dtype=o_parts.dtype, device=o_parts.device)
        lse = torch.empty(H, R_, dtype=torch.float32, device=o_parts.device) if want_lse else None
        _lib.call("edl_attn_combine", o_parts.data_ptr(), R_ * H * D, lse_parts.contiguous().data_ptr(), S_, R_,
                  H, D, _lib.ptr(sinks), out.data_ptr(), _lib.ptr(lse), _lib.stream_ptr())
        return (out, lse) if want_lse else out
    l = lse_parts.float().permute(0, 2, 1)                      # [S, R, H]
    if sinks is not None:
        l_all = torch.cat([l, sinks.float()[None, None].expand(1, R_, H)], 0)
    else:
        l_all = l
    tot = torch.logsumexp(l_all, 0)                             # [R, H]
    w = torch.exp(l - tot[None]).nan_to_num(0.0)
    out = (w[..., None] * o_parts.float()).sum(0).to(o_parts.dtype)
    return (out, tot.t().contiguous()) if want_lse else out


def paged_attention_splitkv(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, kv_lens: torch.Tensor,
                            page_table: torch.Tensor, num_splits: int, *, scale: float | None = None,
                            softcap: float = 0.0, sinks=None) -> torch.Tensor:
    """Decode attention (one query token per sequence) with every sequence's keys cut into ``num_splits`` page
    ranges that run as independent rows of the paged kernel and are merged by :func:`attn_combine`.

    With few sequences and long contexts the plain kernel has ``B * Hkv`` CTAs walking thousands of keys each;
    splitting gives the idle SMs work. q ``[B, Hq, D]``; the page table's width is padded to a multiple of
    ``num_splits`` pages so that each split is a strided view of it.
    """
    B, Hq, D = q.shape
    S_ = int(num_splits)
    MP = page_table.shape[1]
    cp = (MP + S_ - 1) // S_
    if cp * S_ != MP:
        page_table = torch.nn.functional.pad(page_table, (0, cp * S_ - MP))
    pt = page_table.contiguous().view(B * S_, cp)
    chunk = cp * PAGE_SIZE
    starts = torch.arange(S_, device=q.device, dtype=torch.int32) * chunk
    lens = (kv_lens.to(torch.int32)[:, None] - starts[None]).clamp(0, chunk).reshape(-1).contiguous()
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        o = paged_attention_reference(q, k_pages, v_pages, torch.arange(B + 1, dtype=torch.int32), kv_lens,
                                      page_table[:, :MP], scale=scale, causal=True, softcap=softcap, sinks=sinks)
        return o
    qr = q.repeat_interleave(S_, 0).contiguous()
    cu = torch.arange(B * S_ + 1, device=q.device, dtype=torch.int32)
    o_parts = torch.empty(B * S_, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(Hq, B * S_, dtype=torch.float32, device=q.device)
    _lib.call("edl_attn_paged_lse", qr.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), o_parts.data_ptr(),
              lse.data_ptr(), qr.stride(0), k_pages.stride(1), o_parts.stride(0), cu.data_ptr(), lens.data_ptr(),
              pt.data_ptr(), pt.stride(0), B * S_, 1, B * S_, k_pages.shape[0], Hq, k_pages.shape[2], D, float(scale),
              1, 0, float(softcap or 0.0), None, _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
    # [B*S, Hq, D] -> [S, B, Hq, D]; lse [Hq, B*S] -> [S, Hq, B]
    op = o_parts.view(B, S_, Hq, D).transpose(0, 1).contiguous()
    lp = lse.view(Hq, B, S_).permute(2, 0, 1).contiguous()
    return attn_combine(op, lp, sinks)


def paged_attention_reference(q, k_pages, v_pages, cu_q, kv_lens, page_table, *, scale=None, causal=True, window=0,
                              softcap=0.0, sinks=None):
    """Dense oracle: gathers each sequence's keys/values from its pages and runs reference attention."""
    from . import reference as R

    page = k_pages.shape[1]
    outs = []
    cu = cu_q.tolist()
    for b, L in enumerate(kv_lens.tolist()):
        qs = q[cu[b]:cu[b + 1]]
        if qs.shape[0] == 0:
            continue
        n_pages = (L + page - 1) // page
        ids = page_table[b, :n_pages].long()
        ks = k_pages[ids].reshape(-1, *k_pages.shape[2:])[:L]
        vs = v_pages[ids].reshape(-1, *v_pages.shape[2:])[:L]
        o = R.attention(qs[None], ks[None].to(qs.dtype), vs[None].to(qs.dtype), causal=causal, scale=scale,
                        sliding_window=window or None, softcap=softcap, sinks=sinks)
        outs.append(o[0])
    return torch.cat(outs, dim=0)


def sample(logits: torch.Tensor, *, temperature=None, top_k=None, top_p=None, min_p=None, presence=None,
           frequency=None, repetition=None, counts=None, seeds=None, steps=None, want_logprob: bool = False):
    """Samples one token per row of ``[R, V]`` logits. All per-row parameter tensors are optional
    (absent = greedy, no penalties). Returns (tokens int32 [R], logprobs fp32 [R] or None)."""
    R_, V = logits.shape
    if logits.is_cuda:
        assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
        out = torch.empty(R_, dtype=torch.int32, device=logits.device)
        lp = torch.empty(R_, dtype=torch.float32, device=logits.device) if want_logprob else None
        _lib.call("edl_sample", logits.data_ptr(), int(logits.dtype == torch.float32), logits.stride(0), R_, V,
                  _lib.ptr(temperature), _lib.ptr(top_k), _lib.ptr(top_p), _lib.ptr(min_p), _lib.ptr(presence),
                  _lib.ptr(frequency), _lib.ptr(repetition), _lib.ptr(counts),
                  counts.stride(0) if counts is not None else 0, _lib.ptr(seeds), _lib.ptr(steps), out.data_ptr(),
                  _lib.ptr(lp), _lib.stream_ptr())
        return out, lp
    return sample_reference(logits, temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                            presence=presence, frequency=frequency, repetition=repetition, counts=counts,
                            seeds=seeds, steps=steps, want_logprob=want_logprob)


def apply_penalties_reference(z: torch.Tensor, counts, presence, frequency, repetition) -> torch.Tensor:
    z = z.float().clone()
    if counts is None:
        return z
    seen = counts[: z.shape[0], : z.shape[1]] > 0
    if repetition is not None:
        rep = repetition[:, None]
        z = torch.where(seen, torch.where(z > 0, z / rep, z * rep), z)
    c = counts[: z.shape[0], : z.shape[1]].float()
    if presence is not None:
        z = z - presence[:, None] * seen
    if frequency is not None:
        z = z - frequency[:, None] * c
    return z


def sample_reference(logits, *, temperature=None, top_k=None, top_p=None, min_p=None, presence=None, frequency=None,
                     repetition=None, counts=None, seeds=None, steps=None, want_logprob=False):
    """CPU oracle with the kernel's order: penalties -> top-k (<= 64) -> temperature -> top-p -> min-p -> draw."""
    z = apply_penalties_reference(logits, counts, presence, frequency, repetition)
    R_, V = z.shape
    out = torch.empty(R_, dtype=torch.int32)
    lps = torch.empty(R_, dtype=torch.float32)
    for r in range(R_):
        t = float(temperature[r]) if temperature is not None else 0.0
        k = int(top_k[r]) if top_k is not None else 0
        if t <= 0 or k == 1:
            i = int(torch.argmax(z[r]))
            out[r] = i
            lps[r] = torch.log_softmax(z[r], -1)[i]
            continue
        k = 64 if (k <= 0 or k > 64) else k
        vals, idx = torch.topk(z[r], min(k, V))
        p = torch.softmax(vals / t, -1)
        keep = torch.ones_like(p, dtype=torch.bool)
        tp = float(top_p[r]) if top_p is not None else 1.0
        mp = float(min_p[r]) if min_p is not None else 0.0
        cum = torch.cumsum(p, 0) - p
        keep &= (cum < tp)
        keep &= p >= mp * p[0]
        keep[0] = True
        p = torch.where(keep, p, torch.zeros_like(p))
        g = torch.Generator().manual_seed(int(seeds[r]) + 7919 * int(steps[r] if steps is not None else 0)
                                          if seeds is not None else r)
        j = int(torch.multinomial(p / p.sum(), 1, generator=g))
        out[r] = int(idx[j])
        lps[r] = torch.log_softmax(z[r] / t, -1)[idx[j]]
    return out, (lps if want_logprob else None)


def count_update(counts: torch.Tensor, tokens: torch.Tensor, row_slots: torch.Tensor | None = None) -> None:
    if counts.is_cuda:
        _lib.call("edl_count_update", counts.data_ptr(), counts.stride(0), tokens.data_ptr(), _lib.ptr(row_slots),
                  tokens.numel(), counts.shape[1], _lib.stream_ptr())
        return
    rows = row_slots.long() if row_slots is not None else torch.arange(tokens.numel())
    ok = (tokens >= 0) & (rows >= 0)
    counts.index_put_((rows[ok], tokens[ok].long()), torch.ones(int(ok.sum()), dtype=counts.dtype), accumulate=True)


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``src[idx]`` for a 2-D bf16 matrix (last hidden state of every sequence)."""
    if src.is_cuda and src.dtype == torch.bfloat16:
        out = torch.empty((idx.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
        _lib.call("edl_gather_rows", src.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), src.shape[1],
                  src.stride(0), _lib.stream_ptr())
        return out
    return src[idx.long()]
