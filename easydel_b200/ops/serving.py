"""Python entry points of the serving kernels (paged attention, KV append, sampling)."""

from __future__ import annotations

import math

import torch

from . import _lib

vp, i32, i64, f32 = _lib.vp, _lib.i32, _lib.i64, _lib.f32
_lib.register("edl_attn_paged", i32, [vp, vp, vp, vp, i64, i64, i64, vp, vp, vp, i32, i32, i32, i64, i64, i32, i32,
                                      i32, f32, i32, i32, f32, vp, vp, vp])
_lib.register("edl_paged_kv_append", i32, [vp, vp, vp, vp, vp, i32, i32, i64, i64, i64, i64, vp, vp])
_lib.register("edl_sample", i32, [vp, i32, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, vp, vp, vp, vp, vp])
_lib.register("edl_count_update", i32, [vp, i64, vp, vp, i32, i32, vp])
_lib.register("edl_gather_rows", i32, [vp, vp, vp, i32, i32, i64, vp])

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
