"""``model.generate``: greedy / sampling / beam decoding over the dense KV cache.

The reference implements these as ``lax.while_loop`` programs (easydel/infra/mixins/generation.py:3418-4400);
here they are host loops: one prefill call, then one single-token call per step, sampling with the
same kernel the serving engine uses.
"""

from __future__ import annotations

import torch

from ..infra.modeling_outputs import BeamSearchOutput, GreedySearchOutput, SampleOutput
from ..ops import serving as S


def _as_list(x):
    if x is None:
        return []
    return list(x) if isinstance(x, (list, tuple)) else [x]


@torch.no_grad()
def generate(model, input_ids, attention_mask=None, max_new_tokens=None, max_length=None, do_sample=False,
             temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repetition_penalty=1.0, eos_token_id=None,
             pad_token_id=None, num_beams=1, seed=None, generation_config=None):
    dev = model.device
    input_ids = input_ids.to(dev)
    if input_ids.dim() == 1:
        input_ids = input_ids[None]
    B, T = input_ids.shape
    if generation_config is not None:
        max_new_tokens = max_new_tokens or getattr(generation_config, "max_new_tokens", None)
        eos_token_id = eos_token_id if eos_token_id is not None else getattr(generation_config, "eos_token_id", None)
    if max_new_tokens is None:
        max_new_tokens = (max_length - T) if max_length else 32
    eos = set(_as_list(eos_token_id if eos_token_id is not None else getattr(model.config, "eos_token_id", None)))
    pad = pad_token_id if pad_token_id is not None else (getattr(model.config, "pad_token_id", None) or 0)
    if num_beams > 1:
        return _beam_search(model, input_ids, max_new_tokens, num_beams, eos, pad)
    was_training = model.training
    model.eval()
    cache = model.init_cache(B, T + max_new_tokens)
    meta = None
    pos = None
    if attention_mask is not None and not bool(attention_mask.all()):
        attention_mask = attention_mask.to(dev)
        pos = (attention_mask.long().cumsum(-1) - 1).clamp_min(0)
        seg = torch.ones(B, T + max_new_tokens, dtype=torch.int32, device=dev)
        seg[:, :T] = attention_mask.to(torch.int32)
        meta = {"kv_segment_ids": seg}
    out = model(input_ids=input_ids, position_ids=pos, past_key_values=cache, cache_metadata=meta)
    cache.advance(T)
    logits = out.logits[:, -1]
    seqs = input_ids
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    counts = None
    if repetition_penalty != 1.0:
        counts = torch.zeros(B, logits.shape[-1], dtype=torch.int32, device=dev)
        counts.scatter_add_(1, input_ids, torch.ones_like(input_ids, dtype=torch.int32))
    next_pos = pos[:, -1] + 1 if pos is not None else None
    for step in range(max_new_tokens):
        kw = {}
        if do_sample:
            kw = dict(temperature=torch.full((B,), float(temperature), device=dev),
                      top_k=torch.full((B,), int(top_k), dtype=torch.int32, device=dev),
                      top_p=torch.full((B,), float(top_p), device=dev),
                      min_p=torch.full((B,), float(min_p), device=dev),
                      seeds=torch.arange(B, dtype=torch.int64, device=dev) + (seed or 0),
                      steps=torch.full((B,), step, dtype=torch.int32, device=dev))
        if counts is not None:
            kw.update(repetition=torch.full((B,), float(repetition_penalty), device=dev), counts=counts)
        lg = logits if logits.dtype in (torch.bfloat16, torch.float32) else logits.float()
        tok, _ = S.sample(lg.contiguous(), **kw)
        tok = tok.long().to(dev)
        tok = torch.where(done, torch.full_like(tok, pad), tok)
        seqs = torch.cat([seqs, tok[:, None]], dim=1)
        if counts is not None:
            counts.scatter_add_(1, tok[:, None], torch.ones(B, 1, dtype=torch.int32, device=dev))
        if eos:
            done |= torch.isin(tok, torch.tensor(sorted(eos), device=dev))
            if bool(done.all()):
                break
        if step == max_new_tokens - 1:
            break
        p = next_pos[:, None] if next_pos is not None else None
        out = model(input_ids=tok[:, None], position_ids=p, past_key_values=cache, cache_metadata=meta)
        cache.advance(1)
        if next_pos is not None:
            next_pos = next_pos + 1
        logits = out.logits[:, -1]
    if was_training:
        model.train()
    return (SampleOutput if do_sample else GreedySearchOutput)(sequences=seqs)


def _beam_search(model, input_ids, max_new_tokens, num_beams, eos, pad):
    dev = model.device
    B, T = input_ids.shape
    ids = input_ids.repeat_interleave(num_beams, dim=0)
    cache = model.init_cache(B * num_beams, T + max_new_tokens)
    out = model(input_ids=ids, past_key_values=cache)
    cache.advance(T)
    lp = torch.log_softmax(out.logits[:, -1].float(), -1)
    scores = torch.zeros(B, num_beams, device=dev)
    scores[:, 1:] = -1e9
    done = torch.zeros(B * num_beams, dtype=torch.bool, device=dev)
    seqs = ids
    V = lp.shape[-1]
    for step in range(max_new_tokens):
        lp = torch.where(done[:, None], torch.full_like(lp, -1e9), lp)
        if done.any():
            lp[done, pad] = 0.0
        cand = (scores.view(-1, 1) + lp).view(B, num_beams * V)
        top, idx = cand.topk(num_beams, dim=-1)
        beam, tok = idx // V, idx % V
        base = (torch.arange(B, device=dev) * num_beams)[:, None]
        sel = (base + beam).view(-1)
        seqs = torch.cat([seqs[sel], tok.view(-1, 1)], dim=1)
        cache.reorder(sel)
        done = done[sel]
        scores = top
        if eos:
            done |= torch.isin(tok.view(-1), torch.tensor(sorted(eos), device=dev))
        if bool(done.all()) or step == max_new_tokens - 1:
            break
        out = model(input_ids=tok.view(-1, 1), past_key_values=cache)
        cache.advance(1)
        lp = torch.log_softmax(out.logits[:, -1].float(), -1)
    best = scores.argmax(-1)
    pick = (torch.arange(B, device=dev) * num_beams + best)
    return BeamSearchOutput(sequences=seqs[pick], scores=scores.gather(1, best[:, None]).squeeze(1))
