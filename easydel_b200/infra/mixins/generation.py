"""Text generation on top of a model: cache factories, ``generate`` and the eSurge hand-off.

Covers the surface of easydel/infra/mixins/generation.py:1116-5492 (``init_cache``,
``prepare_inputs_for_generation``, greedy / sampling / beam ``generate``, ``get_esurge``,
``esurge_generate``). The decoding loops are host loops over CUDA kernels (optionally replayed
from a CUDA graph by the serving engine) rather than traced ``while_loop`` programs.
"""

from __future__ import annotations

import typing as tp

import torch


class EasyGenerationMixin:
    # ------------------------------------------------------------------ caches
    def init_cache(self, batch_size: int, max_length: int, dtype=None, device=None, **_):
        from ...caching.transformer import TransformerCache

        spec = getattr(self, "spec", None)
        if spec is not None and getattr(spec, "mla", None) is not None:
            from ...layers.mla import MLACache

            cache = MLACache(spec.num_layers, batch_size, max_length, spec.mla["kv_lora_rank"],
                             spec.mla["qk_rope_head_dim"], dtype or self.dtype, device or self.device)
            for i, layer in enumerate(getattr(getattr(self, "model", self), "layers", ())):
                mixer = getattr(layer, "linear_attn", None)
                if mixer is not None:     # hybrids: recurrent state of the linear-attention layers
                    cache.linear[i] = mixer.make_state(batch_size, dtype or self.dtype, device or self.device)
            return cache
        return TransformerCache.init_for_model(self, batch_size, max_length, dtype=dtype, device=device)

    def init_ragged_pages(self, num_pages: int | None = None, page_size: int = 128, hbm_utilization: float = 0.85,
                          max_model_length: int | None = None, dtype=None, device=None, **_):
        from ...caching.paged import PagedKVCache

        return PagedKVCache.init_for_model(self, num_pages=num_pages, page_size=page_size,
                                           hbm_utilization=hbm_utilization, max_model_length=max_model_length,
                                           dtype=dtype, device=device)

    init_unified_attention_cache = init_ragged_pages
    init_operations_cache = init_cache

    def prepare_inputs_for_generation(self, input_ids: torch.Tensor, max_length: int,
                                      attention_mask: torch.Tensor | None = None, **_):
        B, T = input_ids.shape
        cache = self.init_cache(B, max_length)
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        position_ids = (attention_mask.long().cumsum(-1) - 1).clamp_min(0)
        return {"past_key_values": cache, "attention_mask": attention_mask, "position_ids": position_ids}

    # ------------------------------------------------------------------ generate
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None,
                 max_new_tokens: int | None = None, max_length: int | None = None, do_sample: bool = False,
                 temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
                 repetition_penalty: float = 1.0, eos_token_id: int | list[int] | None = None,
                 pad_token_id: int | None = None, num_beams: int = 1, seed: int | None = None,
                 generation_config=None, **_):
        """Greedy / sampled / beam decoding with a dense KV cache. Returns an output with ``sequences``."""
        from ...inference.generate_loop import generate as _generate

        return _generate(self, input_ids, attention_mask=attention_mask, max_new_tokens=max_new_tokens,
                         max_length=max_length, do_sample=do_sample, temperature=temperature, top_k=top_k,
                         top_p=top_p, min_p=min_p, repetition_penalty=repetition_penalty, eos_token_id=eos_token_id,
                         pad_token_id=pad_token_id, num_beams=num_beams, seed=seed,
                         generation_config=generation_config)

    # ------------------------------------------------------------------ eSurge
    @property
    def esurge_compatible_model(self):
        return self

    def get_esurge(self, tokenizer=None, **kw):
        from ...inference.esurge import eSurge

        eng = getattr(self, "_esurge_engine", None)
        if eng is None or kw.pop("force_new", False):
            eng = eSurge(model=self, tokenizer=tokenizer, **kw)
            object.__setattr__(self, "_esurge_engine", eng)
        return eng

    def esurge_generate(self, prompts, tokenizer=None, sampling_params=None, stream: bool = False, **kw):
        eng = self.get_esurge(tokenizer=tokenizer, **kw)
        if stream:
            return eng.stream(prompts, sampling_params)
        return eng.generate(prompts, sampling_params)

    def pause_esurge(self):
        eng = getattr(self, "_esurge_engine", None)
        if eng is not None:
            eng.pause()

    def resume_esurge(self):
        eng = getattr(self, "_esurge_engine", None)
        if eng is not None:
            eng.resume()
