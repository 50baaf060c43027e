"""Saving, loading and converting models (``save_pretrained`` / ``from_pretrained`` / ``push_to_hub``).

Implements the behaviour of easydel/infra/mixins/bridge.py:557-2919 on top of the checkpoint
package :mod:`easydel_b200.io`: the on-disk layout is the reference's (``config.json``,
``generation_config.json``, ``README.md``, ``tensorstore_index.json`` and one zarr array per
parameter under ``model/``), Hugging Face safetensors checkpoints are converted on load.
"""

from __future__ import annotations

import os
import typing as tp

import torch


class EasyBridgeMixin:
    def save_pretrained(self, save_directory: str | os.PathLike, push_to_hub: bool = False, float_dtype=None,
                        gather_fns=None, verbose: bool = True, step: int | None = None, **kwargs):
        from ...io.checkpoint import save_model

        return save_model(self, str(save_directory), float_dtype=float_dtype, step=step, **kwargs)

    def push_to_hub(self, repo_id: str, **kwargs):
        raise RuntimeError("push_to_hub needs network access to the Hugging Face hub, which this environment "
                           "does not have; save_pretrained() the model and upload the directory instead.")

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str | os.PathLike, dtype=torch.bfloat16,
                        param_dtype=None, precision=None, sharding_axis_dims=None, sharding_axis_names=None,
                        sharding_dcn_axis_dims=None, partition_axis=None, config_kwargs: dict | None = None,
                        auto_shard_model: bool = True, partition_rules=None, quantization_config=None,
                        apply_quantization: bool = False, from_torch: bool | None = None, backend=None,
                        platform=None, device=None, verbose: bool = True, **kwargs):
        from ...io.checkpoint import load_model

        return load_model(cls, str(pretrained_model_name_or_path), dtype=dtype, param_dtype=param_dtype,
                          sharding_axis_dims=sharding_axis_dims, sharding_axis_names=sharding_axis_names,
                          sharding_dcn_axis_dims=sharding_dcn_axis_dims, partition_axis=partition_axis,
                          config_kwargs=config_kwargs, auto_shard_model=auto_shard_model,
                          quantization_config=quantization_config, apply_quantization=apply_quantization,
                          from_torch=from_torch, device=device, **kwargs)

    @classmethod
    def _from_torch_pretrained(cls, path: str, **kw):
        kw["from_torch"] = True
        return cls.from_pretrained(path, **kw)

    def can_generate(self) -> bool:
        """True for models with a language-model head and a ``generate`` method (causal LMs, sequence-to-sequence
        and vision-language wrappers); such models get a ``generation_config.json`` next to their weights."""
        if not callable(getattr(self, "generate", None)):
            return False
        lm = getattr(self, "language_model", self)
        return any(hasattr(m, a) for m in (self, lm) for a in ("apply_lm_head", "lm_head", "proj_out"))

    @staticmethod
    def convert_hf_checkpoint_streaming(source: str, out: str, dtype=None, task=None, verbose: bool = False) -> dict:
        """Hugging Face safetensors -> EasyDeL layout tensor by tensor, without building the model
        (:func:`easydel_b200.io.streaming_convert.stream_hf_to_easydel`)."""
        from ...io.streaming_convert import stream_hf_to_easydel

        return stream_hf_to_easydel(source, out, dtype=dtype, task=task, verbose=verbose)
