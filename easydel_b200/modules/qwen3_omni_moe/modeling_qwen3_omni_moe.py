"""Qwen3-Omni-MoE thinker (easydel/modules/qwen3_omni_moe/modeling_qwen3_omni_moe.py:120-660, 3635-4580): the
Qwen3-VL vision tower with DeepStack, a Whisper-style audio tower, and a Qwen3-MoE language model with interleaved
three-stream rotary positions.

Audio tower: the mel frames of every clip are cut into windows of ``2 * n_window`` frames; each window passes three
stride-2 3x3 convolutions over (mel, time) and a linear layer, gets sinusoidal positions that restart in every window,
and the valid frames of all windows are packed into one sequence. Attention is bidirectional inside blocks of
``n_window_infer / (2 * n_window)`` windows of one clip. A LayerNorm and a two-layer projection give one row per
audio placeholder token. Audio tokens advance the three position streams together, like text.

The talker (speech-token language model with its code predictor) and the code-to-waveform decoder of the reference
are separate models downstream of the thinker's hidden states and are not part of this module.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import TaskType, register_config, register_module
from ...ops import functional as F
from ...ops import reference as R
from .._base.vlm import VLMConfig
from ..qwen2_vl.modeling_qwen2_vl import mrope_positions
from ..qwen3_vl.modeling_qwen3_vl import Qwen3VLForConditionalGeneration


@register_config("qwen3_omni_moe_audio_encoder")
class Qwen3OmniMoeAudioEncoderConfig(EasyDeLBaseConfig):
    model_type = "qwen3_omni_moe_audio_encoder"
    hf_config_keys = ("num_mel_bins", "encoder_layers", "encoder_attention_heads", "encoder_ffn_dim", "d_model",
                      "activation_function", "scale_embedding", "max_source_positions", "n_window", "output_dim",
                      "n_window_infer", "conv_chunksize", "downsample_hidden_size")

    def __init__(self, num_mel_bins=128, encoder_layers=32, encoder_attention_heads=20, encoder_ffn_dim=5120,
                 d_model=1280, activation_function="gelu", scale_embedding=False, initializer_range=0.02,
                 max_source_positions=1500, n_window=100, output_dim=3584, n_window_infer=400, conv_chunksize=500,
                 downsample_hidden_size=480, **kw):
        self.num_mel_bins, self.encoder_layers = num_mel_bins, encoder_layers
        self.encoder_attention_heads, self.encoder_ffn_dim, self.d_model = encoder_attention_heads, \
            encoder_ffn_dim, d_model
        self.activation_function, self.scale_embedding = activation_function, scale_embedding
        self.initializer_range, self.max_source_positions = initializer_range, max_source_positions
        self.n_window, self.output_dim, self.n_window_infer = n_window, output_dim, n_window_infer
        self.conv_chunksize, self.downsample_hidden_size = conv_chunksize, downsample_hidden_size
        super().__init__(**kw)


def audio_output_lengths(frames: torch.Tensor) -> torch.Tensor:
    """Tokens produced for ``frames`` mel frames: 13 per full block of 100 frames plus the three stride-2
    convolutions applied to the remainder."""
    rest = frames % 100
    feat = (rest - 1) // 2 + 1
    return ((feat - 1) // 2 + 1 - 1) // 2 + 1 + (frames // 100) * 13


class _AudioLayer(nn.Module):
    def __init__(self, c: Qwen3OmniMoeAudioEncoderConfig, dtype):
        super().__init__()
        d = c.d_model
        self.heads, self.act = c.encoder_attention_heads, c.activation_function
        self.self_attn = nn.Module()
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            setattr(self.self_attn, n, nn.Linear(d, d, dtype=dtype))
        self.self_attn_layer_norm = nn.LayerNorm(d, dtype=dtype)
        self.fc1, self.fc2 = nn.Linear(d, c.encoder_ffn_dim, dtype=dtype), nn.Linear(c.encoder_ffn_dim, d, dtype=dtype)
        self.final_layer_norm = nn.LayerNorm(d, dtype=dtype)

    def forward(self, x, seg):
        T, d = x.shape
        a = self.self_attn
        h = self.self_attn_layer_norm(x)
        q, k, v = (F.linear(h, p.weight, p.bias).view(1, T, self.heads, d // self.heads)
                   for p in (a.q_proj, a.k_proj, a.v_proj))
        o = F.attention(q, k, v, causal=False, segment_ids=seg).reshape(T, d)
        x = x + F.linear(o, a.out_proj.weight, a.out_proj.bias)
        h = R.ACT2FN[self.act](F.linear(self.final_layer_norm(x), self.fc1.weight, self.fc1.bias))
        return x + F.linear(h, self.fc2.weight, self.fc2.bias)


class Qwen3OmniMoeAudioEncoder(nn.Module):
    """``input_features`` ``[mel, total_frames]`` (the clips concatenated along time) + ``feature_lens`` ``[clips]``
    -> ``[total_tokens, output_dim]``."""

    def __init__(self, c: Qwen3OmniMoeAudioEncoderConfig, dtype):
        super().__init__()
        self.cfg = c
        h = c.downsample_hidden_size
        self.conv2d1 = nn.Conv2d(1, h, 3, 2, padding=1, dtype=dtype)
        self.conv2d2 = nn.Conv2d(h, h, 3, 2, padding=1, dtype=dtype)
        self.conv2d3 = nn.Conv2d(h, h, 3, 2, padding=1, dtype=dtype)
        self.conv_out = nn.Linear(h * ((((c.num_mel_bins + 1) // 2 + 1) // 2 + 1) // 2), c.d_model, bias=False,
                                  dtype=dtype)
        self.layers = nn.ModuleList([_AudioLayer(c, dtype) for _ in range(c.encoder_layers)])
        self.ln_post = nn.LayerNorm(c.d_model, dtype=dtype)
        self.proj1 = nn.Linear(c.d_model, c.d_model, dtype=dtype)
        self.proj2 = nn.Linear(c.d_model, c.output_dim, dtype=dtype)
        inc = math.log(10000.0) / (c.d_model // 2 - 1)
        t = torch.arange(c.max_source_positions)[:, None] * torch.exp(-inc * torch.arange(c.d_model // 2))[None]
        self.register_buffer("positional_embedding", torch.cat([t.sin(), t.cos()], 1), persistent=False)

    def forward(self, input_features, feature_lens):
        c = self.cfg
        win = c.n_window * 2
        lens = feature_lens.to(torch.long).cpu()
        n_chunks = torch.ceil(lens / win).long()
        chunk_len = torch.full((int(n_chunks.sum()),), win, dtype=torch.long)
        tail = torch.nn.functional.pad(n_chunks, (1, 0), value=-1).cumsum(0)[1:]
        chunk_len[tail] = lens % win
        chunk_len[chunk_len == 0] = win
        pieces = input_features.T.split(chunk_len.tolist(), dim=0)
        x = nn.utils.rnn.pad_sequence(pieces, batch_first=True).transpose(1, 2)[:, None]      # [chunks, 1, mel, win]
        after = audio_output_lengths(chunk_len)
        dt = self.conv2d1.weight.dtype
        outs = []
        for part in x.to(dt).split(c.conv_chunksize, dim=0):
            y = torch.nn.functional.gelu(self.conv2d1(part))
            y = torch.nn.functional.gelu(self.conv2d2(y))
            outs.append(torch.nn.functional.gelu(self.conv2d3(y)))
        y = torch.cat(outs, 0)
        b, ch, f, t = y.shape
        y = F.linear(y.permute(0, 3, 1, 2).reshape(b, t, ch * f), self.conv_out.weight)
        y = y + self.positional_embedding[:t].to(y.dtype)[None]
        keep = torch.arange(t)[None, :] < after[:, None]
        h = y[keep.to(y.device)]
        # attention blocks: groups of (n_window_infer / win) windows of one clip
        block = t * (c.n_window_infer // win)
        seg, sid = [], 1
        for n in audio_output_lengths(lens).tolist():
            full, rem = divmod(n, block)
            for ln in [block] * full + ([rem] if rem else []):
                seg.append(torch.full((ln,), sid, dtype=torch.int32))
                sid += 1
        seg = torch.cat(seg)[None].to(h.device) if sid > 2 else None
        for layer in self.layers:
            h = layer(h, seg)
        h = self.ln_post(h)
        h = R.ACT2FN[c.activation_function](F.linear(h, self.proj1.weight, self.proj1.bias))
        return F.linear(h, self.proj2.weight, self.proj2.bias)


@register_config("qwen3_omni_moe_thinker")
class Qwen3OmniMoeThinkerConfig(VLMConfig):
    model_type = "qwen3_omni_moe_thinker"
    vision_default, text_default = "qwen3_vl_vision", "qwen3_moe"

    def __init__(self, audio_config=None, vision_config=None, text_config=None, position_id_per_seconds=25,
                 audio_start_token_id=151647, user_token_id=872, audio_token_id=151646, image_token_id=151655,
                 video_token_id=151656, **kw):
        if isinstance(vision_config, dict):
            vision_config = dict(vision_config, model_type="qwen3_vl_vision")
        if isinstance(text_config, dict):
            text_config = dict(text_config, model_type="qwen3_moe")
            rp = text_config.pop("rope_parameters", None)
            if rp:      # one dict in newer checkpoints: base frequency + the three-stream sections
                rp = dict(rp)
                text_config.setdefault("rope_theta", rp.pop("rope_theta", 1000000.0))
                text_config.setdefault("rope_scaling", rp)
            text_config.setdefault("rope_theta", 1000000.0)
            text_config.setdefault("norm_topk_prob", True)
        if audio_config is None:
            audio_config = {}
        if isinstance(audio_config, dict):
            audio_config = Qwen3OmniMoeAudioEncoderConfig(**{k: v for k, v in audio_config.items()
                                                             if k != "model_type"})
        self.audio_config = audio_config
        kw.setdefault("tie_word_embeddings", False)
        kw = self._init_parts(vision_config, text_config, image_token_id, kw)
        self.position_id_per_seconds, self.audio_start_token_id = position_id_per_seconds, audio_start_token_id
        self.user_token_id, self.audio_token_id = user_token_id, audio_token_id
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        super().__init__(**kw)

    def to_dict(self):
        d = super().to_dict()
        d["audio_config"] = self.audio_config.to_dict()
        return d


@register_config("qwen3_omni_moe")
class Qwen3OmniMoeConfig(EasyDeLBaseConfig):
    """Top-level checkpoint configuration: thinker, talker (with its code predictor) and code-to-waveform decoder,
    plus the chat-template and text-to-speech marker ids the hand-over between them needs."""

    model_type = "qwen3_omni_moe"

    def __init__(self, thinker_config=None, talker_config=None, code2wav_config=None, enable_audio_output=False,
                 im_start_token_id=151644, im_end_token_id=151645, tts_pad_token_id=151671, tts_bos_token_id=151672,
                 tts_eos_token_id=151673, system_token_id=8948, user_token_id=872, assistant_token_id=77091, **kw):
        from .speech import Qwen3OmniMoeCode2WavConfig, Qwen3OmniMoeTalkerConfig

        if thinker_config is None:
            thinker_config = {}
        if isinstance(thinker_config, dict):
            thinker_config = Qwen3OmniMoeThinkerConfig(**{k: v for k, v in thinker_config.items()
                                                          if k != "model_type"})
        if isinstance(talker_config, dict):
            talker_config = Qwen3OmniMoeTalkerConfig(**{k: v for k, v in talker_config.items() if k != "model_type"})
        if isinstance(code2wav_config, dict):
            code2wav_config = Qwen3OmniMoeCode2WavConfig(**{k: v for k, v in code2wav_config.items()
                                                            if k != "model_type"})
        self.thinker_config, self.talker_config, self.code2wav_config = thinker_config, talker_config, code2wav_config
        self.enable_audio_output = enable_audio_output
        self.im_start_token_id, self.im_end_token_id = im_start_token_id, im_end_token_id
        self.tts_pad_token_id, self.tts_bos_token_id, self.tts_eos_token_id = tts_pad_token_id, tts_bos_token_id, \
            tts_eos_token_id
        self.system_token_id, self.user_token_id, self.assistant_token_id = system_token_id, user_token_id, \
            assistant_token_id
        super().__init__(**kw)

    def to_dict(self):
        d = super().to_dict()
        d["thinker_config"] = self.thinker_config.to_dict()
        for k in ("talker_config", "code2wav_config"):
            v = getattr(self, k)
            d[k] = v.to_dict() if hasattr(v, "to_dict") else v
        return d


_MERGER_NAMES = [(".ln_q.", ".norm."), (".mlp.0.", ".linear_fc1."), (".mlp.2.", ".linear_fc2.")]


@register_module(TaskType.ANY_TO_ANY, config=Qwen3OmniMoeThinkerConfig, model_type="qwen3_omni_moe_thinker")
@register_module(TaskType.IMAGE_TEXT_TO_TEXT, config=Qwen3OmniMoeThinkerConfig, model_type="qwen3_omni_moe_thinker")
class Qwen3OmniMoeThinkerForConditionalGeneration(Qwen3VLForConditionalGeneration):
    outer_rules = [("model.", "language_model.model."), ("lm_head.", "language_model.lm_head.")]
    hf_keeps_fused = ("visual.",)
    checkpoint_prefix = ""          # "thinker." inside a full Qwen3-Omni checkpoint

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.audio_tower = Qwen3OmniMoeAudioEncoder(config.audio_config, self.param_dtype)

    # ------------------------------------------------------------------ checkpoint names
    def hf_rename_in(self, sd):
        out = {}
        for k, v in sd.items():
            if k.startswith("thinker."):
                k = k[len("thinker."):]
            elif k.startswith(("talker.", "code2wav.")):
                continue
            if k.startswith("visual.merger"):
                k = k.replace("visual.merger_list.", "visual.deepstack_merger_list.")
                for a, b in _MERGER_NAMES:
                    k = k.replace(a, b)
            out[k] = v
        return super().hf_rename_in(out)

    def hf_rename_out(self, sd):
        out = {}
        for k, v in super().hf_rename_out(sd).items():
            if k.startswith("visual."):
                k = k.replace(".attn.qkv_proj.", ".attn.qkv.").replace(".attn.o_proj.", ".attn.proj.")
            if k.startswith("visual.merger") or k.startswith("visual.deepstack_merger_list."):
                k = k.replace("visual.deepstack_merger_list.", "visual.merger_list.")
                for a, b in _MERGER_NAMES:
                    k = k.replace(b, a)
            out[k] = v
        return out

    # ------------------------------------------------------------------ audio
    def get_audio_features(self, input_features, feature_attention_mask=None, audio_feature_lengths=None):
        """``input_features`` ``[clips, mel, frames]`` with ``feature_attention_mask`` ``[clips, frames]``, or already
        packed ``[mel, total_frames]`` with ``audio_feature_lengths``."""
        if feature_attention_mask is not None:
            audio_feature_lengths = feature_attention_mask.sum(1)
            input_features = input_features.permute(0, 2, 1)[feature_attention_mask.bool()].permute(1, 0)
        return self.audio_tower(input_features, audio_feature_lengths)

    def _merge(self, input_ids, pixel_values, image_grid_thw, input_features=None, feature_attention_mask=None,
               audio_feature_lengths=None):
        emb, stacks = super()._merge(input_ids, pixel_values, image_grid_thw)
        if input_features is not None:
            feats = self.get_audio_features(input_features, feature_attention_mask, audio_feature_lengths)
            mask = input_ids == self.config.audio_token_id
            if int(mask.sum()) != feats.shape[0]:
                raise ValueError(f"{int(mask.sum())} audio placeholder tokens for {feats.shape[0]} audio feature rows")
            emb = emb.clone()
            emb[mask] = feats.to(emb.dtype)
        return emb, stacks

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                past_key_values=None, image_grid_thw=None, input_features=None, feature_attention_mask=None,
                audio_feature_lengths=None, **kw):
        first = past_key_values is None or past_key_values.seq_len() == 0
        if inputs_embeds is None:
            inputs_embeds, stacks = self._merge(input_ids, pixel_values if first else None, image_grid_thw,
                                                input_features if first else None, feature_attention_mask,
                                                audio_feature_lengths)
            if stacks:
                kw["deepstack_embeds"] = stacks
        return super().forward(input_ids=input_ids, pixel_values=pixel_values, attention_mask=attention_mask,
                               position_ids=position_ids, inputs_embeds=inputs_embeds,
                               past_key_values=past_key_values, image_grid_thw=image_grid_thw, **kw)

    def _compute_task_loss(self, labels, loss_config, loss_scale, call, loss_kwargs):
        call = dict(call)
        ids = call.pop("input_ids")
        grid, pix = call.pop("image_grid_thw", None), call.pop("pixel_values", None)
        audio = {k: call.pop(k, None) for k in ("input_features", "feature_attention_mask", "audio_feature_lengths")}
        if call.get("position_ids") is None:
            call["position_ids"], _ = mrope_positions(ids, self.config.image_token_id, grid if pix is not None else
                                                      None, self.config.vision_config.spatial_merge_size,
                                                      call.get("attention_mask"))
        emb, stacks = self._merge(ids, pix, grid, **audio)
        if stacks:
            call["deepstack_embeds"] = stacks
        call["inputs_embeds"] = emb
        labels = labels.masked_fill((ids == self.config.image_token_id) | (ids == self.config.audio_token_id),
                                    loss_config.ignore_index)
        return self.language_model._compute_task_loss(labels, loss_config, loss_scale, call, loss_kwargs)


@register_module(TaskType.ANY_TO_ANY, config=Qwen3OmniMoeConfig, model_type="qwen3_omni_moe")
class Qwen3OmniMoeForConditionalGeneration(Qwen3OmniMoeThinkerForConditionalGeneration):
    """The full checkpoint's entry point. The module itself is the thinker (text output; ``thinker.*`` tensors go
    through the regular checkpoint path). With ``enable_audio_output`` (or after :meth:`enable_talker`) it also owns
    the talker and the code-to-waveform decoder (``speech.py``), loaded with :meth:`load_speech_hf_state`, and
    :meth:`generate_speech` runs thinker -> talker -> waveform."""

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config.thinker_config if hasattr(config, "thinker_config") else config, dtype, param_dtype,
                         precision, rngs)
        self.omni_config = config if hasattr(config, "thinker_config") else None
        self.talker = self.code2wav = None
        if self.omni_config is not None and getattr(config, "enable_audio_output", False) \
                and config.talker_config is not None and config.code2wav_config is not None:
            self.enable_talker()

    def hf_rename_out(self, sd):
        return {"thinker." + k: v for k, v in super().hf_rename_out(sd).items()
                if not k.startswith(("talker.", "code2wav."))}

    # ------------------------------------------------------------------ speech
    def enable_talker(self) -> None:
        from .speech import Qwen3OmniMoeCode2Wav, Qwen3OmniMoeTalkerForConditionalGeneration

        c = self.omni_config
        if c is None or c.talker_config is None or c.code2wav_config is None:
            raise ValueError("the configuration has no talker / code2wav sections")
        dev = next(self.parameters()).device
        self.talker = Qwen3OmniMoeTalkerForConditionalGeneration(c.talker_config, dtype=self.dtype,
                                                                 param_dtype=self.param_dtype).to(dev).eval()
        self.code2wav = Qwen3OmniMoeCode2Wav(c.code2wav_config, dtype=torch.float32).to(dev).eval()

    def disable_talker(self) -> None:
        self.talker = self.code2wav = None

    def load_speech_hf_state(self, sd: dict) -> None:
        """``talker.*`` and ``code2wav.*`` tensors of a Hugging Face Qwen3-Omni checkpoint."""
        if self.talker is None:
            self.enable_talker()
        self.talker.load_hf_state(sd, prefix="talker.")
        self.code2wav.load_hf_state(sd, prefix="code2wav.")

    def state_dict(self, *a, **kw):
        sd = super().state_dict(*a, **kw)
        return type(sd)((k, v) for k, v in sd.items() if not k.startswith(("talker.", "code2wav.")))

    @torch.no_grad()
    def generate_speech(self, input_ids: torch.Tensor, speaker: str | int = 0, thinker_max_new_tokens: int = 256,
                        talker_max_new_tokens: int = 1024, do_sample: bool = True, temperature: float = 0.9,
                        top_k: int = 50, top_p: float = 1.0, seed: int | None = None, **thinker_inputs):
        """One conversation (batch 1) -> (token sequence ``[1, T]``, waveform ``[1, 1, samples]``). ``speaker``: a
        name from ``talker_config.speaker_id`` or a codec token id. ``thinker_inputs``: the multimodal tensors of the
        prompt (``pixel_values``, ``image_grid_thw``, ``input_features`` ...)."""
        from ..qwen2_vl import mrope_positions
        from .speech import SpeechTokenIds, talker_inputs, top_k_top_p_sampler

        if self.talker is None:
            raise ValueError("speech output needs the talker: enable_talker() and load_speech_hf_state()")
        if input_ids.shape[0] != 1:
            raise NotImplementedError("speech output is generated one conversation at a time")
        c, tc = self.omni_config, self.omni_config.talker_config
        if isinstance(speaker, str):
            table = {k.lower(): v for k, v in (tc.speaker_id or {}).items()}
            if speaker.lower() not in table:
                raise ValueError(f"unknown speaker {speaker!r}; known: {sorted(table)}")
            speaker = table[speaker.lower()]
        seqs = self.generate(input_ids, max_new_tokens=thinker_max_new_tokens, eos_token_id=c.im_end_token_id,
                             **thinker_inputs).sequences
        # one pass over prompt + reply for the two things the talker is conditioned on
        out = self(input_ids=seqs, output_hidden_states=True, **thinker_inputs)
        hs = out.hidden_states
        ids = SpeechTokenIds(im_start=c.im_start_token_id, system=c.system_token_id, user=c.user_token_id,
                             assistant=c.assistant_token_id, tts_pad=c.tts_pad_token_id, tts_bos=c.tts_bos_token_id,
                             tts_eos=c.tts_eos_token_id, audio=self.config.audio_token_id,
                             image=self.config.image_token_id, video=self.config.video_token_id)
        emb, tids, trailing, pad_e = talker_inputs(self.talker, seqs, input_ids, hs[0], hs[tc.accept_hidden_layer],
                                                   self.get_input_embeddings(), ids, int(speaker))
        grid = thinker_inputs.get("image_grid_thw")
        pos, delta = mrope_positions(tids, self.config.image_token_id, grid,
                                     self.config.vision_config.spatial_merge_size,
                                     video_token_id=self.config.video_token_id,
                                     video_grid_thw=thinker_inputs.get("video_grid_thw"))
        V = tc.text_config.vocab_size
        banned = [i for i in range(V - 1024, V) if i != tc.codec_eos_token_id and i >= 0]
        sampler = top_k_top_p_sampler(temperature, top_k, top_p, seed) if do_sample else None
        residual = top_k_top_p_sampler(1.0, 50, 0.8, seed) if do_sample else None
        codes = self.talker.generate_codes(emb, trailing, pad_e, max_new_tokens=talker_max_new_tokens,
                                           position_ids=pos, rope_delta=int(delta[0]), sample=sampler,
                                           residual_sample=residual, suppress_tokens=banned)
        if codes.shape[-1] == 0:
            return seqs, torch.zeros(1, 1, 0)
        return seqs, self.code2wav.chunked_decode(codes.clamp_max(self.code2wav.config.codebook_size - 1)).float()
