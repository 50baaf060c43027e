"""Speech output of Qwen3-Omni: the talker, its code predictor and the code-to-waveform decoder.

The thinker (``modeling_qwen3_omni_moe.py``) writes text; for speech its hidden states and token embeddings are
projected into the talker, a small MoE decoder that emits one token of the first codebook per audio frame. For every
frame the code predictor, a five-layer dense decoder with one embedding table and one output head per remaining
codebook, fills in the other codebooks autoregressively from the talker's last hidden state; the sum of the frame's
code embeddings (plus the next text embedding while text remains) is the talker's next input. ``Code2Wav`` turns the
``[codebooks, frames]`` code matrix into a waveform: averaged code embeddings, a sliding-window transformer with
layer scale, two transposed-convolution + ConvNeXt up-samplers and a SnakeBeta convolutional decoder.

Counterpart of the talker / code predictor / code2wav classes of
easydel/modules/qwen3_omni_moe/modeling_qwen3_omni_moe.py:1679-3633. The two decoder bodies come from the spec table
(``define_family``), so they run on the same attention / MoE / cache code as every other decoder here.
"""

from __future__ import annotations

import math
import typing as tp

import torch
import torch.nn.functional as tF
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.factory import register_config
from ...ops import functional as F
from .._base.families import base_spec, define_family, moe_spec

_DENSE = dict(vocab_size=2048, hidden_size=1024, intermediate_size=3072, num_hidden_layers=5, num_attention_heads=16,
              num_key_value_heads=8, head_dim=128, hidden_act="silu", max_position_embeddings=32768,
              initializer_range=0.02, rms_norm_eps=1e-6, use_cache=True, rope_theta=10000.0, rope_scaling=None,
              attention_bias=False, attention_dropout=0.0, mlp_bias=False, tie_word_embeddings=False,
              sliding_window=None, layer_types=None, num_code_groups=32)


def _rope_from_parameters(kw: dict) -> dict:
    """Newer checkpoints carry one ``rope_parameters`` dict: base frequency plus (for the talker) the three-stream
    sections. Split it into the ``rope_theta`` / ``rope_scaling`` pair the spec table reads."""
    rp = kw.pop("rope_parameters", None)
    if rp:
        rp = dict(rp)
        kw.setdefault("rope_theta", rp.pop("rope_theta", 10000.0))
        rp.pop("rope_type", None)
        if rp:
            kw.setdefault("rope_scaling", dict(rp, type="default"))
    return kw


_PRED = define_family("qwen3_omni_moe_talker_code_predictor", _DENSE, lambda c: base_spec(c, qk_norm="rms_head"),
                      class_prefix="Qwen3OmniMoeTalkerCodePredictor", with_classifier=False)

_TEXT_DEFAULTS = dict(_DENSE, vocab_size=3072, intermediate_size=2048, num_hidden_layers=20, num_key_value_heads=2,
                      head_dim=None, decoder_sparse_step=1, moe_intermediate_size=384,
                      shared_expert_intermediate_size=768, num_experts_per_tok=8, num_experts=128,
                      norm_topk_prob=False, output_router_logits=False, router_aux_loss_coef=0.001,
                      mlp_only_layers=None)


def _talker_text_spec(c):
    only = set(getattr(c, "mlp_only_layers", None) or [])
    step = getattr(c, "decoder_sparse_step", 1) or 1
    layers = tuple(i for i in range(c.num_hidden_layers) if i not in only and (i + 1) % step == 0)
    return base_spec(c, qk_norm="rms_head",
                     moe=moe_spec(c, num_experts=c.num_experts, top_k=c.num_experts_per_tok,
                                  intermediate=c.moe_intermediate_size, norm_topk=c.norm_topk_prob,
                                  shared=c.shared_expert_intermediate_size, shared_gate=True, layers=layers,
                                  aux_coef=c.router_aux_loss_coef))


_TEXT = define_family("qwen3_omni_moe_talker_text", _TEXT_DEFAULTS, _talker_text_spec,
                      class_prefix="Qwen3OmniMoeTalkerText", with_classifier=False,
                      rules=[("mlp.shared_expert.", "mlp.shared_experts."),
                             ("model.codec_embedding.", "model.embed_tokens."), ("codec_head.", "lm_head.")])

Qwen3OmniMoeTalkerCodePredictorConfig = _PRED["Qwen3OmniMoeTalkerCodePredictorConfig"]
Qwen3OmniMoeTalkerTextConfig = _TEXT["Qwen3OmniMoeTalkerTextConfig"]
Qwen3OmniMoeTalkerTextForCausalLM = _TEXT["Qwen3OmniMoeTalkerTextForCausalLM"]


@register_config("qwen3_omni_moe_talker")
class Qwen3OmniMoeTalkerConfig(EasyDeLBaseConfig):
    model_type = "qwen3_omni_moe_talker"

    def __init__(self, code_predictor_config=None, text_config=None, num_code_groups=32, thinker_hidden_size=2048,
                 codec_eos_token_id=4198, accept_hidden_layer=18, codec_nothink_id=4203, codec_think_bos_id=4204,
                 codec_think_eos_id=4205, codec_pad_id=4196, codec_bos_id=4197, audio_token_id=151646,
                 image_token_id=151655, video_token_id=151656, vision_start_token_id=151652,
                 position_id_per_seconds=25, audio_start_token_id=151669, speaker_id=None, spatial_merge_size=2, **kw):
        if isinstance(code_predictor_config, dict) or code_predictor_config is None:
            d = _rope_from_parameters({k: v for k, v in (code_predictor_config or {}).items() if k != "model_type"})
            d.setdefault("num_code_groups", num_code_groups)
            code_predictor_config = Qwen3OmniMoeTalkerCodePredictorConfig(**d)
        if isinstance(text_config, dict) or text_config is None:
            d = _rope_from_parameters({k: v for k, v in (text_config or {}).items() if k != "model_type"})
            if "num_local_experts" in d:
                d.setdefault("num_experts", d.pop("num_local_experts"))
            text_config = Qwen3OmniMoeTalkerTextConfig(**d)
        self.code_predictor_config, self.text_config = code_predictor_config, text_config
        self.num_code_groups, self.thinker_hidden_size = num_code_groups, thinker_hidden_size
        self.codec_eos_token_id, self.accept_hidden_layer = codec_eos_token_id, accept_hidden_layer
        self.codec_nothink_id, self.codec_think_bos_id = codec_nothink_id, codec_think_bos_id
        self.codec_think_eos_id, self.codec_pad_id, self.codec_bos_id = codec_think_eos_id, codec_pad_id, codec_bos_id
        self.audio_token_id, self.image_token_id, self.video_token_id = audio_token_id, image_token_id, video_token_id
        self.vision_start_token_id, self.position_id_per_seconds = vision_start_token_id, position_id_per_seconds
        self.audio_start_token_id, self.speaker_id, self.spatial_merge_size = audio_start_token_id, speaker_id, \
            spatial_merge_size
        super().__init__(**kw)

    def to_dict(self):
        d = super().to_dict()
        d["code_predictor_config"] = self.code_predictor_config.to_dict()
        d["text_config"] = self.text_config.to_dict()
        return d


@register_config("qwen3_omni_moe_code2wav")
class Qwen3OmniMoeCode2WavConfig(EasyDeLBaseConfig):
    model_type = "qwen3_omni_moe_code2wav"

    def __init__(self, codebook_size=2048, hidden_size=1024, max_position_embeddings=8000, rope_theta=10000.0,
                 num_attention_heads=16, num_key_value_heads=16, attention_bias=False, sliding_window=72,
                 intermediate_size=3072, hidden_act="silu", layer_scale_initial_scale=0.01, rms_norm_eps=1e-5,
                 num_hidden_layers=8, num_quantizers=16, upsample_rates=(8, 5, 4, 3), upsampling_ratios=(2, 2),
                 decoder_dim=1536, attention_dropout=0.0, head_dim=None, **kw):
        kw = _rope_from_parameters(dict(kw, rope_theta=rope_theta) if "rope_parameters" not in kw else dict(kw))
        self.rope_theta = kw.pop("rope_theta", rope_theta)
        kw.pop("rope_scaling", None)
        self.codebook_size, self.hidden_size, self.max_position_embeddings = codebook_size, hidden_size, \
            max_position_embeddings
        self.num_attention_heads, self.num_key_value_heads = num_attention_heads, num_key_value_heads
        self.attention_bias, self.sliding_window, self.intermediate_size = attention_bias, sliding_window, \
            intermediate_size
        self.hidden_act, self.layer_scale_initial_scale, self.rms_norm_eps = hidden_act, layer_scale_initial_scale, \
            rms_norm_eps
        self.num_hidden_layers, self.num_quantizers = num_hidden_layers, num_quantizers
        self.upsample_rates, self.upsampling_ratios = list(upsample_rates), list(upsampling_ratios)
        self.decoder_dim, self.attention_dropout = decoder_dim, attention_dropout
        self.head_dim = head_dim or hidden_size // num_attention_heads
        super().__init__(**kw)


# --------------------------------------------------------------------------------------------- code predictor
class Qwen3OmniMoeTalkerCodePredictor(nn.Module):
    """Fills in codebooks 1 .. G-1 of one audio frame. Its input sequence is (talker hidden state, embedding of the
    frame's first code, embedding of code 1, ...); position ``s + 1`` of the output, read through head ``s``, scores
    codebook ``s + 1``. The sequence never exceeds G + 1 positions, so every step recomputes it (no cache)."""

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None):
        super().__init__()
        self.config = config
        pd = param_dtype or dtype
        self.model = _PRED["Qwen3OmniMoeTalkerCodePredictorModel"](config, dtype=dtype, param_dtype=pd)
        del self.model.embed_tokens          # inputs are always embeddings
        G = config.num_code_groups
        self.codec_embedding = nn.ModuleList([nn.Embedding(config.vocab_size, config.hidden_size, dtype=pd)
                                              for _ in range(G - 1)])
        self.lm_head = nn.ModuleList([nn.Linear(config.hidden_size, config.vocab_size, bias=False, dtype=pd)
                                      for _ in range(G - 1)])

    def forward(self, inputs_embeds: torch.Tensor, generation_step: int | None = None) -> torch.Tensor:
        """Logits of codebook ``generation_step + 1`` at every position (``generation_step`` defaults to the one the
        sequence length implies: length - 2)."""
        s = inputs_embeds.shape[1] - 2 if generation_step is None else generation_step
        h = self.model(inputs_embeds=inputs_embeds).last_hidden_state
        return self.lm_head[s](h)

    @torch.no_grad()
    def predict(self, past_hidden: torch.Tensor, first_code_embed: torch.Tensor,
                sample: tp.Callable[[torch.Tensor], torch.Tensor] | None = None):
        """``past_hidden``, ``first_code_embed``: ``[B, 1, H]``. -> (codes ``[B, G-1]``, the embeddings of those codes
        ``[B, G-1, H]``). ``sample`` maps ``[B, V]`` logits to ``[B]`` tokens (greedy when None)."""
        seq = torch.cat([past_hidden, first_code_embed], dim=1)
        codes, embeds = [], []
        for s in range(self.config.num_code_groups - 1):
            logits = self.forward(seq, s)[:, -1].float()
            tok = logits.argmax(-1) if sample is None else sample(logits)
            e = self.codec_embedding[s](tok)[:, None]
            codes.append(tok)
            embeds.append(e)
            seq = torch.cat([seq, e.to(seq.dtype)], dim=1)
        return torch.stack(codes, 1), torch.cat(embeds, 1)

    def load_hf_state(self, sd: dict[str, torch.Tensor], prefix: str = "") -> None:
        """``sd``: tensors named as in the Hugging Face checkpoint below ``talker.code_predictor.``."""
        from ...utils.parameters_transformation import hf_to_internal

        own = {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}
        body = {k: v for k, v in own.items() if k.startswith("model.") and not k.startswith("model.codec_embedding.")}
        self.model.load_state_dict(hf_to_internal(self.model, {k[len("model."):]: v for k, v in body.items()},
                                                  strict=False), strict=True)
        for i, emb in enumerate(self.codec_embedding):
            emb.weight.data.copy_(own[f"model.codec_embedding.{i}.weight"])
        for i, head in enumerate(self.lm_head):
            head.weight.data.copy_(own[f"lm_head.{i}.weight"])


# ------------------------------------------------------------------------------------------------------ talker
class Qwen3OmniMoeTalkerResizeMLP(nn.Module):
    """Thinker width -> talker width (one for text embeddings, one for multimodal hidden states)."""

    def __init__(self, thinker_hidden: int, intermediate: int, hidden: int, act: str, dtype):
        super().__init__()
        self.linear_fc1 = nn.Linear(thinker_hidden, intermediate, bias=True, dtype=dtype)
        self.linear_fc2 = nn.Linear(intermediate, hidden, bias=True, dtype=dtype)
        self.act = act

    def forward(self, x):
        h = self.linear_fc1(x)
        h = tF.silu(h) if self.act == "silu" else tF.gelu(h)
        return self.linear_fc2(h)


class Qwen3OmniMoeTalkerForConditionalGeneration(nn.Module):
    """The talker: MoE decoder over codec tokens (its token table is the codec embedding, its head the codec head),
    the two projections from the thinker's width, and the code predictor."""

    def __init__(self, config: Qwen3OmniMoeTalkerConfig, dtype=torch.bfloat16, param_dtype=None):
        super().__init__()
        self.config = config
        pd = param_dtype or dtype
        tc = config.text_config
        self.lm = Qwen3OmniMoeTalkerTextForCausalLM(tc, dtype=dtype, param_dtype=pd)
        self.text_projection = Qwen3OmniMoeTalkerResizeMLP(config.thinker_hidden_size, tc.intermediate_size,
                                                           tc.hidden_size, tc.hidden_act, pd)
        self.hidden_projection = Qwen3OmniMoeTalkerResizeMLP(config.thinker_hidden_size, tc.intermediate_size,
                                                             tc.hidden_size, tc.hidden_act, pd)
        self.code_predictor = Qwen3OmniMoeTalkerCodePredictor(config.code_predictor_config, dtype=dtype, param_dtype=pd)

    @property
    def codec_embedding(self):
        return self.lm.get_input_embeddings()

    def forward(self, inputs_embeds, position_ids=None, past_key_values=None, attention_mask=None):
        """-> (codec logits ``[B, T, V]``, last hidden states ``[B, T, H]``). ``position_ids``: ``[3, B, T]`` rotary
        streams (or ``[B, T]`` / None for plain positions)."""
        out = self.lm(inputs_embeds=inputs_embeds, position_ids=position_ids, past_key_values=past_key_values,
                      attention_mask=attention_mask, apply_lm_head=False)
        h = out.last_hidden_state
        return self.lm.apply_lm_head(h), h

    @torch.no_grad()
    def generate_codes(self, prefill_embeds: torch.Tensor, trailing_text_hidden: torch.Tensor,
                       tts_pad_embed: torch.Tensor, max_new_tokens: int = 256, position_ids: torch.Tensor | None = None,
                       rope_delta: int = 0, sample: tp.Callable | None = None, residual_sample: tp.Callable | None = None,
                       suppress_tokens: tp.Sequence[int] = ()) -> torch.Tensor:
        """Autoregressive speech-code generation for one utterance (batch 1).

        ``prefill_embeds`` ``[1, T, H]``: the projected conversation ending in the codec begin-of-speech position;
        ``trailing_text_hidden`` ``[1, L, H]``: projected embeddings of the reply's remaining text tokens, one added
        per generated frame, ``tts_pad_embed`` ``[1, 1, H]`` after they run out. Every frame: first-codebook token from
        the talker, the other codebooks from the code predictor, next input = sum of the frame's code embeddings +
        text (or pad) embedding. Stops at ``codec_eos_token_id``. -> codes ``[1, G, frames]``."""
        cfg = self.config
        T = prefill_embeds.shape[1]
        cache = self.lm.init_cache(1, T + max_new_tokens + 1)
        logits, hidden = self.forward(prefill_embeds, position_ids=position_ids, past_key_values=cache)
        cache.advance(T)
        frames = []
        banned = torch.tensor(sorted(suppress_tokens), dtype=torch.long, device=prefill_embeds.device)
        for step in range(max_new_tokens):
            lg = logits[:, -1].float()
            if banned.numel():
                lg[:, banned] = float("-inf")
            tok = lg.argmax(-1) if sample is None else sample(lg)
            if int(tok[0]) == cfg.codec_eos_token_id:
                break
            first = self.codec_embedding(tok)[:, None]
            rest, rest_emb = self.code_predictor.predict(hidden[:, -1:], first.to(hidden.dtype), residual_sample)
            frames.append(torch.cat([tok[:, None], rest], dim=1))
            nxt = first.float() + rest_emb.float().sum(1, keepdim=True)
            nxt = nxt + (trailing_text_hidden[:, step:step + 1] if step < trailing_text_hidden.shape[1]
                         else tts_pad_embed).float()
            pos = None
            if position_ids is not None:
                p = T + step + rope_delta
                pos = torch.full((3, 1, 1), p, dtype=torch.long, device=prefill_embeds.device)
            logits, hidden = self.forward(nxt.to(prefill_embeds.dtype), position_ids=pos, past_key_values=cache)
            cache.advance(1)
        if not frames:
            return torch.zeros(1, cfg.num_code_groups, 0, dtype=torch.long, device=prefill_embeds.device)
        return torch.stack(frames, dim=-1)

    def load_hf_state(self, sd: dict[str, torch.Tensor], prefix: str = "talker.") -> None:
        """Loads ``talker.*`` tensors of a Hugging Face Qwen3-Omni checkpoint."""
        from ...utils.parameters_transformation import hf_to_internal

        own = {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}
        lm = {k: v for k, v in own.items() if k.startswith(("model.", "codec_head."))}
        self.lm.load_state_dict(hf_to_internal(self.lm, lm, strict=False), strict=True)
        for name in ("text_projection", "hidden_projection"):
            getattr(self, name).load_state_dict({k[len(name) + 1:]: v for k, v in own.items()
                                                 if k.startswith(name + ".")})
        self.code_predictor.load_hf_state(own, prefix="code_predictor.")


# ---------------------------------------------------------------------------------------------------- code2wav
class _CausalConv1d(nn.Module):
    """Convolution that only looks back: left padding of (receptive field - stride), right padding up to a whole
    number of frames."""

    def __init__(self, cin, cout, kernel, dilation=1, stride=1, groups=1, dtype=None):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, kernel, stride=stride, dilation=dilation, groups=groups, dtype=dtype)
        self.stride = stride
        self.field = (kernel - 1) * dilation + 1
        self.left = self.field - stride

    def forward(self, x):
        n = x.shape[-1]
        frames = math.ceil((n - self.field + self.left) / self.stride + 1)
        right = (frames - 1) * self.stride + (self.field - self.left) - n
        return self.conv(tF.pad(x, (self.left, right)))


class _CausalConvTranspose1d(nn.Module):
    """Transposed convolution trimmed by (kernel - stride) samples on both sides, so that frame t of the input only
    shapes output samples from t * stride on."""

    def __init__(self, cin, cout, kernel, stride, dtype=None):
        super().__init__()
        self.conv = nn.ConvTranspose1d(cin, cout, kernel, stride=stride, dtype=dtype)
        self.trim = math.ceil(kernel - stride)

    def forward(self, x):
        y = self.conv(x)
        return y[..., self.trim:y.shape[-1] - self.trim] if self.trim else y


class SnakeBeta(nn.Module):
    """x + sin^2(alpha x) / beta with per-channel alpha, beta stored as logarithms."""

    def __init__(self, channels, dtype=None):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(channels, dtype=dtype))
        self.beta = nn.Parameter(torch.zeros(channels, dtype=dtype))

    def forward(self, x):
        a, b = self.alpha.exp()[None, :, None], self.beta.exp()[None, :, None]
        return x + torch.sin(x * a).pow(2) / (b + 1e-9)


class _ConvNeXtBlock(nn.Module):
    def __init__(self, dim, dtype=None):
        super().__init__()
        self.dwconv = _CausalConv1d(dim, dim, 7, groups=dim, dtype=dtype)
        self.norm = nn.LayerNorm(dim, eps=1e-6, dtype=dtype)
        self.pwconv1 = nn.Linear(dim, 4 * dim, dtype=dtype)
        self.pwconv2 = nn.Linear(4 * dim, dim, dtype=dtype)
        self.gamma = nn.Parameter(1e-6 * torch.ones(dim, dtype=dtype))

    def forward(self, x):
        h = self.dwconv(x).transpose(1, 2)
        h = self.pwconv2(tF.gelu(self.pwconv1(self.norm(h)))) * self.gamma
        return x + h.transpose(1, 2)


class _ResidualUnit(nn.Module):
    def __init__(self, dim, dilation, dtype=None):
        super().__init__()
        self.act1, self.conv1 = SnakeBeta(dim, dtype), _CausalConv1d(dim, dim, 7, dilation=dilation, dtype=dtype)
        self.act2, self.conv2 = SnakeBeta(dim, dtype), _CausalConv1d(dim, dim, 1, dtype=dtype)

    def forward(self, x):
        return x + self.conv2(self.act2(self.conv1(self.act1(x))))


class _DecoderBlock(nn.Module):
    """SnakeBeta, up-sampling transposed convolution (channels halve), three dilated residual units."""

    def __init__(self, cin, cout, rate, dtype=None):
        super().__init__()
        self.block = nn.ModuleList([SnakeBeta(cin, dtype), _CausalConvTranspose1d(cin, cout, 2 * rate, rate, dtype)]
                                   + [_ResidualUnit(cout, d, dtype) for d in (1, 3, 9)])

    def forward(self, x):
        for b in self.block:
            x = b(x)
        return x


class _RMSNorm(nn.Module):
    def __init__(self, dim, eps, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class _Code2WavLayer(nn.Module):
    """Pre-norm transformer layer with causal sliding-window attention and a learnt per-channel scale on both
    residual branches."""

    def __init__(self, cfg: Qwen3OmniMoeCode2WavConfig, dtype=None):
        super().__init__()
        H, D = cfg.num_attention_heads, cfg.head_dim
        self.heads, self.kv_heads, self.head_dim, self.window = H, cfg.num_key_value_heads, D, cfg.sliding_window
        self.q_proj = nn.Linear(cfg.hidden_size, H * D, bias=cfg.attention_bias, dtype=dtype)
        self.k_proj = nn.Linear(cfg.hidden_size, self.kv_heads * D, bias=cfg.attention_bias, dtype=dtype)
        self.v_proj = nn.Linear(cfg.hidden_size, self.kv_heads * D, bias=cfg.attention_bias, dtype=dtype)
        self.o_proj = nn.Linear(H * D, cfg.hidden_size, bias=cfg.attention_bias, dtype=dtype)
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False, dtype=dtype)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False, dtype=dtype)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False, dtype=dtype)
        self.input_layernorm = _RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype)
        self.post_attention_layernorm = _RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype)
        self.attn_scale = nn.Parameter(torch.full((cfg.hidden_size,), cfg.layer_scale_initial_scale, dtype=dtype))
        self.mlp_scale = nn.Parameter(torch.full((cfg.hidden_size,), cfg.layer_scale_initial_scale, dtype=dtype))

    def forward(self, x, cos, sin):
        B, T, _ = x.shape
        h = self.input_layernorm(x)
        q = self.q_proj(h).view(B, T, self.heads, self.head_dim)
        k = self.k_proj(h).view(B, T, self.kv_heads, self.head_dim)
        v = self.v_proj(h).view(B, T, self.kv_heads, self.head_dim)

        def rot(t):
            a, b = t[..., : self.head_dim // 2], t[..., self.head_dim // 2:]
            return (t.float() * cos + torch.cat([-b, a], -1).float() * sin).to(t.dtype)

        o = F.attention(rot(q), rot(k), v, causal=True, sliding_window=self.window)
        x = x + self.o_proj(o.reshape(B, T, -1)) * self.attn_scale
        h = self.post_attention_layernorm(x)
        return x + self.down_proj(tF.silu(self.gate_proj(h)) * self.up_proj(h)) * self.mlp_scale


class Qwen3OmniMoeCode2Wav(nn.Module):
    """Codes ``[B, num_quantizers, frames]`` -> waveform ``[B, 1, frames * prod(upsampling_ratios + upsample_rates)]``
    in [-1, 1]."""

    def __init__(self, config: Qwen3OmniMoeCode2WavConfig, dtype=torch.float32):
        super().__init__()
        self.config = config
        c = config
        self.total_upsample = int(math.prod(list(c.upsample_rates) + list(c.upsampling_ratios)))
        self.code_embedding = nn.Embedding(c.codebook_size * c.num_quantizers, c.hidden_size, dtype=dtype)
        self.layers = nn.ModuleList([_Code2WavLayer(c, dtype) for _ in range(c.num_hidden_layers)])
        self.norm = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype)
        self.upsample = nn.ModuleList([nn.ModuleList([_CausalConvTranspose1d(c.hidden_size, c.hidden_size, f, f, dtype),
                                                      _ConvNeXtBlock(c.hidden_size, dtype)])
                                       for f in c.upsampling_ratios])
        dec: list[nn.Module] = [_CausalConv1d(c.hidden_size, c.decoder_dim, 7, dtype=dtype)]
        for i, rate in enumerate(c.upsample_rates):
            dec.append(_DecoderBlock(c.decoder_dim // 2 ** i, c.decoder_dim // 2 ** (i + 1), rate, dtype))
        out_dim = c.decoder_dim // 2 ** len(c.upsample_rates)
        dec += [SnakeBeta(out_dim, dtype), _CausalConv1d(out_dim, 1, 7, dtype=dtype)]
        self.decoder = nn.ModuleList(dec)

    def _rope(self, T, device):
        D = self.config.head_dim
        inv = 1.0 / (self.config.rope_theta ** (torch.arange(0, D, 2, device=device).float() / D))
        ang = torch.arange(T, device=device).float()[:, None] * inv[None]
        ang = torch.cat([ang, ang], -1)
        return ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def forward(self, codes: torch.Tensor) -> torch.Tensor:
        c = self.config
        if codes.shape[1] != c.num_quantizers:
            raise ValueError(f"expected {c.num_quantizers} rows of codes, got {codes.shape[1]}")
        offset = torch.arange(c.num_quantizers, device=codes.device)[None, :, None] * c.codebook_size
        h = self.code_embedding(codes + offset).mean(1)
        cos, sin = self._rope(h.shape[1], h.device)
        for layer in self.layers:
            h = layer(h, cos, sin)
        h = self.norm(h).transpose(1, 2)
        for up, block in self.upsample:
            h = block(up(h))
        for b in self.decoder:
            h = b(h)
        return h.clamp(-1, 1)

    def chunked_decode(self, codes: torch.Tensor, chunk_size: int = 300, left_context_size: int = 25) -> torch.Tensor:
        """Decodes long code sequences in chunks that each see ``left_context_size`` earlier frames."""
        outs, start = [], 0
        n = codes.shape[-1]
        while start < n:
            end = min(start + chunk_size, n)
            ctx = left_context_size if start - left_context_size > 0 else start
            wav = self(codes[..., start - ctx:end])
            outs.append(wav[..., ctx * self.total_upsample:])
            start = end
        return torch.cat(outs, dim=-1)

    def load_hf_state(self, sd: dict[str, torch.Tensor], prefix: str = "code2wav.") -> None:
        """Loads ``code2wav.*`` tensors of a Hugging Face Qwen3-Omni checkpoint."""
        out = {}
        for k, v in sd.items():
            if not k.startswith(prefix):
                continue
            k = k[len(prefix):]
            k = k.replace("pre_transformer.layers.", "layers.").replace("pre_transformer.norm.", "norm.")
            k = k.replace(".self_attn.", ".").replace(".mlp.", ".")
            k = k.replace(".self_attn_layer_scale.scale", ".attn_scale").replace(".mlp_layer_scale.scale", ".mlp_scale")
            if k.startswith("layers.") and ".attn_scale" not in k and ".mlp_scale" not in k:
                k = k.replace("layers.", "layers.", 1)
            out[k] = v
        self.load_state_dict(out, strict=True)


# ------------------------------------------------------------------------------- thinker -> talker hand-over
class SpeechTokenIds(tp.NamedTuple):
    """Token ids of the chat template and of the text-to-speech markers (top-level checkpoint configuration)."""
    im_start: int = 151644
    system: int = 8948
    user: int = 872
    assistant: int = 77091
    tts_pad: int = 151671
    tts_bos: int = 151672
    tts_eos: int = 151673
    audio: int = 151646
    image: int = 151655
    video: int = 151656


def talker_inputs(talker: Qwen3OmniMoeTalkerForConditionalGeneration, sequences: torch.Tensor, prompt_ids: torch.Tensor,
                  thinker_embed: torch.Tensor, thinker_hidden: torch.Tensor, embed_tokens: tp.Callable,
                  ids: SpeechTokenIds, speaker_id: int):
    """What the talker is conditioned on, from one finished thinker run (batch 1).

    ``sequences`` ``[1, T]``: prompt + reply tokens; ``prompt_ids`` ``[1, P]``: the prompt alone (turn boundaries are
    looked up there); ``thinker_embed`` / ``thinker_hidden`` ``[1, T, Ht]``: the thinker's input embeddings and its
    hidden states at ``accept_hidden_layer``; ``embed_tokens``: the thinker's token embedding. System turns and earlier
    assistant turns are skipped. A user turn contributes, position by position, the projected hidden state where the
    token is an audio / image / video placeholder and the projected embedding elsewhere. The final assistant turn
    contributes nine positions: its three template tokens, four pads, the speech-begin marker and the first reply
    token on the text side, added to (nothing x 3, no-think, think-begin, think-end, speaker, codec pad, codec
    begin) on the codec side; the rest of the reply plus the speech-end marker is handed out one token per generated
    frame. -> (embeddings ``[1, T', H]``, ids for position bookkeeping ``[1, T']``, trailing text ``[1, L, H]``,
    pad embedding ``[1, 1, H]``)."""
    cfg = talker.config
    dev = sequences.device
    T = sequences.shape[1]
    starts = (prompt_ids[0] == ids.im_start).nonzero().flatten().tolist() + [T]
    mm = (sequences == ids.audio) | (sequences == ids.image) | (sequences == ids.video)
    special = torch.tensor([[ids.tts_bos, ids.tts_eos, ids.tts_pad]], device=dev)
    bos_e, eos_e, pad_e = talker.text_projection(embed_tokens(special)).chunk(3, dim=1)
    parts, part_ids, trailing = [], [], None
    for i in range(len(starts) - 1):
        a, z = starts[i], starts[i + 1]
        role = int(prompt_ids[0, a + 1])
        last = i == len(starts) - 2
        if role == ids.system or (role == ids.assistant and not last):
            continue
        if role == ids.user:
            seg_mm = mm[:, a:z]
            text = talker.text_projection(thinker_embed[:, a:z])
            if bool(seg_mm.any()):
                text = torch.where(seg_mm[..., None], talker.hidden_projection(thinker_hidden[:, a:z]), text)
            parts.append(text)
            part_ids.append(sequences[:, a:z])
        elif role == ids.assistant:
            reply = talker.text_projection(thinker_embed[:, a:z])
            text_side = torch.cat([reply[:, :3], pad_e.expand(-1, 4, -1), bos_e, reply[:, 3:4]], dim=1)
            codec = torch.tensor([[cfg.codec_nothink_id, cfg.codec_think_bos_id, cfg.codec_think_eos_id, speaker_id,
                                   cfg.codec_pad_id, cfg.codec_bos_id]], device=dev)
            codec_side = torch.cat([torch.zeros_like(text_side[:, :3]),
                                    talker.codec_embedding(codec).to(text_side.dtype)], dim=1)
            parts.append(text_side + codec_side)
            part_ids.append(torch.full((1, text_side.shape[1]), ids.tts_pad, dtype=sequences.dtype, device=dev))
            trailing = torch.cat([reply[:, 4:], eos_e], dim=1)
        else:
            raise ValueError(f"token {role} after the turn-start marker is not a system, user or assistant role")
    if trailing is None:
        raise ValueError("the prompt does not end in an assistant turn")
    return torch.cat(parts, dim=1), torch.cat(part_ids, dim=1), trailing, pad_e


def top_k_top_p_sampler(temperature: float = 0.9, top_k: int = 50, top_p: float = 1.0, seed: int | None = None):
    """``[B, V]`` logits -> ``[B]`` tokens."""
    gen = torch.Generator().manual_seed(seed) if seed is not None else None

    def sample(logits: torch.Tensor) -> torch.Tensor:
        lg = logits.float() / max(temperature, 1e-5)
        if top_k and top_k < lg.shape[-1]:
            kth = lg.topk(top_k, dim=-1).values[..., -1:]
            lg = lg.masked_fill(lg < kth, float("-inf"))
        if top_p < 1.0:
            srt, idx = lg.sort(dim=-1, descending=True)
            cum = srt.softmax(-1).cumsum(-1)
            drop = cum - srt.softmax(-1) > top_p
            lg = lg.masked_fill(torch.zeros_like(drop).scatter(-1, idx, drop), float("-inf"))
        p = lg.softmax(-1)
        return torch.multinomial(p.cpu(), 1, generator=gen).to(logits.device)[:, 0]

    return sample
