"""Whisper: convolutional audio front end + pre-LayerNorm encoder, causal decoder with cross-attention
(easydel/modules/whisper/modeling_whisper.py:141-2144, whisper_configuration.py).

Encoder: ``gelu(conv1d(k=3)) -> gelu(conv1d(k=3, stride 2)) + positions -> N x [x += attn(LN x); x += mlp(LN x)] -> LN``.
Decoder: token + learned position embeddings, each layer ``self-attention (causal) -> cross-attention over the
encoder output -> MLP``, all pre-LayerNorm; the output projection is tied to the token embedding. The key projections
carry no bias (as in the original checkpoints). Parameter names are the Hugging Face names, so checkpoints load
without a renaming table; only ``proj_out.weight`` is dropped on load and re-emitted on save (tied).

Generation keeps one self-attention K/V buffer per layer, preallocated at the maximum target length, and computes
the cross-attention K/V once per utterance.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from ...infra.base_config import EasyDeLBaseConfig
from ...infra.base_module import EasyDeLBaseModule
from ...infra.factory import TaskType, register_config, register_module
from ...infra.loss_utils import LossConfig, LossMetrics
from ...infra.modeling_outputs import BaseModelOutput, Seq2SeqLMOutput, Seq2SeqModelOutput, SequenceClassifierOutput
from ...layers.embeddings import Embed
from ...layers.linears import ColumnParallelLinear
from ...layers.norms import LayerNorm
from ...ops import functional as F
from ...ops.reference import ACT2FN


@register_config("whisper")
class WhisperConfig(EasyDeLBaseConfig):
    model_type = "whisper"
    attribute_map = {"num_attention_heads": "encoder_attention_heads", "hidden_size": "d_model",
                     "num_hidden_layers": "encoder_layers"}
    hf_config_keys = ("vocab_size", "num_mel_bins", "encoder_layers", "encoder_attention_heads", "decoder_layers",
                      "decoder_attention_heads", "decoder_ffn_dim", "encoder_ffn_dim", "activation_function",
                      "d_model", "dropout", "attention_dropout", "activation_dropout", "init_std", "scale_embedding",
                      "max_source_positions", "max_target_positions", "decoder_start_token_id",
                      "use_weighted_layer_sum", "classifier_proj_size", "suppress_tokens", "begin_suppress_tokens")

    def __init__(self, vocab_size=51865, num_mel_bins=80, encoder_layers=4, encoder_attention_heads=6,
                 decoder_layers=4, decoder_attention_heads=6, decoder_ffn_dim=1536, encoder_ffn_dim=1536,
                 activation_function="gelu", d_model=384, dropout=0.0, attention_dropout=0.0, activation_dropout=0.0,
                 init_std=0.02, scale_embedding=False, max_source_positions=1500, max_target_positions=448,
                 pad_token_id=50256, bos_token_id=50256, eos_token_id=50256, decoder_start_token_id=50257,
                 use_weighted_layer_sum=False, classifier_proj_size=256, suppress_tokens=None,
                 begin_suppress_tokens=None, tie_word_embeddings=True, is_encoder_decoder=True, **kw):
        self.vocab_size, self.num_mel_bins, self.d_model = vocab_size, num_mel_bins, d_model
        self.encoder_layers, self.encoder_attention_heads = encoder_layers, encoder_attention_heads
        self.decoder_layers, self.decoder_attention_heads = decoder_layers, decoder_attention_heads
        self.decoder_ffn_dim, self.encoder_ffn_dim = decoder_ffn_dim, encoder_ffn_dim
        self.activation_function, self.init_std, self.scale_embedding = activation_function, init_std, scale_embedding
        self.dropout, self.attention_dropout, self.activation_dropout = dropout, attention_dropout, activation_dropout
        self.max_source_positions, self.max_target_positions = max_source_positions, max_target_positions
        self.use_weighted_layer_sum, self.classifier_proj_size = use_weighted_layer_sum, classifier_proj_size
        self.suppress_tokens, self.begin_suppress_tokens = suppress_tokens, begin_suppress_tokens
        super().__init__(pad_token_id=pad_token_id, bos_token_id=bos_token_id, eos_token_id=eos_token_id,
                         decoder_start_token_id=decoder_start_token_id, tie_word_embeddings=tie_word_embeddings,
                         is_encoder_decoder=is_encoder_decoder, **kw)
        self.decoder_start_token_id = decoder_start_token_id


def _lin(i, o, bias, dtype, std):
    return ColumnParallelLinear(i, o, bias=bias, dtype=dtype, init_std=std)


class WhisperAttention(nn.Module):
    """Multi-head attention with separate projections; ``kv`` is the encoder output for cross-attention."""

    def __init__(self, d_model: int, heads: int, dtype, std: float, causal: bool = False):
        super().__init__()
        self.h, self.hd, self.causal = heads, d_model // heads, causal
        self.q_proj = _lin(d_model, d_model, True, dtype, std)
        self.k_proj = _lin(d_model, d_model, False, dtype, std)
        self.v_proj = _lin(d_model, d_model, True, dtype, std)
        self.out_proj = _lin(d_model, d_model, True, dtype, std)

    def project_kv(self, src):
        B, S, _ = src.shape
        return self.k_proj(src).view(B, S, self.h, self.hd), self.v_proj(src).view(B, S, self.h, self.hd)

    def forward(self, x, kv=None, cached_kv=None, cache=None, cache_len: int = 0):
        """``cached_kv``: precomputed (k, v) of a cross-attention. ``cache``: (k_buf, v_buf) ``[B,Tmax,H,D]`` of a
        causal self-attention that already holds ``cache_len`` positions; the new ones are appended in place."""
        B, T, _ = x.shape
        q = self.q_proj(x).view(B, T, self.h, self.hd)
        if cached_kv is not None:
            k, v = cached_kv
            causal = False
        elif cache is not None:
            kn, vn = self.project_kv(x)
            cache[0][:, cache_len:cache_len + T] = kn
            cache[1][:, cache_len:cache_len + T] = vn
            k, v = cache[0][:, :cache_len + T], cache[1][:, :cache_len + T]
            causal = self.causal and T > 1
            if causal and cache_len:
                # a multi-token continuation: the oracle path handles the offset causal mask
                from ...ops import reference as R

                o = R.attention(q, k, v, causal=True)
                return self.out_proj(o.reshape(B, T, -1))
        else:
            k, v = self.project_kv(x if kv is None else kv)
            causal = self.causal and kv is None
        if B > 1 and cache is not None:
            k, v = k.contiguous(), v.contiguous()   # rows of a batch must be equally spaced for the kernel
        o = F.attention(q, k, v, causal=causal)
        return self.out_proj(o.reshape(B, T, -1))


class WhisperEncoderLayer(nn.Module):
    def __init__(self, c: WhisperConfig, dtype):
        super().__init__()
        d, s = c.d_model, c.init_std
        self.self_attn = WhisperAttention(d, c.encoder_attention_heads, dtype, s)
        self.self_attn_layer_norm = LayerNorm(d, 1e-5, dtype=dtype)
        self.fc1, self.fc2 = _lin(d, c.encoder_ffn_dim, True, dtype, s), _lin(c.encoder_ffn_dim, d, True, dtype, s)
        self.final_layer_norm = LayerNorm(d, 1e-5, dtype=dtype)
        self.act = ACT2FN[c.activation_function]

    def forward(self, x):
        x = x + self.self_attn(self.self_attn_layer_norm(x))
        return x + self.fc2(self.act(self.fc1(self.final_layer_norm(x))))


class WhisperDecoderLayer(nn.Module):
    def __init__(self, c: WhisperConfig, dtype):
        super().__init__()
        d, s = c.d_model, c.init_std
        self.self_attn = WhisperAttention(d, c.decoder_attention_heads, dtype, s, causal=True)
        self.self_attn_layer_norm = LayerNorm(d, 1e-5, dtype=dtype)
        self.encoder_attn = WhisperAttention(d, c.decoder_attention_heads, dtype, s)
        self.encoder_attn_layer_norm = LayerNorm(d, 1e-5, dtype=dtype)
        self.fc1, self.fc2 = _lin(d, c.decoder_ffn_dim, True, dtype, s), _lin(c.decoder_ffn_dim, d, True, dtype, s)
        self.final_layer_norm = LayerNorm(d, 1e-5, dtype=dtype)
        self.act = ACT2FN[c.activation_function]

    def forward(self, x, enc, cross_kv=None, cache=None, cache_len: int = 0):
        x = x + self.self_attn(self.self_attn_layer_norm(x), cache=cache, cache_len=cache_len)
        x = x + self.encoder_attn(self.encoder_attn_layer_norm(x), kv=enc, cached_kv=cross_kv)
        return x + self.fc2(self.act(self.fc1(self.final_layer_norm(x))))


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """The fixed sinusoidal table the encoder's position embedding is initialised with."""
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None]
    return torch.cat([t.sin(), t.cos()], dim=1)


class WhisperEncoder(nn.Module):
    def __init__(self, c: WhisperConfig, dtype):
        super().__init__()
        d = c.d_model
        self.conv1 = nn.Conv1d(c.num_mel_bins, d, 3, padding=1, dtype=dtype)
        self.conv2 = nn.Conv1d(d, d, 3, stride=2, padding=1, dtype=dtype)
        self.embed_positions = Embed(c.max_source_positions, d, dtype, c.init_std)
        with torch.no_grad():
            self.embed_positions.weight.copy_(sinusoids(c.max_source_positions, d))
        self.layers = nn.ModuleList([WhisperEncoderLayer(c, dtype) for _ in range(c.encoder_layers)])
        self.layer_norm = LayerNorm(d, 1e-5, dtype=dtype)

    def forward(self, input_features, output_hidden_states=False):
        """``input_features`` ``[B, n_mels, frames]`` -> ``[B, frames/2, d_model]``."""
        x = input_features.to(self.conv1.weight.dtype)
        x = torch.nn.functional.gelu(self.conv1(x))
        x = torch.nn.functional.gelu(self.conv2(x)).transpose(1, 2).contiguous()
        if x.shape[1] > self.embed_positions.weight.shape[0]:
            raise ValueError(f"{x.shape[1]} encoder positions exceed max_source_positions "
                             f"{self.embed_positions.weight.shape[0]}")
        x = x + self.embed_positions.weight[: x.shape[1]].to(x.dtype)
        hs = [] if output_hidden_states else None
        for layer in self.layers:
            if hs is not None:
                hs.append(x)
            x = layer(x)
        x = self.layer_norm(x)
        if hs is not None:
            hs.append(x)
        return BaseModelOutput(last_hidden_state=x, hidden_states=tuple(hs) if hs else None)


class WhisperDecoder(nn.Module):
    def __init__(self, c: WhisperConfig, dtype):
        super().__init__()
        d = c.d_model
        self.scale = math.sqrt(d) if c.scale_embedding else 1.0
        self.embed_tokens = Embed(c.vocab_size, d, dtype, c.init_std)
        self.embed_positions = Embed(c.max_target_positions, d, dtype, c.init_std)
        self.layers = nn.ModuleList([WhisperDecoderLayer(c, dtype) for _ in range(c.decoder_layers)])
        self.layer_norm = LayerNorm(d, 1e-5, dtype=dtype)

    def forward(self, input_ids, enc, cross_kv=None, caches=None, cache_len: int = 0, position_ids=None):
        B, T = input_ids.shape
        if position_ids is None:
            position_ids = torch.arange(cache_len, cache_len + T, device=input_ids.device)
        x = self.embed_tokens(input_ids) * self.scale + self.embed_positions(position_ids)
        for i, layer in enumerate(self.layers):
            x = layer(x, enc, None if cross_kv is None else cross_kv[i], None if caches is None else caches[i],
                      cache_len)
        return self.layer_norm(x)


def shift_tokens_right(labels: torch.Tensor, pad: int, start: int) -> torch.Tensor:
    out = labels.new_empty(labels.shape)
    out[:, 1:] = labels[:, :-1]
    out[:, 0] = start
    return out.masked_fill(out == -100, pad)


class _WhisperBase(EasyDeLBaseModule):
    hf_keeps_fused = ()

    def hf_rename_in(self, sd):
        return {k: v for k, v in sd.items() if k != "proj_out.weight"}

    def hf_rename_out(self, sd):
        return dict(sd)


@register_module(TaskType.BASE_MODULE, config=WhisperConfig, model_type="whisper",
                 layernorm_names=["self_attn_layer_norm", "encoder_attn_layer_norm", "final_layer_norm", "layer_norm"])
class WhisperModel(_WhisperBase):
    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.encoder = WhisperEncoder(config, self.param_dtype)
        self.decoder = WhisperDecoder(config, self.param_dtype)

    def get_input_embeddings(self):
        return self.decoder.embed_tokens

    def forward(self, input_features=None, decoder_input_ids=None, encoder_outputs=None,
                output_hidden_states=False, **_):
        if encoder_outputs is None:
            encoder_outputs = self.encoder(input_features, output_hidden_states)
        enc = encoder_outputs.last_hidden_state if hasattr(encoder_outputs, "last_hidden_state") else encoder_outputs
        h = self.decoder(decoder_input_ids, enc)
        return Seq2SeqModelOutput(last_hidden_state=h, encoder_last_hidden_state=enc,
                                  encoder_hidden_states=getattr(encoder_outputs, "hidden_states", None))


@register_module(TaskType.SPEECH_SEQUENCE_TO_SEQUENCE, config=WhisperConfig, model_type="whisper")
class WhisperForConditionalGeneration(_WhisperBase):
    """Speech-to-text head: logits over the vocabulary through the (tied) token embedding."""

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        self.model = WhisperModel(config, dtype, param_dtype, precision, rngs)

    def get_input_embeddings(self):
        return self.model.decoder.embed_tokens

    def get_encoder(self):
        return self.model.encoder

    def get_decoder(self):
        return self.model.decoder

    def hf_rename_out(self, sd):
        sd = dict(sd)
        sd["proj_out.weight"] = sd["model.decoder.embed_tokens.weight"]
        return sd

    def _logits(self, h):
        return F.linear(h, self.model.decoder.embed_tokens.weight)

    def forward(self, input_features=None, decoder_input_ids=None, labels=None, encoder_outputs=None, **kw):
        if decoder_input_ids is None and labels is not None:
            decoder_input_ids = shift_tokens_right(labels, self.config.pad_token_id,
                                                   self.config.decoder_start_token_id)
        out = self.model(input_features=input_features, decoder_input_ids=decoder_input_ids,
                         encoder_outputs=encoder_outputs, **kw)
        logits = self._logits(out.last_hidden_state)
        loss = None
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.reshape(-1),
                                                     ignore_index=-100)
        return Seq2SeqLMOutput(logits=logits, loss=loss, last_hidden_state=out.last_hidden_state,
                               encoder_last_hidden_state=out.encoder_last_hidden_state,
                               encoder_hidden_states=out.encoder_hidden_states)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        call = {k: v for k, v in call.items() if k not in ("input_ids", "attention_mask")}
        out = self(labels=labels, **call)
        return out, LossMetrics(loss=out.loss * loss_scale)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, input_features, decoder_input_ids=None, max_new_tokens: int | None = None,
                 forced_decoder_ids=None, suppress_tokens=None, begin_suppress_tokens=None,
                 no_timestamps_token_id: int | None = None, return_timestamps: bool = False,
                 temperature: float = 0.0, generator: torch.Generator | None = None, eos_token_id=None):
        """Greedy (or temperature) decoding of ``[B, n_mels, frames]`` features.

        ``forced_decoder_ids``: ``[(position, token), ...]`` as in Hugging Face generation configs (language, task,
        no-timestamps prompt tokens). With ``return_timestamps`` the timestamp rules of the original decoder hold:
        timestamps come in pairs, never decrease, and win when their total probability exceeds every text token's.
        Returns token ids ``[B, T]`` including the prompt, padded with ``pad_token_id`` after EOS.
        """
        c = self.config
        dev = input_features.device
        B = input_features.shape[0]
        enc = self.model.encoder(input_features).last_hidden_state
        dec = self.model.decoder
        cross = [layer.encoder_attn.project_kv(enc) for layer in dec.layers]
        if decoder_input_ids is None:
            decoder_input_ids = torch.full((B, 1), c.decoder_start_token_id, dtype=torch.long, device=dev)
        forced = dict(forced_decoder_ids or [])
        eos = c.eos_token_id if eos_token_id is None else eos_token_id
        suppress = list(c.suppress_tokens or []) if suppress_tokens is None else list(suppress_tokens)
        begin_suppress = list(c.begin_suppress_tokens or []) if begin_suppress_tokens is None else \
            list(begin_suppress_tokens)
        t_max = c.max_target_positions
        budget = t_max - decoder_input_ids.shape[1]
        n_new = budget if max_new_tokens is None else min(max_new_tokens, budget)
        h, hd = c.decoder_attention_heads, c.d_model // c.decoder_attention_heads
        caches = [(torch.zeros(B, t_max, h, hd, dtype=enc.dtype, device=dev),
                   torch.zeros(B, t_max, h, hd, dtype=enc.dtype, device=dev)) for _ in dec.layers]
        ids = decoder_input_ids
        done = torch.zeros(B, dtype=torch.bool, device=dev)
        n_cached = 0
        first_free = None        # index of the first position that is not forced
        ts_begin = None if no_timestamps_token_id is None else no_timestamps_token_id + 1
        for _ in range(n_new):
            step_in = ids[:, n_cached:]
            hcur = dec(step_in, enc, cross, caches, n_cached)
            n_cached = ids.shape[1]
            logits = self._logits(hcur[:, -1]).float()
            pos = ids.shape[1]
            if pos in forced:
                nxt = torch.full((B,), forced[pos], dtype=torch.long, device=dev)
            else:
                if first_free is None:
                    first_free = pos
                if suppress:
                    logits[:, suppress] = -float("inf")
                if pos == first_free and begin_suppress:
                    logits[:, begin_suppress] = -float("inf")
                if ts_begin is not None:
                    if return_timestamps:
                        logits = _timestamp_rules(logits, ids, first_free, ts_begin, eos, no_timestamps_token_id)
                    else:
                        logits[:, no_timestamps_token_id:] = -float("inf")
                if temperature and temperature > 0:
                    p = torch.softmax(logits / temperature, -1)
                    nxt = torch.multinomial(p, 1, generator=generator).squeeze(1)
                else:
                    nxt = logits.argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, c.pad_token_id), nxt)
            ids = torch.cat([ids, nxt[:, None]], 1)
            done = done | (nxt == eos)
            if bool(done.all()):
                break
        return ids


def _timestamp_rules(logits, ids, first_free, ts_begin, eos, no_ts):
    """Timestamp constraints of Whisper decoding, applied to one step's fp32 logits ``[B, V]``."""
    B = logits.shape[0]
    logits[:, no_ts] = -float("inf")
    for b in range(B):
        seq = ids[b, first_free:].tolist()
        last_ts = len(seq) >= 1 and seq[-1] >= ts_begin
        pen_ts = len(seq) < 2 or seq[-2] >= ts_begin
        if last_ts:
            if pen_ts:      # a closed pair: text (or EOS) must follow
                logits[b, ts_begin:] = -float("inf")
            else:           # an opened segment has text inside: the closing timestamp or EOS
                logits[b, :eos] = -float("inf")
        stamps = [t for t in seq if t >= ts_begin]
        if stamps:          # timestamps never go backwards; a segment has positive length
            floor = stamps[-1] if last_ts and not pen_ts else stamps[-1] + 1
            logits[b, ts_begin:floor] = -float("inf")
        if not seq:         # the first free token is a timestamp (at most 1 s in)
            logits[b, :ts_begin] = -float("inf")
            logits[b, ts_begin + 51:] = -float("inf")
    lp = torch.log_softmax(logits, -1)
    ts_lp = torch.logsumexp(lp[:, ts_begin:], -1)
    text_max = lp[:, :ts_begin].max(-1).values
    force_ts = ts_lp > text_max
    logits[force_ts, :ts_begin] = -float("inf")
    return logits


@register_module(TaskType.AUDIO_CLASSIFICATION, config=WhisperConfig, model_type="whisper")
class WhisperForAudioClassification(_WhisperBase):
    """Encoder + mean pooling + linear classifier (optionally a learned mixture of all encoder layers)."""

    loss_type = "ForSequenceClassification"

    def __init__(self, config, dtype=torch.bfloat16, param_dtype=None, precision=None, rngs=None):
        super().__init__(config, dtype, param_dtype, precision, rngs)
        pd = self.param_dtype
        self.num_labels = getattr(config, "num_labels", 2)
        self.encoder = WhisperEncoder(config, pd)
        if config.use_weighted_layer_sum:
            self.layer_weights = nn.Parameter(torch.ones(config.encoder_layers + 1, dtype=pd) /
                                              (config.encoder_layers + 1))
        self.projector = _lin(config.d_model, config.classifier_proj_size, True, pd, config.init_std)
        self.classifier = _lin(config.classifier_proj_size, self.num_labels, True, pd, config.init_std)

    def forward(self, input_features=None, labels=None, **_):
        out = self.encoder(input_features, output_hidden_states=self.config.use_weighted_layer_sum)
        if self.config.use_weighted_layer_sum:
            hs = torch.stack(out.hidden_states, 1)
            w = torch.softmax(self.layer_weights.float(), -1).to(hs.dtype)
            h = (hs * w.view(1, -1, 1, 1)).sum(1)
        else:
            h = out.last_hidden_state
        logits = self.classifier(self.projector(h).mean(1))
        loss = None
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits.float(), labels.view(-1))
        return SequenceClassifierOutput(logits=logits, loss=loss, hidden_states=out.hidden_states)

    def _compute_task_loss(self, labels, loss_config: LossConfig, loss_scale, call, loss_kwargs):
        out = self(labels=labels, **{k: v for k, v in call.items() if k == "input_features"})
        return out, LossMetrics(loss=out.loss * loss_scale)
