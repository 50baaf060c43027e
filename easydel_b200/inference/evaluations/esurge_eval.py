"""lm-eval adapter over an eSurge engine (easydel/inference/evaluations/esurge_eval.py).

Implements the three request types of the ``lm_eval`` ``LM`` interface: ``generate_until`` (batched greedy
generation with stop strings), ``loglikelihood`` (sum of continuation log-probabilities and whether the continuation
is the greedy choice, from one teacher-forced forward pass per batch) and ``loglikelihood_rolling``. The class does
not import ``lm_eval`` itself; :func:`run_lm_eval` does, and explains what is missing when the package is absent.
"""

from __future__ import annotations

import typing as tp

import torch


def _args(req):
    return req.args if hasattr(req, "args") else req


class eSurgeLMEvalAdapter:
    def __init__(self, engine, max_new_tokens: int = 256, batch_size: int = 8, temperature: float = 0.0):
        self.engine, self.tok, self.model = engine, engine.tokenizer, engine.model
        self.max_new_tokens, self.batch_size, self.temperature = max_new_tokens, batch_size, temperature
        self.max_length = engine.max_model_len

    # ---- generation ------------------------------------------------------------------------------------------
    def generate_until(self, requests) -> list[str]:
        from ..sampling_params import SamplingParams

        outs: list[str] = []
        for s in range(0, len(requests), self.batch_size):
            chunk = [_args(r) for r in requests[s:s + self.batch_size]]
            sps = []
            for _, gen in chunk:
                gen = gen or {}
                until = gen.get("until") or []
                sps.append(SamplingParams(max_tokens=gen.get("max_gen_toks", self.max_new_tokens),
                                          temperature=gen.get("temperature", self.temperature),
                                          stop=[until] if isinstance(until, str) else list(until)))
            res = self.engine.generate([c[0] for c in chunk], sps)
            outs += [r.get_text() for r in res]
        return outs

    # ---- scoring -----------------------------------------------------------------------------------------------
    def _encode_pair(self, context: str, continuation: str) -> tuple[list[int], list[int]]:
        n_space = len(context) - len(context.rstrip())
        if n_space:
            continuation, context = context[-n_space:] + continuation, context[:-n_space]
        whole = self.tok(context + continuation, add_special_tokens=False)["input_ids"]
        ctx = self.tok(context, add_special_tokens=False)["input_ids"] if context else []
        if not ctx:
            bos = getattr(self.tok, "bos_token_id", None) or getattr(self.tok, "eos_token_id", 0)
            ctx, whole = [bos], [bos] + whole
        return ctx, whole[len(ctx):]

    @torch.no_grad()
    def _score(self, pairs: list[tuple[list[int], list[int]]]) -> list[tuple[float, bool]]:
        dev = self.model.device
        out = []
        for s in range(0, len(pairs), self.batch_size):
            chunk = pairs[s:s + self.batch_size]
            rows = [(c + t)[-self.max_length:] for c, t in chunk]
            L = max(len(r) for r in rows)
            ids = torch.zeros(len(rows), L, dtype=torch.long)
            att = torch.zeros(len(rows), L, dtype=torch.long)
            for i, r in enumerate(rows):
                ids[i, :len(r)] = torch.tensor(r)
                att[i, :len(r)] = 1
            logits = self.model(input_ids=ids.to(dev), attention_mask=att.to(dev)).logits.float()
            lsm = torch.log_softmax(logits, -1)
            for i, (c, t) in enumerate(chunk):
                n, end = len(t), len(rows[i])
                tgt = torch.tensor(t[-min(n, end - 1):], device=dev)
                sl = lsm[i, end - len(tgt) - 1:end - 1]
                lp = sl.gather(-1, tgt[:, None])[:, 0]
                out.append((float(lp.sum()), bool((sl.argmax(-1) == tgt).all())))
        return out

    def loglikelihood(self, requests) -> list[tuple[float, bool]]:
        return self._score([self._encode_pair(*_args(r)) for r in requests])

    def loglikelihood_rolling(self, requests) -> list[float]:
        res = []
        for r in requests:
            (text,) = _args(r)
            toks = self.tok(text, add_special_tokens=False)["input_ids"]
            bos = getattr(self.tok, "bos_token_id", None) or getattr(self.tok, "eos_token_id", 0)
            total, pos = 0.0, 0
            win = self.max_length - 1
            while pos < len(toks):
                piece = toks[pos:pos + win]
                ctx = [bos] if pos == 0 else toks[pos - 1:pos]
                total += self._score([(ctx, piece)])[0][0]
                pos += win
            res.append(total)
        return res


def run_lm_eval(adapter: eSurgeLMEvalAdapter, tasks: tp.Sequence[str], num_fewshot: int = 0, limit=None) -> dict:
    try:
        import lm_eval
        from lm_eval.api.model import LM
    except ImportError as e:
        raise RuntimeError("the `lm_eval` package is not installed; the adapter's generate_until / loglikelihood / "
                           "loglikelihood_rolling methods can still be called directly") from e

    class _Wrapped(LM):
        def generate_until(self, requests):
            return adapter.generate_until(requests)

        def loglikelihood(self, requests):
            return adapter.loglikelihood(requests)

        def loglikelihood_rolling(self, requests):
            return adapter.loglikelihood_rolling(requests)

    return lm_eval.simple_evaluate(model=_Wrapped(), tasks=list(tasks), num_fewshot=num_fewshot, limit=limit)
