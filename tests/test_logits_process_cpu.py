"""Logits processors and warpers against hand-computed expectations, and the list built from a ``SamplingParams``."""

import math

import pytest
import torch

from easydel_b200.inference import logits_process as LP
from easydel_b200.inference.sampling_params import SamplingParams

NEG = -float("inf")


def _scores():
    return torch.tensor([[1.0, 2.0, 3.0, 4.0, 0.5, -1.0]])


def test_temperature_scales_and_rejects_non_positive():
    s = _scores()
    assert torch.equal(LP.TemperatureLogitsWarper(2.0)(None, s), s / 2)
    with pytest.raises(ValueError):
        LP.TemperatureLogitsWarper(0.0)


def test_top_k_keeps_k_largest_and_ties():
    s = _scores()
    out = LP.TopKLogitsWarper(2)(None, s)
    assert out.tolist() == [[NEG, NEG, 3.0, 4.0, NEG, NEG]]
    # k above the vocabulary is a no-op; min_tokens_to_keep lifts a smaller k
    assert torch.equal(LP.TopKLogitsWarper(100)(None, s), s)
    assert (LP.TopKLogitsWarper(1, min_tokens_to_keep=3)(None, s) > NEG).sum() == 3
    tie = torch.tensor([[1.0, 1.0, 0.0]])
    assert (LP.TopKLogitsWarper(1)(None, tie) > NEG).sum() == 2     # equal to the k-th value survives


def test_top_p_smallest_set_reaching_mass():
    probs = torch.tensor([[0.5, 0.3, 0.15, 0.05]])
    s = probs.log()
    keep = lambda p: (LP.TopPLogitsWarper(p)(None, s) > NEG)[0].tolist()     # noqa: E731
    assert keep(0.4) == [True, False, False, False]
    assert keep(0.6) == [True, True, False, False]
    assert keep(0.9) == [True, True, True, False]
    assert keep(1.0) == [True, True, True, True]
    # works on a permuted row, and min_tokens_to_keep overrides a tiny p
    perm = torch.tensor([2, 0, 3, 1])
    out = LP.TopPLogitsWarper(0.6)(None, s[:, perm])
    assert (out > NEG)[0].tolist() == [False, True, False, True]
    assert (LP.TopPLogitsWarper(0.01, min_tokens_to_keep=2)(None, s) > NEG).sum() == 2


def test_min_p_relative_to_the_mode():
    probs = torch.tensor([[0.6, 0.25, 0.1, 0.05]])
    out = LP.MinPLogitsWarper(0.2)(None, probs.log())          # threshold 0.12
    assert (out > NEG)[0].tolist() == [True, True, False, False]


def test_repetition_penalty_sign_rule():
    s = torch.tensor([[2.0, -2.0, 1.0, -1.0]])
    ids = torch.tensor([[0, 1]])
    out = LP.RepetitionPenaltyLogitsProcessor(2.0)(ids, s)
    assert out.tolist() == [[1.0, -4.0, 1.0, -1.0]]


def test_presence_and_frequency_penalties_count_tokens():
    s = torch.zeros(1, 5)
    ids = torch.tensor([[1, 1, 1, 3]])
    assert LP.PresencePenaltyLogitsProcessor(0.5)(ids, s).tolist() == [[0, -0.5, 0, -0.5, 0]]
    assert LP.FrequencyPenaltyLogitsProcessor(0.5)(ids, s).tolist() == [[0, -1.5, 0, -0.5, 0]]


def test_min_length_blocks_eos_until_reached():
    s = _scores()
    p = LP.MinLengthLogitsProcessor(3, [1, 5])
    early = p(None, s, cur_len=2)
    assert early[0, 1] == NEG and early[0, 5] == NEG and early[0, 0] == 1.0
    assert torch.equal(p(None, s, cur_len=3), s)
    assert s[0, 1] == 2.0                                       # the input is not modified


def test_forced_bos_and_eos_positions():
    s = _scores()
    bos = LP.ForcedBOSTokenLogitsProcessor(2)
    assert torch.equal(bos(None, s, cur_len=0), s)
    forced = bos(None, s, cur_len=1)
    assert forced.argmax(-1).item() == 2 and (forced > NEG).sum() == 1
    eos = LP.ForcedEOSTokenLogitsProcessor(max_length=8, eos_token_id=4)
    assert torch.equal(eos(None, s, cur_len=6), s)
    forced = eos(None, s, cur_len=7)
    assert forced.argmax(-1).item() == 4 and (forced > NEG).sum() == 1


def test_suppress_tokens_always_and_at_begin():
    s = _scores()
    assert LP.SuppressTokensLogitsProcessor([3])(None, s).argmax(-1).item() == 2
    at = LP.SuppressTokensAtBeginLogitsProcessor([3], begin_index=4)
    assert torch.equal(at(None, s, cur_len=3), s)
    assert at(None, s, cur_len=4)[0, 3] == NEG


def test_no_repeat_ngram_bans_the_completing_token():
    ids = torch.tensor([[5, 1, 2, 3, 1, 2]])
    s = torch.zeros(1, 6)
    out = LP.NoRepeatNGramLogitsProcessor(3)(ids, s)
    assert (out[0] == NEG).nonzero().flatten().tolist() == [3]           # "1 2 3" was seen
    out = LP.NoRepeatNGramLogitsProcessor(1)(ids, s)
    assert sorted((out[0] == NEG).nonzero().flatten().tolist()) == [1, 2, 3, 5]
    short = torch.tensor([[1]])
    assert torch.equal(LP.NoRepeatNGramLogitsProcessor(3)(short, s), s)  # too short to hold an n-gram


def test_logit_bias_and_allowed_tokens():
    s = _scores()
    out = LP.LogitBiasProcessor({0: 10.0, 3: -10.0})(None, s)
    assert out[0, 0] == 11.0 and out[0, 3] == -6.0 and out[0, 1] == 2.0
    out = LP.AllowedTokensLogitsProcessor([1, 4])(None, s)
    assert (out > NEG)[0].tolist() == [False, True, False, False, True, False]
    assert out[0, 1] == 2.0


def test_list_applies_in_order():
    s = torch.tensor([[0.0, 1.0, 2.0]])
    a = LP.LogitsProcessorList([LP.LogitBiasProcessor({0: 5.0}), LP.TopKLogitsWarper(1)])
    b = LP.LogitsProcessorList([LP.TopKLogitsWarper(1), LP.LogitBiasProcessor({0: 5.0})])
    assert a(None, s).argmax(-1).item() == 0
    assert b(None, s).argmax(-1).item() == 2 and b(None, s)[0, 0] == NEG


def test_processors_from_sampling_params_selection_and_order():
    assert len(LP.processors_from_sampling_params(SamplingParams())) == 0
    assert len(LP.processors_from_sampling_params(SamplingParams(temperature=0.0))) == 0
    sp = SamplingParams(repetition_penalty=1.2, presence_penalty=0.1, frequency_penalty=0.2, logit_bias={1: 2.0},
                        allowed_token_ids=[1, 2], min_tokens=2, max_tokens=8, temperature=0.7, top_k=5, top_p=0.9,
                        min_p=0.05)
    kinds = [type(p).__name__ for p in LP.processors_from_sampling_params(sp, eos_token_id=0)]
    assert kinds == ["RepetitionPenaltyLogitsProcessor", "PresencePenaltyLogitsProcessor",
                     "FrequencyPenaltyLogitsProcessor", "LogitBiasProcessor", "AllowedTokensLogitsProcessor",
                     "MinLengthLogitsProcessor", "TemperatureLogitsWarper", "TopKLogitsWarper", "TopPLogitsWarper",
                     "MinPLogitsWarper"]
    # without an end-of-sequence id there is nothing to hold back
    assert "MinLengthLogitsProcessor" not in [type(p).__name__ for p in LP.processors_from_sampling_params(sp)]


def test_processed_distribution_matches_manual_pipeline():
    torch.manual_seed(0)
    logits = torch.randn(3, 50)
    ids = torch.randint(0, 50, (3, 7))
    sp = SamplingParams(repetition_penalty=1.3, temperature=0.8, top_k=10, top_p=0.8)
    got = LP.processors_from_sampling_params(sp)(ids, logits)
    want = logits.clone()
    for b in range(3):
        for t in set(ids[b].tolist()):
            want[b, t] = want[b, t] * 1.3 if want[b, t] < 0 else want[b, t] / 1.3
    want = want / 0.8
    kth = want.topk(10, -1).values[:, -1:]
    want = want.masked_fill(want < kth, NEG)
    srt, idx = want.sort(-1, descending=True)
    pr = srt.softmax(-1)
    drop = (pr.cumsum(-1) - pr) > 0.8
    want = want.masked_fill(torch.zeros_like(drop).scatter(-1, idx, drop), NEG)
    assert torch.equal(got == NEG, want == NEG)
    assert torch.allclose(got[got > NEG], want[want > NEG])
    assert math.isclose(float(got.softmax(-1).sum()), 3.0, rel_tol=1e-5)


@pytest.mark.parametrize("kwargs", [dict(n=0), dict(n=2, best_of=1), dict(temperature=-0.1), dict(top_p=0.0),
                                    dict(top_p=1.5), dict(min_p=-0.1), dict(top_k=-2), dict(repetition_penalty=0.0),
                                    dict(presence_penalty=3.0), dict(frequency_penalty=-3.0), dict(max_tokens=0),
                                    dict(min_tokens=5, max_tokens=4)])
def test_sampling_params_rejects(kwargs):
    with pytest.raises(ValueError):
        SamplingParams(**kwargs)


def test_sampling_params_normalises():
    sp = SamplingParams(stop="END", top_k=-1)
    assert sp.stop == ["END"] and sp.top_k == 0 and sp.stop_token_ids == []
    assert SamplingParams(temperature=0.0).is_greedy and SamplingParams(top_k=1).is_greedy
    assert not SamplingParams(temperature=0.5).is_greedy
