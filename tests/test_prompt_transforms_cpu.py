"""Per-example preprocessing: the rows each transform produces feed the trainers' collators unchanged."""

import easydel_b200 as ed
from easydel_b200.trainers import prompt_transforms as PT
from easydel_b200.trainers.preference import DPODataCollator, RewardCollator, UnpairedCollator


class Tok:
    pad_token_id, bos_token_id, eos_token_id = 0, 1, 2

    def __call__(self, text, add_special_tokens=True, **_):
        return {"input_ids": ([1] if add_special_tokens else []) + [3 + (ord(c) % 90) for c in text]}

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=False, **_):
        s = "".join(f"<{m['role']}>{m['content']}" for m in messages) + ("<assistant>" if add_generation_prompt else "")
        return self(s, add_special_tokens=True)["input_ids"] if tokenize else s


CHAT = [{"role": "user", "content": "hi"}]


def test_prompt_extraction_and_templates():
    ex = {"chosen": CHAT + [{"role": "assistant", "content": "good"}],
          "rejected": CHAT + [{"role": "assistant", "content": "bad"}], "extra": None}
    ex = PT.extract_prompt_from_preference(PT.purify_example(ex))
    assert ex["prompt"] == CHAT and ex["chosen"][0]["content"] == "good" and "extra" not in ex
    out = PT.apply_chat_template_to_preference(ex, Tok())
    assert out["prompt"] == "<user>hi<assistant>" and out["chosen"] == "good" and out["rejected"] == "bad"
    assert PT.extract_prompt_from_preference({"prompt": "p", "chosen": "a", "rejected": "b"})["prompt"] == "p"


def test_dpo_rows_truncate_and_collate():
    t = ed.DPOPreprocessTransform(Tok(), max_prompt_length=4, max_completion_length=3)
    row = t({"prompt": "abcdefgh", "chosen": "xyzw", "rejected": "q", "margin": 0.5})
    full = Tok()("abcdefgh")["input_ids"]
    assert row["prompt_input_ids"] == full[-4:]                       # the end of the prompt is kept
    assert row["chosen_input_ids"] == Tok()("xyzw", add_special_tokens=False)["input_ids"][:3]
    assert row["rejected_input_ids"][-1] == 2 and row["margin"] == 0.5    # an end-of-sequence token is appended
    batch = DPODataCollator(0)([row, t({"prompt": "ab", "chosen": "c", "rejected": "dd", "margin": 0.0})])
    assert batch["prompt_input_ids"].shape == (2, 4) and batch["prompt_attention_mask"][1].tolist() == [0, 1, 1, 1]
    chat = ed.ORPOPreprocessTransform(Tok())({"chosen": CHAT + [{"role": "assistant", "content": "good"}],
                                              "rejected": CHAT + [{"role": "assistant", "content": "bad"}]})
    assert chat["prompt_input_ids"] == Tok()("<user>hi<assistant>")["input_ids"]
    assert issubclass(ed.CPOPreprocessTransform, ed.DPOPreprocessTransform)


def test_unpaired_rows_and_pair_expansion():
    k = ed.KTOPreprocessTransform(Tok())
    row = k({"prompt": "p", "completion": "c", "label": False})
    assert row["label"] is False and row["completion_input_ids"][-1] == 2
    rows = ed.BCOPreprocessTransform(Tok())({"prompt": "p", "chosen": "good", "rejected": "bad"})
    assert [r["label"] for r in rows] == [True, False]
    assert rows[0]["completion_input_ids"] != rows[1]["completion_input_ids"]
    assert len(ed.BCOPreprocessTransform(Tok())({"prompt": "p", "completion": "c", "label": True})) == 1
    batch = UnpairedCollator(0)(rows)
    assert batch["label"].tolist() == [True, False] and batch["completion_input_ids"].shape[0] == 2


def test_reward_grpo_sft_and_embedding_rows():
    r = ed.RewardPreprocessTransform(Tok(), max_length=6)({"prompt": "pp", "chosen": "aaaa", "rejected": "b",
                                                          "margin": 1})
    assert len(r["input_ids_chosen"]) == 6 and r["input_ids_chosen"][:3] == r["input_ids_rejected"][:3]
    assert RewardCollator(0)([r])["margin"].tolist() == [1.0]
    g = ed.GRPOPreprocessTransform(Tok(), max_prompt_length=5)({"prompt": CHAT, "answer": "42"})
    assert g["answer"] == "42" and g["prompt"] == "<user>hi<assistant>" and len(g["prompt_input_ids"]) == 5
    assert g["attention_mask"] == [1] * 5 and issubclass(ed.PPOPreprocessTransform, ed.GRPOPreprocessTransform)
    s = ed.SFTPreprocessTransform(Tok(), max_length=8)({"prompt": "abc", "completion": "de"})
    assert len(s["input_ids"]) == len(s["completion_mask"]) <= 8 and s["completion_mask"][:3] == [0, 0, 0]
    s = ed.SFTPreprocessTransform(Tok(), assistant_only_loss=True)(
        {"messages": CHAT + [{"role": "assistant", "content": "ok"}]})
    assert 0 < sum(s["assistant_masks"]) < len(s["input_ids"])        # only the assistant turn is marked
    e = PT.EmbeddingPreprocessTransform(Tok(), max_length=5, query_prefix="q: ")(
        {"query": "what", "positive": "this", "negative": ["that", "those"]})
    assert set(e) == {"query_input_ids", "positive_input_ids", "negative_input_ids"}
    assert e["query_input_ids"] == Tok()("q: what")["input_ids"][:5]
