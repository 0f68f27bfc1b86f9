"""Rule rewards (GSM8K text rule, synthetic token rule) and the data pipelines (local records, DP sharding,
prompt templates, seeded synthetic tokens)."""
import json

import pytest

from b200fw.data.pipeline import (PROMPT_TEMPLATES, GRPOBatch, GSM8KDataPipeline, SimpleTokenizer,
                                  SyntheticTokenPipeline)
from b200fw.reward import GSM8KRewardFunction, SyntheticTokenReward
from b200fw.reward.gsm8k import check_format, extract_answer


@pytest.mark.parametrize("text,value", [
    ("Step 1 ... so 3 + 4 = 7.\n#### 7", 7.0),
    ("We get $1,234.50 in total. #### $1,234.50", 1234.5),
    ("Thus the result is \\boxed{42}.", 42.0),
    ("The answer is -3.5 metres", -3.5),
    ("Final answer: 3/4", 0.75),
    ("所以答案是 18 个", 18.0),
    ("first 5 apples then 12 pears and finally 9", 9.0),        # falls back to the last number
    ("#### 5\nchecking again: #### 6", 6.0),                      # the last marker wins
])
def test_answer_extraction_patterns(text, value):
    assert extract_answer(text) == pytest.approx(value)


def test_answer_extraction_misses_and_format():
    assert extract_answer("no digits here") is None
    assert extract_answer("") is None
    assert check_format("#### 7") and check_format("\\boxed{3}") and check_format("the answer is 4")
    assert check_format("Step 1: add the apples") and check_format("1. first thing") and check_format("a\nb\nc")
    assert check_format("第 2 步：相加") and not check_format("maybe 7?") and not check_format("")


def test_gsm8k_reward_values_and_stats():
    from b200fw.reward import compute_batch_rewards, compute_reward
    # correct: +1; wrong or missing answer: -0.5 when well formed, -1 otherwise
    assert compute_batch_rewards(["... #### 72", "I think it is 70", "cannot tell", "Step 1: add\nStep 2: 71", "#### 71"],
                                 ["#### 72"] * 5) == [1.0, -1.0, -1.0, -0.5, -0.5]
    assert compute_reward("so 72 it is", 72) == 1.0                 # the last number counts when nothing marks the answer
    with pytest.raises(AssertionError):
        compute_batch_rewards(["a"], [])
    rf = GSM8KRewardFunction()
    rewards = rf([["... #### 72", "I think it is 70", "cannot tell"],
                  ["\\boxed{10}", "#### 10.00004", "#### 11"]], ["#### 72", 10])
    assert rewards == [[1.0, -1.0, -1.0], [1.0, 1.0, -0.5]]
    st = rf.get_stats()
    assert st["total"] == 6 and st["accuracy"] == pytest.approx(3 / 6) and st["format_rate"] == pytest.approx(4 / 6)
    assert rf.format_accuracy == pytest.approx(4 / 6) and rf.average_reward == pytest.approx(0.5 / 6)
    rf.reset_stats()
    assert rf.get_stats()["total"] == 0 and rf.accuracy == 0.0 and rf.average_reward == 0.0
    assert GSM8KRewardFunction(correct=2.0, wrong=0.0, no_answer=-2.0).score("#### 1", 1) == 2.0


def test_synthetic_token_reward_rule():
    rw = SyntheticTokenReward(vocab_size=1000, seed=3, eos_token_id=2)
    tgt = rw.target_for(5)
    assert len(tgt) == 3 and tgt == rw.target_for(5) and tgt != rw.target_for(6)
    assert rw.score([9, 9] + tgt + [7, 2], 5) == pytest.approx(1.1)            # target found and EOS-terminated
    assert rw.score([9, 9] + tgt[:2] + [7], 5) == 0.0
    assert rw.score([2], 5) == pytest.approx(0.1) and rw.score([], 5) == 0.0
    assert rw([[tgt, [1]], [[4, 4]]], [5, 6]) == [[1.0, 0.0], [0.0]]
    assert rw.get_stats()["total"] == 7 and rw.get_stats()["hit_rate"] == pytest.approx(2 / 7)
    dense = SyntheticTokenReward(vocab_size=1000, seed=3, dense_weight=0.5)
    assert dense.score([7, 14, 8, 9], 0) == pytest.approx(0.5 * 2 / 4)           # ids congruent to 0 mod 7


def _records(n):
    return [{"question": f"What is {i} + {i}?", "answer": f"It is {2 * i}. #### {2 * i}", "input": ""} for i in range(n)]


def test_gsm8k_pipeline_contract_and_dp_sharding(tmp_path):
    p = tmp_path / "gsm.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in _records(10)))
    pipes = [GSM8KDataPipeline(None, str(p), dataset_config="main", split="train", max_samples=9,
                               prompt_template="qwen3_math", dp_rank=r, dp_size=2) for r in range(2)]
    assert [len(x) for x in pipes] == [5, 4] and isinstance(pipes[0].tokenizer, SimpleTokenizer)
    seen = []
    for x in pipes:
        batches = list(x.get_batches(2))
        assert all(isinstance(b, GRPOBatch) and len(b.prompts) == 2 for b in batches)
        assert len(batches) == len(x) // 2                                         # the ragged tail is dropped
        for b in batches:
            assert all("<|im_start|>assistant" in s and "####" in s for s in b.prompts)
            assert b.prompt_tokens[0] == x.tokenizer.encode(b.prompts[0])
            assert all(str(gt).endswith(f"#### {2 * i}") for gt, i in zip(b.ground_truths, b.prompt_indices))
            assert b.reference_responses == b.ground_truths
            seen += b.prompt_indices
    assert sorted(seen) == [0, 1, 2, 3, 4, 5, 6, 7] and len(set(seen)) == len(seen)  # ranks see disjoint samples
    a = [b.prompt_indices for b in pipes[0].get_batches(2, shuffle=True, seed=1)]
    assert a == [b.prompt_indices for b in pipes[0].get_batches(2, shuffle=True, seed=1)]
    assert a != [b.prompt_indices for b in pipes[0].get_batches(2, shuffle=True, seed=2)]
    # the reward function scores the pipeline's reference responses as correct
    rf = GSM8KRewardFunction()
    b = next(pipes[0].get_batches(2))
    assert rf([[r] for r in b.reference_responses], b.ground_truths) == [[1.0], [1.0]]


def test_json_split_file_templates_and_truncation(tmp_path):
    p = tmp_path / "d.json"
    p.write_text(json.dumps({"train": _records(3), "test": [{"instruction": "Add", "ctx": "1 and 2", "out": "3"}]}))
    x = GSM8KDataPipeline(None, str(p), split="test", prompt_template="qwen3_instruction", prompt_field="instruction",
                          input_field="ctx", response_field="out", answer_field="out", max_prompt_tokens=16)
    b = next(x.get_batches(1))
    assert b.prompts[0] == PROMPT_TEMPLATES["qwen3_instruction"].format(prompt="Add", input="\n1 and 2")
    assert len(b.prompt_tokens[0]) == 16 and b.ground_truths == ["3"]               # keeps the prompt's tail
    y = GSM8KDataPipeline(records=_records(2), prompt_template="Q: {prompt} A:")
    assert next(y.get_batches(2)).prompts[1] == "Q: What is 1 + 1? A:"
    with pytest.raises(FileNotFoundError):
        GSM8KDataPipeline(None, "gsm8k")                                            # nothing is fetched from a hub


def test_synthetic_pipeline_is_seeded_and_shares_prefixes():
    a = SyntheticTokenPipeline(1000, num_samples=16, prompt_len=64, seed=4, prefix_len=32, group=4, min_prompt_len=40)
    b = SyntheticTokenPipeline(1000, num_samples=16, prompt_len=64, seed=4, prefix_len=32, group=4, min_prompt_len=40)
    assert a.samples == b.samples and len(a) == 16
    assert all(40 <= len(s) <= 64 and all(3 <= t < 1000 for t in s) for s in a.samples)
    for g in range(0, 16, 4):
        assert all(a.samples[g + j][:32] == a.samples[g][:32] for j in range(4))
    assert a.samples[0][:32] != a.samples[4][:32]
    halves = [SyntheticTokenPipeline(1000, num_samples=16, prompt_len=8, seed=4, dp_rank=r, dp_size=2) for r in range(2)]
    idx = [i for h in halves for bt in h.get_batches(4) for i in bt.prompt_indices]
    assert sorted(idx) == list(range(16))
    bt = next(halves[1].get_batches(4))
    assert bt.ground_truths == bt.prompt_indices == [1, 3, 5, 7] and len(bt.prompt_tokens[0]) == 8
    tok = SimpleTokenizer()
    assert tok.decode(tok.encode("héllo #### 7")) == "héllo #### 7" and tok.encode("a", add_special_tokens=True)[0] == 1


def test_records_without_a_prompt_are_left_out_before_sharding():
    """A record whose prompt field is missing, ``None`` or blank would become an empty request: it is dropped when the
    pipeline is built, before the data-parallel shards are cut (so both ranks drop the same records and the shards
    still partition what is left)."""
    from b200fw.data.pipeline import GSM8KDataPipeline
    recs = [{"question": f"{i}+1?", "answer": f"#### {i + 1}"} for i in range(6)]
    recs[1] = {"answer": "#### 9"}
    recs[3] = {"question": "   ", "answer": "#### 9"}
    recs[4] = {"question": None, "answer": "#### 9"}
    whole = GSM8KDataPipeline(records=recs, prompt_template="plain")
    assert len(whole) == 3
    shards = [GSM8KDataPipeline(records=recs, prompt_template="plain", dp_rank=r, dp_size=2) for r in range(2)]
    got = sorted(b.prompts[0] for s in shards for b in s.get_batches(1))
    assert got == sorted(b.prompts[0] for b in whole.get_batches(1)) and len(got) == 3
    assert all(len(t) > 0 for s in shards for b in s.get_batches(1) for t in b.prompt_tokens)
