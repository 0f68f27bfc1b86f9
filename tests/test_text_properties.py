"""Property tests (hypothesis) of the text-side helpers: the GSM8K rule reward and the evaluation metrics accept any
string without raising, stay inside their value ranges, and recognise a correct answer however it is decorated."""
import math

import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from b200fw.obs.eval_utils import compute_bleu4, compute_exact_match, compute_token_f1, normalize_text  # noqa: E402
from b200fw.reward.gsm8k import GSM8KRewardFunction, check_format, compute_reward, extract_answer  # noqa: E402

TEXT = st.text(alphabet=st.characters(blacklist_categories=("Cs",)), max_size=200)
NUMBERISH = st.text(alphabet="0123456789.,-+$#/ eE\nansweris=\\boxed{}", max_size=80)


@settings(max_examples=400, deadline=None)
@given(st.one_of(TEXT, NUMBERISH), st.one_of(st.integers(-10 ** 9, 10 ** 9), st.floats(allow_nan=False, allow_infinity=False,
                                                                                           width=32), TEXT))
def test_reward_accepts_anything_and_stays_in_range(response, truth):
    r = compute_reward(response, truth)
    assert r in (1.0, -0.5, -1.0)
    a = extract_answer(response)
    assert a is None or (isinstance(a, float) and not math.isnan(a))
    assert check_format(response) in (True, False)
    fn = GSM8KRewardFunction()
    out = fn([[response, response]], [truth])
    assert out == [[r, r]] and 0.0 <= fn.accuracy <= 1.0 and 0.0 <= fn.format_accuracy <= 1.0


@settings(max_examples=300, deadline=None)
@given(st.integers(-10 ** 6, 10 ** 6), st.sampled_from(["#### {}", "The answer is {}.", "so we get\n#### {}\n", "= {} \n#### {}",
                                                          "final answer: {}", "\\boxed{{{}}}"]), TEXT)
def test_a_correct_answer_is_recognised_whatever_surrounds_it(n, template, noise):
    noise = "".join(ch for ch in noise if not (ch.isdigit() or ch in "#$\\=-+.,/"))     # no second number, no markers
    text = noise + " " + template.format(*([n] * template.count("{}"))) if "boxed" not in template else \
        noise + " " + template.format(n)
    assert extract_answer(text) == float(n), text
    assert compute_reward(text, n) == 1.0 and compute_reward(text, str(n)) == 1.0
    assert compute_reward(text, n + 1) == -0.5          # well formed but wrong


@settings(max_examples=300, deadline=None)
@given(TEXT, TEXT)
def test_eval_metrics_are_bounded_and_symmetric_where_they_should_be(a, b):
    for f in (compute_exact_match, compute_token_f1, compute_bleu4):
        v = f(a, b)
        assert 0.0 <= v <= 1.0 + 1e-9, (f.__name__, v)
    assert compute_exact_match(a, a) == 1.0
    assert abs(compute_token_f1(a, b) - compute_token_f1(b, a)) < 1e-9
    if normalize_text(a):
        assert compute_token_f1(a, a) == pytest.approx(1.0)
    assert normalize_text(normalize_text(a)) == normalize_text(a)


@settings(max_examples=150, deadline=None)
@given(st.integers(1, 60), st.integers(1, 8), st.integers(1, 7), st.booleans(), st.integers(0, 99))
def test_data_parallel_shards_partition_the_dataset(num_records, dp_size, batch_size, shuffle, seed):
    """Every record goes to exactly one data-parallel rank, a rank's batches never repeat or invent a record, and the
    global indices a batch reports point back at the records it carries (text and synthetic pipelines)."""
    from b200fw.data.pipeline import GSM8KDataPipeline, SimpleTokenizer, SyntheticTokenPipeline
    records = [{"question": f"what is {i} plus 1 ?", "answer": f"#### {i + 1}"} for i in range(num_records)]
    seen = []
    for rank in range(dp_size):
        p = GSM8KDataPipeline(records=records, tokenizer=SimpleTokenizer(), dp_rank=rank, dp_size=dp_size)
        assert len(p) == len(records[rank::dp_size])
        mine = []
        for b in p.get_batches(batch_size, shuffle=shuffle, seed=seed):
            assert len(b.prompt_tokens) == batch_size == len(b.prompt_indices)
            for text, gi, truth in zip(b.prompts, b.prompt_indices, b.ground_truths):
                assert gi % dp_size == rank and f"what is {gi} plus 1" in text and truth == f"#### {gi + 1}"
            mine += list(b.prompt_indices)
        assert len(mine) == len(set(mine)) == (len(p) // batch_size) * batch_size
        seen.append(set(range(rank, num_records, dp_size)))
        assert set(mine) <= seen[-1]
    assert set().union(*seen) == set(range(num_records)) and sum(len(s) for s in seen) == num_records
    syn = [SyntheticTokenPipeline(64, num_samples=num_records, prompt_len=8, seed=seed, dp_rank=r, dp_size=dp_size)
           for r in range(dp_size)]
    idx = [i for s in syn for b in s.get_batches(batch_size, shuffle, seed) for i in b.prompt_indices]
    assert len(idx) == len(set(idx)) and set(idx) <= set(range(num_records))
    assert all(a.samples == syn[0].samples for a in syn)            # the same seeded corpus on every rank
