"""IcePop and C3PO++ host-side logic."""
import torch

from b200fw.train import C3POConfig, C3POPlusScheduler, IcePopConfig, IcePopFilter


def test_icepop_threshold_and_cap():
    f = IcePopFilter(IcePopConfig(True, divergence_threshold=0.5, max_mask_ratio=0.5))
    train = torch.tensor([-1.0, -1.0, -1.0, -1.0])
    infer = torch.tensor([-1.1, -2.0, -4.0, -1.7])
    adv = torch.tensor([1.0, -1.0, 0.5, 2.0])
    out, d = f.filter_divergent_responses(train, infer, adv)
    # three exceed 0.5, only 2 (50 %) may be masked: the most divergent ones (idx 2 then 1)
    assert out.tolist() == [1.0, 0.0, 0.0, 2.0]
    assert d["icepop_num_masked"] == 2 and d["icepop_masked_ratio"] == 0.5 and abs(d["icepop_max_divergence"] - 3.0) < 1e-6
    assert set(d) == {"icepop_masked_ratio", "icepop_mean_divergence", "icepop_max_divergence", "icepop_num_masked", "icepop_threshold"}
    out, d = f.filter_divergent_responses(train, train, adv)
    assert torch.equal(out, adv) and d["icepop_num_masked"] == 0


def test_c3po_no_split_and_split_sizes():
    s = C3POPlusScheduler(C3POConfig(True, token_budget=4, target_batch_tokens=64))
    prompts = [[1, 2, 3]]
    chunks = s.split(prompts, [[[7] * 3, [8] * 10]], [[0.5, 1.5]], [[-1.0, 1.0]])
    assert [len(c.response_tokens) for c in chunks] == [3, 4, 4, 2]
    assert [len(c.response_prefix) for c in chunks] == [0, 0, 4, 8]
    assert chunks[3].reward == 1.5 and chunks[3].advantage == 1.0 and chunks[3].source_idx == (0, 1)


def test_c3po_ffd_respects_bin_limit_and_schema():
    s = C3POPlusScheduler(C3POConfig(True, token_budget=8, target_batch_tokens=40))
    prompts = [[0] * 5, [1] * 7]
    responses = [[[2] * 20, [3] * 6], [[4] * 9, [5] * 30]]
    rewards = [[1.0, 0.0], [0.3, 0.7]]
    advs = [[1.0, -1.0], [-1.0, 1.0]]
    subs = s.split_and_pack(prompts, responses, rewards, advs)
    total_chunks = 0
    for sb in subs:
        assert set(sb) == {"prompts_tokens", "responses_group", "rewards_group", "precomputed_advantages"}
        n = len(sb["prompts_tokens"])
        assert n == len(sb["responses_group"]) == len(sb["rewards_group"]) == len(sb["precomputed_advantages"])
        tokens = sum(len(p) + len(r[0]) for p, r in zip(sb["prompts_tokens"], sb["responses_group"]))
        assert tokens <= 40 or n == 1           # an over-sized chunk sits alone in its bin
        total_chunks += n
    assert total_chunks == 3 + 1 + 2 + 4
    # the response tokens reassemble, in order, per (prompt, k)
    rebuilt = {}
    for sb in subs:
        for p, r in zip(sb["prompts_tokens"], sb["responses_group"]):
            rebuilt.setdefault(r[0][0], []).append((len(p), r[0]))
    assert sum(len(x[1]) for x in rebuilt[5]) == 30
    assert s.last_stats["bins"] == len(subs)


def test_icepop_with_c3po_chunk_count():
    s = C3POPlusScheduler(C3POConfig(True, token_budget=16, target_batch_tokens=128))
    subs = s.split_and_pack([[1] * 8], [[[2] * 40, [3] * 10]], [[1.0, 0.0]], [[1.0, -1.0]])
    n = sum(len(sb["prompts_tokens"]) for sb in subs)
    assert n == 3 + 1
    f = IcePopFilter(IcePopConfig(True, 0.5, 0.5))
    adv = torch.tensor([a[0] for sb in subs for a in sb["precomputed_advantages"]])
    out, _ = f.filter_divergent_responses(torch.zeros(n), torch.zeros(n), adv)
    assert torch.equal(out, adv)


def test_c3po_chunks_carry_their_own_mean_rollout_logprob():
    from b200fw.train.c3po import C3POConfig, C3POPlusScheduler
    s = C3POPlusScheduler(C3POConfig(True, token_budget=4, target_batch_tokens=64))
    prompts, resp = [[1, 2, 3]], [[[10, 11, 12, 13, 14, 15], [20, 21]]]
    tlp = [[[-1.0, -1.0, -1.0, -1.0, -3.0, -5.0], [-2.0, -4.0]]]
    chunks = s.split(prompts, resp, [[1.0, 0.0]], [[0.5, -0.5]], tlp)
    got = {(c.source_idx, len(c.response_prefix)): c.infer_logprob for c in chunks}
    assert got == {((0, 0), 0): -1.0, ((0, 0), 4): -4.0, ((0, 1), 0): -3.0}
    subs = s.split_and_pack(prompts, resp, [[1.0, 0.0]], [[0.5, -0.5]], tlp)
    assert all("infer_log_probs" in sb and len(sb["infer_log_probs"]) == len(sb["prompts_tokens"]) for sb in subs)
    assert all("infer_log_probs" not in sb for sb in s.split_and_pack(prompts, resp, [[1.0, 0.0]], [[0.5, -0.5]]))
