"""Property tests (hypothesis) of two pieces of host logic that every RL iteration depends on: C3PO++ splitting /
packing never loses, duplicates or reorders a response token, and a SwiftSync receiver that is fed any sequence of delta
and full syncs (dict or flat payloads, with or without double buffering) ends up holding the trainer's latest adapters."""
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from b200fw.sync import SwiftSyncConfig, SwiftSyncTransfer  # noqa: E402
from b200fw.sync.double_buffer import FlatLayout, FlatState  # noqa: E402
from b200fw.train.c3po import C3POConfig, C3POPlusScheduler  # noqa: E402

GROUPS = st.lists(st.tuples(st.integers(1, 30),                                             # prompt length
                            st.lists(st.integers(0, 70), min_size=1, max_size=4)),            # response lengths
                  min_size=1, max_size=6)


@settings(max_examples=200, deadline=None)
@given(GROUPS, st.integers(1, 40), st.integers(8, 200), st.booleans())
def test_c3po_chunks_cover_every_response_exactly_once(groups, budget, target, with_logprobs):
    prompts, responses, rewards, advs, tlps = [], [], [], [], []
    tok = 0
    for b, (plen, rlens) in enumerate(groups):
        prompts.append([1000 + b] * plen)
        rs = []
        for n in rlens:
            rs.append(list(range(tok, tok + n)))        # globally unique token ids: any loss or duplicate shows
            tok += n
        responses.append(rs)
        rewards.append([float(b + k) for k in range(len(rlens))])
        advs.append([0.5 * (b - k) for k in range(len(rlens))])
        tlps.append([[-0.01 * t for t in r] for r in rs])
    sch = C3POPlusScheduler(C3POConfig(True, budget, target))
    chunks = sch.split(prompts, responses, rewards, advs, tlps if with_logprobs else None)
    seen = {}
    for c in chunks:
        b, k = c.source_idx
        assert c.prompt_tokens == prompts[b] and c.reward == rewards[b][k] and c.advantage == advs[b][k]
        assert len(c.response_tokens) <= budget
        # a chunk's prefix is exactly the response up to where the chunk starts
        assert c.response_prefix + c.response_tokens == responses[b][k][:len(c.response_prefix) + len(c.response_tokens)]
        seen.setdefault((b, k), []).append(c)
        if with_logprobs and c.response_tokens:
            want = sum(-0.01 * t for t in c.response_tokens) / len(c.response_tokens)
            assert c.infer_logprob is not None and abs(c.infer_logprob - want) < 1e-9
    for b, rs in enumerate(responses):
        for k, r in enumerate(rs):
            parts = sorted(seen[(b, k)], key=lambda c: len(c.response_prefix))
            assert [t for c in parts for t in c.response_tokens] == r          # nothing lost, duplicated or reordered
            assert len(parts) == max(1, -(-len(r) // budget))
    bins = sch.pack(chunks)
    assert sorted(id(c) for bn in bins for c in bn) == sorted(id(c) for c in chunks)
    for bn in bins:
        load = sum(c.length for c in bn)
        assert load <= target or len(bn) == 1            # only a chunk that is too long by itself may overflow a bin
    kws = sch.split_and_pack(prompts, responses, rewards, advs)
    assert sum(len(kw["prompts_tokens"]) for kw in kws) == len(chunks)
    for kw in kws:
        assert len(kw["prompts_tokens"]) == len(kw["responses_group"]) == len(kw["rewards_group"]) == len(kw["precomputed_advantages"])


SHAPES = {"l0.q.lora_A": (2, 5), "l0.q.lora_B": (7, 2), "l1.o.lora_A": (2, 3), "l1.o.lora_B": (4, 2)}
LAYOUT = FlatLayout(list(SHAPES), list(SHAPES.values()))


class _Receiver:
    """What an inference worker does with SwiftSync payloads: keep a copy of the adapters, add deltas, replace on full."""

    def __init__(self, fail_on=None):
        self.state, self.calls, self.fail_on = None, 0, fail_on

    def update_weights(self, payload, mode="full"):
        self.calls += 1
        if self.fail_on is not None and self.calls == self.fail_on:
            raise RuntimeError("receiver is unavailable (made up by the test)")
        payload = {k: v.clone() for k, v in payload.items()}
        if mode == "full" or self.state is None:
            self.state = payload
        else:
            for k, v in payload.items():
                self.state[k] = self.state[k] + v


@settings(max_examples=120, deadline=None)
@given(st.lists(st.integers(0, 2 ** 31 - 1), min_size=1, max_size=12), st.integers(1, 5), st.booleans(), st.booleans(),
       st.one_of(st.none(), st.integers(1, 12)))
def test_receiver_tracks_the_trainer_through_any_sync_sequence(seeds, full_every, flat, double_buffer, fail_on):
    recv = _Receiver(fail_on)
    t = SwiftSyncTransfer(recv, SwiftSyncConfig(True, fallback_full_every=full_every, double_buffer=double_buffer))
    last_good_version = 0
    for step, seed in enumerate(seeds):
        cur = torch.randn(LAYOUT.numel, generator=torch.Generator().manual_seed(seed))
        payload = FlatState(LAYOUT, cur.clone()) if flat else {k: v.clone() for k, v in FlatState(LAYOUT, cur).items()}
        try:
            v = int(t.sync(step, payload))
        except RuntimeError:
            # a worker that cannot take the payload must not see a version bump; the next sync repairs the state
            assert t.buffer.version == last_good_version
            continue
        assert v == t.buffer.version == last_good_version + 1
        last_good_version = v
        want = FlatState(LAYOUT, cur)
        active = t.buffer.get_active_state()
        for k in SHAPES:
            assert torch.allclose(recv.state[k], want[k], atol=1e-5), (step, k, t.stats.last_mode)
            assert torch.allclose(active[k], want[k], atol=1e-5), (step, k, t.stats.last_mode)
    assert t.stats.delta_syncs + t.stats.full_syncs == last_good_version


@settings(max_examples=300, deadline=None)
@given(st.lists(st.tuples(st.floats(-5, 5, width=32), st.one_of(st.floats(-5, 5, width=32), st.just(float("nan")), st.just(float("inf"))),
                          st.floats(-3, 3, width=32)), min_size=1, max_size=24),
       st.sampled_from([0.0, 0.1, 0.5, 2.0]), st.sampled_from([0.0, 0.25, 0.5, 1.0]))
def test_icepop_masks_exactly_the_most_divergent_responses_up_to_its_cap(rows, threshold, max_ratio):
    from b200fw.train.icepop import IcePopConfig, IcePopFilter
    train = torch.tensor([r[0] for r in rows])
    infer = torch.tensor([r[1] for r in rows])
    adv = torch.tensor([r[2] for r in rows])
    f = IcePopFilter(IcePopConfig(True, threshold, max_ratio))
    out, diag = f.filter_divergent_responses(train, infer, adv)
    gap = (train - infer).abs()
    gap = torch.where(torch.isfinite(gap), gap, torch.full_like(gap, float("inf")))
    over = gap > threshold
    cap = int(len(rows) * max_ratio)
    k = min(cap, int(over.sum()))
    masked = (out == 0) & (adv != 0)
    assert diag["icepop_num_masked"] == k and f.total_masked == k and f.total_seen == len(rows)
    assert int(masked.sum()) <= k
    # untouched entries keep their advantage bit for bit; every masked one was over the threshold
    assert torch.equal(out[~masked], adv[~masked]) and bool(over[masked].all())
    if k and k < int(over.sum()):
        # the cap was binding: nothing that stayed is more divergent than something that was dropped
        dropped_min = gap[masked].min() if bool(masked.any()) else None
        kept_over = over & ~masked & (adv != 0)
        if dropped_min is not None and bool(kept_over.any()):
            assert float(gap[kept_over].max()) <= float(dropped_min)
    if k == int(over.sum()):
        assert bool(((out == 0) | ~over).all())          # below the cap every divergent response is neutralised
    assert torch.isfinite(torch.tensor(diag["icepop_mean_divergence"])) and f.last_non_finite == int((~torch.isfinite(train - infer)).sum())
