"""Inference runtime on CPU: KV manager, prefix / radix caches, scheduler policy, mock engine, and the
native paged engine against the eager (full re-forward) oracle for every feature switch."""
import pytest
import torch

from b200fw.infer import (BlockPool, ContinuousBatchingScheduler, InferenceConfig, InferenceEngine, KVCacheManager,
                          PrefixCache, RadixAttentionCache, Request, verify_greedy, verify_sampling)
from b200fw.model import PRESETS, ModelConfig, ParallelTransformerModel

MC = ModelConfig(vocab_size=128, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                 intermediate_size=48, max_position_embeddings=256, tie_word_embeddings=True)
PROMPTS = [list(range(5, 23)), [3, 4, 5], [9] * 40, list(range(5, 21)) + [77, 78]]


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    m = ParallelTransformerModel(MC)
    m.init_weights(0, std=0.3)
    return m


def _engine(model, **kw):
    base = dict(num_blocks=64, inference_mode="kv_cache", temperature=0.0, chunk_size=16, max_prefill_tokens=32,
                eos_token_id=None)
    base.update(kw)
    return InferenceEngine(InferenceConfig.from_model_config(MC, **base), model).initialize()


@pytest.fixture(scope="module")
def oracle(model):
    cfg = InferenceConfig.from_model_config(MC, inference_mode="eager", temperature=0.0, eos_token_id=None)
    return InferenceEngine(cfg, model).initialize().generate(PROMPTS, max_tokens=10)


def test_kv_manager_allocation_rollback_and_double_free():
    pool = BlockPool(8, 16, 1, 1, 8, torch.float32, "cpu")
    mgr = KVCacheManager(pool, 16)
    assert mgr.can_allocate(16 * 7) and not mgr.can_allocate(16 * 8)        # one spare block is kept
    t = mgr.allocate_for_sequence("a", 40)
    assert t.num_blocks == 3 and pool.num_free_blocks == 5
    assert mgr.allocate_for_sequence("b", 16 * 6) is None                     # rolled back completely
    assert pool.num_free_blocks == 5 and mgr.alloc_failures == 1
    for _ in range(8):
        assert mgr.append_token("a")
    assert mgr.get_seq_token_count("a") == 48 and t.num_blocks == 3
    assert mgr.append_token("a") and t.num_blocks == 4
    mgr.trim("a", 17)
    assert t.num_blocks == 2 and mgr.get_seq_token_count("a") == 17
    blk = t.blocks[0]
    mgr.free_sequence("a")
    assert pool.num_free_blocks == 8
    pool.free(blk)
    assert pool.double_free_count == 1 and pool.num_free_blocks == 8
    shared = mgr.allocate_for_sequence("c", 32)
    ids = shared.get_physical_block_ids()
    mgr.allocate_for_sequence("d", 48, shared_block_ids=ids)
    assert pool.get_block(ids[0]).ref_count == 2
    mgr.free_sequence("c")
    assert pool.get_block(ids[0]).ref_count == 1 and ids[0] not in pool.free_list


@pytest.mark.parametrize("cls", [PrefixCache, RadixAttentionCache])
def test_prefix_caches(cls):
    c = cls(block_size=4) if cls is RadixAttentionCache else cls(block_size=4, max_cached_blocks=3)
    toks = list(range(1, 14))
    assert c.match_prefix(toks) == (0, [])
    assert c.insert(toks, [10, 11, 12]) == [10, 11, 12]
    assert c.match_prefix(toks) == (12, [10, 11, 12])
    assert c.match_prefix(toks[:8] + [99] * 5) == (8, [10, 11])
    assert c.match_prefix([1, 2, 3, 5] + toks[4:]) == (0, [])
    assert 0 < c.hit_rate < 1
    evicted = []
    c.on_evict = evicted.append
    assert c.evict_lru(1) == []                    # everything is referenced by the matches above
    c.release_blocks([10, 11, 12])
    c.release_blocks([10, 11])
    got = c.evict_lru(1)
    assert len(got) == 1 and evicted == got
    assert set(c.invalidate_all()) | set(got) == {10, 11, 12} and c.size == 0


def test_scheduler_decode_first_chunking_and_preemption():
    s = ContinuousBatchingScheduler(max_num_batched_tokens=64, max_num_sequences=3, max_prefill_tokens=48,
                                    chunk_size=16, enable_adaptive_chunking=True)
    for i, n in enumerate([40, 10, 30, 5]):
        s.add_request(Request(f"r{i}", list(range(n)), arrival_time=float(i)))
    out = s.schedule()
    # idle: chunk doubles to 32; 32 + 10 fit the 48-token prefill budget, the third request does not fit
    # the remaining 6 tokens and only the FIRST request of a step may take a partial chunk
    assert out.chunk_size == 32 and [out.prefill_tokens[r.request_id] for r in out.prefill_requests] == [32, 10]
    assert [r.request_id for r in s.running_queue] == ["r1"]
    for r in out.prefill_requests:
        r.num_computed_tokens += out.prefill_tokens[r.request_id]
    out = s.schedule()
    assert [r.request_id for r in out.decode_requests] == ["r1"]
    assert out.prefill_tokens == {"r0": 8, "r2": 16}            # sequence slots: 3 - 1 running = 2 new
    for r in out.prefill_requests:
        r.num_computed_tokens += out.prefill_tokens[r.request_id]
    assert [r.request_id for r in s.running_queue] == ["r1", "r0"]
    # too many running sequences -> the latest arrival is preempted and returns to the queue head
    s.max_num_sequences = 1
    out = s.schedule()
    assert [r.request_id for r in out.preempted_requests] == ["r1"] and s.waiting_queue[0].request_id == "r1"
    assert s.waiting_queue[0].num_computed_tokens == 0 and s.total_preempted == 1
    s.finish_request("r0")
    assert s.total_finished == 1 and s.has_pending_requests()


def test_mock_engine_lifecycle():
    e = InferenceEngine(InferenceConfig(inference_mode="mock", vocab_size=1000, max_prefill_tokens=64)).initialize()
    outs = e.generate([[1, 2, 3], [4] * 100], max_tokens=7)
    assert [len(o) for o in outs] == [7, 7] and all(3 <= t < 1000 for o in outs for t in o)
    e.add_request("x", [1] * 10, max_tokens=50)
    e.step()
    assert e.has_pending()
    # a weight update keeps running requests (staleness 1 is within the default bound) ...
    e.on_weights_updated()
    assert e.has_pending() and e.get_stats()["weights_version"] == 1 and e.requests["x"].weights_version == 0
    # ... a second one makes the request two versions stale: it is dropped, as is everything on abort_running=True
    e.on_weights_updated()
    assert not e.has_pending() and e.get_stats()["aborted_stale"] == 1
    e.add_request("y", [1] * 10, max_tokens=50)
    e.step()
    e.on_weights_updated(abort_running=True)
    assert not e.has_pending() and e.get_stats()["weights_version"] == 3
    k = e.generate([[7, 8]] * 4, max_tokens=3)           # K samples of one prompt
    assert len(k) == 4


@pytest.mark.parametrize("kw", [
    {}, {"enable_prefix_caching": True}, {"use_radix_cache": True},
    {"enable_partitioned_attention": True, "attention_partition_size": 64},
    {"enable_chunked_prefill": False, "max_prefill_tokens": 256},
    {"speculative_enabled": True, "speculative_num_tokens": 3, "speculative_draft_layers": 1},
    {"max_num_sequences": 2},
])
def test_paged_engine_matches_eager_oracle(model, oracle, kw):
    e = _engine(model, **kw)
    assert e.generate(PROMPTS, max_tokens=10) == oracle
    assert e.generate(PROMPTS, max_tokens=10) == oracle                      # second pass hits the caches
    st = e.get_stats()
    if "prefix_cache" in st:
        assert st["cached_prefix_tokens"] > 0 and st["prefix_cache"]["hits"] > 0
    held = st.get("prefix_cache", {}).get("size", 0)
    assert st["kv_cache"]["used_blocks"] == held and st["kv_cache"]["double_frees"] == 0


def test_fp8_kv_cache_close_to_oracle(model, oracle):
    out = _engine(model, kv_cache_dtype="fp8").generate(PROMPTS, max_tokens=10)
    same = sum(a == b for x, y in zip(out, oracle) for a, b in zip(x, y))
    assert same >= 0.6 * sum(len(o) for o in oracle)


def test_kv_exhaustion_is_isolated_per_request(model):
    e = _engine(model, num_blocks=4)
    outs = e.generate([[1] * 30, [2] * 200], max_tokens=4)
    assert len(outs[0]) == 4 and outs[1] == [] and e.get_stats()["request_errors"] == 1
    assert e.get_stats()["kv_cache"]["used_blocks"] == 0


def test_kv_pressure_preempts_the_newest_request_instead_of_failing_it(model):
    """Two requests that each fit the pool but not together once they grow: the newer one is preempted (blocks freed,
    recomputed later), nothing fails, both give the oracle's tokens; a third that can only be admitted after the
    others finished waits instead of failing."""
    prompts = [[7] * 40, [9] * 40, [11] * 60]
    ref = InferenceEngine(InferenceConfig.from_model_config(MC, inference_mode="eager", temperature=0.0, eos_token_id=None),
                          model).initialize()
    want = [ref.generate([p], max_tokens=30)[0] for p in prompts]
    e = _engine(model, num_blocks=7, chunk_size=64, max_prefill_tokens=128, max_num_batched_tokens=256)
    for i, p in enumerate(prompts):
        e.add_request(f"r{i}", p, 30)
    steps = 0
    while e.has_pending():
        e.step()
        steps += 1
        assert steps < 2000
    st = e.get_stats()
    assert [e.finished[f"r{i}"].output_tokens for i in range(3)] == want
    assert st["request_errors"] == 0 and st.get("memory_preemptions", 0) >= 1 and st.get("admission_deferrals", 0) >= 1
    assert st["kv_cache"]["used_blocks"] == 0 and e.finished["r1"].preemptions >= 1 and e.finished["r0"].preemptions == 0


def test_speculative_decoding_gives_way_under_kv_pressure(model):
    """A pool too small for a speculative round of every sequence: the engine drops the draft state of those sequences and
    decodes them normally (preempting if it must) instead of raising out of ``step``; the tokens stay the oracle's."""
    prompts = [[5, 6, 7, 8, 9] * 3, [11] * 20, list(range(3, 40))]
    ref = InferenceEngine(InferenceConfig.from_model_config(MC, inference_mode="eager", temperature=0.0, eos_token_id=None),
                          model).initialize()
    want = ref.generate(prompts, max_tokens=12)
    for blocks in (64, 6):
        e = _engine(model, num_blocks=blocks, speculative_enabled=True, speculative_num_tokens=3, speculative_draft_layers=1,
                    chunk_size=64, max_prefill_tokens=128, max_num_batched_tokens=256)
        assert e.generate(prompts, max_tokens=12) == want
        st = e.get_stats()
        assert st["request_errors"] == 0 and st["spec_rounds"] >= 1
        assert (st.get("spec_fallbacks", 0) >= 1) == (blocks == 6)
        assert st["kv_cache"]["used_blocks"] == 0 and e.draft_runner.mgr.pool.num_used_blocks == 0


def test_weight_update_in_place_changes_outputs(model, oracle):
    import copy
    m2 = ParallelTransformerModel(MC)
    m2.load_state_dict(copy.deepcopy(model.state_dict()))
    e = _engine(m2, enable_prefix_caching=True)
    assert e.generate(PROMPTS, max_tokens=10) == oracle
    from b200fw.model.hf_io import hf_named_tensors
    new = {k: v + 0.05 * torch.randn_like(v) for k, v in hf_named_tensors(m2)}
    assert e.load_weights(new) == len(new)
    assert e.get_stats()["prefix_cache"]["size"] == 0 and e.weights_version == 1
    assert e.generate(PROMPTS, max_tokens=10) != oracle


def test_speculative_verification_rules():
    logits = torch.full((4, 10), -5.0)
    for i, t in enumerate([3, 4, 7, 1]):
        logits[i, t] = 5.0
    assert verify_greedy(torch.tensor([3, 4, 5]), logits) == (2, 7)
    assert verify_greedy(torch.tensor([3, 4, 7]), logits) == (3, 1)
    assert verify_greedy(torch.tensor([9, 4, 7]), logits) == (0, 3)
    g = torch.Generator().manual_seed(0)
    probs = torch.softmax(logits[:3], -1)
    n, nxt = verify_sampling(torch.tensor([3, 4, 7]), probs, logits, 1.0, g)     # draft == target: all accepted
    assert n == 3 and 0 <= nxt < 10
    wrong = torch.zeros(3, 10)
    wrong[:, 0] = 1.0
    n, nxt = verify_sampling(torch.tensor([0, 0, 0]), wrong, logits, 1.0, g)     # p_t(0) ~ 0: reject at once
    assert n == 0 and nxt == 3
    # batched forms agree with the per-sequence rules
    from b200fw.infer.spec import verify_greedy_batch, verify_sampling_batch
    drafts = torch.tensor([[3, 4, 5], [3, 4, 7], [9, 4, 7]])
    nb, tb = verify_greedy_batch(drafts, logits[None].repeat(3, 1, 1))
    assert nb.tolist() == [2, 3, 0] and tb.tolist() == [7, 1, 3]
    dp = torch.stack([probs, wrong])
    nb, tb = verify_sampling_batch(torch.tensor([[3, 4, 7], [0, 0, 0]]), dp, logits[None].repeat(2, 1, 1), 1.0, g)
    assert nb.tolist() == [3, 0] and tb[1] == 3 and 0 <= int(tb[0]) < 10


def test_requests_with_a_shared_prefix_wait_for_the_first_prefill_and_share_its_blocks():
    cfg = PRESETS["tiny"]
    torch.manual_seed(0)
    m = ParallelTransformerModel(cfg)
    m.init_weights(1)
    e = InferenceEngine(InferenceConfig(inference_mode="kv_cache", block_size=16, num_blocks=128, use_radix_cache=True,
                                        max_num_batched_tokens=512, max_prefill_tokens=512, dtype="float32"), model=m)
    e.initialize()
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(3, cfg.vocab_size, (48,), generator=g).tolist()
    prompts = [shared + torch.randint(3, cfg.vocab_size, (5 + i,), generator=g).tolist() for i in range(4)]
    outs = e.generate(prompts, max_tokens=6, temperature=0.0)
    assert e.stats["cached_prefix_tokens"] == 3 * 48          # three of the four reused the 48-token prefix
    ref = InferenceEngine(InferenceConfig(inference_mode="kv_cache", block_size=16, num_blocks=128,
                                          enable_prefix_reuse=False, dtype="float32"), model=m).initialize()
    assert ref.generate(prompts, max_tokens=6, temperature=0.0) == outs
    assert not e._inflight_prefix


def test_one_step_late_decode_bookkeeping_on_cpu(model, oracle):
    """The one-step-late decode path (sampled ids consumed by the next launch before the host has read them) with
    its bookkeeping forced on the CPU: same tokens as the synchronous engine, EOS cuts, per-request lengths, a
    weight update in the middle, and nothing unresolved ever leaves the engine."""
    e = _engine(model, async_decode="force")
    assert e.generate(PROMPTS, max_tokens=10) == oracle
    assert e._inflight is None
    # EOS in the middle of the stream: the token after it (sampled one step ahead) is dropped
    eos = oracle[0][4]
    cut = [o[:o.index(eos) + 1] if eos in o else o for o in oracle]
    for flag in (False, "force"):
        assert _engine(model, async_decode=flag, eos_token_id=eos).generate(PROMPTS, max_tokens=10) == cut, flag
    # different lengths: some requests finish by count while others have a launch in flight
    e2 = _engine(model, async_decode="force")
    want_len = [3 + 2 * i for i in range(len(PROMPTS))]
    for i, (p, n) in enumerate(zip(PROMPTS, want_len)):
        e2.add_request(f"r{i}", p, max_tokens=n)
    seen = {}
    while e2.has_pending():
        for rid, toks in e2.step().items():
            seen.setdefault(rid, []).extend(toks)
    for i, n in enumerate(want_len):
        out = e2.finished[f"r{i}"].output_tokens
        assert out == oracle[i][:n] and all(t >= 0 for t in out) and seen[f"r{i}"] == out
    # a weight update between steps settles the launch in flight first; requests go on
    e3 = _engine(model, async_decode="force")
    for i, p in enumerate(PROMPTS):
        e3.add_request(f"q{i}", p, max_tokens=8)
    for _ in range(6):
        e3.step()
    e3.on_weights_updated()
    assert e3._inflight is None and e3.has_pending()
    while e3.has_pending():
        e3.step()
    assert all(len(e3.finished[f"q{i}"].output_tokens) == 8 and min(e3.finished[f"q{i}"].output_tokens) >= 0
               for i in range(len(PROMPTS)))


def test_fused_norm_rope_store_path_equals_the_two_step_path(model, oracle):
    """The runner stores the new K / V rows from the norm + RoPE op when the cache is 16-bit; with the switch off it
    runs the separate store.  Both give the oracle's tokens, and the op's cache rows equal ``kv_store``'s."""
    from b200fw.ops import kv_store, qknorm_rope, qknorm_rope_store, rope_tables
    e = _engine(model)
    assert e.runner.fuse_kv_store
    assert e.generate(PROMPTS, max_tokens=10) == oracle
    e2 = _engine(model)
    e2.runner.fuse_kv_store = False
    assert e2.generate(PROMPTS, max_tokens=10) == oracle
    torch.manual_seed(0)
    Hq, Hkv, D, M = 4, 2, 8, 21
    qkv = torch.randn(M, (Hq + 2 * Hkv) * D)
    qw, kw = torch.rand(D) + 0.5, torch.rand(D) + 0.5
    pos = torch.arange(M, dtype=torch.int32)
    cos, sin = rope_tables(64, D, 1e4, torch.device("cpu"))
    kc, vc = torch.zeros(3, 16, Hkv, D), torch.zeros(3, 16, Hkv, D)
    slots = torch.tensor([32 + i for i in range(16)] + [-1] + [3, 4, 5, 6], dtype=torch.int32)
    q, k, v = qknorm_rope_store(qkv, qw, kw, pos, cos, sin, Hq, Hkv, D, 1e-6, kc, vc, slots)
    q0, k0, v0 = qknorm_rope(qkv, qw, kw, pos, cos, sin, Hq, Hkv, D, 1e-6)
    kc0, vc0 = torch.zeros_like(kc), torch.zeros_like(vc)
    kv_store(k0, v0, kc0, vc0, torch.tensor([[2, 0, 16, 0], [0, 17, 4, 3]], dtype=torch.int32))
    assert torch.equal(q, q0) and torch.equal(kc, kc0) and torch.equal(vc, vc0)


def test_bad_requests_are_refused_at_submission_and_leave_the_engine_serving(model, oracle):
    """An empty prompt, a token outside the vocabulary, a prompt that fills the position table or a request id that is
    still in flight raises at ``add_request`` (these values index device tables unchecked); a ``max_tokens`` beyond the
    position table is shortened; ``generate`` queues nothing if one prompt of the batch is bad; the requests already
    in flight finish as if nothing happened."""
    eng = _engine(model)
    eng.add_request("good", PROMPTS[0], 10)
    eng.step()
    for rid, prompt, err in [("e", [], "empty prompt"), ("v", [5, MC.vocab_size, 7], "outside the vocabulary"),
                             ("n", [5, -1], "outside the vocabulary"), ("good", [5, 6], "already in flight"),
                             ("l", [9] * MC.max_position_embeddings, "no room")]:
        with pytest.raises(ValueError, match=err):
            eng.add_request(rid, prompt, 4)
    with pytest.raises(ValueError, match="max_tokens"):
        eng.add_request("neg", [4, 5], -1)
    with pytest.raises(ValueError, match="empty prompt"):
        eng.generate([[4, 5], []], max_tokens=3)
    assert set(eng.requests) == {"good"}                       # the good half of that batch was not queued either
    r = eng.add_request("long", [9] * (MC.max_position_embeddings - 5), 50)
    assert r.max_tokens == 5
    while eng.has_pending():
        eng.step()
    assert eng.finished["good"].output_tokens == oracle[0]
    assert len(eng.finished["long"].output_tokens) == 5
    assert eng.pool.num_free_blocks == eng.pool.num_blocks
    eng.add_request("good", PROMPTS[1], 2)                      # a finished id may be used again
    # sampling parameters are made sane: NaN / negative / vanishing temperature is greedy, top_p is clamped to [0, 1]
    odd = eng.add_request("odd", PROMPTS[1], 2, temperature=float("nan"), top_p=7.0)
    tiny = eng.add_request("tiny", PROMPTS[1], 2, temperature=1e-30, top_p=float("nan"))
    assert (odd.temperature, odd.top_p, tiny.temperature, tiny.top_p) == (0.0, 1.0, 0.0, 1.0)
    # the eager oracle applies the same checks
    cfg = InferenceConfig.from_model_config(MC, inference_mode="eager", temperature=0.0, eos_token_id=None)
    with pytest.raises(ValueError, match="empty prompt"):
        InferenceEngine(cfg, model).initialize().generate([[]], max_tokens=2)
    # mock mode has no tables to index: only the structural checks apply
    mock = InferenceEngine(InferenceConfig(inference_mode="mock", num_blocks=8)).initialize()
    mock.add_request("m", [10 ** 9], 2)
    with pytest.raises(ValueError, match="empty prompt"):
        mock.add_request("m2", [], 2)


@pytest.mark.parametrize("kw", [dict(), dict(async_decode="force"), dict(enable_prefix_caching=True),
                                dict(speculative_enabled=True, speculative_num_tokens=2, speculative_draft_layers=1)])
def test_out_of_memory_in_a_step_drops_the_batch_and_leaves_a_clean_engine(model, oracle, kw):
    """The error is made on the host (the runner's forward raises ``torch.cuda.OutOfMemoryError`` once): the step
    returns, the requests in flight are handed back with the tokens they had (no unread placeholder among them, each a
    prefix of the oracle's output), every block of every pool is free again, and the next batch is served in full."""
    eng = _engine(model, **kw)
    for i, p in enumerate(PROMPTS):
        eng.add_request(f"r{i}", p, 10)
    real, calls = eng.runner.forward, []

    def flaky(*a, **k):
        calls.append(1)
        if len(calls) == 6:
            raise torch.cuda.OutOfMemoryError("CUDA out of memory (made up by the test)")
        return real(*a, **k)
    eng.runner.forward = flaky
    steps = 0
    while eng.has_pending():
        eng.step()
        steps += 1
        assert steps < 500
    assert eng.stats["oom_recoveries"] == 1
    assert set(eng.finished) == {f"r{i}" for i in range(len(PROMPTS))} and not eng.requests
    for i in range(len(PROMPTS)):
        out = eng.finished[f"r{i}"].output_tokens
        assert -1 not in out and out == oracle[i][:len(out)]
    assert eng.pool.num_free_blocks == eng.pool.num_blocks and not eng.kv.tables
    if eng.spec is not None:
        dp = eng.draft_runner.pool
        assert dp.num_free_blocks == dp.num_blocks and not eng.draft_runner.mgr.tables
    eng.runner.forward = real
    assert eng.generate(PROMPTS, max_tokens=10) == oracle


def test_weight_updates_and_cancellations_from_another_thread_take_turns_with_the_steps(model, oracle):
    """A rollout (``generate``) runs on a worker thread while this thread announces weight updates (same weights, so the
    oracle holds), adds a request and cancels it again, hundreds of times: the engine's entry points take turns under
    its lock, the rollout's outputs equal the oracle's and the pool comes back whole."""
    import threading
    eng = _engine(model, async_decode="force", enable_prefix_caching=True, max_weight_staleness=10 ** 9)
    out, err = {}, []

    def rollout():
        try:
            for i in range(6):
                out[i] = eng.generate(PROMPTS, max_tokens=10)
        except Exception as e:  # noqa: BLE001
            err.append(e)
    t = threading.Thread(target=rollout)
    t.start()
    n = 0
    while t.is_alive():
        eng.on_weights_updated()
        eng.add_request(f"extra{n}", [7, 8, 9], 50)
        # cancelled here, unless the rollout thread's steps already carried it to its end
        assert eng.abort_request(f"extra{n}") or f"extra{n}" in eng.finished
        assert -1 not in eng.finished[f"extra{n}"].output_tokens
        n += 1
    t.join()
    assert not err, err
    assert n >= 1 and all(out[i] == oracle for i in range(6))
    for k in [k for k in eng.finished if k.startswith("extra")]:
        del eng.finished[k]
    if eng.prefix_cache is not None:
        eng.prefix_cache.evict_lru(eng.pool.num_blocks)
    assert eng.pool.num_free_blocks == eng.pool.num_blocks and not eng.kv.tables and not eng.requests


def test_radix_cache_at_capacity_never_hangs_a_block_under_an_evicted_node():
    """A path longer than the cache's capacity: making room for block i must not evict block i-1 (the only leaf), or
    block i ends up under a detached node - counted, holding its pool reference, unreachable and never evicted."""
    cache = RadixAttentionCache(2, 3)
    gone = []
    cache.on_evict = gone.append
    toks = [0, 0, 0, 1, 0, 0, 0, 1]
    new = cache.insert(toks, [10, 11, 12, 13])
    assert new == [10, 11, 12] and not gone and cache.size == 3           # the fourth block does not fit: left out
    assert cache.match_prefix(toks) == (6, [10, 11, 12])
    cache.release_blocks([10, 11, 12])
    assert cache.insert(toks, [20, 21, 22, 23]) == []                     # nothing new, nothing orphaned
    assert sorted(cache.invalidate_all()) == [10, 11, 12] and sorted(gone) == [10, 11, 12]
    # with another branch to give up, room is made from that branch
    cache = RadixAttentionCache(2, 3)
    cache.on_evict = gone.append
    del gone[:]
    cache.insert([5, 5], [1])
    assert cache.insert([0, 0, 0, 1, 0, 0], [2, 3, 4]) == [2, 3, 4] and gone == [1]
    assert cache.match_prefix([0, 0, 0, 1, 0, 0]) == (6, [2, 3, 4])
