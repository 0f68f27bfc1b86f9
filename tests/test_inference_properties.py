"""Property tests of the inference runtime's host logic (hypothesis): block accounting of the paged KV manager under
random operation sequences, and the paged engine against the eager oracle for random workloads under memory pressure
(preemption, chunked prefill, prefix sharing, one-step-late decode)."""
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

from b200fw.infer import BlockPool, InferenceConfig, InferenceEngine, KVCacheManager  # noqa: E402
from b200fw.model import ModelConfig, ParallelTransformerModel  # noqa: E402

BS = 4      # tokens per block in the accounting test


def _check_pool(pool: BlockPool, mgr: KVCacheManager, extra_refs):
    refs = {}
    for table in mgr.tables.values():
        for b in table.blocks:
            refs[b.block_id] = refs.get(b.block_id, 0) + 1
        assert table.capacity >= table.num_tokens
    for bid, n in extra_refs.items():
        refs[bid] = refs.get(bid, 0) + n
    free = list(pool.free_list)
    assert len(free) == len(set(free)), "a block sits in the free list twice"
    for b in pool.blocks:
        assert b.ref_count == refs.get(b.block_id, 0), (b.block_id, b.ref_count, refs.get(b.block_id, 0))
        assert (b.block_id in free) == (b.ref_count == 0)
    assert pool.num_free_blocks + sum(1 for b in pool.blocks if b.ref_count > 0) == pool.num_blocks
    assert pool.double_free_count == 0


OPS = st.lists(st.tuples(st.sampled_from(["new", "new_shared", "append", "grow", "trim", "free", "hold", "drop"]),
                         st.integers(0, 7), st.integers(0, 40)), min_size=1, max_size=60)


@settings(max_examples=150, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(OPS, st.integers(3, 24))
def test_block_accounting_survives_any_operation_sequence(ops, num_blocks):
    pool = BlockPool(num_blocks, BS, 1, 1, 4, torch.float32, "cpu", allocate=False)
    mgr = KVCacheManager(pool, BS)
    held = {}           # references a prefix cache would hold: block id -> count
    next_id = 0
    for op, which, n in ops:
        ids = sorted(mgr.tables)
        sid = ids[which % len(ids)] if ids else None
        free_before = pool.num_free_blocks
        if op == "new":
            t = mgr.allocate_for_sequence(next_id, n)
            if t is None:
                assert pool.num_free_blocks == free_before, "a failed allocation must roll back completely"
            else:
                assert t.num_blocks == mgr.blocks_needed(n) and t.num_tokens == n
            next_id += 1
        elif op == "new_shared" and sid is not None:
            src = mgr.tables[sid]
            full = [b.block_id for b in src.blocks[:src.num_tokens // BS]]
            shared = full[:which % (len(full) + 1)]
            total = len(shared) * BS + n
            t = mgr.allocate_for_sequence(next_id, total, shared_block_ids=shared)
            if t is None:
                assert pool.num_free_blocks == free_before
            else:
                assert t.get_physical_block_ids()[:len(shared)] == shared
            next_id += 1
        elif op == "append" and sid is not None:
            before = mgr.get_seq_token_count(sid)
            ok = mgr.append_token(sid)
            assert mgr.get_seq_token_count(sid) == before + (1 if ok else 0)
            if not ok:
                assert pool.num_free_blocks == free_before
        elif op == "grow" and sid is not None:
            ok = mgr.ensure_capacity(sid, mgr.get_seq_token_count(sid) + n)
            if not ok:
                assert pool.num_free_blocks == free_before
        elif op == "trim" and sid is not None:
            keep = min(mgr.get_seq_token_count(sid), n)
            mgr.trim(sid, keep)
            assert mgr.get_seq_token_count(sid) == keep
            assert mgr.tables[sid].num_blocks <= max(1, mgr.blocks_needed(keep)) or mgr.tables[sid].num_blocks == 0
        elif op == "free" and sid is not None:
            mgr.free_sequence(sid)
            assert sid not in mgr.tables
        elif op == "hold" and sid is not None and mgr.tables[sid].blocks:
            b = mgr.tables[sid].blocks[which % mgr.tables[sid].num_blocks]
            pool.share(b.block_id)
            held[b.block_id] = held.get(b.block_id, 0) + 1
        elif op == "drop" and held:
            bid = sorted(held)[which % len(held)]
            pool.free(pool.get_block(bid))
            held[bid] -= 1
            if held[bid] == 0:
                del held[bid]
        _check_pool(pool, mgr, held)
    mgr.reset()
    for bid, k in list(held.items()):
        for _ in range(k):
            pool.free(pool.get_block(bid))
    assert pool.num_free_blocks == pool.num_blocks and pool.double_free_count == 0


MC = ModelConfig(vocab_size=96, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                 intermediate_size=48, max_position_embeddings=256, tie_word_embeddings=True)


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    m = ParallelTransformerModel(MC)
    m.init_weights(0, std=0.3)
    return m


def _engine(model, **kw):
    base = dict(inference_mode="kv_cache", temperature=0.0, eos_token_id=None, num_blocks=256, block_size=16)
    base.update(kw)
    return InferenceEngine(InferenceConfig.from_model_config(MC, **base), model).initialize()


WORKLOAD = st.lists(st.tuples(st.integers(1, 70), st.integers(1, 24), st.booleans()), min_size=1, max_size=10)


@settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(WORKLOAD, st.integers(0, 3), st.sampled_from([8, 16, 48]), st.sampled_from(["none", "hash", "radix"]), st.booleans(),
       st.sampled_from([2, 3, 256]), st.sampled_from([0, 0, 2, 4]), st.sets(st.integers(1, 60), max_size=3),
       st.sampled_from([100, 100, 1, 0]), st.dictionaries(st.integers(1, 40), st.integers(0, 9), max_size=2))
def test_paged_engine_equals_eager_oracle_under_memory_pressure(model, workload, slack, chunk, cache, late, max_seqs, spec_k,
                                                                update_at, staleness, abort_at):
    """Random prompts (some sharing a 32-token prefix), a block pool barely larger than the largest single request
    (so running sequences get preempted and recomputed), small prefill chunks, no / hash / radix prefix cache, read-back one
    step late or not, greedy speculative decoding with a one-layer draft or none: outputs must equal the eager full-recompute oracle, and every block must come back."""
    g = torch.Generator().manual_seed(len(workload) * 1000 + slack)
    prefix = torch.randint(3, 96, (32,), generator=g).tolist()
    prompts, outs = [], []
    for plen, out_len, shared in workload:
        body = torch.randint(3, 96, (plen,), generator=g).tolist()
        prompts.append((prefix + body) if shared else body)
        outs.append(out_len)
    longest = max(len(p) + o for p, o in zip(prompts, outs))
    blocks = (longest + 15) // 16 + 2 + slack              # the biggest request fits, several at once usually do not
    oracle = _engine(model, inference_mode="eager")
    want = [oracle.generate([p], max_tokens=o)[0] for p, o in zip(prompts, outs)]
    eng = _engine(model, num_blocks=blocks, chunk_size=chunk, max_prefill_tokens=max(chunk, 16),
                  max_num_batched_tokens=max(chunk, 16) + 8, use_radix_cache=cache == "radix",
                  enable_prefix_caching=cache != "none",
                  max_cached_blocks=blocks, async_decode="force" if late else False, adaptive_chunking=False,
                  max_num_sequences=max_seqs, speculative_enabled=spec_k > 0, speculative_num_tokens=max(1, spec_k),
                  speculative_draft_layers=1, max_weight_staleness=staleness)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        eng.add_request(f"r{i}", p, o)
    steps = cancelled = 0
    while eng.has_pending():
        eng.step()
        steps += 1
        if steps in update_at:
            eng.on_weights_updated()
        if steps in abort_at:
            rid = f"r{abort_at[steps] % len(prompts)}"
            was_live = rid in eng.requests
            assert eng.abort_request(rid) == was_live
            cancelled += int(was_live)
            assert rid not in eng.requests and rid in eng.finished and not eng.abort_request(rid)
        assert steps < 5000, "the engine stopped making progress"
    dropped = eng.stats.get("aborted_stale", 0)
    assert dropped == 0 or staleness < 100
    got = [eng.finished[f"r{i}"].output_tokens for i in range(len(prompts))]
    short = 0
    for i, (a, b) in enumerate(zip(got, want)):
        assert -1 not in a, "a placeholder of the one-step-late decode left the engine"
        if len(a) < len(b):
            short += 1
            assert list(a) == list(b[:len(a)]), (i, a, b)
        else:
            assert list(a) == list(b), (i, prompts[i][:6], a, b)
    assert short <= dropped + cancelled
    # every block is back in the pool except those the prefix cache still references; evicting them frees the rest
    if eng.prefix_cache is not None:
        eng.prefix_cache.evict_lru(blocks)
    assert eng.pool.num_free_blocks == eng.pool.num_blocks, (eng.pool.num_free_blocks, eng.pool.num_blocks)
    assert eng.pool.double_free_count == 0 and not eng.kv.tables


@settings(max_examples=200, deadline=None)
@given(st.lists(st.floats(-30, 30, allow_nan=False, width=32), min_size=2, max_size=40),
       st.floats(-1.0, 4.0, allow_nan=False), st.floats(-0.5, 1.5, allow_nan=False), st.floats(0.0, 1.0, allow_nan=False))
def test_cpu_sampler_picks_inside_the_nucleus(row, temp, top_p, u):
    """The CPU sampler (the oracle of the sampling kernel): the pick is a valid index; greedy at temperature <= 0; at
    top_p <= 0 the most likely token; otherwise a token of the smallest set of most likely tokens whose mass reaches
    top_p; the reported log-prob is the tempered full-softmax one."""
    from b200fw.ops import topp_sample
    if 0 < temp < 1e-3:
        temp = 0.0                  # the engine maps vanishing temperatures to greedy before they reach the sampler
    logits = torch.tensor([row], dtype=torch.float32)
    ids, lps = topp_sample(logits, torch.tensor([temp]), torch.tensor([top_p]), torch.tensor([u]), return_logprob=True)
    pick = int(ids[0])
    assert 0 <= pick < len(row)
    if temp <= 0:
        assert logits[0, pick] == logits.max()
        return
    lp = torch.log_softmax(logits[0] / temp, -1)
    assert abs(float(lps[0]) - float(lp[pick])) < 1e-5
    p = lp.exp()
    sp, _ = p.sort(descending=True)
    before = sp.cumsum(0) - sp
    nucleus = sp[before < min(max(top_p, 0.0), 1.0)]
    floor = float(nucleus[-1]) if nucleus.numel() else float(sp[0])
    assert float(p[pick]) >= floor * (1 - 1e-5), (pick, float(p[pick]), floor)
    if top_p <= 0:
        assert float(p[pick]) >= float(sp[0]) * (1 - 1e-6)


CACHE_OPS = st.lists(st.tuples(st.sampled_from(["insert", "match", "release", "evict", "clear"]),
                               st.lists(st.integers(0, 2), min_size=0, max_size=14), st.integers(0, 5)),
                     min_size=1, max_size=50)


@settings(max_examples=150, deadline=None)
@given(CACHE_OPS, st.sampled_from(["hash", "radix"]), st.integers(2, 8))
def test_prefix_caches_agree_with_a_plain_model_of_them(ops, kind, capacity):
    """Random insert / match / release / evict / clear sequences on the hash-chain and the radix cache (blocks of 2
    tokens over a 3-letter alphabet, so prefixes collide all the time) against a dictionary model: a match returns the
    block that was registered FIRST for each block-aligned prefix, whole blocks only and never past a gap; a block
    leaves the cache exactly once (eviction callback), never while a match holds it; the cache never exceeds its
    capacity."""
    from b200fw.infer import PrefixCache, RadixAttentionCache
    BSZ = 2
    cache = PrefixCache(BSZ, capacity) if kind == "hash" else RadixAttentionCache(BSZ, capacity)
    registered = {}          # prefix tuple (k whole blocks) -> block id in the cache
    held = {}                # block id -> outstanding matches
    gone = []
    cache.on_evict = gone.append
    next_block = [0]

    def live_prefixes():
        return {p: b for p, b in registered.items() if b not in gone}
    for op, toks, n in ops:
        nblocks = len(toks) // BSZ
        if op == "insert":
            ids = list(range(next_block[0], next_block[0] + nblocks))
            next_block[0] += nblocks
            new = cache.insert(toks, ids)
            assert set(new) <= set(ids)
            for i, bid in enumerate(ids):
                if bid in new:
                    p = tuple(toks[:(i + 1) * BSZ])
                    assert p not in live_prefixes(), "a second block was cached for a prefix that is already there"
                    registered[p] = bid
        elif op == "match":
            matched, ids = cache.match_prefix(toks)
            assert matched == len(ids) * BSZ and matched <= nblocks * BSZ
            live = live_prefixes()
            for i, bid in enumerate(ids):
                assert live.get(tuple(toks[:(i + 1) * BSZ])) == bid
            if len(ids) < nblocks and kind == "radix":
                assert tuple(toks[:(len(ids) + 1) * BSZ]) not in live      # the radix tree stops only at a real gap
            for bid in ids:
                held[bid] = held.get(bid, 0) + 1
        elif op == "release" and held:
            bid = sorted(held)[n % len(held)]
            cache.release_blocks([bid])
            held[bid] -= 1
            if held[bid] == 0:
                del held[bid]
        elif op == "evict":
            before = len(gone)
            out = cache.evict_lru(n)
            assert len(out) <= n and gone[before:] == out
            assert not (set(out) & set(held)), "a block that a match still holds was evicted"
        elif op == "clear" and n == 0 and not held:
            cache.invalidate_all()
            registered = {p: b for p, b in registered.items() if b in gone}
        assert len(gone) == len(set(gone)), "a block left the cache twice"
        size = len(cache.entries) if kind == "hash" else cache.size
        assert size <= capacity
        assert size == len(live_prefixes()), (size, live_prefixes())


@settings(max_examples=100, deadline=None)
@given(st.lists(st.tuples(st.integers(1, 300), st.integers(1, 40), st.integers(0, 30)), min_size=1, max_size=40),
       st.sampled_from([16, 64, 256]), st.sampled_from([1, 2, 8, 64]), st.sampled_from([8, 32, 512]), st.booleans(),
       st.booleans())
def test_scheduler_budgets_hold_every_step_and_every_request_finishes(reqs, max_tokens, max_seqs, chunk, chunked, adaptive):
    """The mock engine (scheduler and bookkeeping only, no model) over random arrivals: every step's batch respects the
    token, prefill and sequence budgets, a prefill chunk never exceeds what is left of its prompt, decode requests are
    scheduled before new prefills, and every request finishes with exactly ``max_tokens`` tokens."""
    cfg = InferenceConfig(inference_mode="mock", num_blocks=8, max_num_batched_tokens=max_tokens, max_num_sequences=max_seqs,
                          max_prefill_tokens=max(8, max_tokens // 2), chunk_size=chunk, enable_chunked_prefill=chunked,
                          adaptive_chunking=adaptive, eos_token_id=None)
    eng = InferenceEngine(cfg).initialize()
    real = eng.scheduler.schedule

    def checked():
        out = real()
        assert len(out.decode_requests) <= max_seqs
        fresh = [r for r in out.prefill_requests if r not in out.decode_requests]
        assert len(out.decode_requests) + len(fresh) <= max(max_seqs, len(out.decode_requests))
        assert out.num_prefill_tokens <= cfg.max_prefill_tokens
        assert out.total_tokens <= max(max_tokens, len(out.decode_requests) + 1)
        for r in out.prefill_requests:
            n = out.prefill_tokens[r.request_id]
            assert 0 < n <= r.remaining_prefill_tokens
        return out
    eng.scheduler.schedule = checked
    arrivals = sorted(((at, i, p, o) for i, (p, o, at) in enumerate(reqs)))
    step, k = 0, 0
    while k < len(arrivals) or eng.has_pending():
        while k < len(arrivals) and arrivals[k][0] <= step:
            _, i, p, o = arrivals[k]
            eng.add_request(f"r{i}", [3 + (j % 90) for j in range(p)], o)
            k += 1
        eng.step()
        step += 1
        assert step < 20000, "the scheduler stopped making progress"
    assert len(eng.finished) == len(reqs) and not eng.requests
    for i, (p, o, _) in enumerate(reqs):
        assert len(eng.finished[f"r{i}"].output_tokens) == o
