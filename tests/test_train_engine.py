"""TrainEngine end to end on CPU: the tiny-Qwen3 DP2 + ZeRO-1 plumbing configuration, 1F1B pipeline
equivalence, GRPO step against a plain PyTorch oracle, checkpoints, truncation."""
import math
import tempfile

import pytest
import torch

from _dist_util import run_ranks
from b200fw.model import PRESETS, ModelConfig, ParallelTransformerModel
from b200fw.train import TrainConfig, TrainEngine

SMALL = ModelConfig(vocab_size=256, hidden_size=32, num_layers=4, num_heads=2, num_kv_heads=2, head_dim=16,
                    intermediate_size=48, max_position_embeddings=128, tie_word_embeddings=False)


def _tiny_batch(step, rank, n, seq, vocab):
    g = torch.Generator().manual_seed(step * 17 + rank)
    ids = torch.randint(0, vocab, (n, seq), generator=g)
    labels = ids.clone()
    labels[:, : seq // 2] = -100
    return ids, labels


def _tiny_worker(rank, world, steps, seq):
    cfg = TrainConfig(model_preset="tiny", dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-4,
                      gradient_accumulation_steps=1, zero_stage=1, use_amp=False, amp_dtype="fp32",
                      warmup_steps=max(1, steps // 20), total_training_steps=steps, lr_scheduler_type="cosine",
                      max_seq_len=seq, backend="gloo", bucket_mb=4.0)
    eng = TrainEngine(cfg).initialize()
    assert eng.optimizer.stage == 1 and eng.optimizer.world == world
    out = []
    for s in range(steps):
        ids, labels = _tiny_batch(s, rank, 4 // world, seq, 8192)
        m = eng.sft_step_tensors(ids, labels)
        out.append((m.loss, m.grad_norm, m.learning_rate))
    return out


def test_tiny_qwen3_sft_dp2_zero1_matches_single_process():
    """4 layers / hidden 256 / 4q-2kv heads of 64 / FFN 704 / vocab 8192 / tied; batch 4 x seq 256 (seq
    shortened to 64 here for CPU time), loss on the second half, AdamW 1e-4, 5 % warm-up, cosine."""
    steps, seq = 20, 64
    dp = run_ranks(_tiny_worker, 2, steps, seq, timeout=900)
    # oracle: one process, plain torch AdamW, whole global batch
    torch.manual_seed(0)
    model = ParallelTransformerModel(PRESETS["tiny"])
    model.init_weights(0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    from b200fw.optim import LRSchedule
    sched = LRSchedule(1e-4, "cosine", 1, steps, 0.1)
    for s in range(steps):
        for g in opt.param_groups:
            g["lr"] = sched.lr_at(s)
        losses = []
        for r in range(2):
            ids, labels = _tiny_batch(s, r, 2, seq, 8192)
            l = model.loss(ids, labels)
            (l / 2).backward()
            losses.append(l.item())
        gn = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        for r in range(2):
            assert abs(dp[r][s][0] - losses[r]) < 2e-4, (s, r, dp[r][s][0], losses[r])
            assert abs(dp[r][s][1] - float(gn)) / float(gn) < 1e-3
            assert abs(dp[r][s][2] - sched.lr_at(s)) < 1e-12


def _pp_worker(rank, world, path):
    from b200fw.model import load_from_hf_checkpoint
    cfg = TrainConfig(model_config=SMALL, pp_size=world, num_micro_batches=4, lora_rank=0, grpo_beta=0.0,
                      learning_rate=1e-3, gradient_accumulation_steps=1, zero_stage=1, use_amp=False,
                      amp_dtype="fp32", warmup_steps=0, max_seq_len=32, backend="gloo", max_grad_norm=0.0)
    eng = TrainEngine(cfg).initialize()
    load_from_hf_checkpoint(eng.model, path, strict=False)
    eng.optimizer.refresh_masters_from_params()
    m = eng.model
    assert (m.embed_tokens is not None) == (rank == 0) and (m.lm_head is not None) == (rank == world - 1)
    assert len(m.layers) == 2
    ids, labels = _tiny_batch(0, 0, 8, 16, SMALL.vocab_size)
    eng.optimizer.begin_backward(True)
    loss = eng.pipeline_scheduler.run_1f1b_schedule(ids, labels)
    loss = eng.pipeline_scheduler.broadcast_loss(loss)
    grads = {f"{m.layer_start + i}": l.mlp.down_proj.weight.grad.clone() for i, l in enumerate(m.layers)}
    met = eng.sft_step_tensors(ids, labels)     # a full step through the public API also works
    return float(loss), {k: v.tolist() for k, v in grads.items()}, met.loss


def test_pipeline_1f1b_matches_single_process():
    from b200fw.model import save_hf_checkpoint
    with tempfile.TemporaryDirectory() as d:
        ref = ParallelTransformerModel(SMALL)
        ref.init_weights(11)
        save_hf_checkpoint(ref, d)
        res = run_ranks(_pp_worker, 2, d, timeout=600)
        ids, labels = _tiny_batch(0, 0, 8, 16, SMALL.vocab_size)
        # mean of per-micro-batch means, as the schedule computes it
        total = 0.0
        for mb_ids, mb_labels in zip(ids.chunk(4), labels.chunk(4)):
            l = ref.loss(mb_ids, mb_labels)
            (l / 4).backward()
            total += l.item() / 4
        assert abs(res[0][0] - total) < 1e-5 and abs(res[1][0] - total) < 1e-5
        for r in range(2):
            for k, g in res[r][1].items():
                want = ref.layers[int(k)].mlp.down_proj.weight.grad
                assert (torch.tensor(g) - want).abs().max() < 1e-6
        assert abs(res[0][2] - res[1][2]) < 1e-7


def test_grpo_step_matches_oracle_and_icepop_masks():
    torch.manual_seed(0)
    cfg = TrainConfig(model_config=SMALL, lora_rank=0, grpo_beta=0.05, grpo_clip_eps=0.2, learning_rate=1e-3,
                      gradient_accumulation_steps=1, use_amp=False, amp_dtype="fp32", warmup_steps=0,
                      max_seq_len=64, icepop_enabled=True, icepop_divergence_threshold=1e9)
    eng = TrainEngine(cfg).initialize()
    assert eng.ref_model is not None
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 256, (6,), generator=g).tolist() for _ in range(2)]
    groups = [[torch.randint(0, 256, (5 + k,), generator=g).tolist() for k in range(3)] for _ in range(2)]
    rewards = [[1.0, 0.0, 0.5], [0.2, 0.2, 0.2]]
    # oracle on a clone of the initial weights
    oracle = eng.model.clone(requires_grad=True)
    m = eng.grpo_step(prompts, groups, rewards)
    adv = TrainEngine.group_advantages(rewards[0]) + TrainEngine.group_advantages(rewards[1])
    assert adv[3:] == [0.0, 0.0, 0.0] and abs(sum(adv[:3])) < 1e-5
    seqs = [p + r for p, rs in zip(prompts, groups) for r in rs]
    L = max(len(s) for s in seqs)
    ids = torch.tensor([s + [0] * (L - len(s)) for s in seqs])
    labels = torch.full_like(ids, -100)
    i = 0
    for p, rs in zip(prompts, groups):
        for r in rs:
            labels[i, len(p):len(p) + len(r)] = torch.tensor(r)
            i += 1
    lp = torch.log_softmax(oracle(ids)[:, :-1].float(), -1).gather(-1, labels[:, 1:].clamp(min=0)[..., None]).squeeze(-1)
    mask = (labels[:, 1:] != -100).float()
    lp = lp * mask
    ratio = torch.exp(lp - lp.detach())
    a = torch.tensor(adv)[:, None]
    pol = (-torch.min(ratio * a, ratio.clamp(0.8, 1.2) * a) * mask).sum() / (mask.sum() + 1e-8)
    assert abs(m.policy_loss - pol.item()) < 1e-5 and m.kl_divergence == 0.0     # ref == policy at step 0
    assert abs(m.extras["ratio_mean"] - 1.0) < 1e-6 and m.grad_norm > 0
    assert m.extras["icepop_num_masked"] == 0
    # second step: behaviour baseline kept -> ratio != 1, KL >= 0
    m2 = eng.grpo_step(prompts, groups, rewards, reset_behavior_baseline=False)
    assert m2.extras["ratio_max"] != 1.0 and m2.kl_divergence >= 0.0
    # IcePop: rollout log-probs far from the trainer's mask at most max_mask_ratio of the responses
    eng.icepop.config.divergence_threshold = 0.1
    fake = torch.full((6,), -100.0)
    m3 = eng.grpo_step(prompts, groups, rewards, infer_log_probs=fake)
    assert m3.extras["icepop_num_masked"] == 3 and m3.extras["icepop_masked_ratio"] == 0.5
    # skip_optimizer_step leaves the weights alone and keeps accumulating
    before = [p.detach().clone() for p in eng.model.parameters()]
    step_before = eng.step_count
    eng.grpo_step(prompts, groups, rewards, skip_optimizer_step=True)
    assert all(torch.equal(a, b) for a, b in zip(before, eng.model.parameters())) and eng.step_count == step_before


def test_checkpoint_roundtrip_full_and_lora():
    for rank_ in (0, 4):
        cfg = TrainConfig(model_config=SMALL, lora_rank=rank_, grpo_beta=0.0, learning_rate=1e-2,
                          gradient_accumulation_steps=1, use_amp=False, amp_dtype="fp32", warmup_steps=0, max_seq_len=32)
        eng = TrainEngine(cfg).initialize()
        ids, labels = _tiny_batch(0, 0, 2, 16, 256)
        for _ in range(2):
            eng.sft_step_tensors(ids, labels)
        with tempfile.TemporaryDirectory() as d:
            eng.save_checkpoint(d)
            import os
            files = set(os.listdir(d))
            assert {"optimizer_state.pt", "trainer_state.json"} <= files
            assert ("lora_weights.pt" in files) == (rank_ > 0) and ("model.safetensors" in files) == (rank_ == 0)
            eng2 = TrainEngine(cfg).initialize()
            if rank_ > 0:
                # base weights are not part of a LoRA checkpoint: start both from the same base
                for a, b in zip(eng2.model.parameters(), eng.model.parameters()):
                    if not a.requires_grad:
                        a.data.copy_(b.data)
            assert eng2.load_checkpoint(d)
            assert eng2.step_count == 2 and eng2.optimizer.step_count == 2
            a = eng.sft_step_tensors(ids, labels)
            b = eng2.sft_step_tensors(ids, labels)
            assert abs(a.loss - b.loss) < 1e-6 and abs(a.grad_norm - b.grad_norm) < 1e-5
        assert not eng.load_checkpoint("/nonexistent/dir")


def test_truncation_and_sampling_helpers():
    eng = TrainEngine(TrainConfig(model_config=SMALL, max_seq_len=32, min_prompt_len=4))
    p, r = eng._truncate_prompt_response(list(range(10)), list(range(10)))
    assert (len(p), len(r)) == (10, 10)
    p, r = eng._truncate_prompt_response(list(range(30)), list(range(10)))
    assert (len(p), len(r)) == (22, 10)                         # prompt tail trimmed, response kept
    p, r = eng._truncate_prompt_response(list(range(30)), list(range(40)))
    assert (len(p), len(r)) == (4, 28)                          # response cut, min prompt kept
    logits = torch.tensor([[0.0, 5.0, 1.0, -2.0]])
    assert int(TrainEngine.sample_next_token(logits, 0.0, 1.0)) == 1
    g = torch.Generator().manual_seed(0)
    picks = {int(TrainEngine.sample_next_token(logits, 1.0, 0.5, g)) for _ in range(50)}
    assert picks == {1}                                        # nucleus 0.5 keeps only the top token
    assert int(TrainEngine.sample_next_token(logits, 1.0, 0.0, g)) == 1      # top_p 0: the top token, not a NaN draw
    assert math.isclose(sum(TrainEngine.group_advantages([1.0, 2.0, 3.0])), 0.0, abs_tol=1e-6)
    full = TrainEngine(TrainConfig(model_config=SMALL, max_seq_len=32, lora_rank=0, grpo_beta=0.0, amp_dtype="fp32")).initialize()
    import pytest as _pytest
    with _pytest.raises(ValueError, match="empty prompt"):
        full.generate([], 2)
    with _pytest.raises(ValueError, match="outside the vocabulary"):
        full.generate([3, SMALL.vocab_size], 2)
    assert full.generate([3, 4], 0) == [] and len(full.generate([3, 4], 3, temperature=0.0)) == 3


def test_export_weights_leaves_the_lora_base_bit_identical():
    """The merged export is built out of place: N exports (one per RL weight sync) must not move the frozen
    base, which under LoRA is also the KL reference.  bf16 makes an in-place merge + unmerge lossy."""
    cfg = TrainConfig(model_config=SMALL, lora_rank=4, grpo_beta=0.0, learning_rate=1e-2,
                      gradient_accumulation_steps=1, use_amp=False, amp_dtype="fp32", warmup_steps=0, max_seq_len=32)
    eng = TrainEngine(cfg).initialize()
    eng.model.to(torch.bfloat16)
    from b200fw.model.lora import LinearWithLoRA
    mods = [m for m in eng.model.modules() if isinstance(m, LinearWithLoRA)]
    assert mods
    with torch.no_grad():
        for m in mods:
            for ad in m.adapters.values():
                ad.lora_B.normal_(0, 0.3)                      # a delta large enough to round in bf16
    before = [m.base.weight.detach().clone() for m in mods]
    first = eng.export_weights()
    for _ in range(4):
        again = eng.export_weights()
    for m, w0 in zip(mods, before):
        assert torch.equal(m.base.weight, w0)
        assert not m.merged
    k = "model.layers.0.self_attn.q_proj.weight"
    assert torch.equal(first[k], again[k])
    hq = mods[0].ranges["q_proj"]
    assert not torch.equal(first[k], before[0][hq[0]:hq[1]])   # the export does carry the adapters


def test_resolve_step_takes_back_the_bookkeeping_of_a_skipped_step():
    cfg = TrainConfig(model_config=SMALL, lora_rank=0, grpo_beta=0.0, learning_rate=1e-2, warmup_steps=0,
                      gradient_accumulation_steps=1, use_amp=False, amp_dtype="fp32", max_seq_len=32)
    eng = TrainEngine(cfg).initialize()
    ids, labels = _tiny_batch(0, 0, 2, 16, 256)
    loss, gn = eng.sft_step_tensors(ids, labels, sync=False)
    assert eng.step_count == 1 and eng.resolve_step(gn) > 0 and eng.step_count == 1
    assert eng.optimizer.step_count == 1 and eng.lr_scheduler.step_count == 1
    # a non-finite norm arrives as -1: counters, schedule and the optimizer's bias-correction step go back
    eng.step_count, eng.optimizer.step_count, eng.lr_scheduler.step_count = 2, 2, 2
    assert eng.resolve_step(torch.tensor(-1.0)) < 0
    assert (eng.step_count, eng.optimizer.step_count, eng.lr_scheduler.step_count) == (1, 1, 1)
    assert eng.resolve_step(None) == 0.0


def test_close_window_steps_after_any_number_of_chunks():
    cfg = TrainConfig(model_config=SMALL, lora_rank=0, grpo_beta=0.0, learning_rate=1e-2, warmup_steps=0,
                      gradient_accumulation_steps=4, use_amp=False, amp_dtype="fp32", max_seq_len=32)
    eng = TrainEngine(cfg).initialize()
    P, R, W = [[1, 2, 3]], [[[4, 5], [6, 7]]], [[1.0, 0.0]]
    eng.grpo_step(P, R, W, skip_optimizer_step=True)
    assert eng.step_count == 0
    m = eng.grpo_step(P, R, W, close_window=True)
    assert eng.step_count == 1 and m.grad_norm > 0 and eng._accumulation_count == 0


def _empty_rank_worker(rank, world):
    """Rank 1's responses are all empty (nothing to score); rank 0 has a normal batch."""
    import hashlib
    cfg = TrainConfig(model_preset="tiny", dp_size=world, lora_rank=0, grpo_beta=0.01, learning_rate=1e-3,
                      gradient_accumulation_steps=1, zero_stage=1, use_amp=False, amp_dtype="fp32", warmup_steps=0,
                      max_seq_len=32, backend="gloo", bucket_mb=4.0)
    eng = TrainEngine(cfg).initialize()
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(3, 8192, (6,), generator=g).tolist()
    resp = [torch.randint(3, 8192, (n,), generator=g).tolist() for n in (5, 7)]
    mine = resp if rank == 0 else [[], []]
    out = []
    m = eng.grpo_step([prompt], [mine], [[0.0, 1.0]])
    out.append((m.loss, m.grad_norm))
    m = eng.sft_step([prompt, prompt], mine)
    out.append((m.loss, m.grad_norm))
    with eng.optimizer.eval_mode():
        flat = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
    return out, hashlib.sha256(flat.numpy().tobytes()).hexdigest()


def test_a_rank_with_nothing_to_score_still_takes_part_in_the_step():
    """A data-parallel rank whose responses are all empty contributes zero gradients instead of failing in backward
    (which would leave its peers waiting in the gradient reduction); the ranks stay bit-identical."""
    res = run_ranks(_empty_rank_worker, 2, timeout=600)
    (out0, h0), (out1, h1) = res
    assert h0 == h1
    for (l0, g0), (l1, g1) in zip(out0, out1):
        assert l1 == 0.0 and math.isfinite(l0) and l0 != 0.0
        assert g0 > 0 and abs(g0 - g1) < 1e-6 * max(1.0, g0)      # one global norm, seen by both


def test_token_ids_and_lengths_are_checked_while_the_batch_is_on_the_host():
    """The embedding, rotary and loss kernels index their tables with ids / positions / labels unchecked: a bad value
    is refused before the batch leaves host memory, and the step that follows a refusal runs normally."""
    import pytest
    cfg = TrainConfig(model_config=SMALL, lora_rank=0, grpo_beta=0.0, gradient_accumulation_steps=1, zero_stage=1,
                      use_amp=False, amp_dtype="fp32", warmup_steps=0, max_seq_len=32)
    eng = TrainEngine(cfg).initialize()
    V = SMALL.vocab_size
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.sft_step([[3, 4, V]], [[5, 6]])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.sft_step([[3, 4]], [[5, -2]])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.grpo_step([[3, 4]], [[[5, V + 7], [6]]], [[0.0, 1.0]])
    ids = torch.randint(0, V, (2, 16))
    bad_labels = ids.clone()
    bad_labels[0, 3] = V
    with pytest.raises(ValueError, match="labels must be"):
        eng.sft_step_tensors(ids, bad_labels)
    bad_labels[0, 3] = -1
    with pytest.raises(ValueError, match="labels must be"):
        eng.sft_step_tensors(ids, bad_labels)
    long = torch.randint(0, V, (1, SMALL.max_position_embeddings + 1))
    with pytest.raises(ValueError, match="max_position_embeddings"):
        eng.sft_step_tensors(long, long.clone())
    with pytest.raises(ValueError, match="max_position_embeddings"):
        eng.model(long)
    assert eng.step_count == 0
    m = eng.sft_step([[3, 4, 5]], [[5, 6]])
    assert math.isfinite(m.loss) and eng.step_count == 1
    # a max_seq_len beyond the position table is brought down to it: batches are truncated to what the model addresses
    wide = TrainEngine(TrainConfig(model_config=SMALL, max_seq_len=SMALL.max_position_embeddings + 50, lora_rank=0,
                                   grpo_beta=0.0, amp_dtype="fp32")).initialize()
    assert wide.config.max_seq_len == SMALL.max_position_embeddings
    m = wide.sft_step([[3] * 100], [[4] * 100])
    assert math.isfinite(m.loss)


def _ckpt_agreement_worker(rank, world, path):
    import os
    import shutil
    cfg = TrainConfig(model_config=SMALL, dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=1, zero_stage=1, use_amp=False, amp_dtype="fp32", warmup_steps=0,
                      max_seq_len=32, backend="gloo", bucket_mb=0.02)
    eng = TrainEngine(cfg).initialize()
    ids, labels = _tiny_batch(0, rank, 2, 16, SMALL.vocab_size)
    eng.sft_step_tensors(ids, labels)
    good = os.path.join(path, "good")
    eng.save_checkpoint(good)
    assert not [f for f in os.listdir(good) if ".tmp" in f]            # the temporaries were renamed away
    with eng.optimizer.eval_mode():
        saved = torch.cat([p.detach().reshape(-1).clone() for p in eng.model.parameters()])
    saved_m = eng.optimizer.exp_avg.clone()
    eng.sft_step_tensors(ids, labels)                                   # move on: step 2
    out = {}
    # (1) the complete checkpoint restores everything
    out["good"] = eng.load_checkpoint(good)
    with eng.optimizer.eval_mode():
        now = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
    out["good_exact"] = bool(torch.equal(now, saved) and torch.equal(eng.optimizer.exp_avg, saved_m)) and eng.step_count == 1
    # (2) rank 1's shard is gone (only rank 0's file and its copy remain): rank 1 must not take rank 0's shard, and
    #     rank 0 must not walk alone into the parameter re-publication
    eng.parallel_ctx.barrier()
    if rank == 0:
        shutil.copytree(good, os.path.join(path, "lost"))
        os.remove(os.path.join(path, "lost", "optimizer_state_rank1.pt"))
    eng.parallel_ctx.barrier()
    eng.sft_step_tensors(ids, labels)
    before = eng.optimizer.exp_avg.clone()
    out["lost"] = eng.load_checkpoint(os.path.join(path, "lost"))
    out["lost_moments_kept"] = bool(torch.equal(eng.optimizer.exp_avg, before))
    with eng.optimizer.eval_mode():
        now = torch.cat([p.detach().reshape(-1) for p in eng.model.parameters()])
    out["lost_weights_restored"] = bool(torch.equal(now, saved))      # the weights came back, the optimizer did not
    # (3) a save that was interrupted between the shards and the state file: shards of step 4, state file of step 1
    eng.sft_step_tensors(ids, labels)
    torn = os.path.join(path, "torn")
    eng.save_checkpoint(torn)
    eng.parallel_ctx.barrier()
    if rank == 0:
        shutil.copy(os.path.join(good, "trainer_state.json"), os.path.join(torn, "trainer_state.json"))
    eng.parallel_ctx.barrier()
    out["torn"] = eng.load_checkpoint(torn)
    # (4) a directory that does not exist
    out["missing"] = eng.load_checkpoint(os.path.join(path, "nothing-here"))
    # the ranks are still in step with each other
    m = eng.sft_step_tensors(ids, labels)
    out["alive"] = math.isfinite(m.loss)
    return out


def test_checkpoint_restore_is_agreed_between_ranks():
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks(_ckpt_agreement_worker, 2, d, timeout=600)
    for out in res:
        assert out == {"good": True, "good_exact": True, "lost": False, "lost_moments_kept": True,
                       "lost_weights_restored": True, "torn": False, "missing": False, "alive": True}, out


def test_lora_delta_export_sequence_logprobs_and_closing_a_window_early():
    """Three entry points the orchestration layer relies on: ``export_lora_delta`` (full state first, then exactly the
    change since the previous export), ``compute_sequence_log_probs`` (mean response log-prob, equal to a plain
    log-softmax evaluation) and ``close_accumulation_window`` (the optimizer step over however many micro-batches have
    accumulated; nothing when none has)."""
    from b200fw.model import get_lora_state_dict
    cfg = TrainConfig(model_config=SMALL, lora_rank=4, lora_alpha=8.0, grpo_beta=0.0, gradient_accumulation_steps=4,
                      zero_stage=1, use_amp=False, amp_dtype="fp32", warmup_steps=0, max_seq_len=32, learning_rate=1e-2)
    eng = TrainEngine(cfg).initialize()
    assert 0 < eng.trainable_params_count < eng.total_params_count
    first = eng.export_lora_delta()
    state0 = {k: v.clone() for k, v in get_lora_state_dict(eng.model).items()}
    assert first.keys() == state0.keys() and all(torch.equal(first[k], state0[k]) for k in first)
    assert all(float(v.abs().max()) == 0.0 for v in eng.export_lora_delta().values())      # nothing changed since
    # nothing pending: closing the window is a no-op
    m0 = eng.close_accumulation_window()
    assert m0.grad_norm == 0.0 and eng.step_count == 0
    # two of four micro-batches, then close: one optimizer step over the two
    P, R = [[3, 4, 5], [6, 7]], [[8, 9, 10], [11, 12]]
    eng.sft_step(P, R)
    eng.sft_step(P, R)
    assert eng.step_count == 0 and eng._accumulation_count == 2
    m = eng.close_accumulation_window()
    assert eng.step_count == 1 and eng._accumulation_count == 0 and m.grad_norm > 0
    delta = eng.export_lora_delta()
    state1 = get_lora_state_dict(eng.model)
    assert any(float(v.abs().max()) > 0 for v in delta.values())
    for k in delta:
        assert torch.allclose(state0[k] + delta[k], state1[k], atol=1e-7)
    # sequence log-probs against a plain evaluation
    got = eng.compute_sequence_log_probs(P, R)
    for i, (p, r) in enumerate(zip(P, R)):
        ids = torch.tensor([p + r])
        with eng.optimizer.eval_mode():
            lp = torch.log_softmax(eng.model(ids).float(), -1)[0].detach()
        want = sum(float(lp[len(p) - 1 + j, t]) for j, t in enumerate(r)) / len(r)
        assert abs(float(got[i]) - want) < 1e-4, (i, float(got[i]), want)


DEEP = ModelConfig(vocab_size=128, hidden_size=32, num_layers=5, num_heads=2, num_kv_heads=2, head_dim=16,
                   intermediate_size=48, max_position_embeddings=64, tie_word_embeddings=False)


def _pp_shape_worker(rank, world, path, num_micro, batch):
    from b200fw.model import load_from_hf_checkpoint
    cfg = TrainConfig(model_config=DEEP, pp_size=world, num_micro_batches=num_micro, lora_rank=0, grpo_beta=0.0,
                      learning_rate=1e-3, gradient_accumulation_steps=1, zero_stage=1, use_amp=False,
                      amp_dtype="fp32", warmup_steps=0, max_seq_len=32, backend="gloo", max_grad_norm=0.0)
    eng = TrainEngine(cfg).initialize()
    load_from_hf_checkpoint(eng.model, path, strict=False)
    eng.optimizer.refresh_masters_from_params()
    m = eng.model
    ids, labels = _tiny_batch(3, 0, batch, 12, DEEP.vocab_size)
    eng.optimizer.begin_backward(True)
    loss = eng.pipeline_scheduler.broadcast_loss(eng.pipeline_scheduler.run_1f1b_schedule(ids, labels))
    grads = {m.layer_start + i: l.mlp.down_proj.weight.grad.clone().tolist() for i, l in enumerate(m.layers)}
    return float(loss), grads, (m.layer_start, len(m.layers))


@pytest.mark.parametrize("world,num_micro", [(3, 3), (3, 5), (4, 4), (4, 6)])
def test_pipeline_1f1b_other_stage_and_micro_batch_counts(world, num_micro):
    """Five layers over 3 or 4 stages (uneven split), as many micro-batches as stages or more: the schedule's
    warm-up / steady / cool-down phases line up (no rank waits for a message nobody sends), every layer is owned by
    exactly one stage, and loss and gradients equal the single-process accumulation."""
    from b200fw.model import save_hf_checkpoint
    with tempfile.TemporaryDirectory() as d:
        ref = ParallelTransformerModel(DEEP)
        ref.init_weights(5)
        save_hf_checkpoint(ref, d)
        batch = 2 * num_micro
        res = run_ranks(_pp_shape_worker, world, d, num_micro, batch, timeout=300)
        ids, labels = _tiny_batch(3, 0, batch, 12, DEEP.vocab_size)
        total = 0.0
        for mb_ids, mb_labels in zip(ids.chunk(num_micro), labels.chunk(num_micro)):
            l = ref.loss(mb_ids, mb_labels)
            (l / num_micro).backward()
            total += l.item() / num_micro
        owned = sorted(k for r in res for k in r[1])
        assert owned == list(range(DEEP.num_layers)), [r[2] for r in res]
        for r in res:
            assert abs(r[0] - total) < 1e-5
            for k, g in r[1].items():
                assert (torch.tensor(g) - ref.layers[k].mlp.down_proj.weight.grad).abs().max() < 1e-6


def _heartbeat_worker(rank, world, silent):
    """Two data-parallel ranks train two steps; then rank 1 leaves between steps (with a word, or silently: its
    heartbeat just stops).  Rank 0's next step must raise before it launches anything."""
    import time
    from b200fw.dist import PeerLostError
    cfg = TrainConfig(model_config=SMALL, dp_size=world, lora_rank=0, grpo_beta=0.0, learning_rate=1e-3,
                      gradient_accumulation_steps=1, zero_stage=1, use_amp=False, amp_dtype="fp32", warmup_steps=0,
                      max_seq_len=32, backend="gloo", bucket_mb=0.02, heartbeat_interval_s=0.05, heartbeat_timeout_s=2.0)
    eng = TrainEngine(cfg).initialize()
    assert eng.heartbeat is not None
    ids, labels = _tiny_batch(0, rank, 2, 16, SMALL.vocab_size)
    for _ in range(2):
        eng.sft_step_tensors(ids, labels)
    if rank == 1:
        if silent:
            eng.heartbeat.stop()
        else:
            eng.heartbeat.announce_leave("made up by the test")
        time.sleep(6.0)                  # stays around (its process group alive) while rank 0 notices
        return "left"
    deadline = time.time() + 20
    while eng.heartbeat.lost is None and time.time() < deadline:
        time.sleep(0.02)
    t0 = time.time()
    try:
        eng.sft_step_tensors(ids, labels)
    except PeerLostError as e:
        return ("raised", e.rank, e.reason, time.time() - t0, eng.step_count)
    return ("trained", None, None, time.time() - t0, eng.step_count)


@pytest.mark.parametrize("silent", [False, True])
def test_a_step_is_refused_once_the_heartbeat_has_lost_a_peer(silent):
    res = run_ranks(_heartbeat_worker, 2, silent, timeout=120)
    kind, who, reason, took, steps = res[0]
    assert kind == "raised" and who == 1 and steps == 2
    assert ("no heartbeat" in reason) if silent else ("made up by the test" in reason)
    assert took < 0.5                    # refused on the host at once: nothing was launched, nothing timed out
    assert res[1] == "left"
