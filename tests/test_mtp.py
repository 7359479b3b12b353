"""MTP speculative decoding: verification / rejection-sampling numerics (modelled on the reference's
tests/test_mtp_linear.py:33-391) and end-to-end equivalence with plain greedy decoding on the CPU engine."""
import torch

from nanoengine_b200 import Config, LLM, SamplingParams
from nanoengine_b200.runtime.mtp_runner import linear_greedy_verify, linear_rejection_sample


def _logits_for(targets, V=16):
    """[B, N+1, V] logits whose argmax per row is targets[b][i]."""
    B, N1 = len(targets), len(targets[0])
    lg = torch.zeros(B, N1, V)
    for b in range(B):
        for i in range(N1):
            lg[b, i, targets[b][i]] = 10.0
    return lg


def test_greedy_verify_every_acceptance_length():
    N = 5
    target = [3, 4, 5, 6, 7, 8]
    for a in range(N + 1):
        drafts = target[:a] + [0] * (N - a)          # first `a` drafts match, then a mismatch
        acc, nxt = linear_greedy_verify(_logits_for([target]), torch.tensor([drafts]))
        assert int(acc) == a and int(nxt) == target[a]
    # a later match after a mismatch does not count
    acc, nxt = linear_greedy_verify(_logits_for([target]), torch.tensor([[3, 0, 5, 6, 7]]))
    assert int(acc) == 1 and int(nxt) == 4


def test_rejection_sampling_accepts_by_target_probability_and_masks_the_rejected_draft():
    V, N = 4, 2
    logits = torch.log(torch.tensor([[[0.7, 0.1, 0.1, 0.1], [0.25, 0.25, 0.25, 0.25], [0.1, 0.2, 0.3, 0.4]]]))
    drafts = torch.tensor([[0, 2]])
    temps = torch.ones(1)
    # coins below the draft probabilities -> both accepted, bonus row sampled unmasked
    acc, nxt, lp = linear_rejection_sample(logits, drafts, temps, uniforms=torch.tensor([[0.5, 0.2]]))
    assert int(acc) == 2 and lp.item() <= 0
    # first coin above p(d1)=0.7 -> rejected at once; the recovery token can never be the rejected draft
    g = torch.Generator().manual_seed(0)
    for _ in range(50):
        acc, nxt, _ = linear_rejection_sample(logits, drafts, temps, generator=g, uniforms=torch.tensor([[0.9, 0.0]]))
        assert int(acc) == 0 and int(nxt) != 0
    # temperature 0 falls back to greedy verification
    acc, nxt, _ = linear_rejection_sample(logits, torch.tensor([[0, 1]]), torch.zeros(1), uniforms=torch.tensor([[0.99, 0.99]]))
    assert int(acc) == 1 and int(nxt) in (0, 1, 2, 3)


def test_rejection_sampling_preserves_the_target_distribution():
    torch.manual_seed(0)
    V = 5
    p = torch.tensor([0.5, 0.2, 0.15, 0.1, 0.05])
    logits = torch.log(p).view(1, 1, V).repeat(20000, 2, 1)
    drafts = torch.zeros(20000, 1, dtype=torch.long)            # the draft model always proposes token 0
    g = torch.Generator().manual_seed(1)
    acc, nxt, _ = linear_rejection_sample(logits, drafts, torch.ones(20000), generator=g)
    first = torch.where(acc == 1, torch.zeros_like(nxt), nxt)   # token emitted at position 0
    freq = torch.bincount(first, minlength=V).float() / 20000
    assert torch.allclose(freq, p, atol=0.02)


def _make(n_spec, **kw):
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8,
                num_kvcache_blocks=96, seed=0, hf_overrides={"num_nextn_predict_layers": 1}, num_speculative_tokens=n_spec)
    base.update(kw)
    return LLM(Config(**base))


def test_speculative_decoding_emits_exactly_the_greedy_tokens():
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 33, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True)
    want = {o["seq_id"]: o["token_ids"] for o in _make(0).generate(prompts, sp)}
    for n in (1, 2):
        llm = _make(n)
        got = {o["seq_id"]: o["token_ids"] for o in llm.generate(prompts, sp)}
        assert got == want, n
        mr = llm.engine.executor.runner.mtp_runner
        assert mr.verify_steps > 0


def test_forced_acceptance_shortens_the_run():
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 1024, (16,), generator=g).tolist() for _ in range(2)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    llm = _make(2)
    llm.engine.executor.runner.mtp_runner.force_accept = 2
    steps = 0
    for p in prompts:
        llm.add_request(p, sp)
    while not llm.is_finished():
        llm.step(); steps += 1
    assert steps <= 1 + 4 + 1      # prefill + ceil(11 / 3) verify steps (+ slack), instead of 12 plain decode steps
