"""EPLB planner: replicas go to the hottest experts, physical slots pack evenly, the logical->physical map is consistent."""
import torch

from nanoengine_b200.parallel.eplb import dummy_balanced_topk, map_logical_to_physical, rebalance_experts


def _check(load, P, G, groups=1, nodes=1):
    phy2log, log2phy, logcnt = rebalance_experts(load, P, G, groups, nodes)
    L, E = load.shape
    assert phy2log.shape == (L, P) and logcnt.sum(-1).eq(P).all()
    for l in range(L):
        assert set(phy2log[l].tolist()) == set(range(E))                 # every logical expert is placed
        for e in range(E):
            reps = log2phy[l, e][log2phy[l, e] >= 0]
            assert reps.numel() == logcnt[l, e] and (phy2log[l][reps] == e).all()
    per_gpu = (load / logcnt).gather(1, phy2log).view(L, G, -1).sum(-1)
    return per_gpu, logcnt


def test_flat_rebalance_evens_out_a_skewed_load():
    torch.manual_seed(0)
    load = torch.rand(2, 16) + torch.tensor([10.0] + [0.0] * 15)          # expert 0 is 10x hotter
    per_gpu, logcnt = _check(load, 20, 4)
    assert (logcnt[:, 0] >= 3).all()                                      # the hot expert got most of the spare slots
    naive = load.view(2, 4, 4).sum(-1)
    assert (per_gpu.max(-1).values < naive.max(-1).values).all()
    assert (per_gpu.max(-1).values / per_gpu.mean(-1) < 1.6).all()


def test_hierarchical_rebalance_keeps_groups_on_a_node():
    torch.manual_seed(1)
    load = torch.rand(1, 32) + 0.1
    phy2log, log2phy, logcnt = rebalance_experts(load, 40, 8, num_groups=4, num_nodes=2)
    _check(load, 40, 8, 4, 2)
    node_of_slot = torch.arange(40) // 20
    group_of = phy2log[0] // 8
    for g in range(4):
        assert node_of_slot[group_of == g].unique().numel() == 1          # all replicas of a group's experts share a node


def test_replica_choice_is_deterministic_and_spreads():
    load = torch.tensor([[8.0, 1.0, 1.0, 1.0]])
    phy2log, log2phy, logcnt = rebalance_experts(load, 8, 2)
    idx = torch.zeros(1000, 1, dtype=torch.int32)
    tok = torch.arange(1000)
    a = map_logical_to_physical(idx, log2phy[0], logcnt[0], tok)
    assert torch.equal(a, map_logical_to_physical(idx, log2phy[0], logcnt[0], tok))
    used = a.unique()
    assert used.numel() == logcnt[0, 0] and (phy2log[0][used.long()] == 0).all()
    assert torch.bincount(dummy_balanced_topk(64, 8, 32).flatten().long(), minlength=32).eq(16).all()


def test_router_remap_picks_a_replica_of_the_chosen_expert():
    import torch
    from nanoengine_b200.ops import reference as ref
    from nanoengine_b200.parallel.eplb import EplbPlan
    torch.manual_seed(0)
    E, K, T = 8, 2, 64
    load = torch.tensor([[10.0, 1, 1, 1, 8, 1, 1, 1]])
    plan = EplbPlan.from_load(load, 4, 2)
    assert plan.num_physical == 12 and int(plan.logcnt[0, 0]) >= 2
    logits = torch.randn(T, E)
    idx_l, w_l = ref.moe_route(logits, None, K, scoring="softmax")
    l2p, cnt = plan.router_tables(0, "cpu")
    idx_p, w_p = ref.moe_route(logits, None, K, scoring="softmax", log2phy=l2p, logcnt=cnt)
    assert torch.equal(w_l, w_p)
    assert torch.equal(plan.phy2log[0][idx_p.long()], idx_l.long())          # every physical id holds the logical expert chosen
    hot = idx_p[idx_l == 0]
    assert len(set(hot.tolist())) >= 2                                       # the hot expert's replicas share its tokens
    # the dummy balance deals ids evenly over the ranks and keeps the weights
    idx_b, w_b = ref.moe_route(logits, None, K, scoring="softmax", balance_ranks=2)
    assert torch.equal(w_b, w_l)
    per_rank = torch.bincount(idx_b.flatten().long() // (E // 2), minlength=2)
    assert per_rank[0] == per_rank[1]


def test_engine_with_redundant_experts_equals_the_plain_engine(tmp_path):
    """Replicas hold the same weights, so an engine serving under a load-balancing plan (10 physical slots for 8 experts,
    a skewed measured load) generates exactly what the plain engine generates."""
    import torch
    from nanoengine_b200 import Config, LLM, SamplingParams
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=4, num_kvcache_blocks=32)
    want = [o["token_ids"] for o in LLM(Config(**base)).generate(prompts, sp)]
    load = torch.ones(2, 8)
    load[1, 3] = 20.0
    torch.save(load, tmp_path / "load.pt")
    llm = LLM(Config(**base, eplb_redundant_experts=2, eplb_load_path=str(tmp_path / "load.pt")))
    ex = llm.engine.executor.runner.model.model.layers["1"].mlp.experts
    assert ex.num_experts == 10 and ex.phy2log.count(3) >= 2
    assert [o["token_ids"] for o in llm.generate(prompts, sp)] == want
    from nanoengine_b200.parallel import eplb
    eplb.set_active_plan(None)
