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
