"""Round-robin page dealing of context-parallel decode: every token lands on exactly one rank, in order."""
import pytest

from nanoengine_b200.parallel.decode_cp import shard_pages


@pytest.mark.parametrize("ctx", [1, 63, 64, 65, 129, 1000, 4096])
@pytest.mark.parametrize("cp", [1, 2, 4, 8])
def test_shard_pages_partitions_the_context(ctx, cp):
    bs = 64
    n_pages = -(-ctx // bs)
    table = list(range(100, 100 + n_pages))
    seen, total = [], 0
    for r in range(cp):
        pages, tokens = shard_pages(table, ctx, bs, cp, r)
        assert pages == table[r::cp]
        # all of a rank's pages are full except, on one rank, the last page of the sequence
        full = sum(bs for p in pages if p != table[-1])
        last = (ctx - (n_pages - 1) * bs) if table[-1] in pages else 0
        assert tokens == full + last
        seen += pages
        total += tokens
    assert sorted(seen) == table and total == ctx
