"""Randomised model check of the C++ block pool and table: after any sequence of grow / share / adopt / free / cache
operations every block's reference count equals the number of holders the test knows about, rows never hold a free
block, and releasing everything returns the pool to full."""
import random

import pytest

cpp = pytest.importorskip("deepseek_v4_2080ti_b200.pocketllm_cpp")


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_reference_counts_follow_a_python_model(seed):
    rng = random.Random(seed)
    n_blocks, block_tokens, slots, max_blocks = 24, 4, 5, 8
    pool = cpp.BlockPool(n_blocks + 1, block_tokens)
    table = cpp.BlockTable(pool, slots, max_blocks)
    rows: list[list[int]] = [[] for _ in range(slots)]       # the model: blocks per slot, in order
    cache: list[list[int]] = []                              # block lists a prefix cache holds its own reference to

    def check():
        holders: dict[int, int] = {}
        for r in rows:
            for b in r:
                holders[b] = holders.get(b, 0) + 1
        for entry in cache:
            for b in entry:
                holders[b] = holders.get(b, 0) + 1
        for b in range(1, n_blocks + 1):
            assert pool.refcount(b) == holders.get(b, 0), (b, pool.refcount(b), holders.get(b, 0))
        assert pool.free_blocks == n_blocks - len(holders)
        for s in range(slots):
            assert table.blocks_in(s) == len(rows[s]) and [table.block_at(s, i) for i in range(len(rows[s]))] == rows[s]

    for step in range(600):
        op = rng.choice(["grow", "grow", "share", "adopt", "free", "cache", "drop"])
        s = rng.randrange(slots)
        if op == "grow":
            tokens = rng.randrange(1, max_blocks * block_tokens + 6)
            need = (tokens + block_tokens - 1) // block_tokens
            free_before = pool.free_blocks
            ok = table.ensure_capacity(s, tokens)                      # all or nothing
            if ok:
                assert need <= max_blocks
                rows[s] = [table.block_at(s, i) for i in range(table.blocks_in(s))]
                assert len(rows[s]) >= need
            else:
                assert need > max_blocks or need - len(rows[s]) > free_before
        elif op == "share":
            src = rng.randrange(slots)
            n = rng.randrange(0, max_blocks + 2)
            if src != s and table.share_prefix(s, src, n):
                assert not rows[s] and n <= len(rows[src])
                rows[s] = rows[src][:n]
        elif op == "adopt" and cache:
            entry = rng.choice(cache)
            ok = table.adopt(s, entry)
            if ok:
                assert not rows[s]
                rows[s] = list(entry)
            else:
                assert rows[s] or len(entry) > max_blocks
        elif op == "free":
            table.free_slot(s)
            rows[s] = []
        elif op == "cache" and rows[s]:
            entry = rows[s][:rng.randrange(1, len(rows[s]) + 1)]
            for b in entry:
                pool.retain(b)
            cache.append(entry)
        elif op == "drop" and cache:
            entry = cache.pop(rng.randrange(len(cache)))
            for b in entry:
                pool.release(b)
        check()
    for s in range(slots):
        table.free_slot(s)
        rows[s] = []
    for entry in cache:
        for b in entry:
            pool.release(b)
    cache.clear()
    check()
    assert pool.free_blocks == n_blocks
    # a block that went back to the pool cannot be retained, released again or adopted
    with pytest.raises(Exception):
        pool.release(1)
    assert not table.adopt(0, [1])
