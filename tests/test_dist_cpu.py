"""Host-side logic of the multi-GPU path on CPU: frame sharding and the uneven row all-gather over a 2-rank gloo
group (the attention itself needs a GPU and is covered by the row-range test there)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_shard_range_is_contiguous_and_balanced():
    from come_b200.dist import rows_per_rank, shard_range
    for n, world in ((100, 8), (8, 8), (5, 8), (256, 3), (1, 1)):
        ranges = [shard_range(n, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
        sizes = [hi - lo for lo, hi in ranges]
        assert max(sizes) - min(sizes) <= 1
    offsets = [0, 10, 25, 31, 40, 58]  # 5 frames
    assert rows_per_rank(offsets, 2) == [31, 27]
    assert rows_per_rank(offsets, 5) == [10, 15, 6, 9, 18]
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from come_b200.dist import gather_rows
        local = torch.arange(rows[rank] * 6, dtype=torch.float32).reshape(rows[rank], 2, 3) + 1000 * rank
        got = gather_rows(local, rows)
        want = torch.cat([torch.arange(rows[r] * 6, dtype=torch.float32).reshape(rows[r], 2, 3) + 1000 * r for r in range(world)])
        ok = torch.equal(got, want)
        # remote-first order: the other ranks' blocks (rank + 1, ..., rank - 1) in front, the local block last
        from come_b200.dist import block_order
        order = block_order(world, rank, True)
        got_rf = gather_rows(local, rows, remote_first=True)
        want_rf = torch.cat([torch.arange(rows[r] * 6, dtype=torch.float32).reshape(rows[r], 2, 3) + 1000 * r for r in order])
        ok = ok and order[-1] == rank and sorted(order) == list(range(world)) and torch.equal(got_rf, want_rf)
        ok = ok and torch.equal(got_rf[sum(rows) - rows[rank]:], local)
        # an inconsistent row table is reported on the host before any collective is started
        try:
            gather_rows(local, list(rows) + [1])
            ok = False
        except ValueError:
            pass
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows", [[5, 3], [4, 4], [0, 7]])
def test_gather_rows_uneven_gloo(rows):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, rows, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(2))
    assert results == {0: True, 1: True}


def _exchange_worker(rank, world, port, rows, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from come_b200.dist import GlobalExchange
        total = sum(rows)
        weight_all = torch.where(torch.arange(total) % 3 == 0, 9.0, 1.0)
        ex = GlobalExchange(rows, rank, weight_all)
        local = torch.arange(rows[rank] * 4, dtype=torch.float32).reshape(rows[rank], 2, 2) + 100 * rank
        got = ex.gather(local)
        want = torch.cat([torch.arange(rows[r] * 4, dtype=torch.float32).reshape(rows[r], 2, 2) + 100 * r for r in range(world)])
        ok = torch.equal(got, want) and ex.row_begin == sum(rows[:rank]) and ex.total == total
        ok = ok and ex.cu_seqlens.tolist() == [0, total] and torch.equal(ex.bias(torch.float32), weight_all.log())
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_global_exchange_gloo():
    """The exchange object of a frame-sharded global block over two gloo ranks: row bookkeeping, replicated bias, gather."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_exchange_worker, args=(r, 2, port, [5, 3], q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(q.get(timeout=10) for _ in range(2)) == {0: True, 1: True}


def test_global_exchange_checks_and_custom_gather():
    from come_b200.dist import GlobalExchange
    w = torch.ones(7)
    calls = []
    ex = GlobalExchange([3, 4], 1, w, gather=lambda local, rows, rank: calls.append((tuple(local.shape), rows, rank)) or torch.zeros(7, 2))
    assert ex.row_begin == 3 and ex.gather(torch.zeros(4, 2)).shape == (7, 2) and calls == [((4, 2), [3, 4], 1)]
    with pytest.raises(ValueError):
        ex.gather(torch.zeros(3, 2))       # not this rank's row count
    with pytest.raises(ValueError):
        GlobalExchange([3, 4], 0, torch.ones(6))
    single = GlobalExchange([7], 0, w)
    t = torch.zeros(7, 2)
    assert single.gather(t) is t           # one rank: nothing to exchange


def test_block_order():
    from come_b200.dist import block_order
    assert block_order(4, 1, False) == [0, 1, 2, 3]
    assert block_order(4, 1, True) == [2, 3, 0, 1]
    assert block_order(1, 0, True) == [0]


def test_exchange_bias_split_follows_the_remote_first_order():
    """The per-key bias handed to the attention over the gathered remote rows is laid out like those rows."""
    from come_b200.dist import GlobalExchange
    rows = [3, 2, 4]
    weight = torch.tensor([1., 9, 1, 9, 9, 1, 1, 9, 1])
    ex = GlobalExchange(rows, 1, weight, overlap=True)
    local, remote = ex.bias_local_remote(torch.float32)
    assert torch.equal(local, weight[3:5].log())
    assert torch.equal(remote, torch.cat([weight[5:9], weight[0:3]]).log())  # rank 2's rows, then rank 0's
    assert ex.overlap and not GlobalExchange([9], 0, weight, overlap=True).overlap


def test_hiding_the_exchange_pays_only_while_local_attention_is_long():
    """The two-line model of a global layer: for the 100-frame scene (80,672 rows of 4 KB, 16 heads x 64) hiding the
    exchange pays on 2 to 4 ranks and not on 8; never on one rank; never for a small scene, where no attention launch is
    long enough to cover a slowed exchange; and a faster hidden exchange moves the boundary."""
    from come_b200.dist import hiding_exchange_pays
    big = dict(total_rows=80672, row_bytes=4096, num_heads=16, head_dim=64)
    assert [hiding_exchange_pays(world=w, **big) for w in (1, 2, 4, 8)] == [False, True, True, False]
    assert not hiding_exchange_pays(total_rows=6448, world=2, row_bytes=1024, num_heads=4, head_dim=64)
    assert hiding_exchange_pays(world=8, exchange_hidden_gbs=380.0, **big)
    from come_b200.dist import pulls_first_pays
    assert pulls_first_pays(world=8, **big) and not pulls_first_pays(world=1, **big)
    assert not pulls_first_pays(total_rows=6448, world=8, row_bytes=1024, num_heads=4, head_dim=64)  # nothing to hide behind


def test_global_exchange_rejects_unknown_transport():
    import torch
    from come_b200.dist import GlobalExchange
    with pytest.raises(ValueError, match="transport"):
        GlobalExchange([2, 2], 0, torch.ones(4), transport="carrier-pigeon")
