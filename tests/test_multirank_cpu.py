"""The N > 1 host logic on CPU: two gloo ranks exchange handles and routes, build their schedules
with the oracle, and the union must place every (rank, token, slot) exactly once; context-parallel
work lists must tile the causal triangle exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import routing
        from pipelink_b200 import ep
        # 1. handle exchange (bootstrap): rank r contributes 64 bytes of value r
        handles = ep.exchange_handles(bytes([rank]) * 64, world)
        assert [h[0] for h in handles] == list(range(world))
        # 2. routes all-gather + per-rank schedule
        tokens, topk, experts = 96, 2, 8
        rng = np.random.default_rng(100 + rank)
        mine = np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)]).astype(np.int32)
        bucket = [torch.zeros(tokens, topk, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(bucket, torch.from_numpy(mine))
        routes = torch.stack(bucket).numpy()
        assert np.array_equal(routes[rank], mine)
        El = experts // world
        sched = routing.build_schedule(routes, rank * El, El, 1024, 256)
        total = int(sched["num_tokens"][0])
        live = sched["peer_rank"][:total] >= 0
        placed = np.stack([sched["peer_rank"][:total][live], sched["dest_row"][:total][live]], axis=1)
        np.save(os.path.join(tmp, f"placed{rank}.npy"), placed)
        np.save(os.path.join(tmp, f"routes{rank}.npy"), routes)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_schedule_every_route_once(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    routes = np.load(tmp_path / "routes0.npy")
    assert np.array_equal(routes, np.load(tmp_path / "routes1.npy"))
    tokens, topk = routes.shape[1:]
    seen = np.zeros((world, tokens * topk), int)
    for r in range(world):
        placed = np.load(tmp_path / f"placed{r}.npy")
        for src, dest in placed:
            seen[src, dest] += 1
            assert routes[src, dest // topk, dest % topk] // 4 == r     # the row went to the owner of its expert
    assert (seen == 1).all()


@pytest.mark.parametrize("world,seq", [(2, 1024), (4, 4096), (8, 131072)])
def test_zigzag_work_tiles_the_causal_triangle(world, seq):
    from oracle import attention as oa
    from pipelink_b200 import attention as att
    covered = np.zeros(seq // 128, int)
    total_blocks = 0
    for r in range(world):
        w = att.zigzag_work(seq, world, r, q_heads=1)
        pos = oa.zigzag_rows(seq, world, r)
        for q_row0, q_pos0, kv_row0, kv_pos0, kv_blocks, head, batch, _ in w:
            assert pos[q_row0] == q_pos0 and kv_blocks == q_pos0 // 128 + 1 and kv_row0 == 0 and kv_pos0 == 0
            covered[q_pos0 // 128] += 1
            total_blocks += kv_blocks
        per_rank = sum(row[4] for row in w)
        # zigzag balances the causal work: every rank visits the same number of KV blocks
        assert per_rank == (seq // 128) * (seq // 128 + 1) // 2 // world
    assert (covered == 1).all() and total_blocks == (seq // 128) * (seq // 128 + 1) // 2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_slab_layout_regions_do_not_overlap(world):
    """Peer-visible regions of one rank's symmetric slab (forward and training) are 256-byte
    aligned, disjoint and inside the allocation."""
    from pipelink_b200 import ep, mok
    shape = mok.Shape("slab", 64, 4096, 2048, 8, 1024)
    for train in (False, True):
        lay = ep.SlabLayout(shape, world, train)
        L, H, k = shape.tokens, shape.hidden, shape.topk
        regions = [("flags", lay.flags, 4 * 32), ("xq", lay.xq, L * H), ("xsc", lay.xsc, L // 128 * (H // 128) * 512),
                   ("routes_all", lay.routes_all, world * L * k * 4), ("combine", lay.combine, L * k * H * 2)]
        if train:
            regions += [("x_bf16", lay.x_bf16, L * H * 2), ("d_out", lay.d_out, L * H * 2),
                        ("router_w", lay.router_w, L * k * 4), ("d_x_rows", lay.d_x_rows, L * k * H * 2)]
        regions.sort(key=lambda r: r[1])
        for (name, off, size), nxt in zip(regions, regions[1:] + [("end", lay.nbytes, 0)]):
            assert off % 256 == 0, name
            assert off + size <= nxt[1], (name, nxt[0])


def test_push_rotation_separates_the_ranks():
    """Rows are ordered by (expert, source rank). With the rotation every rank starts its pushing
    GEMM at a different source-rank block, so at equal progress no two ranks address the same home
    rank (balanced routing: a block is L * k / E rows)."""
    L, k, E, world = 8192, 8, 64, 8
    block_tiles = max(1, (L * k // E) // 256)
    tiles_per_expert = block_tiles * world
    for step in range(0, tiles_per_expert * 2, block_tiles):
        homes = set()
        for rank in range(world):
            rot = rank * block_tiles                     # ep.EpMoKHost.push_rotation
            tile = (step + rot) % tiles_per_expert       # position inside an expert's segment
            homes.add(tile // block_tiles)               # source (= home) rank of that block
        assert len(homes) == world


def _bootstrap_with_a_missing_rank(rank, world, port, tmp):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from pipelink_b200 import ep
    outcome = "left"
    if rank == 0:
        # rank 1 leaves before the handle exchange: the bootstrap must end with an error on the host,
        # well before any kernel could wait on a peer that is not there
        try:
            ep.exchange_handles(bytes([rank]) * 64, world)
            outcome = "completed"
        except Exception as e:   # gloo reports the lost peer or the timeout
            outcome = "error:" + type(e).__name__
    with open(os.path.join(tmp, f"outcome{rank}.txt"), "w") as f:
        f.write(outcome)
    if rank == 0:
        os._exit(0)     # the group is broken; skip the collective teardown


def test_bootstrap_fails_on_the_host_when_a_rank_never_joins(tmp_path):
    """Failure made on the host: one rank exits before contributing its IPC handle."""
    world, port = 2, _free_port()
    ctx = mp.spawn(_bootstrap_with_a_missing_rank, args=(world, port, str(tmp_path)), nprocs=world, join=False)
    ctx.join(timeout=60)
    assert (tmp_path / "outcome1.txt").read_text() == "left"
    assert (tmp_path / "outcome0.txt").read_text().startswith("error:")


def test_exchange_rejects_a_malformed_handle():
    from pipelink_b200 import ep
    with pytest.raises(ValueError):
        ep.exchange_handles(b"short", 2)


def test_tp_layout_regions_are_disjoint_and_aligned():
    """Slab layout of the tensor-parallel compositions: two parities of counters, gathered buffers
    and receive slots, none overlapping; shapes that do not tile are refused."""
    from pipelink_b200.tp import TILE, TpLayout
    lay = TpLayout(2048, 1024, 1024, 4)
    regions = [(lay.flags, 16)]
    for p in range(2):
        regions += [(lay.ready[p], 4 * (2048 // TILE)), (lay.gather[p], 2048 * 1024 * 2), (lay.slots[p], 2048 * 1024 * 2)]
    regions.sort()
    for (a, n), (b, _) in zip(regions, regions[1:]):
        assert a % 1024 == 0 and a + n <= b
    assert regions[-1][0] + regions[-1][1] <= lay.nbytes
    for bad in ((2048 + 256, 1024, 1024, 4), (2048, 1024 + 256, 1024, 4), (2048, 1024, 1024 + 128, 4)):
        with pytest.raises(ValueError):
            TpLayout(*bad)


def test_tp_reduce_scatter_row_maps():
    """Row i of a rank's partial product goes to owner i // (M / W), slot row (i % (M / W)) * W + rank:
    together the W ranks fill every [row, source] slot of every owner exactly once."""
    m, w = 1024, 4
    ms = m // w
    seen = set()
    for rank in range(w):
        for i in range(m):
            owner, dest = i // ms, (i % ms) * w + rank
            assert 0 <= dest < ms * w
            seen.add((owner, dest))
    assert len(seen) == w * ms * w
