"""CPU tests (gloo, world_size 2 and 3) of the expert-parallel dispatch/combine plan: rows
grouped by expert go to the rank that owns the expert and come back in the sender's order."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import trismoe_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, num_experts, top_k, tokens, out):
    import trismoe_b200  # noqa: F401
    from trismoe_b200 import expert_parallel as ep

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(100 + rank)
        T = tokens[rank]
        sel = np.stack([rng.choice(num_experts, size=top_k, replace=False) for _ in range(T)]).astype(np.int64) \
            if T else np.zeros((0, top_k), np.int64)
        route = orc.build_route(sel, num_experts)
        grouped_ids = torch.from_numpy(route["grouped_expert_ids"].astype(np.int32))
        rows = torch.from_numpy(rng.standard_normal((T * top_k, 6)).astype(np.float32))
        lo, hi = ep.expert_range(num_experts, rank, world)
        seen = []

        def compute(recv_rows, recv_local_ids):
            assert recv_rows.shape[0] == recv_local_ids.shape[0]
            if recv_local_ids.numel():
                assert int(recv_local_ids.min()) >= 0 and int(recv_local_ids.max()) < hi - lo
            seen.append(int(recv_rows.shape[0]))
            return recv_rows * (recv_local_ids.to(torch.float32) + lo + 1).unsqueeze(1)

        back = ep.expert_parallel_exchange(rows, grouped_ids, num_experts, compute)
        want = rows * (grouped_ids.to(torch.float32) + 1).unsqueeze(1)
        ok = bool(torch.equal(back, want))
        # every routed row of every rank is processed by exactly one owner
        total = torch.tensor([seen[0], T * top_k], dtype=torch.long)
        dist.all_reduce(total)
        ok = ok and int(total[0]) == int(total[1])
        out[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,num_experts,top_k,tokens", [
    (2, 8, 2, [5, 3]),
    (2, 7, 3, [4, 0]),      # uneven expert split, one rank without tokens
    (3, 64, 8, [6, 1, 9]),
])
def test_dispatch_combine_round_trip(world, num_experts, top_k, tokens):
    port = _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, num_experts, top_k, tokens, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(out.get(r) for r in range(world)), dict(out)


def test_partition_and_payload_sharding(lib):
    from trismoe_b200 import expert_parallel as ep, synth

    for E, world in ((64, 8), (7, 2), (8, 3), (256, 4), (3, 4)):
        covered = []
        for r in range(world):
            lo, hi = ep.expert_range(E, r, world)
            covered += list(range(lo, hi))
            if hi > lo:
                owners = ep.owner_of(torch.arange(lo, hi), E, world)
                assert torch.all(owners == r), (E, world, r)
        assert covered == list(range(E))
    layer = synth.synth_layer(synth.LayerShape(64, 96, 6, 2, rank=32, group_size=32), seed=0)
    full = layer["gate"]
    parts = [ep.shard_payload(full, r, 4) for r in range(4)]
    assert sum(int(p["qweight1"].shape[0]) for p in parts) == 6
    assert torch.equal(torch.cat([p["qweight1"] for p in parts]), full["qweight1"])
    assert torch.equal(torch.cat([p["q_gmap_gr_offsets"] for p in parts]), full["q_gmap_gr_offsets"])
    assert parts[0]["compact3_use_block_gr"] is True


def test_balanced_rows_per_peer_bounds():
    import trismoe_b200  # noqa: F401
    from trismoe_b200 import expert_parallel as ep

    for tokens, k, world in [(128, 8, 2), (128, 8, 8), (1, 8, 4), (9, 2, 2), (4096, 2, 8)]:
        rows = tokens * k
        c = ep.balanced_rows_per_peer(tokens, k, world)
        assert c <= rows and (c % 8 == 0 or c == rows)
        assert c >= min(rows, rows / world)          # never below the mean
    assert ep.balanced_rows_per_peer(128, 8, 2) == 616   # 512 + 6 * 16 = 608 -> next multiple of 8 above it
    assert ep.balanced_rows_per_peer(128, 8, 1) == 1024  # one rank: everything stays


@pytest.mark.parametrize("world,num_experts,top_k,tokens,capacity", [
    (2, 8, 2, [9, 5], 18),
    (3, 7, 3, [4, 0, 6], 18),   # uneven expert split, a rank without tokens
    (4, 64, 8, [16, 16, 16, 16], 56),  # fewer slots than the worst case (128): nothing overflows at this seed
])
def test_fixed_capacity_slot_layout(world, num_experts, top_k, tokens, capacity):
    """The slot arithmetic of the fixed-capacity exchange (tris_ep_pack_rows /
    tris_ep_dispatch_peer / tris_ep_return_peer), all ranks emulated in one process: rank s puts
    row `off` of its rows for owner d into slot (s, off) of d's receive buffer, d answers into
    slot (d, off) of s's result buffer, and combine_index[flat] = d * capacity + off finds it."""
    import trismoe_b200  # noqa: F401
    from trismoe_b200 import expert_parallel as ep

    rng = np.random.default_rng(7)
    recv = [np.full((world * capacity, 3), np.nan) for _ in range(world)]       # [value, expert id, unused]
    recv_id = [np.full((world * capacity,), -1, np.int64) for _ in range(world)]
    back = [np.full((world * capacity,), np.nan) for _ in range(world)]
    routes, values, indexes, overflow = [], [], [], False
    for s in range(world):
        T = tokens[s]
        sel = np.stack([rng.choice(num_experts, size=top_k, replace=False) for _ in range(T)]).astype(np.int64) \
            if T else np.zeros((0, top_k), np.int64)
        route = orc.build_route(sel, num_experts)
        gid = route["grouped_expert_ids"].astype(np.int64)
        val = rng.standard_normal(T * top_k)           # one number per flat (token, slot) entry
        owner = ep.owner_of(torch.from_numpy(gid), num_experts, world).numpy() if gid.size else gid
        first = np.searchsorted(owner, np.arange(world), side="left")
        index = np.full((T * top_k,), -1, np.int64)
        for d in range(world):
            end = first[d + 1] if d + 1 < world else gid.size
            overflow |= (end - first[d]) > capacity
            for off in range(capacity):
                row = first[d] + off
                if row < end:
                    flat = route["perm"][row]
                    recv[d][s * capacity + off, 0] = val[flat]
                    recv_id[d][s * capacity + off] = gid[row]
                    index[flat] = d * capacity + off
                else:
                    recv_id[d][s * capacity + off] = -1
        routes.append(sel)
        values.append(val)
        indexes.append(index)
    assert not overflow
    for d in range(world):  # every rank processes what it received and sends it back
        lo, hi = ep.expert_range(num_experts, d, world)
        for pos in range(world * capacity):
            e = recv_id[d][pos]
            if e < 0:
                continue
            assert lo <= e < hi
            s, off = divmod(pos, capacity)
            back[s][d * capacity + off] = recv[d][pos, 0] * (e + 1)
    for s in range(world):
        sel = routes[s].reshape(-1)
        got = back[s][indexes[s]] if sel.size else np.zeros((0,))
        assert np.array_equal(got, values[s] * (sel + 1))
