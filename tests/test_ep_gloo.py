"""Host logic of the expert-parallel exchange on CPU: two gloo ranks route synthetic pairs, exchange rows with the splits
`plan_exchange` computes, and check the orderings the device kernels rely on (source-major, expert order inside a source;
the return path restores the sender's order). No GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ingot_b200 import ep
from oracle import qref

E, K, T, D = 32, 4, 11, 8


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def routing_of(rank):
    rng = np.random.default_rng(100 + rank)
    return np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)


def worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        inds = routing_of(rank)
        offsets, row_map, pos = qref.group_pairs(inds, E)
        counts = torch.from_numpy(np.diff(offsets.astype(np.int64)).astype(np.int32))
        counts_all = torch.zeros(world * E, dtype=torch.int32)
        dist.all_gather_into_tensor(counts_all, counts)
        ca = counts_all.view(world, E).numpy()
        send, recv = ep.plan_exchange(ca, rank)
        P = T * K
        assert sum(send) == P
        # a row carries (source rank, pair id, expert) so the receiver can check what it got
        rows = torch.zeros(P, D, dtype=torch.float32)
        flat = inds.reshape(-1)
        for pair in range(P):
            rows[pos[pair], 0] = rank
            rows[pos[pair], 1] = pair
            rows[pos[pair], 2] = float(flat[pair])
        R = sum(recv)
        got = torch.zeros(R, D, dtype=torch.float32)
        dist.all_to_all_single(got, rows, recv, send)
        lo, per = ep.expert_range(rank, world, E)
        # source-major, then ascending expert, then ascending pair id; every expert is one of mine
        keys = [(int(r[0]), int(r[2]), int(r[1])) for r in got]
        assert keys == sorted(keys)
        assert all(lo <= e < lo + per for _, e, _ in keys)
        # per (source, expert) counts agree with the gathered matrix: what the tile builder relies on
        for s in range(world):
            for e in range(lo, lo + per):
                assert sum(1 for k in keys if k[0] == s and k[1] == e) == ca[s, e]
        # the return path restores the sender's expert order
        back = torch.zeros(P, D, dtype=torch.float32)
        dist.all_to_all_single(back, got, send, recv)
        assert torch.equal(back, rows)
        q.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_exchange_plan_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def colsplit_worker(rank, world, port, q):
    """The column-split linear's host logic: every rank cuts its shard of the same seeded matrix, computes its slice of y
    (with the CPU oracle standing in for the kernels), the slices are all-gathered and assembled."""
    from ingot_b200 import synth

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)  # the same tensors on every rank
        N, Kin, rows, max_rows = 96, 128, 3, 4
        w, s, b = synth.affine_np(rng, N, Kin, 4)
        x = synth.activations_np(rng, rows, Kin)
        lo, per = ep.column_shard(rank, world, N)
        assert (lo, per) == (rank * N // world, N // world)
        ws, ss, bs = ep.shard_tensors(w[0], s[0], b[0], rank, world, N)
        assert ws.shape == (per, Kin // 8) and ss.shape == (per, Kin // 64)
        # a shard is one contiguous byte range of each tensor
        assert ws.tobytes() == w[0].tobytes()[lo * Kin // 2:(lo + per) * Kin // 2]
        y_local = torch.zeros(max_rows, per)
        y_local[:rows] = torch.from_numpy(qref.matmul_t(x, qref.dequant_affine(ws, ss, bs, 4)))
        y_all = torch.zeros(world, max_rows, per)
        dist.all_gather_into_tensor(y_all.view(world * max_rows, per), y_local)
        y = ep.assemble_columns(y_all, rows)
        ref = qref.matmul_t(x, qref.dequant_affine(w[0], s[0], b[0], 4))
        assert y.shape == (rows, N) and np.array_equal(y.numpy(), ref)
        q.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_column_split_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=colsplit_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res


def test_column_shard_guards():
    assert ep.column_shard(3, 8, 14336) == (5376, 1792)
    with pytest.raises(ValueError):
        ep.column_shard(0, 3, 64)      # 64 features do not make three shards of whole 16-row blocks
    with pytest.raises(ValueError):
        ep.column_shard(2, 2, 64)


def test_plan_exchange_and_slices():
    ca = np.arange(4 * 8).reshape(4, 8)
    send, recv = ep.plan_exchange(ca, 1)
    assert send == [int(ca[1, 0:2].sum()), int(ca[1, 2:4].sum()), int(ca[1, 4:6].sum()), int(ca[1, 6:8].sum())]
    assert recv == [int(ca[s, 2:4].sum()) for s in range(4)]
    assert ep.expert_range(3, 8, 128) == (48, 16)
    with pytest.raises(ValueError):
        ep.expert_range(0, 3, 128)
    assert [ep.token_slice(r, 4, 10) for r in range(4)] == [(0, 3), (3, 3), (6, 2), (8, 2)]
