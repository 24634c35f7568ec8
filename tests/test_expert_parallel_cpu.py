"""Dispatch / combine layout of the expert-parallel layer on two gloo ranks (CPU): which rows go
where, in which order they arrive, and that the way back restores the owner's order."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_expert_blocks_and_rows_per_rank():
    from inference_b200 import expert_parallel as ep
    assert ep.expert_bounds(256, 8, 3) == (96, 128)
    with pytest.raises(ValueError):
        ep.expert_bounds(10, 4, 0)
    counts = torch.tensor([1, 2, 3, 4, 5, 6, 7, 8])
    assert ep.rows_per_rank(counts, 2).tolist() == [10, 26]
    assert ep.rows_per_rank(counts, 4).tolist() == [3, 7, 11, 15]


def _worker(rank, world, port, out_dir):
    from inference_b200 import expert_parallel as ep
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    experts, topk, tokens, width = 8, 2, 13 + rank, 4
    rng = np.random.default_rng(100 + rank)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    ids, _ = oracle.topk_softmax(logits, topk)
    counts, offsets, pos, src_token, _, _ = oracle.moe_align(ids, experts)
    # sorted rows: row pos[t*topk+k] carries (rank, token, k, expert)
    send = torch.zeros((tokens * topk, width), dtype=torch.int64)
    for t in range(tokens):
        for k in range(topk):
            send[pos[t * topk + k]] = torch.tensor([rank, t, k, int(ids[t, k])])
    send_counts = ep.rows_per_rank(torch.from_numpy(counts.astype(np.int64)), world)
    all_counts = [torch.zeros(world, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_counts, send_counts)
    recv_counts = [int(all_counts[s][rank]) for s in range(world)]
    got = ep.exchange_rows(send, send_counts.tolist(), recv_counts)
    lo, hi = ep.expert_bounds(experts, world, rank)
    ok = got.shape[0] == sum(recv_counts)
    ok &= bool(((got[:, 3] >= lo) & (got[:, 3] < hi)).all())            # only this rank's experts arrive
    src = got[:, 0]
    ok &= bool((src[1:] >= src[:-1]).all())                               # source-major arrival order
    for s in range(world):                                                # and expert-sorted within a source
        e = got[src == s][:, 3]
        ok &= bool((e[1:] >= e[:-1]).all())
    back = ep.exchange_rows(got * 10, recv_counts, send_counts.tolist())  # "results" travel home
    ok &= bool(torch.equal(back, send * 10))                              # in the owner's sorted order
    np.save(os.path.join(out_dir, f"ep{rank}.npy"), np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_dispatch_and_way_back(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(np.load(tmp_path / f"ep{r}.npy").all() for r in range(world))
