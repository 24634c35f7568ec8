"""N-sharding arithmetic and the gather layout, on two gloo ranks (CPU)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from inference_b200 import shard


def test_shard_bounds_cover_n_in_whole_scale_blocks():
    for n, g in [(73728, 8), (73728, 4), (73728, 2), (73728, 1), (1024, 2)]:
        spans = [shard.shard_bounds(n, g, r) for r in range(g)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % 128 == 0 and hi % 128 == 0 for lo, hi in spans)
    with pytest.raises(ValueError):
        shard.shard_bounds(1000, 2, 0)
    with pytest.raises(ValueError):
        shard.shard_bounds(128 * 3, 2, 0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, m, n, k, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)  # same inputs on every rank: A replicated, W sharded from one matrix
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    bq_l, bs_l = shard.shard_weights(torch.from_numpy(bq), torch.from_numpy(bs), world, rank)
    # the per-rank GEMM (the oracle stands in for the GPU kernel on CPU ranks)
    c_l = torch.from_numpy(oracle.w8a8_block_fp8_gemm(aq, a_s, bq_l.numpy(), bs_l.numpy()))
    blocked = shard.gather_outputs(c_l)
    full = shard.blocked_to_row_major(blocked)
    # the layout contract of the all-gather GEMM: rank r's result occupies columns
    # peer_columns(N/G, r) of every rank's row-major [M, N] buffer (gloo moves the data here)
    parts = [torch.empty_like(c_l) for _ in range(world)]
    dist.all_gather(parts, c_l)
    peer_full = torch.full((m, n), float("nan"))
    for r in range(world):
        lo, hi = shard.peer_columns(n // world, r)
        peer_full[:, lo:hi] = parts[r]
    if rank == 0:
        want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
        np.save(os.path.join(out_dir, "ok.npy"),
                np.array([np.array_equal(full.numpy(), want), blocked.shape == (world, m, n // world),
                          np.array_equal(peer_full.numpy(), want)]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_gemm_and_gather_equals_unsharded(tmp_path):
    world, m, n, k = 2, 8, 512, 256
    mp.spawn(_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    ok = np.load(tmp_path / "ok.npy")
    assert ok.all()


def test_peer_output_without_a_process_group_is_one_local_buffer():
    out = shard.PeerOutput(4, 256, torch.float16, device="cpu")
    assert out.world == 1 and out.rank == 0 and out.ptrs == [out.local.data_ptr()]
    assert out.local.shape == (4, 256)
    out.barrier()   # nothing to meet
    assert shard.peer_columns(128, 3) == (384, 512)


def _k_worker(rank, world, port, m, n, k, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(1)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (0.02 * rng.standard_normal((n, k))).astype(np.float32)
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    t = [torch.from_numpy(x) for x in (aq, a_s, bq, bs)]
    mine = [x.numpy() for x in shard.shard_k(*t, world, rank)]
    part = torch.from_numpy(oracle.w8a8_block_fp8_gemm(*mine))          # this rank's partial [M, N]
    # the contract of the scatter GEMM: owner d receives rows owner_rows(d) of every rank's partial
    # in slot [source rank]; gloo gathers move the row blocks here
    rows = [shard.owner_rows(m, world, d) for d in range(world)]
    send = [part[lo:hi].contiguous() for lo, hi in rows]
    recv = []
    for d in range(world):                  # gloo has no all-to-all: one gather per owner
        got = [torch.empty_like(send[d]) for _ in range(world)] if rank == d else None
        dist.gather(send[d], got, dst=d)
        if rank == d:
            recv = got
    acc = recv[0].clone()
    for r in range(1, world):
        acc = acc + recv[r]
    lo, hi = rows[rank]
    want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)[lo:hi]
    ok = np.allclose(acc.numpy(), want, rtol=1e-5, atol=1e-6)
    np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_k_sharded_gemm_scatter_and_sum_equals_unsharded(tmp_path):
    world, m, n, k = 2, 256, 96, 512
    mp.spawn(_k_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    assert all(np.load(tmp_path / f"ok{r}.npy").all() for r in range(world))


def test_k_shard_and_owner_bounds():
    assert shard.k_shard_bounds(1024, 4, 1) == (256, 512)
    assert shard.owner_rows(512, 2, 1) == (256, 512)
    with pytest.raises(ValueError):
        shard.k_shard_bounds(384, 2, 0)
    with pytest.raises(ValueError):
        shard.owner_rows(384, 2, 0)


# ------------------------------------------------------------------ row-split upload of the host front end
def _rows_worker(rank, world, port, rows, k, out_dir):
    """What inference_b200.host.HostLinearFP8 does with a panel at N > 1: every rank quantises its
    rank_rows chunk, the ranks all-gather bytes and scales; the result must equal quantising the
    whole panel in one place."""
    from inference_b200 import host
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)                       # the same host activations on every rank
    x = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((rows, k)).astype(np.float32)))
    lo, hi = host.rank_rows(rows, world, rank)
    q_part, s_part = (torch.from_numpy(t) for t in oracle.quant_fp8_per_token_group(x[lo:hi]))
    q = torch.empty((rows, k), dtype=torch.uint8)
    s = torch.empty((rows, k // 128), dtype=torch.float32)
    dist.all_gather_into_tensor(q, q_part)
    dist.all_gather_into_tensor(s, s_part)
    want_q, want_s = oracle.quant_fp8_per_token_group(x)
    np.save(os.path.join(out_dir, f"rows{rank}.npy"),
            np.array([np.array_equal(q.numpy(), want_q), np.array_equal(s.numpy(), want_s)]))
    dist.barrier()
    dist.destroy_process_group()


def test_row_split_quantisation_all_gathers_to_the_whole_panel(tmp_path):
    from inference_b200 import host
    assert host.rank_rows(2048, 8, 3) == (768, 1024)
    with pytest.raises(ValueError):
        host.rank_rows(100, 8, 0)
    world, rows, k = 2, 64, 512
    mp.spawn(_rows_worker, args=(world, _free_port(), rows, k, str(tmp_path)), nprocs=world, join=True)
    assert all(np.load(tmp_path / f"rows{r}.npy").all() for r in range(world))
