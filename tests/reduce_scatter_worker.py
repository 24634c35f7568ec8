"""One rank of the multi-GPU check of the scatter GEMM + ordered sum (started by
test_reduce_scatter_gpu.py through torch.distributed.run).  Every rank builds the same seeded case,
runs its K shard with the epilogue that stores fp32 partial tiles into the row owners' slots,
meets the others, sums its own slots and compares with the sum of the partial GEMMs that it
recomputes locally for all ranks."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from inference_b200 import ops, shard, synth
    ops.set_option("gemm_path", 1)

    ok = True
    for (m, n, k) in [(128 * world, 256, 128 * world), (1024 * world // 2, 1152, 512 * world), (2048, 7168, 2048)]:
        if m % (128 * world) or k % (128 * world):
            continue
        x = synth.activations(m, k, seed=3, device=dev)
        b_q, b_s = synth.quantised_weights(n, k, seed=4, device=dev)
        a_q, a_s = ops.quant_fp8_per_token_group(x)
        mine = shard.shard_k(a_q, a_s, b_q, b_s, world, rank)
        slots = shard.PeerSlots(m, n, dev)
        lo, hi = shard.owner_rows(m, world, rank)
        want = None
        for r in range(world):
            part = ops.w8a8_block_fp8_gemm(*shard.shard_k(a_q, a_s, b_q, b_s, world, r), out_dtype=torch.float32)[lo:hi]
            want = part.clone() if want is None else want + part
        want = want.to(torch.bfloat16)
        for rep in range(3):
            slots.local.fill_(float(rep))
            slots.barrier()
            ops.w8a8_block_fp8_gemm_scatter(slots.ptrs, rank, *mine)
            slots.barrier()
            got = ops.reduce_slots(slots.local)
            torch.cuda.synchronize()
            same = torch.equal(got, want)
            ok &= same
            if not same:
                print(f"rank {rank}: {m}x{n}x{k} rep {rep}: {(got != want).sum().item()} elements differ", flush=True)
        assert ops.device_status()[0] == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("reduce-scatter parity ok", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
