"""One rank of the multi-GPU check of the all-gather GEMM (started by test_allgather_gpu.py
through torch.distributed.run).  Every rank builds the same seeded case, runs its column shard
with the epilogue that stores into every rank's buffer, meets the others, and compares its own
full buffer with the unsharded GEMM computed locally."""
import os
import sys

import numpy as np
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

    ok = True
    for (m, n_shard, k) in [(256, 256, 512), (1000, 1152, 1024), (4096, 2304, 2048)]:
        n = n_shard * world
        x = synth.activations(m, k, seed=3, device=dev)
        b_q, b_s = synth.quantised_weights(n, k, seed=4, device=dev)
        a_q, a_s = ops.quant_fp8_per_token_group(x)
        want = ops.w8a8_block_fp8_gemm(a_q, a_s, b_q, b_s)
        wq, ws = shard.shard_weights(b_q, b_s, world, rank)
        out = shard.PeerOutput(m, n, torch.bfloat16, dev)
        assert out.world == world and out.rank == rank and len(out.ptrs) == world
        for rep in range(3):
            out.local.fill_(float(rep))
            out.barrier()                       # nobody stores into a buffer that is still being reset
            ops.w8a8_block_fp8_gemm_allgather(out.ptrs, rank, a_q, a_s, wq, ws)
            out.barrier()
            torch.cuda.synchronize()
            same = torch.equal(out.local, want)
            ok &= same
            if not same:
                bad = (out.local != want).nonzero()
                print(f"rank {rank}: {m}x{n}x{k} rep {rep}: {bad.shape[0]} elements differ, first {bad[0].tolist()}",
                      flush=True)
        # the same gather done by the copy engines, panel by panel
        pg = shard.PanelGather(m, n, torch.bfloat16, dev, panels=4)
        for rep in range(2):
            pg.out.local.fill_(float(rep))
            pg.out.barrier()
            got = pg(a_q, a_s, wq, ws)
            torch.cuda.synchronize()
            same = torch.equal(got, want)
            ok &= same
            if not same:
                print(f"rank {rank}: panel gather {m}x{n}x{k} rep {rep} differs", flush=True)
        assert ops.device_status()[0] == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("allgather parity ok", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
