"""One rank of the multi-GPU check of the expert-parallel MoE layer (started by
test_expert_parallel_gpu.py through torch.distributed.run).  Every rank holds the full seeded
weights only to compute the single-device answer for its own tokens; the expert-parallel layer
gets this rank's experts."""
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
    from inference_b200 import ops, synth
    from inference_b200.expert_parallel import ExpertParallelMoE, expert_bounds
    from inference_b200.moe import MoEFP8Layer

    ok = True
    for (tokens, experts, topk, hidden, inter) in [(256, 8 * world, 2, 512, 256), (1000, 16 * world, 8, 1024, 384)]:
        wgu, sgu = synth.quantised_weights(experts * 2 * inter, hidden, seed=1, device=dev)
        wd, sd = synth.quantised_weights(experts * hidden, inter, seed=2, device=dev)
        wgu, sgu = wgu.view(experts, 2 * inter, hidden), sgu.view(experts, 2 * inter // 128, hidden // 128)
        wd, sd = wd.view(experts, hidden, inter), sd.view(experts, hidden // 128, inter // 128)
        lo, hi = expert_bounds(experts, world, rank)
        layer = ExpertParallelMoE(wgu[lo:hi].contiguous(), sgu[lo:hi].contiguous(), wd[lo:hi].contiguous(),
                                  sd[lo:hi].contiguous(), experts, topk, world, rank)
        x = synth.activations(tokens, hidden, seed=10 + rank, device=dev)          # this rank's own tokens
        g = torch.Generator(device="cpu").manual_seed(20 + rank)
        logits = torch.randn((tokens, experts), generator=g).to(dev)
        want = MoEFP8Layer(wgu, sgu, wd, sd, topk, tokens).forward(x, logits)
        for _ in range(2):
            got = layer.forward(x, logits)
            torch.cuda.synchronize()
            ok &= bool(torch.equal(got, want))
        assert ops.device_status()[0] == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("expert-parallel parity ok", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
