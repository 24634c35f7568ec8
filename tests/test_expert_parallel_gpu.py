"""Expert-parallel MoE layer against the single-device layer, bit for bit.

On one GPU the ranks are emulated: every rank's share (its token slice, its experts' weights)
runs through the same three stages as the real thing (route -> run_experts -> combine), and
the two exchanges between the stages are done by slicing on the host side of the test, in
exactly the order an all-to-all delivers (source-major).  With two or more GPUs a worker per
GPU runs ExpertParallelMoE.forward over NCCL (tests/expert_parallel_worker.py)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def build_layers(world, experts, hidden, inter, topk, seed=0):
    from inference_b200 import synth
    from inference_b200.expert_parallel import ExpertParallelMoE, expert_bounds
    from inference_b200.moe import MoEFP8Layer
    wgu, sgu = synth.quantised_weights(experts * 2 * inter, hidden, seed=seed + 1)
    wd, sd = synth.quantised_weights(experts * hidden, inter, seed=seed + 2)
    wgu, sgu = wgu.view(experts, 2 * inter, hidden), sgu.view(experts, 2 * inter // 128, hidden // 128)
    wd, sd = wd.view(experts, hidden, inter), sd.view(experts, hidden // 128, inter // 128)
    parts = []
    for r in range(world):
        lo, hi = expert_bounds(experts, world, r)
        parts.append(ExpertParallelMoE(wgu[lo:hi].contiguous(), sgu[lo:hi].contiguous(), wd[lo:hi].contiguous(),
                                       sd[lo:hi].contiguous(), experts, topk, world, r))
    return (wgu, sgu, wd, sd), parts


def emulate(parts, xs, logits):
    """All ranks' forward on one device: the exchanges become slices and concatenations."""
    world = len(parts)
    routed = [p.route(x, l) for p, x, l in zip(parts, xs, logits)]
    counts = [r.send_counts.cpu().tolist() for r in routed]                    # counts[s][d]
    starts = [np.concatenate([[0], np.cumsum(c)]) for c in counts]
    outs = []
    arrived = []
    for d in range(world):                                                     # what rank d receives, source-major
        seg = lambda t, s: t[int(starts[s][d]):int(starts[s][d + 1])]
        rq = torch.cat([seg(routed[s].xq, s) for s in range(world)])
        rs = torch.cat([seg(routed[s].xs, s) for s in range(world)])
        rid = torch.cat([seg(routed[s].sorted_ids, s) for s in range(world)])
        arrived.append(parts[d].run_experts(rq, rs, rid))
    for s in range(world):                                                     # the way back, destination-major
        back = []
        for d in range(world):
            first = sum(counts[t][d] for t in range(s))
            back.append(arrived[d][first:first + counts[s][d]])
        outs.append(parts[s].combine(torch.cat(back), routed[s]))
    return outs


@pytest.mark.parametrize("world,tokens,experts,topk,hidden,inter", [(2, 300, 8, 2, 512, 256), (4, 512, 32, 4, 1024, 384),
                                                                    (8, 1024, 64, 8, 512, 128), (2, 64, 4, 1, 256, 128)])
def test_emulated_ranks_equal_the_single_device_layer(world, tokens, experts, topk, hidden, inter):
    from inference_b200 import ops, synth
    from inference_b200.moe import MoEFP8Layer
    assert ops.has_cuda() and ops.device_sm_version(0) == 100, "needs a B200"
    (wgu, sgu, wd, sd), parts = build_layers(world, experts, hidden, inter, topk, seed=world)
    x = synth.activations(tokens, hidden, seed=9)
    g = torch.Generator(device="cpu").manual_seed(world + tokens)
    logits = torch.randn((tokens, experts), generator=g).cuda()
    if experts >= 8:
        logits[:, 1] = -60.0            # an expert nobody picks
    want = MoEFP8Layer(wgu, sgu, wd, sd, topk, tokens).forward(x, logits)
    per = tokens // world
    xs = [x[r * per:(r + 1) * per].contiguous() for r in range(world)]
    ls = [logits[r * per:(r + 1) * per].contiguous() for r in range(world)]
    got = torch.cat(emulate(parts, xs, ls))
    assert ops.device_status()[0] == 0
    assert torch.equal(got, want)


def test_permute_rows_scatter_and_gather(ops=None):
    from inference_b200 import ops
    rng = np.random.default_rng(1)
    rows, width = 1000, 96
    src = torch.from_numpy(rng.integers(0, 255, (rows, width), dtype=np.uint8)).cuda()
    perm = torch.from_numpy(rng.permutation(rows).astype(np.int32)).cuda()
    perm[5] = -1
    dst = torch.full((rows, width), 7, dtype=torch.uint8, device="cuda")
    ops.moe_permute_rows(src, perm, dst, gather=False)
    keep = perm >= 0
    assert torch.equal(dst[perm[keep].long()], src[keep])
    back = torch.zeros_like(src)
    ops.moe_permute_rows(dst, perm, back, gather=True)
    assert torch.equal(back[keep], src[keep]) and bool((back[5] == 0).all())
    with pytest.raises(Exception):
        ops.moe_permute_rows(src[:, :10].contiguous(), perm, dst[:, :10].contiguous(), gather=False)   # rows of 10 bytes


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_processes_over_nccl_equal_the_single_device_layer():
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29741", os.path.join(HERE, "expert_parallel_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "expert-parallel parity ok" in res.stdout
