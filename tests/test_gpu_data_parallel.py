"""Two-GPU data-parallel check (skipped with fewer than two devices): with identical data on both ranks the
reduced, 1/world-scaled gradient equals the single-GPU gradient bit for bit (x + x and /2 are exact), so after an
optimizer step both replicas hold exactly the single-GPU parameters.  With bf16 gradient buckets every rank's
gradient is rounded once before the sum: the replicas still agree with each other bit for bit and stay within bf16
rounding of the single-GPU parameters."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NNB_ROOT"])
import __graft_entry__ as entry
from oracle import gpt_oracle as go
nnb = entry.load_package()
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
oc = go.GptConfig(256, 128, 2, 2, 256, 128, 2, go.ACT_SWIGLU, go.NORM_RMS, go.POS_ALIBI)
params = go.init_params(oc, 42)
mbs = go.make_batches(oc, 2, seed=3, dist="zipf")
def run(pg, buckets="fp32"):
    cfg = nnb.GptConfig(oc.vocab, oc.d_model, oc.heads, oc.layers, oc.d_ff, oc.seq, oc.batch, oc.act, oc.norm, oc.pos, nnb.FP32)
    tr = nnb.GptTrainer(cfg, lr=1e-3, process_group=pg, grad_reduce_dtype=buckets)
    tr.load_params(params)
    for step in range(2):
        tr.micro_step(mbs[step]["tokens"], mbs[step]["labels"], mbs[step]["mask"])
        tr.optimizer_step(clip=1.0)
    torch.cuda.synchronize()
    return tr.params.clone()
p_dp = run(dist.group.WORLD)
p_single = run(None)
ok = torch.equal(p_dp, p_single)
print("RANK", rank, "EQUAL", ok, flush=True)
p_bf = run(dist.group.WORLD, "bf16")
both = [torch.empty_like(p_bf) for _ in range(world)]
dist.all_gather(both, p_bf)
same = all(torch.equal(both[0], b) for b in both[1:])
rel = float((p_bf - p_single).norm() / p_single.norm())
print("RANK", rank, "BF16_REPLICAS_EQUAL", same, "REL", rel, flush=True)
ok = ok and same and rel < 1e-3
dist.destroy_process_group()
sys.exit(0 if ok else 3)
'''


def test_two_replicas_match_single_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "dp_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NNB_ROOT=root, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29533", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count(" EQUAL True") == 2
    assert r.stdout.count("BF16_REPLICAS_EQUAL True") == 2
