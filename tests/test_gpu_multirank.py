"""The batch x heads sharding of the multi-GPU benchmark on real GPUs.

Every (batch, head) pair of an attention call is independent, so N ranks each
run a contiguous range of b * H + h units (heads as strided views of the full
tensors) and the gathered results must equal the unsharded result bit for bit.
The first test plays both ranks of a 2-way split on one GPU, one after the
other; the second launches two real ranks over NCCL when the machine has two
GPUs and is skipped otherwise."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import bench
from rgd_triton_b200 import ops
from tests._util import gen, randn

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [2, 3, 8])
def test_sharded_units_equal_the_unsharded_result_on_one_gpu(world):
    g = gen(31)
    B, Tn, H, D = 2, 384, 6, 128
    q, k, v, do = (randn(g, B, Tn, H, D, dtype=torch.bfloat16).cuda() for _ in range(4))
    attn = ops.FlashAttention()
    qi, ki, vi = (t.clone().requires_grad_(True) for t in (q, k, v))
    o = attn(qi, ki, vi)
    full = (o.detach(), *torch.autograd.grad(o, (qi, ki, vi), do))
    shards = [bench.run_shard(q.device, attn, q, k, v, do, world, r) for r in range(world)]
    buckets = [[shards[r][t] for r in range(world)] for t in range(4)]
    res = bench.compare_gathered(buckets, full, world)
    assert res["ok"], res


def test_two_ranks_over_nccl_gather_and_compare():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "bench.py"),
                          "--gpus", "2", "--steps", "3", "--warmup", "3", "--attn-only"],
                         capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads([ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["verify"]["ok"] and line["verify"]["ranks"] == 2, line["verify"]
