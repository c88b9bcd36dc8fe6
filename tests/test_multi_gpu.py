"""Two-GPU check (NCCL) of the query-row-sharded path: every rank ends with the full output and the
full gradients, equal to the single-GPU result.  Skipped when fewer than two GPUs are visible."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "flash-3-way-attention_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flash_trittention import _native, flash_trittention, parallel
        from oracle import trittention_oracle as orc

        B, N, T, D, alpha = 1, 2, 320, 64, 1 / 64
        ins = orc.make_inputs(B, N, T, D, scale=0.5, seed=7, dtype=torch.bfloat16)
        q, k1, k2, v1, v2, dz = (t.to(dev) for t in ins)
        ref_leaves = [t.clone().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
        ref = flash_trittention(*ref_leaves, alpha, None, None, None, None, True)
        ref.backward(dz)
        leaves = [t.clone().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
        out = parallel.flash_trittention_query_sharded(*leaves, alpha, True)
        out.backward(dz)
        torch.cuda.synchronize()
        ok = _native.read_status(dev) == 0
        ok = ok and float((out.float() - ref.float()).abs().max()) <= 2e-2 * float(ref.float().abs().max())
        for a, b in zip(leaves, ref_leaves):
            ok = ok and float((a.grad.float() - b.grad.float()).abs().max()) <= 2e-2 * float(b.grad.float().abs().max())
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_query_sharded_two_gpus_matches_single_gpu():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert all(results.get(r) for r in range(world)), dict(results)
