"""Host-side logic of the multi-GPU paths on CPU ranks (gloo, world_size 2).

The kernels cannot run here, so the two native calls the sharded path makes are replaced IN THIS
TEST by stand-ins built on the CPU oracle that honour the same contract (interleaved query rows,
fp32 partial key-side sums in the workspace).  What is under test is the distributed plumbing of
``flash_trittention/parallel.py``: row ownership, the all-gather of output and dQ rows (with a sequence
length that does not divide by the world size), the forward that exchanges nothing when the caller does not ask for
the gathered output, the all-reduce of the partial sums and the finalisation, and head sharding."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "flash-3-way-attention_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_trittention import _native, parallel
        from oracle import trittention_oracle as orc

        B, N, T, D, alpha = 1, 2, 25, 8, 0.25
        q, k1, k2, v1, v2, dz = orc.make_inputs(B, N, T, D, seed=3)

        def fake_fwd(q, k1, k2, v1, v2, o, lse, alpha, causal, *w, q_mod=1, q_rem=0, flags=0):
            z, l = orc.tdp_forward(q, k1, k2, v1, v2, alpha, causal)
            rows = parallel.owned_rows(T, q_rem, q_mod)
            o[:, :, rows] = z[:, :, rows]
            lse[:, :, rows] = l[:, :, rows]

        def fake_bwd(q, k1, k2, v1, v2, o, do, lse, dq, dk1, dk2, dv1, dv2, alpha, causal, *w, q_mod=1, q_rem=0,
                     flags=0, ws=None):
            assert flags & _native.FLAG_BWD_PARTIAL
            rows = parallel.owned_rows(T, q_rem, q_mod)
            mask = torch.zeros(T, dtype=torch.bool)
            mask[rows] = True
            # gradient contribution of the owned query rows only: zero the upstream gradient elsewhere
            do_own = do * mask.view(1, 1, T, 1)
            g = orc.tdp_backward(q, k1, k2, v1, v2, do_own, alpha, causal)
            dq[:, :, rows] = g[0][:, :, rows]
            sv1 = torch.nn.functional.silu(v1)
            sig = torch.sigmoid(v1)
            dsv1 = g[3] / (sig * (1 + v1 * (1 - sig)))  # undo SiLU' to get the partial w.r.t. SiLU(V1)
            n = q.numel()
            ws = torch.zeros(16 * n, dtype=torch.uint8)
            ws.view(torch.float32)[: 4 * n] = torch.cat([g[1].flatten(), g[2].flatten(), dsv1.flatten(), g[4].flatten()])
            return ws

        def fake_finalize(v1, dk1, dk2, dv1, dv2, ws):
            n = v1.numel()
            part = ws.view(torch.float32)
            sig = torch.sigmoid(v1)
            dk1.copy_(part[:n].view_as(v1))
            dk2.copy_(part[n:2 * n].view_as(v1))
            dv1.copy_(part[2 * n:3 * n].view_as(v1) * sig * (1 + v1 * (1 - sig)))
            dv2.copy_(part[3 * n:4 * n].view_as(v1))

        _native.tdp_fwd, _native.tdp_bwd, _native.tdp_bwd_finalize = fake_fwd, fake_bwd, fake_finalize
        # the product refuses CPU tensors; the stand-ins above do not need a device
        from flash_trittention.triple_dot_product import flash_trittention as ft_mod

        ft_mod._validate = lambda *a: None
        _native.check_status = lambda *a, **k: None
        collectives = []
        for name in ("all_reduce", "all_gather_into_tensor"):
            orig = getattr(dist, name)

            def counted(*a, _orig=orig, _name=name, **k):
                collectives.append(_name)
                return _orig(*a, **k)

            setattr(dist, name, counted)
        leaves = [t.clone().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
        out = parallel.flash_trittention_query_sharded(*leaves, alpha, True)
        out.backward(dz)
        z_ref, _ = orc.tdp_forward(q, k1, k2, v1, v2, alpha, True)
        g_ref = orc.tdp_backward(q, k1, k2, v1, v2, dz, alpha, True)
        ok = torch.allclose(out, z_ref, atol=1e-5)
        for leaf, ref in zip(leaves, g_ref):
            ok = ok and torch.allclose(leaf.grad, ref, atol=2e-4)
        # one gather forward; backward = one all-reduce (the partial sums) + one gather (dQ rows)
        ok = ok and collectives == ["all_gather_into_tensor", "all_reduce", "all_gather_into_tensor"]
        # without the gathered output the forward does not communicate, and only the own rows are filled in
        del collectives[:]
        with torch.no_grad():
            own = parallel.flash_trittention_query_sharded(q, k1, k2, v1, v2, alpha, True, None, False)
        rows = parallel.owned_rows(T, rank, world)
        other = parallel.owned_rows(T, 1 - rank, world)
        ok = ok and collectives == [] and torch.allclose(own[:, :, rows], z_ref[:, :, rows], atol=1e-5)
        ok = ok and bool((own[:, :, other] == 0).all())
        # head sharding: the ranks' slices tile the (batch*head) axis exactly once
        full = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).view(2, 3, 4, 5)
        mine = parallel.shard_heads(full, rank, world)
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        ok = ok and torch.equal(torch.cat(gathered, 1).reshape(2, 3, 4, 5), full)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_query_sharded_and_head_sharded_paths_world_size_2():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert all(results.get(r) for r in range(world)), dict(results)


def test_row_ownership_is_a_partition():
    sys.path.insert(0, os.path.join(ROOT, "flash-3-way-attention_b200"))
    from flash_trittention import parallel

    T = 37
    for world in (1, 2, 4, 8):
        rows = torch.cat([parallel.owned_rows(T, r, world) for r in range(world)])
        assert sorted(rows.tolist()) == list(range(T))
    with pytest.raises(ValueError):
        parallel.shard_heads(torch.zeros(1, 3, 2, 2), 0, 2)
