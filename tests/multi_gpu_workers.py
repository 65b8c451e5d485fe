"""Workers of tests/test_gpu_multi.py, one rank per GPU over NCCL:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        tests/multi_gpu_workers.py {training|rows|heads}

Every rank builds the same seeded graph and features, runs its share through the sharded path and
compares its rows with the single-GPU result of the whole graph computed on the same device, and with
the CPU oracle.
  training: ``ShardedTrainingAttention`` forward + backward (and through ``torch.autograd``);
  rows:     ``ShardedAttention.forward`` (TC-block balanced shards, one all-gather, two-phase kernel);
  heads:    ``HeadShardedPipeline.forward`` (heads over ranks, pipelined all-to-alls)."""
import math
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fused3s_b200 import cabi, graphs, sharding  # noqa: E402


def setup():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import datetime

    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))
    return rank, world, dev


def check_rows_against_oracle(g, q, k, v, out, a, b, scale, seed):
    from oracle import attention_oracle as ao

    rng = np.random.default_rng(seed)
    for r0 in rng.integers(a, max(a + 1, b - 64), size=3):
        r0 = int(r0) // 16 * 16
        r1 = min(b, r0 + 64)
        for h in range(q.shape[1] if q.dim() == 3 else 1):
            sel = (lambda x: x[:, h]) if q.dim() == 3 else (lambda x: x)
            want = ao.edge_attention(g.rowptr, g.colidx, sel(q), sel(k), sel(v), scale, row_begin=r0, row_end=r1)
            m = ao.compare(sel(out[r0 - a:r1 - a]).float().cpu(), want)
            assert m["max_abs"] <= ao.MAX_ABS_TOL and m["mean_rel"] <= ao.MEAN_REL_TOL, (r0, h, m)


def rows():
    rank, world, dev = setup()
    used = []
    for cfg, sc in ((4, 0.05), (5, 0.02)):
        g = graphs.make_config(cfg, scale=sc)
        n = g.num_nodes
        q, k, v = graphs.make_features(g)
        rp, ci = torch.from_numpy(g.rowptr).to(dev), torch.from_numpy(g.colidx).to(dev)
        w = cabi.window_tcb_counts(ci, rp, n).cpu().numpy()
        # cfg4: own columns numbered last, all-gather overlapped with a first launch (NCCL);
        # cfg5: order-preserving numbering, one collective (NVSwitch multicast when it can be set up) + one launch
        shard = sharding.make_shard(g.rowptr, g.colidx, n, rank, world, window_weight=w, local_last=(cfg == 4))
        att = sharding.ShardedAttention(shard, dev, two_phase=(cfg == 4), collective="nccl" if cfg == 4 else "multimem")
        assert att.two_phase == (cfg == 4)
        a, b = shard.row_begin, shard.row_end
        ql = q[a:b].to(dev)
        ks, vs = att.send_buffers(ql)
        ks[: b - a].copy_(k[a:b])
        vs[: b - a].copy_(v[a:b])
        tcb = cabi.preprocess(ci, rp, n, 16)
        one = cabi.forward(tcb, n, q.to(dev), k.to(dev), v.to(dev), 8.0)
        for call in range(3):  # buffers and scratch are reused from call to call
            out = att.forward(ql, ks, vs, 8.0)
            torch.cuda.synchronize()
            assert torch.allclose(out, one[a:b], rtol=2e-3, atol=5e-4), (rank, cfg, call)
        check_rows_against_oracle(g, q, k, v, out, a, b, 8.0, seed=rank)
        # the shares are balanced by TC blocks
        t = torch.tensor([float(att.tcb["nTCB"])], device=dev)
        parts = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        parts = [float(x) for x in parts]
        assert max(parts) <= 1.05 * (sum(parts) / world) + 64, parts
        used.append(att.collective_used)
    if rank == 0:
        print(f"row-sharded forward (collectives: {used}) ok on {world} GPUs")
    dist.destroy_process_group()


def heads():
    rank, world, dev = setup()
    g = graphs.make_config(5, scale=0.03)
    n = g.num_nodes
    q, k, v = graphs.make_features(g)
    hp = sharding.HeadShardedPipeline(g.rowptr, g.colidx, n, g.heads, rank, world, dev, chunks=3)
    a, b = hp.row_begin, hp.row_end
    q_x = hp.to_exchange_layout(q[a:b].to(dev))
    kv_x = hp.kv_to_exchange_layout(k[a:b].to(dev), v[a:b].to(dev))
    rp, ci = torch.from_numpy(g.rowptr).to(dev), torch.from_numpy(g.colidx).to(dev)
    tcb = cabi.preprocess(ci, rp, n, 16)
    one = cabi.forward(tcb, n, q.to(dev), k.to(dev), v.to(dev), 8.0)
    for call in range(3):
        out = hp.from_exchange_layout(hp.forward(q_x, kv_x, 8.0))
        torch.cuda.synchronize()
        assert out.shape == (b - a, g.heads, g.dim)
        assert torch.allclose(out, one[a:b], rtol=2e-3, atol=5e-4), (rank, call)
    check_rows_against_oracle(g, q, k, v, out, a, b, 8.0, seed=10 + rank)
    if rank == 0:
        print(f"head-sharded pipeline ok on {world} GPUs")
    dist.destroy_process_group()


def training():
    rank, world, dev = setup()
    g = graphs.make_config(5, scale=0.02)  # multi-head power-law graph
    n = g.num_nodes
    q, k, v = graphs.make_features(g)
    gen = torch.Generator().manual_seed(11)
    d_out = torch.randn(q.shape, generator=gen)
    scale = math.sqrt(q.shape[-1])

    att = sharding.ShardedTrainingAttention(g.rowptr, g.colidx, n, rank, world, dev)
    a, b = att.shard.row_begin, att.shard.row_end
    out = att.forward(q[a:b].to(dev), k[a:b].to(dev), v[a:b].to(dev), scale)
    dq, dk, dv = att.backward(d_out[a:b].to(dev))

    rp, ci = torch.from_numpy(g.rowptr).to(dev), torch.from_numpy(g.colidx).to(dev)
    tcb = cabi.preprocess(ci, rp, n, 16)
    rp_t, ci_t = cabi.transpose_csr(rp, ci, n)
    tcb_t = cabi.preprocess(ci_t, rp_t, n, 16)
    out1, lse1 = cabi.forward_lse(tcb, n, q.to(dev), k.to(dev), v.to(dev), scale)
    ref = cabi.backward(tcb, tcb_t, n, q.to(dev), k.to(dev), v.to(dev), out1, lse1, d_out.to(dev), scale)
    worst = 0.0
    for name, got, want in (("out", out, out1[a:b]), ("dq", dq, ref[0][a:b]), ("dk", dk, ref[1][a:b]),
                            ("dv", dv, ref[2][a:b])):
        err = float(torch.linalg.norm(got.double() - want.double()) / torch.linalg.norm(want.double()).clamp_min(1e-30))
        worst = max(worst, err)
        assert err <= 2e-3, (rank, name, err)  # the two runs differ only in how heavy windows are chunked
    # the same through torch.autograd
    from fused3s_b200 import autograd as fa

    ql, kl, vl = (x[a:b].to(dev).requires_grad_(True) for x in (q, k, v))
    out_a = fa.sharded_attention(ql, kl, vl, att, scale)
    out_a.backward(d_out[a:b].to(dev))
    for name, got, want in (("q.grad", ql.grad, dq), ("k.grad", kl.grad, dk), ("v.grad", vl.grad, dv)):
        assert got.dtype == torch.float16
        assert torch.equal(got, want.to(torch.float16)), (rank, name)
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"sharded training check ok on {world} GPUs: worst relative difference {float(t):.2e}")
    dist.destroy_process_group()


if __name__ == "__main__":
    {"training": training, "rows": rows, "heads": heads}[sys.argv[1] if len(sys.argv) > 1 else "training"]()
