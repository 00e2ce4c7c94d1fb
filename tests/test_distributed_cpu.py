"""world_size-2 gloo tests (CPU) of the multi-GPU host logic: tensor partitioning for the
whole-model pass and the column-sharded linear with its all-gather."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import voyager_oracle as vo
        from voyager_compiler_b200 import model_quant as mq
        from voyager_compiler_b200 import parallel as par
        from golden_util import golden_table

        # 1. every rank derives the same plan; the shares are disjoint and complete
        shapes = [(64, 128), (32, 128), (512, 64), (8, 64), (300, 128)]
        sizes, rows = [a * b for a, b in shapes], [a for a, _ in shapes]
        plan = mq.shard_plan(sizes, rows, world)
        plans = [None] * world
        dist.all_gather_object(plans, plan)
        assert all(p == plans[0] for p in plans)
        covered = {}
        for r in range(world):
            for i, b, e in plan[r]:
                covered.setdefault(i, []).append((b, e))
        for i, r_ in enumerate(rows):
            spans = sorted(covered[i])
            assert spans[0][0] == 0 and spans[-1][1] == r_ and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        # quantizing the shares with the oracle and stitching them equals quantizing whole tensors
        torch.manual_seed(7)
        ws = [(torch.randn(s) * 0.02).to(torch.bfloat16) for s in shapes]
        tab = golden_table("nf4")
        mine = {}
        for i, b, e in plan[rank]:
            s = vo.mx_scale(ws[i][b:e], (-1,), 64, 1.0, False)
            mine[(i, b, e)] = (s, vo.quantize(ws[i][b:e], s, None, (-1,), 64, tab))
        everything = [None] * world
        dist.all_gather_object(everything, mine)
        for i, w in enumerate(ws):
            parts = sorted((k, v) for d in everything for k, v in d.items() if k[0] == i)
            s_all = torch.cat([v[0] for _, v in parts]); q_all = torch.cat([v[1] for _, v in parts])
            s_ref = vo.mx_scale(w, (-1,), 64, 1.0, False)
            assert torch.equal(s_all, s_ref) and torch.equal(q_all, vo.quantize(w, s_ref, None, (-1,), 64, tab))

        # 2. column-parallel linear: uneven shards (3 tiles over 2 ranks), bias, 3-D input
        torch.manual_seed(3)
        N, K = 600, 128
        x = torch.randn(2, 5, K).to(torch.bfloat16)
        w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
        bias = torch.randn(N).to(torch.bfloat16)
        q = golden_table("int8")
        xs, xq = vo.quantize_mx(x, q, (-1,), 32, 127.0, True)
        wsc, wq = vo.quantize_mx(w, q, (-1,), 32, 127.0, True)
        shards = par.column_shards(N, world)
        assert shards == [(0, 512), (512, 600)]
        wq_r, ws_r = par.shard_weight(wq, wsc, rank, world)
        n0, n1 = shards[rank]
        got = par.column_parallel_linear_mx(xq, xs, wq_r, ws_r, N, 32, bias_shard=bias[n0:n1], gemm=vo.linear_mx)
        want = vo.linear_mx(xq, wq, bias, input_scale=xs, weight_scale=wsc, block_size=32)
        assert got.shape == want.shape and torch.equal(got, want)
        # the prepared form, exchanged in two pieces (512 + 88 columns on rank 0's side, 88 + 0 on rank 1's)
        lin = par.ColumnParallelLinearMX(wq_r, ws_r, N, 32, bias_shard=bias[n0:n1], gemm=vo.linear_mx, chunks=2)
        assert len(lin.pieces) == 2
        assert torch.equal(lin(xq, xs), want) and torch.equal(lin(xq, xs), want)
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo():
    world = 2
    port = 29500 + (os.getpid() % 500)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}, dict(ret)


def test_column_shards_properties():
    from voyager_compiler_b200.parallel import column_shards
    for n in (11008, 256, 255, 1, 4096, 600):
        for g in (1, 2, 4, 8):
            sh = column_shards(n, g)
            assert sh[0][0] == 0 and sh[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(sh, sh[1:]))
            tiles = [-(-(b - a) // 256) for a, b in sh]
            assert max(tiles) - min(tiles) <= 1
            assert all(a % 256 == 0 for a, _ in sh if a < n)
    assert column_shards(11008, 8) == [(0, 1536), (1536, 3072), (3072, 4608), (4608, 5888), (5888, 7168),
                                       (7168, 8448), (8448, 9728), (9728, 11008)]
