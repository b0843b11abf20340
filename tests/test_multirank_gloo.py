"""CPU, world_size 2 over gloo: the host-side logic of the row-sharded paths.

Each rank takes its row shard of E exactly as the GPU path does (Ellpack.shard_rows: contiguous
ranges of ceil(m/G) rows, the parent's r kept), computes its slab with the CPU oracle standing in for
the kernel, places it at rank*ceil(m/G) rows of the padded output and all-gathers in place.  The
gathered buffer must equal the unsharded result bit for bit, for a row count that divides evenly and
one that does not, and for a two-layer row-sharded model where the gathered output of layer 1 is
layer 2's X."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _sparse(rng, m, n, p):
    W = rng.standard_normal((m, n)).astype(np.float32)
    W[rng.random((m, n)) >= p] = 0
    return W


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import oracle
        import sparseops_backend as sb
        orc = oracle.Oracle()

        def sharded_spmm(W, X, bias, act):
            """One row-sharded layer: local slab + in-place all-gather of padded slabs."""
            E = sb.encode_host(W)
            S = E.shard_rows(rank, world, upload=False)
            per = -(-E.m // world)
            assert S.r == E.r and S.m == max(0, min(E.m, (rank + 1) * per) - min(E.m, rank * per))
            lo = min(E.m, rank * per)
            shard = oracle.EllArrays(S.m, S.n, S.r, S.Wd, S.idx, S.nnz)
            slab = orc.spmm(shard, X, None if bias is None else bias[lo:lo + S.m], act=act)
            full = torch.zeros((per * world, X.shape[1]), dtype=torch.float32)
            full[rank * per:rank * per + S.m] = torch.from_numpy(slab)
            dist.all_gather_into_tensor(full, full[rank * per:(rank + 1) * per].clone())
            return full.numpy()[:E.m]

        rng = np.random.default_rng(99)          # same stream on every rank
        results = {}
        for m in (64, 51):                       # 51 rows: the last rank's slab is shorter
            W = _sparse(rng, m, 40, 0.3)
            X = rng.uniform(-1, 1, (40, 12)).astype(np.float32)
            b = rng.standard_normal(m).astype(np.float32)
            got = sharded_spmm(W, X, b, 0)
            want = orc.spmm(orc.encode(W), X, b)
            results[f"spmm_{m}"] = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
        # two row-sharded layers: the gathered output IS the next layer's X (feature-major)
        W1, W2 = _sparse(rng, 37, 40, 0.3), _sparse(rng, 9, 37, 0.4)
        b1 = rng.standard_normal(37).astype(np.float32)
        X = rng.uniform(0, 1, (40, 6)).astype(np.float32)
        h = sharded_spmm(W1, X, b1, 1)
        y = sharded_spmm(W2, np.ascontiguousarray(h), None, 0)
        want = orc.spmm(orc.encode(W2), orc.spmm(orc.encode(W1), X, b1, act=1), None)
        results["mlp"] = bool(np.array_equal(y.view(np.uint32), want.view(np.uint32)))
        # clustered long rows: ranges of near-equal nonzeros (balanced_row_split) instead of equal
        # row counts; slabs are padded to the longest range for the in-place all-gather and the
        # gathered buffer is compacted with the same bounds on every rank
        m, n = 90, 40
        W = _sparse(rng, m, n, 0.1)
        W[:12] = rng.standard_normal((12, n)).astype(np.float32)
        X = rng.uniform(-1, 1, (n, 5)).astype(np.float32)
        b = rng.standard_normal(m).astype(np.float32)
        E = sb.encode_host(W)
        bounds = E.balanced_row_split(world, 0)
        lo, hi = bounds[rank], bounds[rank + 1]
        S = E.shard_range(lo, hi, upload=False)
        slab_rows = max(bounds[g + 1] - bounds[g] for g in range(world))
        full = torch.zeros((slab_rows * world, X.shape[1]), dtype=torch.float32)
        shard = oracle.EllArrays(S.m, S.n, S.r, S.Wd, S.idx, S.nnz)
        full[rank * slab_rows:rank * slab_rows + S.m] = torch.from_numpy(orc.spmm(shard, X, b[lo:hi], act=0))
        dist.all_gather_into_tensor(full, full[rank * slab_rows:(rank + 1) * slab_rows].clone())
        got = np.concatenate([full.numpy()[g * slab_rows:g * slab_rows + bounds[g + 1] - bounds[g]] for g in range(world)])
        want = orc.spmm(orc.encode(W), X, b)
        nz = [int(E.nnz[bounds[g]:bounds[g + 1]].sum()) for g in range(world)]
        results["balanced"] = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32))) and \
            max(nz) <= E.nnz_total / world + int(E.nnz.max()) and bounds[1] < m // world
        # the operand layout of the sharded host-buffer SpMM: every rank places its block of X's
        # rows into a panel-major buffer (panel p = a contiguous [per * world x width] matrix), one
        # in-place all-gather per panel rebuilds X on every rank
        n, Cw, panel = 37, 20, 8
        X = rng.uniform(-1, 1, (n, Cw)).astype(np.float32)
        per = -(-n // world)
        lo, hi = min(n, rank * per), min(n, (rank + 1) * per)
        ok = True
        for c0 in range(0, Cw, panel):
            w = min(panel, Cw - c0)
            buf = torch.zeros((per * world, w), dtype=torch.float32)
            buf[lo:hi] = torch.from_numpy(X[lo:hi, c0:c0 + w])
            dist.all_gather_into_tensor(buf, buf[rank * per:(rank + 1) * per].clone())
            ok = ok and bool(np.array_equal(buf.numpy()[:n], X[:, c0:c0 + w]))
        results["x_panels"] = ok
        # the benchmark's shardable generator: two half ranges equal the whole
        import workloads as wl
        rp, col, val = wl.cfg5_rows(rank * 4096, 4096, n=2048, kmax=128, mean=12)
        cnt = torch.tensor([len(col)], dtype=torch.int64)
        dist.all_reduce(cnt)
        whole = wl.cfg5_rows(0, 8192, n=2048, kmax=128, mean=12)
        results["generator"] = int(cnt.item()) == len(whole[1])
        q.put((rank, results))
        dist.destroy_process_group()
    except Exception as ex:  # surface the failure in the parent
        q.put((rank, {"error": repr(ex)}))


def test_row_sharding_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, res in out:
        assert "error" not in res, f"rank {rank}: {res}"
        assert all(res.values()), f"rank {rank}: {res}"
