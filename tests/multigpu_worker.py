"""Worker of tests/test_multigpu.py: one process per GPU (torchrun), NCCL.  Exits non-zero on any
mismatch.  Checks, against the CPU oracle on the same seeded inputs:
  1. row-sharded SpMM with the library's own in-place all-gather (spx_allgather_rows);
  2. SparseOnnxModel in row-sharded (tensor-parallel) mode: every layer ends with an all-gather;
  3. SparseOnnxModel batch-sharded: each rank runs its own batch columns, no collective;
  4. spx_spmm_host_sharded: host buffers, each rank copies its block of X's rows, all-gather of X
     over NVLink, own rows of Y back -- one panel and several panels, n not divisible by world;
  5. a handle used while another device is current is refused with a status code (no launch)."""
import ctypes as C
import os
import sys
import tempfile

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "sparse-ops_b200")):
    sys.path.insert(0, p)

import onnx_wire  # noqa: E402
import oracle  # noqa: E402
import sparseops_backend as sb  # noqa: E402
import spx_ctypes as sx  # noqa: E402


def sparse(rng, m, n, p, scale=1.0):
    W = (rng.standard_normal((m, n)) * scale).astype(np.float32)
    W[rng.random((m, n)) >= p] = 0
    return W


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    lib = sx.Lib()
    lib.spx_set_device(local)
    sb.set_device(local)
    orc = oracle.Oracle()
    rng = np.random.default_rng(1234)            # identical stream on every rank

    # one NCCL communicator of the library, id made by rank 0
    idbuf = [sb.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(idbuf, src=0)
    comm = C.c_void_p()
    lib.spx_comm_create(rank, world, idbuf[0], C.byref(comm))

    # 1. row-sharded SpMM, m not divisible by world
    m, n, Cc = 1003, 700, 96
    W = sparse(rng, m, n, 0.1)
    X = rng.uniform(-1, 1, (n, Cc)).astype(np.float32)
    b = rng.standard_normal(m).astype(np.float32)
    E = sb.encode_host(W)
    S = E.shard_rows(rank, world, upload=False)
    per = -(-m // world)
    lo = min(m, rank * per)
    h = lib.ell_create(S.Wd, S.idx, S.nnz, n)
    dX = torch.from_numpy(X).to(dev)
    dB = torch.from_numpy(b[lo:lo + S.m].copy()).to(dev)
    dY = torch.zeros((per * world, Cc), device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    h.spmm(dX.data_ptr(), Cc, Cc, dB.data_ptr(), sx.ACT_RELU, dY[rank * per:].data_ptr(), Cc, stream)
    lib.spx_allgather_rows(comm, dY.data_ptr(), per, Cc, stream)
    torch.cuda.synchronize()
    want = orc.spmm(orc.encode(W), X, b, act=1)
    assert np.array_equal(dY.cpu().numpy()[:m].view(np.uint32), want.view(np.uint32)), "row-sharded SpMM differs"

    # 1b. the same exchange fused into the SpMM epilogue: every rank stores its rows straight into
    # all ranks' full buffers (peers' buffers opened over IPC), then a stream-ordered barrier
    buf = C.c_void_p()
    nbytes = per * world * Cc * 4
    lib.spx_malloc(C.byref(buf), nbytes)
    lib.spx_memset(buf, 0xff, nbytes, 0)
    torch.cuda.synchronize()
    handle = C.create_string_buffer(sx.IPC_HANDLE_BYTES)
    lib.spx_ipc_export(buf, handle)
    handles = [None] * world
    dist.all_gather_object(handles, handle.raw)
    ptrs, opened = [], []
    for g in range(world):
        if g == rank:
            ptrs.append(buf.value)
        else:
            pp = C.c_void_p()
            lib.spx_ipc_open(handles[g], C.byref(pp))
            ptrs.append(pp.value)
            opened.append(pp)
    dist.barrier()                                   # every buffer is initialised before anyone writes
    arr = (C.c_void_p * world)(*ptrs)
    lib.spx_spmm_bcast(h.h, dX.data_ptr(), Cc, Cc, dB.data_ptr(), sx.ACT_RELU, arr, world, rank * per, Cc, stream)
    lib.spx_comm_barrier(comm, stream)
    torch.cuda.synchronize()
    got = np.empty((per * world, Cc), np.float32)
    lib.spx_memcpy_d2h(got.ctypes.data_as(C.c_void_p), buf, nbytes, 0)
    lib.spx_device_sync()
    assert np.array_equal(got[:m].view(np.uint32), want.view(np.uint32)), "fused SpMM + all-gather differs"
    # 1c. the same fused exchange on a skewed matrix (rows of 512 and more entries, wide X): the
    # staged kernel, long rows first, the others shortest first; the exchange buffers of 1b are reused
    m2, n2 = 2 * 301, 1200
    W2 = sparse(rng, m2, n2, 0.02)
    for row, cnt in ((5, 600), (310, 1200), (601, 513)):
        W2[row] = 0
        W2[row, rng.choice(n2, cnt, replace=False)] = rng.standard_normal(cnt).astype(np.float32)
    Cw = 132                                         # > 128: the wide kernels
    X2 = rng.uniform(-1, 1, (n2, Cw)).astype(np.float32)
    b2 = rng.standard_normal(m2).astype(np.float32)
    assert m2 * Cw * 4 <= nbytes
    per2 = -(-m2 // world)
    lo2 = min(m2, rank * per2)
    S2 = sb.encode_host(W2).shard_rows(rank, world, upload=False)
    h2 = lib.ell_create(S2.Wd, S2.idx, S2.nnz, n2)
    dX2 = torch.from_numpy(X2).to(dev)
    dB2 = torch.from_numpy(b2[lo2:lo2 + S2.m].copy()).to(dev)
    dist.barrier()
    lib.spx_spmm_bcast(h2.h, dX2.data_ptr(), Cw, Cw, dB2.data_ptr(), sx.ACT_NONE, arr, world, rank * per2, Cw, stream)
    lib.spx_comm_barrier(comm, stream)
    torch.cuda.synchronize()
    got2 = np.empty((per2 * world, Cw), np.float32)
    lib.spx_memcpy_d2h(got2.ctypes.data_as(C.c_void_p), buf, got2.nbytes, 0)
    lib.spx_device_sync()
    want2 = orc.spmm(orc.encode(W2), X2, b2)
    assert np.array_equal(got2[:m2].view(np.uint32), want2.view(np.uint32)), "fused exchange on a skewed matrix differs"
    # 1e. the exchange through the copy engines (spx_spmm_exchange): slices of the rank's rows are
    # copied to the peers while the next slices are multiplied.  The skewed matrix in 3 slices, then
    # the first matrix with a leading dimension wider than C (strided copies) in 5 slices.
    lib.spx_memset(buf, 0xff, nbytes, 0)
    torch.cuda.synchronize()
    dist.barrier()
    lib.spx_spmm_exchange(h2.h, dX2.data_ptr(), Cw, Cw, dB2.data_ptr(), sx.ACT_NONE, arr, world, rank, rank * per2, Cw, 3, stream)
    lib.spx_comm_barrier(comm, stream)
    torch.cuda.synchronize()
    lib.spx_memcpy_d2h(got2.ctypes.data_as(C.c_void_p), buf, got2.nbytes, 0)
    lib.spx_device_sync()
    assert np.array_equal(got2[:m2].view(np.uint32), want2.view(np.uint32)), "copy-engine exchange on a skewed matrix differs"
    dist.barrier()
    Cn = 64                                          # narrower than the leading dimensions
    lib.spx_spmm_exchange(h.h, dX.data_ptr(), Cn, Cc, dB.data_ptr(), sx.ACT_RELU, arr, world, rank, rank * per, Cc, 5, stream)
    lib.spx_comm_barrier(comm, stream)
    torch.cuda.synchronize()
    lib.spx_memcpy_d2h(got.ctypes.data_as(C.c_void_p), buf, nbytes, 0)
    lib.spx_device_sync()
    want_n = orc.spmm(orc.encode(W), np.ascontiguousarray(X[:, :Cn]), b, act=1)
    assert np.array_equal(got[:m, :Cn].view(np.uint32), want_n.view(np.uint32)), "copy-engine exchange with ldy > C differs"
    dist.barrier()
    for pp in opened:
        lib.spx_ipc_close(pp)
    dist.barrier()
    lib.spx_free(buf)

    # 1d. the exchange through an NVLink multicast address (NVLS): the full buffers are torch
    # symmetric-memory allocations bound under one multicast address; every vector is stored once
    # (multimem.st) and the switch replicates it.  Both matrices of 1b / 1c.  Reported as skipped
    # when the rendezvous yields no multicast address on this machine.
    mc_state = "skipped"
    try:
        import torch.distributed._symmetric_memory as symm_mem
        mbuf = symm_mem.empty((per * world, Cc), dtype=torch.float32, device=dev)
        mhdl = symm_mem.rendezvous(mbuf, dist.group.WORLD.group_name)
        mc_ptr = int(mhdl.multicast_ptr or 0)
    except Exception as ex:
        mc_ptr, mbuf = 0, None
        mc_state = f"skipped ({type(ex).__name__})"
    have = torch.tensor([1.0 if mc_ptr else 0.0], device=dev)
    dist.all_reduce(have, op=dist.ReduceOp.MIN)
    if have.item() == 1.0:
        mbuf.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        lib.spx_spmm_mcast(h.h, dX.data_ptr(), Cc, Cc, dB.data_ptr(), sx.ACT_RELU, mc_ptr, rank * per, Cc, stream)
        lib.spx_comm_barrier(comm, stream)
        torch.cuda.synchronize()
        assert np.array_equal(mbuf.cpu().numpy()[:m].view(np.uint32), want.view(np.uint32)), "multicast exchange differs"
        dist.barrier()
        flat = mbuf.view(-1)
        flat.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        lib.spx_spmm_mcast(h2.h, dX2.data_ptr(), Cw, Cw, dB2.data_ptr(), sx.ACT_NONE, mc_ptr, rank * per2, Cw, stream)
        lib.spx_comm_barrier(comm, stream)
        torch.cuda.synchronize()
        gotm = flat[:per2 * world * Cw].view(per2 * world, Cw).cpu().numpy()
        assert np.array_equal(gotm[:m2].view(np.uint32), want2.view(np.uint32)), "multicast exchange on a skewed matrix differs"
        # misuse: a column count that is not a multiple of 4 is refused before any launch
        try:
            lib.spx_spmm_mcast(h.h, dX.data_ptr(), 95, Cc, dB.data_ptr(), sx.ACT_RELU, mc_ptr, rank * per, Cc, stream)
            raise AssertionError("spx_spmm_mcast accepted C = 95")
        except sx.SpxError as err:
            assert err.status == 1
        mc_state = "ok"
        torch.cuda.synchronize()
        dist.barrier()                               # no store in flight when the buffers go away
    if rank == 0:
        print(f"multicast exchange: {mc_state}")
    mbuf = None

    # 4. host buffers, sharded copy of X: several 256-column panels (ragged last one) and a single panel
    for (m4, n4, C4) in ((1003, 701, 772), (64, 50, 36)):
        W4 = sparse(rng, m4, n4, 0.1)
        X4 = rng.uniform(-1, 1, (n4, C4)).astype(np.float32)
        b4 = rng.standard_normal(m4).astype(np.float32)
        E4 = sb.encode_host(W4)
        S4 = E4.shard_rows(rank, world, upload=False)
        per4 = -(-m4 // world)
        lo4 = min(m4, rank * per4)
        h4 = lib.ell_create(S4.Wd, S4.idx, S4.nnz, n4)
        Y4 = np.full((S4.m, C4), np.nan, np.float32)
        phases = (C.c_float * 4)()
        fp = lambda a: a.ctypes.data_as(C.c_void_p)
        bl = np.ascontiguousarray(b4[lo4:lo4 + S4.m])
        lib.spx_spmm_host_sharded(comm, h4.h, fp(X4), C4, fp(bl), sx.ACT_RELU, fp(Y4), phases)
        want4 = orc.spmm(orc.encode(W4), X4, b4, act=1)[lo4:lo4 + S4.m]
        assert np.array_equal(Y4.view(np.uint32), want4.view(np.uint32)), "sharded host SpMM differs"
        assert all(t >= 0.0 for t in phases) and phases[2] > 0.0
        lib.spx_spmm_host_sharded(comm, h4.h, fp(X4), C4, None, sx.ACT_NONE, fp(Y4), None)       # second call: cached staging
        want4 = orc.spmm(orc.encode(W4), X4, None)[lo4:lo4 + S4.m]
        assert np.array_equal(Y4.view(np.uint32), want4.view(np.uint32)), "sharded host SpMM differs (no bias)"
    rk, wd = C.c_int(-1), C.c_int(-1)
    lib.spx_comm_info(comm, C.byref(rk), C.byref(wd))
    assert (rk.value, wd.value) == (rank, world)

    # 5. misuse made on the host: the handle lives on this rank's GPU, another one is current
    other = (local + 1) % torch.cuda.device_count()
    launches = lib.spx_launch_count()
    lib.spx_set_device(other)
    try:
        for call in (lambda: h.spmm(dX.data_ptr(), Cc, Cc, 0, sx.ACT_NONE, dY.data_ptr(), Cc, 0),
                     lambda: h.spmv(dX.data_ptr(), 0, dY.data_ptr(), 0)):
            try:
                call()
                raise AssertionError("a handle of another device was accepted")
            except sx.SpxError as ex:
                assert ex.status == 1
    finally:
        lib.spx_set_device(local)
    assert lib.spx_launch_count() == launches

    # 2. + 3. model: 3 layers, relu/relu/none (bit-exact end to end), out features not divisible by world
    dims, B = [64, 96, 80, 30 + world - 1], 8 * world
    Ws = [sparse(rng, dims[i + 1], dims[i], 0.3, 0.3) for i in range(3)]
    bs = [rng.standard_normal(dims[i + 1]).astype(np.float32) * 0.1 for i in range(3)]
    x = rng.uniform(0, 1, (B, dims[0])).astype(np.float32)
    x_mem = np.ascontiguousarray(x.T)
    a = x_mem
    for Wl, bl, act in zip(Ws, bs, (1, 1, 0)):
        a = orc.spmm(orc.encode(Wl), a, bl, act=act)
    f = tempfile.NamedTemporaryFile(suffix=f".r{rank}.onnx", delete=False)
    f.write(onnx_wire.mlp_model(Ws, bs, ["Relu", "Relu", None], B))
    f.close()
    tp = sb.SparseOnnxModel(f.name)
    tp.shard_rows(rank, world, idbuf2(rank, sb))
    y = tp.run(x_mem.reshape(B, -1)).ravel().reshape(-1, B)
    assert np.array_equal(y.view(np.uint32), a.view(np.uint32)), "row-sharded model differs"
    y2 = tp.run(x_mem.reshape(B, -1)).ravel().reshape(-1, B)          # second run: graph replay
    assert np.array_equal(y2.view(np.uint32), a.view(np.uint32)), "row-sharded model differs on replay"

    bsd = sb.SparseOnnxModel(f.name)
    os.unlink(f.name)
    Bl = B // world
    xl = np.ascontiguousarray(x_mem[:, rank * Bl:(rank + 1) * Bl])
    yl = bsd.run(xl.reshape(Bl, -1)).ravel().reshape(-1, Bl)
    assert np.array_equal(yl.view(np.uint32), a[:, rank * Bl:(rank + 1) * Bl].view(np.uint32)), "batch-sharded model differs"

    lib.spx_comm_destroy(comm)
    dist.barrier()
    if rank == 0:
        print(f"multigpu ok: world {world}")
    dist.destroy_process_group()


def idbuf2(rank, sb_mod):
    """A second communicator id (the model owns its communicator)."""
    buf = [sb_mod.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(buf, src=0)
    return buf[0]


if __name__ == "__main__":
    main()
