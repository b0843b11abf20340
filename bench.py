#!/usr/bin/env python
"""Benchmark of the ELLPACK hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of seeded synthetic
input.  Workloads (the five benchmark configurations):

  cfg5_spmm  (default)  skewed SpMM 262144 x 65536, power-law rows (mean 64, max 2048), C = 1024;
                        the largest single-GPU SpMM configuration.  N > 1: rows of E split over
                        the ranks, X replicated, Y stays row-sharded (strong scaling, no
                        collective in `value`); the NCCL all-gather of Y is timed separately.
  cfg1_spmm / cfg1_spmv 4096^2, p = 0.1 (C = 256 for SpMM).  Fits in L2, so the operands are
                        replicated and the launches rotate through the copies.
  cfg2_spmv             square iid matrix, --size in {4096,16384,65536}, --sparsity.
  cfg3_mlp              sparse MLP 4096-4096-4096-4096-1000, batch 256, via SparseOnnxModel
                        (N > 1: batch-sharded, no collective; --tp: row-sharded + all-gather).
  cfg4_conv             sparse 3x3 conv 256->256, 56x56, batch 32, [C,H,W,B] layout (--nchw: NCHW).
  cfg4_stack            four such layers chained, through SparseOnnxModel.

`value` is measured with operands resident in HBM; `e2e` is the same metric through the
host-buffer entry points (pinned host memory, copies inside the timed region; at N > 1 every rank
copies its block of X, the ranks rebuild X over NVLink, and each copies its own rows of Y back).
After the timed regions sampled rows of every result buffer are compared with the CPU oracle on
every rank (`check`); a mismatch makes the run fail.  The default run also carries the other
configurations under `also` (N = 1: configs 1 - 4; N > 1: the MLP batch- and row-sharded).
`--impl reference` times the reference's own CPU implementation (oracle/_ref, else the C port)
on the whole matrix per step where the host's memory holds it.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "sparse-ops_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
L2_FLUSH_BYTES = 512 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg5_spmm",
                    choices=["cfg5_spmm", "cfg1_spmm", "cfg1_spmv", "cfg2_spmv", "cfg3_mlp", "cfg4_conv", "cfg4_stack"])
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the workload (testing only)")
    ap.add_argument("--size", type=int, default=16384, help="cfg2_spmv: m = n")
    ap.add_argument("--sparsity", type=float, default=0.90, help="cfg2_spmv")
    ap.add_argument("--conv-sparsity", type=float, default=0.80, help="cfg4_conv: fraction of zero weights")
    ap.add_argument("--tp", action="store_true", help="cfg3_mlp at N > 1: row-sharded layers + all-gather")
    ap.add_argument("--batch", type=int, default=0, help="cfg3_mlp / cfg4_conv: override the batch size")
    ap.add_argument("--nchw", action="store_true", help="cfg4_conv: NCHW tensors instead of [C,H,W,B]")
    ap.add_argument("--rows", type=int, default=0, help="cfg5_spmm: override the row count (profiling on a smaller case)")
    ap.add_argument("--cols", type=int, default=0, help="cfg5_spmm: override C, the dense column count")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-also", action="store_true", help="skip the other configurations in the default run")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of the results with the CPU oracle")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# helpers
# ------------------------------------------------------------------------------------------------
def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def recorded_traffic(kernel: str, args, world: int):
    """DRAM bytes per launch from the committed ncu summary -- only where the profiled launch is the
    timed launch: the named workload at its full size on one GPU.  Anything else (a rank's shard, a
    scaled or resized case) has no measured traffic and reports null."""
    if world != 1 or args.scale != 1.0 or args.rows or args.cols or args.batch:
        return None
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            key = f"{kernel}:{args.workload}"
        if args.workload == "cfg2_spmv":
            key += f":{args.size}:{args.sparsity}"
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return json.load(f).get(key)
    except Exception:
        return None


def load_probe():
    """bench_l2_gather_probe of sparse-ops_b200/libspx_bench_probe.so (bench equipment), or None."""
    try:
        dll = ctypes.CDLL(os.path.join(PKG, "libspx_bench_probe.so"))
        fn = dll.bench_l2_gather_probe
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p,
                       ctypes.POINTER(ctypes.c_uint64)]
        return fn
    except (OSError, AttributeError):
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read only)."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
                 "hw_thermal_slowdown": 0x40, "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.005)

    def __enter__(self):
        if self._nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def _count_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# Taken once at start-up: OpenMP thread binding later narrows the main thread's affinity mask.
_HOST_CORES = _count_cores()


def host_cores():
    return _HOST_CORES


# ------------------------------------------------------------------------------------------------
# workload construction (host side, seeded)
# ------------------------------------------------------------------------------------------------
def build_workload(args, rank: int, world: int):
    """Returns a dict describing this rank's share: CSR rows, dense operands, byte/flop counts."""
    import workloads as wl
    s = args.scale
    w = args.workload
    if w == "cfg5_spmm":
        m = max(4096 * world, int(262144 * s) // (4096 * world) * 4096 * world)
        n = max(1024, int(65536 * s))
        C = max(16, int(1024 * s) // 4 * 4)
        if args.rows:
            m = max(4096 * world, args.rows // (4096 * world) * 4096 * world)
        if args.cols:
            C = args.cols
        kmax = min(2048, n // 2)
        per = m // world
        rowptr, col, val = wl.cfg5_rows(rank * per, per, n=n, kmax=kmax, mean=64.0 if kmax >= 512 else kmax / 8)
        X = wl.cfg5_dense_operand(n, C)
        return dict(kind="spmm", m=m, n=n, C=C, rows=per, row0=rank * per, csr=(rowptr, col, val), X=X, bias=None,
                    desc=f"skewed SpMM {m}x{n}, power-law rows (mean 64, max {kmax}), C={C}")
    if w in ("cfg1_spmm", "cfg1_spmv"):
        d = wl.cfg1(s)
        m = d["m"]
        per = (m + world - 1) // world
        lo, hi = min(m, rank * per), min(m, (rank + 1) * per)
        csr = wl.csr_from_blocks([(0, d["W"][lo:hi])], hi - lo)
        if w == "cfg1_spmm":
            return dict(kind="spmm", m=m, n=d["n"], C=d["C"], rows=hi - lo, row0=lo, csr=csr, X=d["X"],
                        bias=d["bias"][lo:hi].copy(),
                        desc=f"SpMM {m}x{d['n']} iid p=0.1, C={d['C']}, bias")
        return dict(kind="spmv", m=m, n=d["n"], C=1, rows=hi - lo, row0=lo, csr=csr, x=d["x"],
                    bias=d["bias"][lo:hi].copy(), desc=f"SpMV {m}x{d['n']} iid p=0.1, bias")
    if w == "cfg2_spmv":
        size = max(256, int(args.size * s))
        d = wl.cfg2_case(size, args.sparsity) if s == 1.0 else None
        if d is None:
            p = 1.0 - args.sparsity
            rp, col, val = wl.bernoulli_csr(43, size, size, p, 1.0 / np.sqrt(max(1.0, p * size)))
            g = np.random.default_rng(43)
            d = dict(m=size, n=size, rowptr=rp, col=col, val=val, x=g.uniform(-1, 1, size).astype(np.float32),
                     bias=g.standard_normal(size).astype(np.float32))
        m = d["m"]
        per = (m + world - 1) // world
        lo, hi = min(m, rank * per), min(m, (rank + 1) * per)
        rp = d["rowptr"]
        a, b = int(rp[lo]), int(rp[hi])
        csr = ((rp[lo:hi + 1] - rp[lo]).astype(np.uint64), d["col"][a:b], d["val"][a:b])
        return dict(kind="spmv", m=m, n=d["n"], C=1, rows=hi - lo, row0=lo, csr=csr, x=d["x"], bias=d["bias"][lo:hi].copy(),
                    desc=f"SpMV {m}x{m} iid sparsity {args.sparsity}, bias")
    if w == "cfg3_mlp":
        d = wl.cfg3(s, batch=args.batch or None)
        return dict(kind="mlp", **d, desc=f"sparse MLP {'-'.join(map(str, d['dims']))}, 90% sparse, batch {d['B']}")
    if w == "cfg4_conv":
        d = wl.cfg4(s, layers=1, density=1.0 - args.conv_sparsity)
        if args.batch:
            d["x_nchw"] = np.ascontiguousarray(d["x_nchw"][:args.batch])
            d["B"] = d["x_nchw"].shape[0]
        return dict(kind="conv", **d, desc=f"sparse conv {d['C']}->{d['C']} 3x3 on {d['H']}x{d['W']}, batch {d['B']}, {args.conv_sparsity:.0%} sparse, bias+ReLU, " + ("NCHW" if args.nchw else "[C,H,W,B]"))
    if w == "cfg4_stack":
        d = wl.cfg4(s, layers=4)
        return dict(kind="convstack", **d, desc=f"4 x (sparse conv {d['C']}->{d['C']} 3x3 + bias + ReLU) on {d['H']}x{d['W']}, batch {d['B']}, 80% sparse, via SparseOnnxModel, [C,H,W,B]")
    raise SystemExit(f"unknown workload {w}")


def sample_rows(rowptr, k_long=6, k_spread=26):
    """Row ids to check: the longest rows of the range and an even spread over the rest."""
    counts = np.diff(rowptr.astype(np.int64))
    m = len(counts)
    if m == 0:
        return np.zeros(0, np.int64)
    longest = np.argsort(counts, kind="stable")[::-1][:k_long]
    spread = np.linspace(0, m - 1, num=min(m, k_spread)).astype(np.int64)
    return np.unique(np.concatenate([longest, spread]))


def oracle_rows_spmm(csr, rows, n, X, bias):
    """The oracle's SpMM (one FMA per stored entry, in order, from the bias) on the given rows."""
    import oracle
    import workloads as wl
    rowptr, col, val = csr
    cnt = np.diff(rowptr.astype(np.int64))[rows]
    rp = np.zeros(len(rows) + 1, np.uint64)
    rp[1:] = np.cumsum(cnt)
    cc = np.concatenate([col[int(rowptr[i]):int(rowptr[i + 1])] for i in rows]) if len(rows) else np.zeros(0, np.uint32)
    vv = np.concatenate([val[int(rowptr[i]):int(rowptr[i + 1])] for i in rows]) if len(rows) else np.zeros(0, np.float32)
    Wd, idx, nnz = wl.csr_to_ell(len(rows), rp, cc, vv)
    E = oracle.EllArrays(len(rows), n, Wd.shape[1], Wd, idx, nnz)
    orc = oracle.Oracle()
    return E, orc, orc.spmm(E, X, None if bias is None else bias[rows])


def bits_equal(a, b) -> bool:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    return a.shape == b.shape and bool(np.array_equal(a.view(np.uint32), b.view(np.uint32)))


def config_of(args, wk, world: int, local_nnz: int):
    """The `config` object of the JSON line -- the same for the product arm and the reference arm --
    together with the L2 protocol it describes: (config, copies of the operands, flush needed)."""
    kind = wk["kind"]
    if kind == "spmm":
        working_set = (wk["n"] * wk["C"] + wk["rows"] * wk["C"]) * 4 + 8 * local_nnz
    elif kind == "spmv":
        working_set = 8 * local_nnz + 4 * wk["n"]
    elif kind == "conv":
        working_set = 2 * (wk["B"] // world) * wk["C"] * wk["H"] * wk["W"] * 4
    else:
        working_set = 64 << 20
    ncopies = rotation_copies(working_set, world) if kind in ("spmm", "spmv") else 1
    rotating = ncopies > 1
    need_flush = working_set < (256 << 20) and not rotating
    cfg = {"workload": args.workload, "desc": wk["desc"],
           "l2": (f"{ncopies} rotating copies of the operands ({ncopies * working_set >> 20} MiB > L2), launches back to back"
                  if rotating else "flushed between timed iterations (512 MiB write)" if need_flush
                  else "inputs larger than L2"),
           "sharding": "rows of E split over ranks, X replicated, Y row-sharded" if kind in ("spmm", "spmv")
           else ("row-sharded layers + all-gather" if args.tp else "batch-sharded, no collective")}
    return cfg, ncopies, need_flush


def rotation_copies(working_set: int, world: int) -> int:
    """Operands that fit L2 are replicated so that consecutive timed launches never touch the same
    copy before it has been evicted (total well above the 126 MB L2); larger operands need one copy."""
    if working_set >= (256 << 20) or world > 1:
        return 1
    return min(64, -(-(384 << 20) // max(1, working_set)) + 1)


def spmm_bytes(nnz, m, n, C, bias):
    return 8 * nnz + 4 * m + (4 * m if bias else 0) + 4 * n * C + 4 * m * C


def spmv_bytes(nnz, m, n):
    return 8 * nnz + 4 * n + 12 * m


# ------------------------------------------------------------------------------------------------
# the reference / CPU arm
# ------------------------------------------------------------------------------------------------
def cpu_engine():
    """(engine, kind): the unmodified reference build when usable here, else the C port."""
    # all host cores, also under torchrun, which presets OMP_NUM_THREADS=1 for every rank (the
    # reference reads the variable on every call)
    os.environ["OMP_NUM_THREADS"] = str(host_cores())
    os.environ.setdefault("OMP_PLACES", "cores")
    os.environ.setdefault("OMP_PROC_BIND", "spread")
    import oracle
    if oracle.reference_available():
        try:
            return oracle.Reference(), "reference"
        except Exception:
            pass
    return oracle.Oracle(), "port"


def host_memory_available() -> int:
    try:
        import psutil
        return int(psutil.virtual_memory().available)
    except Exception:
        return 8 << 30


def cpu_sample_runner(args, wk, fraction=None):
    """Builds the bounded CPU sample of this workload.  Returns (run_fn, work_fraction, kind, text).

    fraction (SpMM / SpMV): share of the matrix's nonzeros the sample should hold, taken as its
    first rows; None = about 4 GFLOP of work (a stable timing in well under a second).  1.0 runs the
    whole matrix.  The share is cut down to what the host's free memory holds (the reference keeps
    three padded m x r arrays: Wd, idx and its Xt scratch, next to the two this script builds)."""
    import oracle
    import workloads as wl
    eng, kind = cpu_engine()
    is_ref = kind == "reference"

    def make_ell(rowptr, col, val, m, n):
        Wd, idx, nnz = wl.csr_to_ell(m, rowptr, col, val)
        E = oracle.EllArrays(m, n, Wd.shape[1], Wd, idx, nnz)
        return eng.from_arrays(E) if is_ref else E

    if wk["kind"] in ("spmm", "spmv"):
        rowptr, col, val = wk["csr"]
        rows = wk["rows"]
        total_nnz = int(rowptr[-1])
        take = rows
        if fraction is None:
            if wk["kind"] == "spmm":
                # about 4 GFLOP of the same matrix: enough for a stable CPU timing, seconds not minutes
                target = 4e9 / (2.0 * wk["C"])
                if total_nnz > target:
                    take = max(1, int(np.searchsorted(rowptr, target)))
            elif total_nnz > 64e6:                  # SpMV: at most 64 M nonzeros (0.5 GB of matrix)
                take = max(1, int(np.searchsorted(rowptr, 64e6)))
        elif fraction < 1.0:
            take = max(1, int(np.searchsorted(rowptr, fraction * total_nnz)))
        take = min(take, rows)
        r_max = int(np.diff(rowptr[:take + 1].astype(np.int64)).max()) if take else 0
        budget = host_memory_available() // 2
        per_row = max(1, r_max) * 4 * 5 + wk["C"] * 4
        if take * per_row > budget:
            take = max(1, budget // per_row)
        sub = (rowptr[:take + 1].copy(), col[:int(rowptr[take])], val[:int(rowptr[take])])
        E = make_ell(*sub, take, wk["n"])
        frac = float(rowptr[take]) / max(1, total_nnz)
        bias = None if wk["bias"] is None else wk["bias"][:take].copy()
        if wk["kind"] == "spmm":
            X = wk["X"]
            Y = np.empty((take, wk["C"]), np.float32)
            run = (lambda: eng.matmul(E, X, bias, out=Y)) if is_ref else (lambda: eng.spmm(E, X, bias))
        else:
            x = wk["x"]
            y = np.empty(take, np.float32)
            run = (lambda: eng.matvec(E, x, bias, out=y)) if is_ref else (lambda: eng.spmv(E, x, bias))
        what = "the whole matrix" if take == rows else f"rows 0..{take - 1} of {rows} of the same matrix ({frac:.3f} of the nonzeros)"
        return run, frac, kind, what + ", full dense operand"
    if wk["kind"] == "mlp":
        import onnx_wire
        import tempfile
        B = wk["B"]
        x_mem = np.ascontiguousarray(wk["x"].T)
        if is_ref:
            f = tempfile.NamedTemporaryFile(suffix=".onnx", delete=False)
            f.write(onnx_wire.mlp_model(wk["weights"], wk["biases"], wk["acts"], B))
            f.close()
            h = eng.model_load(f.name)
            os.unlink(f.name)
            return (lambda: eng.model_run(h, x_mem, B)), 1.0, kind, "the whole forward pass (SparseOnnxModel::run of the reference)"
        Es = [eng.encode(W) for W in wk["weights"]]

        def run():
            a = x_mem
            for E, b, act in zip(Es, wk["biases"], (1, 1, 1, 2)):
                a = eng.spmm(E, a, b, act=1) if act == 1 else eng.activation(eng.spmm(E, a, b), act)
            return a
        return run, 1.0, kind, "the whole forward pass (layer loop over the C port)"
    if wk["kind"] == "conv":
        B, Cc, H, W = wk["B"], wk["C"], wk["H"], wk["W"]
        Bs = max(1, min(B, 4))      # a few images of the batch: the explicit-im2col CPU path is slow
        g = dict(Cin=Cc, kH=3, kW=3, sH=1, sW=1, pH=1, pW=1, dH=1, dW=1, H=H, W=W)
        x_pf = np.ascontiguousarray(wk["x_nchw"][:Bs].transpose(1, 2, 3, 0))
        if is_ref:
            h = eng.conv_create(wk["weights"][0], g, wk["biases"][0], True)
            out = np.empty((Cc, H, W, Bs), np.float32)
            return (lambda: eng.conv_run(h, 0, x_pf, Bs, Cc, out=out)), Bs / B, kind, \
                f"{Bs} of {B} images, conv2d_patchmajor_tiled of the reference"
        E = eng.encode(wk["weights"][0].reshape(Cc, -1))
        return (lambda: eng.conv2d(E, g, 0, x_pf, Bs, wk["biases"][0], 1)), Bs / B, kind, f"{Bs} of {B} images, C port"
    if wk["kind"] == "convstack":
        import onnx_wire
        import tempfile
        B, Cc, H, W = wk["B"], wk["C"], wk["H"], wk["W"]
        Bs = max(1, min(B, 2))
        x_pf = np.ascontiguousarray(wk["x_nchw"][:Bs].transpose(1, 2, 3, 0))
        if is_ref:
            f = tempfile.NamedTemporaryFile(suffix=".onnx", delete=False)
            f.write(onnx_wire.conv_model(wk["weights"], wk["biases"], [True] * len(wk["weights"]), Bs, H, W))
            f.close()
            h = eng.model_load(f.name)
            os.unlink(f.name)
            return (lambda: eng.model_run(h, x_pf, Bs)), Bs / B, kind, f"{Bs} of {B} images, SparseOnnxModel::run of the reference"
        g = dict(Cin=Cc, kH=3, kW=3, sH=1, sW=1, pH=1, pW=1, dH=1, dW=1, H=H, W=W)
        Es = [eng.encode(w.reshape(Cc, -1)) for w in wk["weights"]]

        def run():
            a = x_pf
            for E, b in zip(Es, wk["biases"]):
                a = eng.conv2d(E, g, 0, a, Bs, b, 1)
            return a
        return run, Bs / B, kind, f"{Bs} of {B} images, C port"
    raise SystemExit("no CPU sample for this workload")


def time_cpu(run, repeats, warmup=1, budget_s=25.0):
    """Median wall time of `repeats` runs after `warmup` untimed ones; both are cut short when the
    budget (seconds, warm-up included) runs out, so the leg always ends."""
    t_start = time.perf_counter()
    done_warm = 0
    for _ in range(warmup):
        run()
        done_warm += 1
        if time.perf_counter() - t_start > budget_s / 3:
            break
    ts = []
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        run()
        ts.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    return float(np.median(ts)), len(ts), done_warm


def metric_of(wk, args):
    return {"spmm": ("spmm_effective_hbm_gbs", "GB/s"), "spmv": ("spmv_effective_hbm_gbs", "GB/s"),
            "mlp": ("sparse_mlp_samples_per_s", "samples/s"), "conv": ("conv_effective_hbm_gbs", "GB/s"),
            "convstack": ("conv_effective_hbm_gbs", "GB/s")}[wk["kind"]]


def job_bytes_flops(wk, nnz_total):
    """Algorithmic bytes and flops of the WHOLE job (all ranks), one step."""
    k = wk["kind"]
    if k == "spmm":
        return spmm_bytes(nnz_total, wk["m"], wk["n"], wk["C"], wk["bias"] is not None), 2.0 * nnz_total * wk["C"]
    if k == "spmv":
        return spmv_bytes(nnz_total, wk["m"], wk["n"]), 2.0 * nnz_total
    if k == "mlp":
        B = wk["B"]
        by, fl = 0, 0.0
        for W in wk["weights"]:
            z = int(np.count_nonzero(W))
            by += 8 * z + 8 * W.shape[0] + 4 * B * (W.shape[0] + W.shape[1])
            fl += 2.0 * z * B
        return by, fl
    if k == "conv":
        z = int(np.count_nonzero(wk["weights"][0]))
        cols = wk["B"] * wk["H"] * wk["W"]
        return 4 * cols * 2 * wk["C"] + 8 * z + 8 * wk["C"], 2.0 * z * cols
    if k == "convstack":
        cols = wk["B"] * wk["H"] * wk["W"]
        by, fl = 0, 0.0
        for w_ in wk["weights"]:
            z = int(np.count_nonzero(w_))
            by += 4 * cols * 2 * wk["C"] + 8 * z + 8 * wk["C"]
            fl += 2.0 * z * cols
        return by, fl
    raise SystemExit(k)


def to_value(wk, job_bytes, seconds):
    if wk["kind"] == "mlp":
        return wk["B"] / seconds
    return job_bytes / seconds / 1e9


# ------------------------------------------------------------------------------------------------
def run_reference_arm(args):
    """The reference's own CPU implementation on the host cores.  SpMM / SpMV run the WHOLE matrix
    per step where the host's memory holds the reference's padded arrays (config 5: about 11 GB),
    otherwise the largest share that fits, scaled by its share of the nonzeros and labelled so."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wk = build_workload(args, 0, 1)
    nnz_total = int(wk["csr"][0][-1]) if "csr" in wk else 0
    job_bytes, job_flops = job_bytes_flops(wk, nnz_total)
    run, frac, kind, sample = cpu_sample_runner(args, wk, fraction=1.0)
    med, reps, warm = time_cpu(run, args.steps, warmup=args.warmup, budget_s=240.0)
    sec_full = med / frac
    metric, unit = metric_of(wk, args)
    value = to_value(wk, job_bytes, sec_full)
    cores = host_cores()
    scaled = "" if frac == 1.0 else f", scaled by 1/{frac:.4f} to the whole job"
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": reps,
        "warmup": warm, "ms_per_step": sec_full * 1e3, "measured_ms_per_sample": med * 1e3, "sample_fraction": frac,
        "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_of(args, wk, 1, nnz_total)[0],
        "gflops": job_flops / sec_full / 1e9,
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": kind,
                         "sample": sample + f"; median of {reps} runs of {med * 1e3:.2f} ms" + scaled},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
class Ctx:
    """Process-wide state of the product arm: device, library handle, rank layout."""


def setup_ours(args):
    import torch
    import torch.distributed as dist

    import spx_ctypes as sx

    c = Ctx()
    c.torch, c.dist, c.sx = torch, dist, sx
    c.world = int(os.environ.get("WORLD_SIZE", "1"))
    c.rank = int(os.environ.get("RANK", "0"))
    c.local = int(os.environ.get("LOCAL_RANK", "0"))
    if c.world != args.gpus and c.world > 1:
        args.gpus = c.world
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(c.local)
    c.dev = torch.device("cuda", c.local)
    if c.world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=c.dev)
    c.lib = sx.Lib()
    c.lib.spx_set_device(c.local)
    c.stream = torch.cuda.current_stream().cuda_stream
    return c


def measure(args, c):
    """Runs one workload; returns the JSON line as a dict on rank 0 (None elsewhere)."""
    torch, dist, sx = c.torch, c.dist, c.sx
    world, rank, local, dev, lib, stream = c.world, c.rank, c.local, c.dev, c.lib, c.stream

    wk = build_workload(args, rank, world)
    kind = wk["kind"]
    flush_buf = None
    h2d = d2h = 0
    e2e_step = None
    ag_step = None
    fused_step = None
    mcast_step, mcast_note, mbuf = None, None, None
    exchange_step, xslices = None, 0
    e2e_phases = None
    checks = []                 # (what, rows compared, ok) filled by run_checks after the timed regions
    run_checks = None

    if kind in ("spmm", "spmv"):
        rowptr, col, val = wk["csr"]
        ell = lib.ell_create_csr(wk["rows"], wk["n"], rowptr, col, val)
        local_nnz = torch.tensor([ell.nnz_total], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(local_nnz)
        nnz_total = int(local_nnz.item())
        dB = None if wk["bias"] is None else torch.from_numpy(wk["bias"]).to(dev)
        if kind == "spmm":
            C = wk["C"]
            dX = torch.from_numpy(wk["X"]).to(dev)
            dY = torch.empty((wk["rows"], C), device=dev, dtype=torch.float32)
            config, ncopies, need_flush = config_of(args, wk, world, ell.nnz_total)
            ells = [ell] + [lib.ell_create_csr(wk["rows"], wk["n"], rowptr, col, val) for _ in range(ncopies - 1)]
            dXs = [dX] + [dX.clone() for _ in range(ncopies - 1)]
            dYs = [dY] + [torch.empty_like(dY) for _ in range(ncopies - 1)]
            rot = [0]

            def step():
                i = rot[0] = (rot[0] + 1) % ncopies
                ells[i].spmm(dXs[i].data_ptr(), C, C, 0 if dB is None else dB.data_ptr(), sx.ACT_NONE, dYs[i].data_ptr(), C, stream)
            hX = torch.from_numpy(wk["X"]).pin_memory()
            hY = torch.empty((wk["rows"], C), dtype=torch.float32).pin_memory()
            hB = None if wk["bias"] is None else torch.from_numpy(wk["bias"]).pin_memory()
            d2h = hY.numel() * 4
            rows_lo = wk["row0"]

            def check_rows_against_oracle(Ydev_rows, local_rows, what):
                """Ydev_rows: device tensor whose row i is the output row local_rows[i] of this rank."""
                _, _, want = oracle_rows_spmm(wk["csr"], local_rows, wk["n"], wk["X"], wk["bias"])
                ok = bits_equal(Ydev_rows.cpu().numpy(), want)
                checks.append((what, len(local_rows), ok))
            if not args.no_check:
                picked = sample_rows(rowptr)
                pick_dev = torch.from_numpy(picked).to(dev)
            if world == 1:
                h2d = hX.numel() * 4 + (0 if hB is None else hB.numel() * 4)

                def e2e_step():
                    lib.spx_spmm_host(ell.h, hX.data_ptr(), C, 0 if hB is None else hB.data_ptr(), sx.ACT_NONE, hY.data_ptr())
            else:
                import ctypes as Ct
                idb = [None]
                if rank == 0:
                    ub = Ct.create_string_buffer(sx.UNIQUE_ID_BYTES)
                    lib.spx_comm_unique_id(ub)
                    idb = [ub.raw]
                dist.broadcast_object_list(idb, src=0)
                fcomm = Ct.c_void_p()
                lib.spx_comm_create(rank, world, idb[0], Ct.byref(fcomm))
                # end to end on host buffers: every rank copies its block of X's rows over PCIe, the
                # ranks rebuild X over NVLink, multiply, and copy their own rows of Y back
                per_x = -(-wk["n"] // world)
                h2d = max(0, min(wk["n"], (rank + 1) * per_x) - min(wk["n"], rank * per_x)) * C * 4 + (0 if hB is None else hB.numel() * 4)
                e2e_phases = (Ct.c_float * 4)()

                def e2e_step():
                    lib.spx_spmm_host_sharded(fcomm, ell.h, hX.data_ptr(), C, 0 if hB is None else hB.data_ptr(), sx.ACT_NONE,
                                              hY.data_ptr(), e2e_phases)
                Yfull = torch.empty((wk["m"], C), device=dev, dtype=torch.float32)
                Yslab = Yfull[wk["row0"]:wk["row0"] + wk["rows"]]

                def ag_step():
                    ell.spmm(dX.data_ptr(), C, C, 0 if dB is None else dB.data_ptr(), sx.ACT_NONE, Yslab.data_ptr(), C, stream)
                    lib.spx_allgather_rows(fcomm, Yfull.data_ptr(), wk["rows"], C, stream)
                # the same exchange fused into the epilogue: stores into every rank's full buffer
                # (own + peers' buffers opened over IPC), followed by a stream-ordered barrier
                fbuf = Ct.c_void_p()
                lib.spx_malloc(Ct.byref(fbuf), wk["m"] * C * 4)
                hnd = Ct.create_string_buffer(sx.IPC_HANDLE_BYTES)
                lib.spx_ipc_export(fbuf, hnd)
                hs = [None] * world
                dist.all_gather_object(hs, hnd.raw)
                plist = []
                for g_ in range(world):
                    if g_ == rank:
                        plist.append(fbuf.value)
                    else:
                        pp = Ct.c_void_p()
                        lib.spx_ipc_open(hs[g_], Ct.byref(pp))
                        plist.append(pp.value)
                parr = (Ct.c_void_p * world)(*plist)

                def fused_step():
                    lib.spx_spmm_bcast(ell.h, dX.data_ptr(), C, C, 0 if dB is None else dB.data_ptr(), sx.ACT_NONE, parr, world,
                                       wk["row0"], C, stream)
                    lib.spx_comm_barrier(fcomm, stream)
                # the exchange through the copy engines: slices of the rank's rows go to the peers by
                # asynchronous device-to-device copies while the next slices are multiplied
                xslices = int(os.environ.get("SPX_BENCH_EXCHANGE_SLICES", "4"))

                def exchange_step():
                    lib.spx_spmm_exchange(ell.h, dX.data_ptr(), C, C, 0 if dB is None else dB.data_ptr(), sx.ACT_NONE, parr, world,
                                          rank, wk["row0"], C, xslices, stream)
                    lib.spx_comm_barrier(fcomm, stream)
                # and through an NVLink multicast address (NVLS): the ranks' full buffers are one
                # torch symmetric-memory allocation each, bound under one multicast address by the
                # rendezvous; the epilogue stores every vector once (spx_spmm_mcast, multimem.st)
                try:
                    if os.environ.get("SPX_BENCH_NO_MCAST") == "1":
                        raise RuntimeError("switched off by SPX_BENCH_NO_MCAST")
                    import torch.distributed._symmetric_memory as symm_mem
                    mbuf = symm_mem.empty((wk["m"], C), dtype=torch.float32, device=dev)
                    mhdl = symm_mem.rendezvous(mbuf, dist.group.WORLD.group_name)
                    mc_ptr = int(mhdl.multicast_ptr or 0)
                    if not mc_ptr:
                        mcast_note = "the symmetric-memory rendezvous gave no multicast address"
                except Exception as ex:
                    mc_ptr, mbuf = 0, None
                    mcast_note = f"symmetric memory unavailable: {type(ex).__name__}: {ex}"[:200]
                # every rank takes part in this reduction whatever happened above, and all take the same branch after it
                all_mc = torch.tensor([1.0 if mc_ptr else 0.0], dtype=torch.float64, device=dev)
                dist.all_reduce(all_mc, op=dist.ReduceOp.MIN)
                if all_mc.item() != 1.0:
                    mc_ptr = 0
                    mcast_note = mcast_note or "no multicast address on another rank"
                if mc_ptr:
                    def mcast_step():
                        lib.spx_spmm_mcast(ell.h, dX.data_ptr(), C, C, 0 if dB is None else dB.data_ptr(), sx.ACT_NONE, mc_ptr,
                                           wk["row0"], C, stream)
                        lib.spx_comm_barrier(fcomm, stream)

            def run_checks():
                """After the timed regions: sampled rows of every result buffer against the oracle.
                Gathered buffers are also checked on rows another rank computed."""
                if args.no_check:
                    return
                torch.cuda.synchronize()
                check_rows_against_oracle(dYs[rot[0]][pick_dev], picked, "device-resident Y")
                if e2e_step is not None and not args.no_e2e:
                    check_rows_against_oracle(hY[torch.from_numpy(picked)], picked, "host-buffer Y")
                if world > 1:
                    import workloads as wl
                    nb = (rank + 1) % world                       # a block of the neighbour's rows
                    rp2, c2, v2 = wl.cfg5_rows(nb * wk["rows"], 4096, n=wk["n"], kmax=min(2048, wk["n"] // 2)) \
                        if args.workload == "cfg5_spmm" else (None, None, None)
                    views = [("NCCL-gathered Y", Yfull)]

                    def shared_buffer_copy():
                        v = torch.empty((wk["m"], C), device=dev, dtype=torch.float32)
                        lib.spx_memcpy_d2d(v.data_ptr(), fbuf, wk["m"] * C * 4, stream)
                        torch.cuda.synchronize()
                        return v
                    # the shared buffers hold what the last timed exchange wrote: the copy-engine one;
                    # then they are overwritten with NaN patterns and the fused exchange runs once more
                    views.append(("copy-engine-exchange Y", shared_buffer_copy()))
                    dist.barrier()
                    lib.spx_memset(fbuf, 0xff, wk["m"] * C * 4, stream)
                    torch.cuda.synchronize()
                    dist.barrier()
                    fused_step()
                    views.append(("fused-exchange Y", shared_buffer_copy()))
                    if mcast_step is not None:
                        views.append(("multicast-exchange Y", mbuf))
                    torch.cuda.synchronize()
                    for name, buf in views:
                        check_rows_against_oracle(buf[rows_lo + pick_dev], picked, name + ", own rows")
                        if rp2 is not None:
                            far = sample_rows(rp2, 3, 9)
                            _, _, want = oracle_rows_spmm((rp2, c2, v2), far, wk["n"], wk["X"], None)
                            got = buf[nb * wk["rows"] + torch.from_numpy(far).to(dev)].cpu().numpy()
                            checks.append((name + ", a neighbour's rows", len(far), bits_equal(got, want)))
        else:
            dx = torch.from_numpy(wk["x"]).to(dev)
            dy = torch.empty(wk["rows"], device=dev, dtype=torch.float32)
            config, ncopies, need_flush = config_of(args, wk, world, ell.nnz_total)
            ells = [ell] + [lib.ell_create_csr(wk["rows"], wk["n"], rowptr, col, val) for _ in range(ncopies - 1)]
            dxs = [dx] + [dx.clone() for _ in range(ncopies - 1)]
            dys = [dy] + [torch.empty_like(dy) for _ in range(ncopies - 1)]
            rot = [0]

            def step():
                i = rot[0] = (rot[0] + 1) % ncopies
                ells[i].spmv(dxs[i].data_ptr(), 0 if dB is None else dB.data_ptr(), dys[i].data_ptr(), stream)
            hx = torch.from_numpy(wk["x"]).pin_memory()
            hy = torch.empty(wk["rows"], dtype=torch.float32).pin_memory()
            hB = None if wk["bias"] is None else torch.from_numpy(wk["bias"]).pin_memory()
            h2d = hx.numel() * 4 + (0 if hB is None else hB.numel() * 4)
            d2h = hy.numel() * 4

            def e2e_step():
                lib.spx_spmv_host(ell.h, hx.data_ptr(), 0 if hB is None else hB.data_ptr(), hy.data_ptr())

            def run_checks():
                """Sampled rows against the oracle's SpMV, within 1e-5 * (sum |w||x| + |bias|) per element
                (the summation order differs from the reference's)."""
                if args.no_check:
                    return
                torch.cuda.synchronize()
                picked = sample_rows(rowptr)
                E, orc, _ = oracle_rows_spmm(wk["csr"], picked, wk["n"], wk["x"][:, None], wk["bias"])
                bsub = None if wk["bias"] is None else wk["bias"][picked]
                want, bound = orc.spmv(E, wk["x"], bsub), orc.absbound(E, wk["x"], bsub)
                outs = [("device-resident y", dys[rot[0]].cpu().numpy())]
                if not args.no_e2e:
                    outs.append(("host-buffer y", hy.numpy()))
                for name, y in outs:
                    checks.append((name, len(picked), bool((np.abs(y[picked] - want) <= 1e-5 * bound + 1e-30).all())))
        kernel_name = "spmm" if kind == "spmm" else "spmv"
    elif kind == "mlp":
        import tempfile

        import onnx_wire
        import sparseops_backend as sb
        sb.set_device(local)
        B = wk["B"]
        f = tempfile.NamedTemporaryFile(suffix=".onnx", delete=False)
        f.write(onnx_wire.mlp_model(wk["weights"], wk["biases"], wk["acts"], B))
        f.close()
        model = sb.SparseOnnxModel(f.name)
        os.unlink(f.name)
        nnz_total = 0
        x_mem = np.ascontiguousarray(wk["x"].T)                  # [features][B]
        if world > 1 and args.tp:
            idbuf = [sb.comm_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(idbuf, src=0)
            model.shard_rows(rank, world, idbuf[0])
            Bl, xl = B, x_mem
        else:
            Bl = B // world
            xl = np.ascontiguousarray(x_mem[:, rank * Bl:(rank + 1) * Bl])
        model.resize_buffers(Bl)
        # operands resident in the model's own device buffers; one step = one replay of the captured loop
        dX = torch.from_numpy(xl).to(dev)
        lib.spx_memcpy_d2d(model.device_input_ptr(), dX.data_ptr(), dX.numel() * 4, stream)
        torch.cuda.synchronize()

        def step():
            model.run_resident(stream)
        hX = torch.from_numpy(xl).pin_memory()
        h2d, d2h = hX.numel() * 4, model.out_features * Bl * 4

        e2e_out = [None]

        def e2e_step():
            e2e_out[0] = model.run(hX.numpy().reshape(Bl, -1))

        def run_checks():
            """The whole forward pass against the oracle's layer loop on this rank's batch columns:
            identical chains up to the last layer, whose sigmoid may differ by a few ulp."""
            if args.no_check:
                return
            import oracle
            orc = oracle.Oracle()
            cols = min(Bl, 16)                      # the oracle is scalar C: a few batch columns suffice
            a = np.ascontiguousarray(xl[:, :cols])
            for W_, b_, act in zip(wk["weights"], wk["biases"], wk["acts"]):
                code = {"Relu": 1, "Sigmoid": 2, "Tanh": 3, None: 0}[act]
                a = orc.spmm(orc.encode(W_), a, b_, act=code)
            torch.cuda.synchronize()
            got = np.empty((model.out_features, Bl), np.float32)
            lib.spx_memcpy_d2h(got.ctypes.data_as(ctypes.c_void_p), model.device_output_ptr(), got.nbytes, stream)
            torch.cuda.synchronize()
            checks.append(("device-resident output", cols, bool(np.abs(got[:, :cols] - a).max() <= 1e-6)))
            if e2e_out[0] is not None:
                y = np.asarray(e2e_out[0]).ravel().reshape(model.out_features, Bl)
                checks.append(("host-buffer output", cols, bool(np.abs(y[:, :cols] - a).max() <= 1e-6)))
        kernel_name = "spmm"
    elif kind == "convstack":
        import tempfile

        import onnx_wire
        import sparseops_backend as sb
        sb.set_device(local)
        B, Cc, H, W = wk["B"], wk["C"], wk["H"], wk["W"]
        Bl = B // world
        f = tempfile.NamedTemporaryFile(suffix=".onnx", delete=False)
        f.write(onnx_wire.conv_model(wk["weights"], wk["biases"], [True] * len(wk["weights"]), Bl, H, W))
        f.close()
        model = sb.SparseOnnxModel(f.name)
        os.unlink(f.name)
        nnz_total = 0
        x_pf = np.ascontiguousarray(wk["x_nchw"][rank * Bl:(rank + 1) * Bl].transpose(1, 2, 3, 0))
        model.resize_buffers(Bl)
        dX = torch.from_numpy(x_pf).to(dev)
        lib.spx_memcpy_d2d(model.device_input_ptr(), dX.data_ptr(), dX.numel() * 4, stream)
        torch.cuda.synchronize()

        def step():
            model.run_resident(stream)
        hX = torch.from_numpy(x_pf).pin_memory()
        h2d, d2h = hX.numel() * 4, model.out_features * Bl * 4

        def e2e_step():
            model.run(hX.numpy().reshape(Bl, Cc, H, W))
        kernel_name = "conv"
    elif kind == "conv":
        B, Cc, H, W = wk["B"], wk["C"], wk["H"], wk["W"]
        import sparseops_backend as sb
        sb.set_device(local)
        Eh = sb.encode_host(wk["weights"][0].reshape(Cc, -1))
        ell = lib.ell_create(Eh.Wd, Eh.idx, Eh.nnz, Eh.n)
        nnz_total = 0
        Bl = B // world
        layout = sx.LAYOUT_NCHW if args.nchw else sx.LAYOUT_PF
        xs = wk["x_nchw"][rank * Bl:(rank + 1) * Bl]
        x_in = np.ascontiguousarray(xs if args.nchw else xs.transpose(1, 2, 3, 0))
        g = sx.conv_geom(Cc, Cc, 3, 3, H, W, pH=1, pW=1)
        dX = torch.from_numpy(x_in).to(dev)
        dB = torch.from_numpy(wk["biases"][0]).to(dev)
        oshape = (Bl, Cc, H, W) if args.nchw else (Cc, H, W, Bl)
        dY = torch.empty(oshape, device=dev, dtype=torch.float32)

        def step():
            ell.conv2d(g, layout, dX.data_ptr(), Bl, dB.data_ptr(), sx.ACT_RELU, dY.data_ptr(), stream)
        hX = torch.from_numpy(x_in).pin_memory()
        hY = torch.empty(oshape, dtype=torch.float32).pin_memory()
        h2d, d2h = hX.numel() * 4, hY.numel() * 4

        def e2e_step():
            dX.copy_(hX, non_blocking=True)
            ell.conv2d(g, layout, dX.data_ptr(), Bl, dB.data_ptr(), sx.ACT_RELU, dY.data_ptr(), stream)
            hY.copy_(dY, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        def run_checks():
            """Six output channels on up to four images against the oracle, bit for bit."""
            if args.no_check:
                return
            import oracle
            orc = oracle.Oracle()
            torch.cuda.synchronize()
            got = dY.cpu().numpy()
            got_pf = got if not args.nchw else got.transpose(1, 2, 3, 0)
            rows = sorted(set(int(v) for v in np.linspace(0, Cc - 1, 6)))
            nb = min(Bl, 4)
            sub = oracle.EllArrays(len(rows), Eh.n, Eh.r, Eh.Wd[rows], Eh.idx[rows], Eh.nnz[rows])
            gd = dict(Cin=Cc, kH=3, kW=3, sH=1, sW=1, pH=1, pW=1, dH=1, dW=1, H=H, W=W)
            x_pf = np.ascontiguousarray(xs[:nb].transpose(1, 2, 3, 0))
            want = orc.conv2d(sub, gd, 0, x_pf, nb, wk["biases"][0][rows], 1)
            checks.append(("device-resident output", len(rows) * nb, bits_equal(got_pf[rows][..., :nb], want)))
        kernel_name = "conv"

    job_bytes, job_flops = job_bytes_flops(wk, nnz_total)
    if kind not in ("spmm", "spmv"):
        config, ncopies, need_flush = config_of(args, wk, world, 0)
    if need_flush:
        flush_buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    counted = {"launches": 0}

    def timed(fn, steps, warmup, flush):
        """Device time of `steps` calls (CUDA events on the launching stream), seconds."""
        for _ in range(warmup):
            fn()
        barrier()
        launches0 = lib.spx_launch_count()
        if flush:
            evs = []
            for _ in range(steps):
                flush_buf.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                evs.append((e0, e1))
            barrier()
            total = sum(a.elapsed_time(b) for a, b in evs) / 1e3
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            barrier()
            total = e0.elapsed_time(e1) / 1e3
        counted["launches"] = lib.spx_launch_count() - launches0
        t = torch.tensor([total], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warm = max(3, args.warmup)
    with ClockSampler(local) as clocks:
        total = timed(step, args.steps, warm, need_flush)
        launches = counted["launches"]
    sec = total / args.steps
    launches_per_step = launches // max(1, args.steps)

    e2e = None
    if not args.no_e2e and e2e_step is not None:
        def e2e_wall(steps, warmup):
            for _ in range(warmup):
                e2e_step()
            barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                e2e_step()          # synchronous: returns after the device->host copy has landed
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            t = torch.tensor([dt], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item()) / steps
        e2e_steps = max(3, min(args.steps, 10))
        e2e_sec = e2e_wall(e2e_steps, 2)
        e2e = {"value": to_value(wk, job_bytes, e2e_sec), "unit": metric_of(wk, args)[1], "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_sec * 1e3, "steps": e2e_steps,
               "timing": "host wall clock around synchronous host-buffer calls, max over ranks"}
        if e2e_phases is not None:
            e2e["phases_ms_rank0"] = {k: round(float(v), 4) for k, v in zip(("h2d_own_rows_of_X", "allgather_X_nvlink", "spmm", "d2h_own_rows_of_Y"), e2e_phases)}
            e2e["path"] = "spx_spmm_host_sharded: 256-column panels pipelined over four streams; stage times overlap"

    ag = None
    if ag_step is not None:
        ag_total = timed(ag_step, max(3, min(args.steps, 10)), 2, False)
        ag_sec = ag_total / max(3, min(args.steps, 10))
        ag = {"ms_per_step": ag_sec * 1e3, "value": to_value(wk, job_bytes, ag_sec),
              "note": "SpMM + in-place NCCL all-gather of Y into every rank's full buffer (spx_allgather_rows)"}

    fused = None
    if fused_step is not None:
        n_f = max(3, min(args.steps, 10))
        f_sec = timed(fused_step, n_f, 2, False) / n_f
        fused = {"ms_per_step": f_sec * 1e3, "value": to_value(wk, job_bytes, f_sec),
                 "note": "SpMM whose epilogue stores Y into every rank's full buffer over NVLink (peer stores) + barrier"}

    mcast = None
    if mcast_step is not None:
        n_f = max(3, min(args.steps, 10))
        m_sec = timed(mcast_step, n_f, 2, False) / n_f
        mcast = {"ms_per_step": m_sec * 1e3, "value": to_value(wk, job_bytes, m_sec),
                 "note": "SpMM whose epilogue stores Y once to an NVLink multicast address (multimem.st, replicated into "
                         "every rank's full buffer by the NVSwitch) + barrier"}
    elif mcast_note:
        mcast = {"unavailable": mcast_note}

    check = None
    if run_checks is not None and not args.no_check:
        run_checks()
        ok_all = torch.tensor([1.0 if all(c[2] for c in checks) else 0.0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
        passed = bool(ok_all.item() == 1.0)
        exact = kind in ("spmm", "conv")
        check = {"rows": int(sum(c[1] for c in checks)), "bit_exact" if exact else "within_tolerance": passed,
                 "against": "CPU oracle (oracle/ellpack_oracle.c) on sampled rows of every result buffer, all ranks",
                 "buffers": [c[0] for c in checks], "failed": [c[0] for c in checks if not c[2]]}
        if not exact:
            check["tolerance"] = "1e-5 * (sum|w||x| + |bias|) per element" if kind == "spmv" else "1e-6 absolute on sigmoid outputs (chains before it are bit-identical)"

    xchg = None
    if exchange_step is not None:
        n_f = max(3, min(args.steps, 10))
        x_sec = timed(exchange_step, n_f, 2, False) / n_f
        xchg = {"ms_per_step": x_sec * 1e3, "value": to_value(wk, job_bytes, x_sec), "slices": xslices,
                "note": "SpMM in row slices, each slice copied into every rank's full buffer by the copy engines over NVLink "
                        "while the next slices are multiplied (spx_spmm_exchange) + barrier"}

    if mcast_step is not None:                  # the same on every rank (decided by an all-reduce)
        # nothing may still be storing to the multicast address when a rank lets go of its buffer
        torch.cuda.synchronize()
        dist.barrier()

    # Measured denominator for the SpMM operand path: random 512-byte gathers from an L2-resident
    # buffer, L1 bypassed (the bench-side probe library), timed here on this GPU right after the workload.
    l2_gather_tbps = None
    probe = load_probe() if rank == 0 and kind in ("spmm", "mlp") else None
    if probe is not None:
        probe_buf = torch.empty(32 << 20, dtype=torch.uint8, device=dev)
        probe_buf.zero_()
        sink = torch.zeros(1, dtype=torch.float32, device=dev)
        nbytes = ctypes.c_uint64(0)
        stream_ptr = torch.cuda.current_stream().cuda_stream
        best = 0.0
        for i in range(5):                              # first pass warms L2; best of the rest
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if probe(probe_buf.data_ptr(), 32 << 20, 200, sink.data_ptr(), stream_ptr, ctypes.byref(nbytes)) != 0:
                break
            e1.record()
            torch.cuda.synchronize()
            if i:
                best = max(best, nbytes.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        l2_gather_tbps = best or None
        del probe_buf

    if rank == 0:
        metric, unit = metric_of(wk, args)
        peak, peak_kind = measured_peak()
        per_gpu_bytes = job_bytes / world if kind != "mlp" else job_bytes
        achieved = per_gpu_bytes / sec / 1e9
        line = {
            "metric": metric, "value": to_value(wk, job_bytes, sec), "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": config,
            "gflops": job_flops / sec / 1e9,
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"of {peak_kind}", "kernel": kernel_name,
                         "algorithmic_bytes_per_launch": per_gpu_bytes / max(1, launches_per_step) if kind != "mlp" else None,
                         "traffic": recorded_traffic(kernel_name, args, world)},
        }
        # SpMM and conv move one 4-byte operand per FMA through the L2 -> SM gather path / shared
        # memory; that path, not HBM, is what their time tracks, so it is reported too.
        if kind in ("spmm", "conv", "convstack", "mlp"):
            op_bytes = job_flops / 2.0 * 4.0 / world
            line["roofline"]["operand_path"] = {
                "what": "X operands consumed, 4 bytes per FMA (gathered L2->SM for SpMM/MLP; for conv read from "
                        "shared memory, once per FMA by the per-row kernel, once per block of 4 rows by the "
                        "row-block-merged kernel)",
                "bytes_per_step": op_bytes, "achieved_tbps": op_bytes / sec / 1e12}
            if l2_gather_tbps:
                line["roofline"]["operand_path"].update({
                    "l2_gather_peak_tbps": l2_gather_tbps,
                    "frac_of_l2_gather_peak": op_bytes / sec / 1e12 / l2_gather_tbps,
                    "peak_source": "bench_l2_gather_probe on this GPU: random 512-byte gathers from a 32 MiB buffer, "
                                   "L1 bypassed; operands served by L1 hits can lift the fraction above 1"})
        if check is not None:
            line["check"] = check
        if e2e:
            line["e2e"] = e2e
        if ag:
            line["with_allgather"] = ag
        if fused:
            line["with_fused_allgather"] = fused
        if xchg:
            line["with_copy_engine_allgather"] = xchg
        if mcast:
            line["with_multicast_allgather"] = mcast
        if not args.no_cpu and world == 1:
            try:
                run, frac, ckind, sample = cpu_sample_runner(args, wk, fraction=0.25 if args.workload == "cfg5_spmm" else None)
                med, reps, _ = time_cpu(run, 5, warmup=1, budget_s=20.0)
                csec = med / frac
                line["cpu_baseline"] = {"value": to_value(wk, job_bytes, csec), "unit": unit, "cores": host_cores(), "kind": ckind,
                                        "sample": sample + f"; median of {reps} runs of {med * 1e3:.2f} ms, scaled by 1/{frac:.4f}",
                                        "gflops": job_flops / csec / 1e9}
            except Exception as ex:  # the CPU leg must never take the GPU line down
                line["cpu_baseline"] = {"value": None, "error": repr(ex)}
        return line
    return None


ALSO = [("cfg1_spmm", {}, "cfg1_spmm"), ("cfg1_spmv", {}, "cfg1_spmv"),
        ("cfg2_spmv", {"size": 16384, "sparsity": 0.90}, "cfg2_spmv_16384_s90"),
        ("cfg2_spmv", {"size": 65536, "sparsity": 0.90}, "cfg2_spmv_65536_s90"),
        ("cfg3_mlp", {}, "cfg3_mlp"), ("cfg4_conv", {}, "cfg4_conv")]
# At N > 1 the second half of the metric rides along: the sparse MLP batch-sharded (no collective)
# and row-sharded (an exchange after every layer), device-resident and through host buffers.
ALSO_MULTI = [("cfg3_mlp", {"tp": False}, "cfg3_mlp_batch_sharded"), ("cfg3_mlp", {"tp": True}, "cfg3_mlp_row_sharded")]


def also_entry(l2):
    e = {"desc": l2["config"]["desc"], "sharding": l2["config"]["sharding"], "metric": l2["metric"], "value": l2["value"],
         "unit": l2["unit"], "n_gpus": l2["n_gpus"], "ms_per_step": l2["ms_per_step"], "gflops": l2["gflops"],
         "hbm_frac": l2["roofline"]["frac"], "l2": l2["config"]["l2"], "gpu_launches": l2["gpu_launches"]}
    for k in ("check", "cpu_baseline"):
        if k in l2:
            e[k] = l2[k]
    if "e2e" in l2:
        e["e2e"] = {k: l2["e2e"][k] for k in ("value", "unit", "ms_per_step", "h2d_bytes_per_step", "d2h_bytes_per_step")}
    return e


def run_ours(args):
    c = setup_ours(args)
    line = measure(args, c)
    # The metric names SpMM, SpMV and the sparse MLP; the headline line carries the largest SpMM
    # configuration, the other configurations ride along in "also".
    default_run = not args.no_also and args.workload == "cfg5_spmm" and args.scale == 1.0 and not args.rows and not args.cols
    if default_run:
        import copy
        also = {}
        for name, over, label in (ALSO if c.world == 1 else ALSO_MULTI):
            a2 = copy.copy(args)
            a2.workload, a2.steps = name, max(args.steps, 20)
            a2.no_e2e = name != "cfg3_mlp"                    # host-buffer timing for the model only
            a2.no_cpu = args.no_cpu
            for k, v in over.items():
                setattr(a2, k, v)
            try:
                l2 = measure(a2, c)                           # collective: every rank takes part
                if c.rank == 0:
                    also[label] = also_entry(l2)
            except Exception as ex:
                also[label] = {"error": repr(ex)}
        if c.rank == 0:
            line["also"] = also
    failed = False
    if c.rank == 0:
        print(json.dumps(line), flush=True)
        bad = [line.get("check")] + [v.get("check") for v in line.get("also", {}).values() if isinstance(v, dict)]
        failed = any(ch is not None and not (ch.get("bit_exact", True) and ch.get("within_tolerance", True)) for ch in bad)
    if c.world > 1:
        c.dist.barrier()
        c.dist.destroy_process_group()
    if failed:
        raise SystemExit("bench.py: a result differs from the CPU oracle (see \"check\" in the line above)")


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
