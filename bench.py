"""Benchmark of the JL projection hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (per GPU): Gaussian JL projection of 128 per-example gradients of a CIFAR
ResNet-18 (D = 11,173,962 features, fp16, N(0, 1e-2)) to k = 4096, seed 17,
148 feature tiles.  One step = one pass of the projection over one such batch.
Multi-GPU: one process per GPU (torchrun), every rank projects its own batch of
128 examples with the same virtual matrix -- the path shards by example, there is
no data-path collective (weak scaling).

After the projection, one featurize step of the CIFAR ResNet-18 configuration (key ``featurize``:
torch.func gradients -> projection from the gradient dict) and the second hot path are measured
too (key ``scoring`` of the same line): the whole C4 scoring job -- X fp32 [1,000,000 x 8192] sharded by rows over the GPUs,
Gram + one all-reduce + Cholesky inverse + features + weighted scores for 10,000 targets (the
reference's ordering; ``scoring.without_features`` times the same scores with the targets taken
through the inverse first, which never forms the features).

Further keys of the same line: ``rademacher`` (the same shape with the Rademacher matrix), ``rows_sweep``
(16 ... 512 rows per call, both matrix types: what one GPU does when the 128-row batch is split over 8 ... 1
GPUs, and what larger batches gain), ``scaling_strong`` (N > 1: the 128-row batch split 128/N rows per rank),
``scoring.e2e`` (the three score-computer calls as TRAKer makes them, train rows in pinned host memory, scores
into a host accumulator), ``scoring.parity`` (this library against the reference's CPU class at k = 8192),
``scoring.multi_gpu_check`` (N > 1: rank 0 recomputes a block of scores alone), ``featurize_job`` (the whole
50,000-example featurize job with its stores) and ``chunked`` (GPT-2-small per-sample gradients through the
chunked projector).

Prints ONE JSON line (rank 0).  ``value`` is examples/s with the batch resident in
HBM; ``e2e`` is the same through the public ``trak_b200.fast_jl.project`` call with every
step's batch copied from pinned host memory and its result read back (the copy of the next
batch overlaps the current projection); ``roofline`` rates the
projection kernel against the tensor-core peak; ``cpu_baseline`` is the reference's
BasicProjector (or its CPU port, see below) timed on a bounded sample on this box.

``--impl reference`` times the reference's CPU path alone (all host threads) on the same
workload, one bounded sample per step: the unmodified ``BasicProjector`` from the reference
package when its offline install is present under ``baseline/_ref`` (``kind`` "reference"),
else the CPU port in ``oracle/`` (``kind`` "port").  ``--scale f`` shrinks D by f (for profiler
captures of the same command on a small case).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D_FULL = 11_173_962
ROWS = 128
K_DIM = 4096
SEED = 17
TILES = 148
BLOCK = 100  # BasicProjector's column block (trak/projectors.py:229)

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the three launches of one projection call on
# the full workload, from the ncu capture summarised in profiles/project_kernel_normal_bench.md: taken at D/10
# (traffic grows in proportion to D) and multiplied by 10.
NCU_TRAFFIC_BYTES_FULL = {"stage_kernel": 5.30e9, "project_kernel": 3.45e9, "reduce_kernel": 0.78e9}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops_sustained", d.get("bf16_tflops"))), "measured (sustained bf16, MEASURED_PEAKS.json)"
    return 1400.0, "fallback (sustained bf16 figure of an earlier measurement on this pool)"


def burst_peak():
    """The bf16 GEMM rate of a kernel timed alone (MEASURED_PEAKS.json), else this pool's earlier figure."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops", 1590.0))
    return 1590.0


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs: through NVML
    (read-only queries, every 20 ms) when the bindings are importable, else with nvidia-smi."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index, pci_bus_id=None):
        self.index, self.pci = index, pci_bus_id
        self.clocks, self.max_mhz, self.reasons = [], None, set()
        self.proc = self.thread = self.handle = self.nvml = None
        self.stop_flag = threading.Event()

    def _nvml_loop(self):
        n = self.nvml
        masks = {"hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag.is_set():
            try:
                self.clocks.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                bits = int(get_reasons(self.handle))
                for name, m in masks.items():
                    if bits & m:
                        self.reasons.add(name)
            except Exception:
                pass
            self.stop_flag.wait(0.02)

    def _smi_loop(self):
        for line in self.proc.stdout:
            r = [c.strip() for c in line.split(",")]
            try:
                self.clocks.append(float(r[0]))
                self.max_mhz = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(self.NAMES, r[2:6]):
                if v.lower().startswith("active"):
                    self.reasons.add(name)

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(self.pci.encode() if self.pci else b"")
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._smi_loop, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if self.nvml is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML bindings and no nvidia-smi"]}
        return {"sm_mhz": statistics.median(self.clocks) if self.clocks else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.clocks),
                "source": "nvml" if self.nvml is not None else "nvidia-smi"}


_cpu_input = {}
_REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def reference_package():
    """The reference's own Python package when its offline install travelled with the repository
    (baseline/_ref, made by __graft_entry__.build() where the reference checkout exists), else None."""
    if not os.path.isdir(os.path.join(_REF_DIR, "trak")):
        return None
    if _REF_DIR not in sys.path:
        sys.path.insert(0, _REF_DIR)
    try:
        import trak
        return trak
    except Exception:
        return None


def cpu_kind():
    return "reference" if reference_package() is not None else "port"


def cpu_port_sample(rows, D, threads, blocks):
    """Times the reference's CPU projection on `blocks` of the ceil(k/100) column blocks of 100: the
    unmodified BasicProjector built with proj_dim = 100 * blocks (it then generates and multiplies exactly
    the first `blocks` blocks of the full projection, same per-block seeds) when the reference package is
    there, else its CPU port."""
    import torch
    torch.set_num_threads(threads)
    if (rows, D) not in _cpu_input:  # the input is made once, outside the timed part
        _cpu_input.clear()
        _cpu_input[(rows, D)] = torch.randn(rows, D, generator=torch.Generator().manual_seed(1000)) * 1e-2
    g = _cpu_input[(rows, D)]
    trak = reference_package()
    if trak is not None:
        proj = trak.projectors.BasicProjector(grad_dim=D, proj_dim=BLOCK * blocks, seed=SEED, proj_type="normal",
                                              device="cpu", block_size=BLOCK, dtype=torch.float32)
        if blocks == 1:  # a one-block projector keeps its matrix from the constructor; generate it in the timed part
            t0 = time.perf_counter()
            proj.generate_sketch_matrix(proj.generator_states[0])
            proj.project(g, model_id=0)
        else:
            t0 = time.perf_counter()
            proj.project(g, model_id=0)
        dt = time.perf_counter() - t0
        proj.free_memory()
    else:
        from oracle import basic_ref
        t0 = time.perf_counter()
        basic_ref.basic_project(g, K_DIM, SEED, "normal", blocks=range(blocks))
        dt = time.perf_counter() - t0
    nblocks = -(-K_DIM // BLOCK)
    return dt * nblocks / blocks, dt  # extrapolated full-step seconds, measured seconds


def run_reference(args, D):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    threads = os.cpu_count() or 1
    blocks = 1   # one of the 41 column blocks per step keeps a --steps 20 --warmup 5 run within minutes
    nblocks = -(-K_DIM // BLOCK)
    for _ in range(args.warmup):
        cpu_port_sample(ROWS, D, threads, blocks)
    full, measured = [], []
    for _ in range(args.steps):
        s, m = cpu_port_sample(ROWS, D, threads, blocks)
        full.append(s)
        measured.append(m)
    sec = sum(full) / len(full)
    value = ROWS / sec
    who = "the reference's unmodified BasicProjector" if cpu_kind() == "reference" else "CPU port of BasicProjector"
    sample = (f"{who}: each step projects all {ROWS} rows x D={D} onto {blocks} of {nblocks} column blocks of "
              f"{BLOCK} (matrix block generated + matmul); value = rows / (measured step time x {nblocks}/{blocks})")
    line = {
        "impl": "reference", "metric": "jl_projected_examples_per_s", "value": value, "unit": "examples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        # the time one timed step actually took (a bounded sample: `sampled` of the column blocks);
        # `extrapolated_ms_per_step` is that time scaled to all blocks, which is what `value` is computed from
        "ms_per_step": sum(measured) / len(measured) * 1e3, "measured_ms_per_step": sum(measured) / len(measured) * 1e3,
        "extrapolated_ms_per_step": sec * 1e3, "sampled": f"{blocks}/{nblocks}",
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(D),
        "cpu_baseline": {"value": value, "unit": "examples/s", "cores": torch.get_num_threads(),
                         "kind": cpu_kind(), "sample": sample},
        "e2e": {"value": value, "unit": "examples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(D, proj_type="normal"):
    name = "gaussian" if proj_type == "normal" else "rademacher"
    return {"workload": f"C2 {name} JL projection: fp16 N(0,1e-2) grads [{ROWS} x {D}] per GPU -> k={K_DIM}, "
                        f"seed {SEED}, {TILES} feature tiles",
            "rows_per_gpu": ROWS, "grad_dim": D, "proj_dim": K_DIM, "proj_type": proj_type,
            "l2": "input batch (2.86 GB at full size) is larger than the 126 MB L2; no flush needed"}


# ---- after-kernel scoring (second hot path) ---------------------------------------------------
SC_N, SC_K, SC_M, SC_LAMBDA, SC_BLOCK = 1_000_000, 8192, 10_000, 1e-3, 65_536


def scoring_flop(n, k, m):
    """Algorithmic work of the whole job: symmetric Gram, inverse, features, scores."""
    return n * k * (k + 1) + k ** 3 + 2.0 * n * k * k + 2.0 * n * m * k


def run_scoring(args, dev, rank, world, scale):
    """Train rows [n, k] fp32 sharded over the ranks: Gram per shard -> one all-reduce -> Cholesky
    inverse with the mean-|.| rescale (replicated) -> features and out-to-loss-weighted scores for
    m targets per shard.  Returns the timing of the whole job (max over ranks)."""
    import torch
    import torch.distributed as dist
    from trak_b200 import _lib, score_computers as sc

    n_total = max(world * 1024, int(SC_N * scale))
    lo, hi = sc.shard_rows(n_total, rank, world)
    n = hi - lo
    k, m = SC_K, max(256, int(SC_M * scale))
    gen = torch.Generator(device=dev).manual_seed(2000 + rank)
    X = torch.empty(n, k, device=dev)
    for i in range(0, n, SC_BLOCK):  # generated block-wise to bound temporary memory
        X[i:i + SC_BLOCK] = torch.randn(min(SC_BLOCK, n - i), k, device=dev, generator=gen) / k ** 0.5
    T = torch.randn(m, k, device=dev, generator=torch.Generator(device=dev).manual_seed(3000)) / k ** 0.5
    w = torch.rand(n, device=dev, generator=torch.Generator(device=dev).manual_seed(4000 + rank))
    scores = torch.empty(n, m, device=dev)
    feats = torch.empty(min(SC_BLOCK, n), k, device=dev)
    gram = torch.empty(k, k, device=dev)
    group = dist.group.WORLD if world > 1 else None

    # Row blocks alternate between two streams (score_computers.StreamPair), as B200ScoreComputer runs them: the
    # memory-bound packing passes of one block overlap the tensor-bound GEMM of the other.  Each stream has its own
    # partial Gram and its own features buffer.
    pair = sc.StreamPair(dev)
    gram2 = torch.empty(k, k, device=dev)
    feats2 = torch.empty_like(feats)
    grams, fbuf = [gram, gram2], [feats, feats2]
    starts = list(range(0, n, SC_BLOCK))

    def gram_phase():
        with pair:
            for j, i in enumerate(starts):
                with pair.stream(j):
                    sc.gram(X[i:i + SC_BLOCK], out=grams[j % 2], accumulate=j >= 2)
        if len(starts) > 1:
            gram.add_(gram2)
        sc.reduce_gram(gram, group)                     # the one exchange of the path (NCCL all-reduce)
        sc.spd_inverse_(gram, SC_LAMBDA, rescale=True)  # gram now holds the rescaled inverse

    def job():
        gram_phase()
        with pair:
            for j, i in enumerate(starts):
                rows = min(SC_BLOCK, n - i)
                with pair.stream(j):
                    sc.gemm_nt(X[i:i + rows], gram, out=fbuf[j % 2][:rows])
                    sc.gemm_nt(fbuf[j % 2][:rows], T, out=scores[i:i + rows], row_scale=w[i:i + rows])

    solved = torch.empty(m, k, device=dev)

    def job_direct():
        # the same scores without the features: targets through the inverse first, one product over the rows
        gram_phase()
        sc.gemm_nt(T, gram, out=solved)
        with pair:
            for j, i in enumerate(starts):
                rows = min(SC_BLOCK, n - i)
                with pair.stream(j):
                    sc.gemm_nt(X[i:i + rows], solved, out=scores[i:i + rows], row_scale=w[i:i + rows])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        fn()
        barrier()
        steps = 2
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        _lib.device_status(dev.index)
        ms = torch.tensor([ev0.elapsed_time(ev1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() * 1e-3

    sec = timed(job)
    check = scores[:256].clone()
    sec_direct = timed(job_direct)
    direct_err = float((scores[:256] - check).norm() / check.norm())
    flop_direct = n_total * k * (k + 1) + k ** 3 + 2.0 * k * k * m + 2.0 * n_total * m * k
    peak, _ = measured_peaks()
    out = {"metric": "scoring_seconds", "value": sec, "unit": "s", "higher_is_better": False, "scaling": "strong",
           "config": {"workload": f"C4 scoring: X fp32 [{n_total} x {k}] N(0,1/k) sharded by rows over {world} GPU(s), "
                                  f"lambda {SC_LAMBDA}, {m} targets, out-to-loss weights fused",
                      "row_block": SC_BLOCK, "streams": "row blocks alternate between two streams",
                      "ordering": "the reference's: Gram, inverse, features X.inv, scores features.targets^T"},
           "algorithmic_tflops": scoring_flop(n_total, k, m) / sec / 1e12,
           "roofline": {"bound": "tensor", "achieved": scoring_flop(n_total, k, m) / sec / 1e12 / world, "peak": peak,
                        "unit": "TFLOP/s", "frac": scoring_flop(n_total, k, m) / sec / 1e12 / world / peak,
                        "frac_burst": scoring_flop(n_total, k, m) / sec / 1e12 / world / burst_peak(),
                        "note": "fp32 inputs run as fp16 hi/lo splits: three tensor-core passes per algorithmic flop, "
                                "so 1/3 of the bf16 peak is the ceiling of this figure"},
           "without_features": {"value": sec_direct, "unit": "s",
                                "ordering": "Gram, inverse, targets.inv, scores X.(targets.inv)^T: the features are "
                                            "never formed (2 k^2 m flop replace 2 n k^2)",
                                "algorithmic_tflops": flop_direct / sec_direct / 1e12,
                                "relative_difference_of_scores": direct_err}}
    if world > 1:
        # Correctness of the sharded job: rank 0 alone regenerates every rank's shard (same seeds), forms the whole
        # Gram by itself, inverts it and recomputes its first 256 rows of scores; the sharded job's all-reduce adds
        # the same partial Grams in another order, so the two agree to fp32 round-off.
        x256, w256 = X[:256].clone(), w[:256].clone()
        del X, feats, feats2, fbuf
        torch.cuda.empty_cache()
        if rank == 0:
            g1 = torch.empty(k, k, device=dev)
            first = True
            for r in range(world):
                lo_r, hi_r = sc.shard_rows(n_total, r, world)
                gen_r = torch.Generator(device=dev).manual_seed(2000 + r)
                for i in range(0, hi_r - lo_r, SC_BLOCK):
                    blk = torch.randn(min(SC_BLOCK, hi_r - lo_r - i), k, device=dev, generator=gen_r) / k ** 0.5
                    sc.gram(blk, out=g1, accumulate=not first)
                    first = False
            sc.spd_inverse_(g1, SC_LAMBDA, rescale=True)
            alone = sc.gemm_nt(x256, sc.gemm_nt(T, g1), row_scale=w256)
            out["multi_gpu_check"] = {
                "rows": 256, "relative_difference": float((scores[:256] - alone).norm() / alone.norm()),
                "what": f"rank 0's first 256 rows of scores from the {world}-GPU job (Gram summed by NCCL through "
                        "score_computers.reduce_gram) against the same rows recomputed by rank 0 alone from all shards"}
        dist.barrier()
    else:
        del X, feats, feats2, fbuf
    del scores
    torch.cuda.empty_cache()
    return out


def run_scoring_e2e(dev, rank, world):
    """The scoring path as TRAKer drives it (trak/traker.py:480-486, 632, 662-667): the train rows of this rank in
    pinned HOST memory, B200ScoreComputer.get_xtx -> get_x_xtx_inv -> get_scores with a host accumulator.  Every
    byte of X crosses PCIe twice (Gram, features), the features come back once and go in once more, and the scores
    leave through the pinned staging pair and are added into the accumulator on the host."""
    import torch
    import torch.distributed as dist
    from trak_b200.score_computers import B200ScoreComputer
    n, k, m = 131_072, SC_K, SC_M
    X = torch.empty(n, k).pin_memory()
    gen = torch.Generator(device=dev).manual_seed(2000 + rank)
    for i in range(0, n, SC_BLOCK):
        X[i:i + SC_BLOCK].copy_(torch.randn(min(SC_BLOCK, n - i), k, device=dev, generator=gen) / k ** 0.5)
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(3000)) / k ** 0.5
    acc = torch.zeros(n, m).pin_memory()
    sc = B200ScoreComputer(torch.float32, dev, lambda_reg=SC_LAMBDA,
                           process_group=dist.group.WORLD if world > 1 else None)

    def job():
        gram = sc.get_xtx(X)
        feats = sc.get_x_xtx_inv(X, gram)
        sc.get_scores(feats, T, acc)

    job()  # warms the pinned staging and the workspaces
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    job()
    torch.cuda.synchronize()
    sec = torch.tensor([time.perf_counter() - t0], device=dev)
    if world > 1:
        dist.all_reduce(sec, op=dist.ReduceOp.MAX)
    sec = sec.item()
    flop = scoring_flop(n * world, k, m)
    out = {"value": sec, "unit": "s", "rows_per_gpu": n, "targets": m,
           "h2d_bytes": 2 * n * k * 4 + m * k * 4, "d2h_bytes": n * m * 4,
           "algorithmic_tflops": flop / sec / 1e12,
           "rows_per_s": n * world / sec,
           "what": "B200ScoreComputer.get_xtx / get_x_xtx_inv / get_scores, X in pinned host memory, features kept on "
                   "the device as the reference does, scores added into a host accumulator (wall clock, max over ranks); "
                   f"the full job is {SC_N // n // world} such shards per GPU"}
    del X, acc
    return out


def scoring_reference_on_gpu(dev):
    """The reference's own GPU path for the same three steps: the unmodified BasicScoreComputer(device="cuda")
    (torch.matmul / torch.linalg.inv, i.e. cuBLAS and cuSOLVER in fp32, trak/score_computers.py:145-189) on one
    131,072-row shard of the C4 job, next to this library on the very same tensors.  Outside every timed region of
    the benchmark; needs the reference package (baseline/_ref)."""
    import torch
    trak = reference_package()
    if trak is None:
        return {"unavailable": "reference package not installed under baseline/_ref"}
    from trak_b200.score_computers import B200ScoreComputer
    n, k, m = 131_072, SC_K, SC_M
    gen = torch.Generator(device=dev).manual_seed(2000)
    X = torch.empty(n, k, device=dev)
    for i in range(0, n, SC_BLOCK):
        X[i:i + SC_BLOCK] = torch.randn(min(SC_BLOCK, n - i), k, device=dev, generator=gen) / k ** 0.5
    T = torch.randn(m, k, device=dev, generator=torch.Generator(device=dev).manual_seed(3000)) / k ** 0.5
    ref = trak.score_computers.BasicScoreComputer(dtype=torch.float32, device=dev, logging_level=40,
                                                  lambda_reg=SC_LAMBDA)
    mine = B200ScoreComputer(torch.float32, dev, lambda_reg=SC_LAMBDA)

    acc = torch.zeros(n, m)   # on the host, where TRAKer keeps it and the reference's get_scores needs it

    def run(sc):
        acc.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        g = sc.get_xtx(X)
        f = sc.get_x_xtx_inv(X, g)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        sc.get_scores(f, T, acc)
        torch.cuda.synchronize()
        return t1 - t0, time.perf_counter() - t1

    run(mine)
    mine_dev, mine_scores = run(mine)
    s_mine = acc[:4096].clone()
    run(ref)
    ref_dev, ref_scores = run(ref)
    diff = float((s_mine - acc[:4096]).norm() / acc[:4096].norm())
    del X
    torch.cuda.empty_cache()
    return {"reference_seconds": ref_dev + ref_scores, "this_library_seconds": mine_dev + mine_scores,
            "ratio": (ref_dev + ref_scores) / (mine_dev + mine_scores),
            "gram_inverse_features": {"reference_seconds": ref_dev, "this_library_seconds": mine_dev},
            "scores_into_host_accumulator": {"reference_seconds": ref_scores, "this_library_seconds": mine_scores},
            "relative_difference_of_scores": diff,
            "what": f"get_xtx + get_x_xtx_inv + get_scores on device-resident X fp32 [{n} x {k}], {m} targets, host "
                    "accumulator (wall clock): the reference's unmodified BasicScoreComputer(device='cuda') -- "
                    "cuBLAS fp32 products, cuSOLVER LU inverse, a pageable copy of the scores -- against "
                    "B200ScoreComputer on the same tensors"}


def scoring_cpu_baseline(threads, dev=None):
    """The reference's BasicScoreComputer on the host cores on a bounded sample (k full, fewer rows and targets),
    scaled to C4 -- and, with `dev`, this library on the very same sample, compared with it (``parity``)."""
    import torch
    from oracle import basic_ref
    torch.set_num_threads(threads)
    n, k, m = 8192, SC_K, 512
    X = torch.randn(n, k, generator=torch.Generator().manual_seed(1)) / k ** 0.5
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(2)) / k ** 0.5
    trak = reference_package()
    if trak is not None:  # the reference's own class on the host cores
        ref = trak.score_computers.BasicScoreComputer(dtype=torch.float32, device="cpu", logging_level=40,
                                                      lambda_reg=SC_LAMBDA)
        xtx, x_xtx_inv, scores = ref.get_xtx, ref.get_x_xtx_inv, ref.get_scores
    else:
        xtx = basic_ref.xtx
        x_xtx_inv = lambda x, g: basic_ref.x_xtx_inv(x, g, SC_LAMBDA)  # noqa: E731
        scores = basic_ref.scores
    ridge = (SC_N / n - 1) * torch.eye(k)  # keeps the sample as well conditioned as the full job's Gram
    t0 = time.perf_counter()
    g = xtx(X)
    t1 = time.perf_counter()
    f = x_xtx_inv(X, g + ridge)
    t2 = time.perf_counter()
    acc = torch.zeros(n, m)
    scores(f, T, acc)
    t3 = time.perf_counter()
    # Gram and features grow with n, scores with n*m; the inverse (part of t2 - t1) is size-independent:
    # timed separately below
    t4 = time.perf_counter()
    torch.linalg.inv(g + (SC_N / n) * torch.eye(k) + SC_LAMBDA * torch.eye(k))
    t_inv = time.perf_counter() - t4
    full = (t1 - t0) * SC_N / n + t_inv + max(0.0, (t2 - t1) - t_inv) * SC_N / n + (t3 - t2) * (SC_N / n) * (SC_M / m)
    who = "the reference's unmodified BasicScoreComputer" if trak is not None else "CPU port of BasicScoreComputer"
    out = {"value": full, "unit": "s", "cores": torch.get_num_threads(), "kind": cpu_kind(),
           "sample": f"{who} at k={k} on {n} rows x {m} targets "
                     f"(gram {t1 - t0:.1f} s, inverse {t_inv:.1f} s, features {t2 - t1 - t_inv:.1f} s, scores {t3 - t2:.1f} s), "
                     f"Gram/features scaled by n, scores by n*m, inverse counted once"}
    parity = None
    if dev is not None:
        from trak_b200.score_computers import B200ScoreComputer
        mine = B200ScoreComputer(torch.float32, dev, lambda_reg=SC_LAMBDA)
        g_m = mine.get_xtx(X)
        f_m = mine.get_x_xtx_inv(X, g_m + ridge.to(dev))
        acc_m = torch.zeros(n, m)
        mine.get_scores(f_m, T, acc_m)

        def rel(a, b):
            a, b = a.double().cpu(), b.double().cpu()
            return float((a - b).norm() / b.norm())

        parity = {"gram": rel(g_m, g), "features": rel(f_m, f), "scores": rel(acc_m, acc), "tolerance": 1e-3,
                  "what": f"Frobenius-relative difference of this library from {who} on that sample "
                          f"(k={k}, {n} rows, {m} targets, lambda {SC_LAMBDA})"}
    return out, parity


# ---- end-to-end featurize step (per-sample gradients -> projection) ------------------------------
def run_featurize(dev, rank, world):
    """One featurize step as TRAKer runs it (trak/traker.py:424-429) on the CIFAR ResNet-18 configuration:
    a batch of 128 synthetic 3x32x32 images copied from pinned host memory, per-example margin gradients from
    torch.func (vmap(grad), fp32, 62 tensors, 11,173,962 features), Rademacher projection to k = 2048 straight
    from the gradient dict with 1/sqrt(D) folded in, features copied back to the host.  Reports examples/s over
    all ranks and how the step splits between PyTorch's gradients and the projection."""
    import torch
    import torch.distributed as dist
    try:
        import torchvision
    except Exception as e:  # no torchvision: nothing to measure
        return {"unavailable": f"torchvision not importable: {e}"}
    from torch.func import functional_call, grad, vmap
    from trak_b200 import fast_jl
    from trak_b200.projectors import CudaProjector, ProjectionType

    torch.manual_seed(0)
    model = torchvision.models.resnet18(num_classes=10)
    model.conv1 = torch.nn.Conv2d(3, 64, 3, 1, 1, bias=False)
    model.maxpool = torch.nn.Identity()
    model = model.to(dev).eval()
    params = {k: v.detach() for k, v in model.named_parameters()}
    buffers = {k: v.detach() for k, v in model.named_buffers()}
    D = sum(p.numel() for p in params.values())
    B, N = 128, 2048
    gen = torch.Generator().manual_seed(rank)
    host_x = torch.rand(B, 3, 32, 32, generator=gen).pin_memory()
    host_y = torch.randint(0, 10, (B,), generator=gen).pin_memory()
    host_out = torch.empty(B, N).pin_memory()

    def margin(p, x, y):
        logits = functional_call(model, (p, buffers), (x.unsqueeze(0),))[0]
        own = torch.arange(logits.numel(), device=logits.device) == y
        rest = torch.logsumexp(torch.where(own, torch.full_like(logits, -torch.inf), logits), 0)
        return (logits * own).sum() - rest

    per_sample = vmap(grad(margin), in_dims=(None, 0, 0))
    proj = CudaProjector(D, N, 0, ProjectionType.rademacher, dev, 32)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]

    def step(timed):
        x = host_x.to(dev, non_blocking=True)
        y = host_y.to(dev, non_blocking=True)
        if timed:
            ev[0].record()
        grads = per_sample(params, x, y)
        if timed:
            ev[1].record()
        feats = proj.project(grads, model_id=0, alpha=1.0 / D ** 0.5)
        if timed:
            ev[2].record()
        host_out.copy_(feats, non_blocking=True)
        del grads

    for _ in range(2):
        step(False)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps, g_ms, p_ms = 5, 0.0, 0.0
    t0 = time.perf_counter()
    for _ in range(steps):
        step(True)
        torch.cuda.synchronize()
        g_ms += ev[0].elapsed_time(ev[1])
        p_ms += ev[1].elapsed_time(ev[2])
    sec = torch.tensor([(time.perf_counter() - t0) / steps], device=dev)
    if world > 1:
        dist.all_reduce(sec, op=dist.ReduceOp.MAX)
    fast_jl.free_workspaces()
    del model, params, proj
    torch.cuda.empty_cache()
    return {"metric": "featurize_examples_per_s", "value": world * B / sec.item(), "unit": "examples/s",
            "config": {"workload": f"CIFAR ResNet-18 ({D} parameters, 62 tensors, fp32), batch {B} per GPU, "
                                   f"vmap(grad) margins -> Rademacher k={N}, host images in, host features out"},
            "ms_per_step": sec.item() * 1e3, "gradients_ms": g_ms / steps, "projection_ms": p_ms / steps}


def time_projection(lib, fast_jl, g, ptype, calls=5, warm=2):
    """(ms per call, ms of the projection kernel alone) of fast_jl.project on a resident batch: the median over
    `calls` calls, each between its own pair of CUDA events on the current stream, and the library's own event
    pair around the dominant kernel (the median keeps the first calls after a clock change out of the figure)."""
    import torch
    out = torch.empty(g.shape[0], K_DIM, device=g.device, dtype=torch.float32)
    for _ in range(warm):
        fast_jl.project(g, K_DIM, SEED, TILES, ptype, out=out, strict=False)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(calls)]
    for quad in ev:
        for e in quad:
            e.record()
    torch.cuda.synchronize()
    for c0, c1, k0, k1 in ev:
        c0.record()
        lib.tb_profile_events(k0.cuda_event, k1.cuda_event)
        fast_jl.project(g, K_DIM, SEED, TILES, ptype, out=out, strict=False)
        c1.record()
    torch.cuda.synchronize()
    return (statistics.median(c0.elapsed_time(c1) for c0, c1, _, _ in ev),
            statistics.median(k0.elapsed_time(k1) for _, _, k0, k1 in ev))


def run_rows_sweep(lib, fast_jl, _lib, dev, D, rows_list=(16, 32, 64, 128, 256, 512)):
    """ms per call and examples/s of one GPU for batches of 16 ... 512 rows of the C2 gradients, both matrix
    types.  16 / 32 / 64 rows are what one GPU gets when the 128-row batch is split over 8 / 4 / 2 GPUs; 256 and
    512 rows show what one generation of the matrix serving more rows gains.  A batch of more than 256 rows is
    one launch for the Gaussian matrix and 256-row passes for the Rademacher matrix."""
    import torch
    peak, _ = measured_peaks()
    gen = torch.Generator(device=dev).manual_seed(1234)
    big = torch.empty(max(rows_list), D, device=dev, dtype=torch.float16)
    for i in range(0, big.shape[0], 64):  # generated block-wise to bound temporary memory
        big[i:i + 64] = (torch.randn(min(64, big.shape[0] - i), D, device=dev, generator=gen) * 1e-2).half()
    out = {"rows": list(rows_list), "unit_ms": "ms per call (restage + project + reduce), median of 5 calls", "proj_dim": K_DIM, "grad_dim": D}
    for name, ptype in (("normal", _lib.TB_NORMAL), ("rademacher", _lib.TB_RADEMACHER)):
        ms, eps, frac = [], [], []
        for r in rows_list:
            time.sleep(0.25)  # lets the SM clock recover from the previous, possibly power-capped, configuration
            t, _ = time_projection(lib, fast_jl, big[:r], ptype)
            ms.append(round(t, 3))
            eps.append(round(r / t * 1e3, 1))
            frac.append(round(2.0 * r * D * K_DIM / (t * 1e-3) / 1e12 / peak, 4))
        out[name] = {"ms": ms, "examples_per_s": eps, "frac_of_sustained_peak": frac}
    _lib.device_status(dev.index)
    del big
    fast_jl.free_workspaces()
    torch.cuda.empty_cache()
    return out


def run_stored_matrix(lib, fast_jl, _lib, dev, D, rows_list=(128, 256, 512)):
    """The Gaussian projection of the C2 shape with the matrix kept in HBM (fast_jl.StoredMatrix: 91.6 GB for
    D = 11,173,962, k = 4096) instead of regenerated in every call -- what a projector that serves many batches
    with one seed can do on a 180 GB GPU.  Reports the one-off generation time and, per batch size, ms per call,
    examples/s and the HBM rate of the matrix stream (a call of up to 256 rows reads the matrix once)."""
    import torch
    peak, _ = measured_peaks()
    need = fast_jl.StoredMatrix.nbytes(D, K_DIM, TILES)
    free, _ = torch.cuda.mem_get_info(dev)
    if need + max(rows_list) * D * 6 > free:
        return {"unavailable": f"needs {need / 1e9:.1f} GB for the matrix, {free / 1e9:.1f} GB free"}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    m = fast_jl.StoredMatrix(D, K_DIM, SEED, TILES, _lib.TB_NORMAL, dtype=torch.float16, device=dev)
    ev1.record()
    torch.cuda.synchronize()
    gen_ms = ev0.elapsed_time(ev1)
    gen = torch.Generator(device=dev).manual_seed(4321)
    big = torch.empty(max(rows_list), D, device=dev, dtype=torch.float16)
    for i in range(0, big.shape[0], 64):
        big[i:i + 64] = (torch.randn(min(64, big.shape[0] - i), D, device=dev, generator=gen) * 1e-2).half()
    res = {"matrix_bytes": need, "generation_ms": gen_ms, "rows": list(rows_list), "ms": [], "examples_per_s": [],
           "frac_of_sustained_peak": [], "matrix_stream_tb_per_s": []}
    for r in rows_list:
        g = big[:r]
        out = torch.empty(r, K_DIM, device=dev)
        for _ in range(2):
            fast_jl.project(g, K_DIM, SEED, TILES, _lib.TB_NORMAL, out=out, strict=False, matrix=m)
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fast_jl.project(g, K_DIM, SEED, TILES, _lib.TB_NORMAL, out=out, strict=False, matrix=m)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        t = statistics.median(times)
        res["ms"].append(round(t, 3))
        res["examples_per_s"].append(round(r / t * 1e3, 1))
        res["frac_of_sustained_peak"].append(round(2.0 * r * D * K_DIM / (t * 1e-3) / 1e12 / peak, 4))
        res["matrix_stream_tb_per_s"].append(round(need * -(-r // 256) / (t * 1e-3) / 1e12, 3))
    # same result as the regenerating path (one-hot row and a random row of the 128-row batch)
    chk = big[:128].clone()
    chk[0].zero_()
    chk[0, D // 3] = 1.0
    a = fast_jl.project(chk, K_DIM, SEED, TILES, _lib.TB_NORMAL, strict=False, matrix=m)
    b = fast_jl.project(chk, K_DIM, SEED, TILES, _lib.TB_NORMAL, strict=False)
    res["one_hot_row_bit_equal"] = bool(torch.equal(a[0], b[0]))
    res["max_row_relative_difference"] = float(((a - b).norm(dim=1) / b.norm(dim=1)).max())
    _lib.device_status(dev.index)
    del m, big, a, b, chk
    fast_jl.free_workspaces()
    torch.cuda.empty_cache()
    res["what"] = ("Gaussian matrix of the benchmark shape generated once and kept in HBM; every call reads it "
                   "(once per 256 rows) instead of regenerating it")
    return res


def run_scaling_strong(lib, fast_jl, _lib, g, rank, world):
    """The 128-row batch of the configuration split over the ranks (128 / N rows each, same virtual matrix, no
    collective): examples/s = 128 / (slowest rank's time per call)."""
    import torch
    import torch.distributed as dist
    rows = max(1, ROWS // world)
    res = {"rows_per_gpu": rows, "scaling": "strong"}
    for name, ptype in (("normal", _lib.TB_NORMAL), ("rademacher", _lib.TB_RADEMACHER)):
        part = g[rank * rows % ROWS: rank * rows % ROWS + rows]
        dist.barrier()
        t, _ = time_projection(lib, fast_jl, part, ptype, calls=7, warm=3)
        tt = torch.tensor([t], device=g.device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        res[name] = {"ms_per_call": tt.item(), "examples_per_s": rows * world / tt.item() * 1e3}
    res["note"] = ("every rank regenerates the whole D x k matrix for its rows, as the reference does per 32 rows "
                   "(fast_jl/fast_jl.cu:51): the Gaussian time does not fall with the rows per GPU")
    return res


def _cifar_resnet18(dev):
    import torch
    import torchvision
    torch.manual_seed(0)
    model = torchvision.models.resnet18(num_classes=10)
    model.conv1 = torch.nn.Conv2d(3, 64, 3, 1, 1, bias=False)
    model.maxpool = torch.nn.Identity()
    return model.to(dev).eval()


def run_featurize_job(dev, rank, world, total=50_000, batch=256):
    """The whole featurize job of the CIFAR ResNet-18 configuration: `total` synthetic images (uniform pixels and
    labels) sharded contiguously over the ranks, per-example margin gradients from torch.func, Rademacher
    projection to k = 2048 with 1/sqrt(D) folded in, margin out-to-loss weights from a second forward
    (trak/modelout_functions.py:153-179), both written into this rank's grads / out_to_loss stores (fp16 npy
    memmaps, the reference's default dtype) through FeatureWriter.  Wall clock from the first batch to the
    flushed stores, max over ranks."""
    import shutil
    import tempfile
    import numpy as np
    import torch
    import torch.distributed as dist
    from torch.func import functional_call, grad, vmap
    from trak_b200 import fast_jl, mmap_io
    from trak_b200.featurize import FeatureWriter
    from trak_b200.projectors import CudaProjector, ProjectionType
    from trak_b200.score_computers import shard_rows

    model = _cifar_resnet18(dev)
    params = {k: v.detach() for k, v in model.named_parameters()}
    buffers = {k: v.detach() for k, v in model.named_buffers()}
    D = sum(p.numel() for p in params.values())
    N = 2048
    lo, hi = shard_rows(total, rank, world)
    n = hi - lo
    gen = torch.Generator().manual_seed(rank)
    host_x = torch.rand(n, 3, 32, 32, generator=gen).pin_memory()
    host_y = torch.randint(0, 10, (n,), generator=gen).pin_memory()

    def margin(p, x, y):
        logits = functional_call(model, (p, buffers), (x.unsqueeze(0),))[0]
        own = torch.arange(logits.numel(), device=logits.device) == y
        rest = torch.logsumexp(torch.where(own, torch.full_like(logits, -torch.inf), logits), 0)
        return (logits * own).sum() - rest

    per_sample = vmap(grad(margin), in_dims=(None, 0, 0))

    def out_to_loss(x, y):
        with torch.no_grad():
            ps = torch.softmax(model(x), dim=-1)[torch.arange(x.shape[0], device=x.device), y]
        return (1.0 - ps).unsqueeze(-1)

    tmp = tempfile.mkdtemp(prefix="trak_b200_featurize_")
    try:
        gs = mmap_io.create_store(os.path.join(tmp, "grads.mmap"), (n, N), torch.float16)
        ws = mmap_io.create_store(os.path.join(tmp, "out_to_loss.mmap"), (n, 1), torch.float16)
        proj = CudaProjector(D, N, 0, ProjectionType.rademacher, dev, 32)
        fw = FeatureWriter(proj, D ** 0.5, torch.float16, dev, max_batch=batch, grads_store=gs, out_to_loss_store=ws)

        def step(i):
            x = host_x[i:i + batch].to(dev, non_blocking=True)
            y = host_y[i:i + batch].to(dev, non_blocking=True)
            grads = per_sample(params, x, y)
            return fw.add(grads, np.arange(i, i + x.shape[0]), model_id=0, loss_grads=out_to_loss(x, y))

        step(0)  # warm-up (the rows are written again below)
        fw.flush()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        last = None
        for i in range(0, n, batch):
            last = step(i)
        fw.flush()
        torch.cuda.synchronize()
        sec = torch.tensor([time.perf_counter() - t0], device=dev)
        if world > 1:
            dist.all_reduce(sec, op=dist.ReduceOp.MAX)
        # the last batch as stored against its device-side result (fp16 rounding only)
        i_last = (n - 1) // batch * batch
        stored = torch.from_numpy(np.array(gs[i_last:n])).float()
        diff = float((stored - last.float().cpu()).abs().max() / last.float().abs().max())
        nz = float((np.array(ws[:64]).astype(np.float32) > 0).mean())
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    fast_jl.free_workspaces()
    del model, params, proj, fw
    torch.cuda.empty_cache()
    return {"metric": "featurize_job_seconds", "value": sec.item(), "unit": "s", "examples_per_s": total / sec.item(),
            "config": {"workload": f"C3 featurize job: {total} synthetic 3x32x32 images over {world} GPU(s) ({n} on rank 0), "
                                   f"CIFAR ResNet-18 ({D} parameters, fp32), batch {batch}, vmap(grad) margins -> "
                                   f"Rademacher k={N} with 1/sqrt(D), margin out-to-loss weights, fp16 grads.mmap / "
                                   "out_to_loss.mmap per rank"},
            "stored_vs_device_last_batch": diff, "out_to_loss_rows_positive": nz}


def run_chunked(dev):
    """GPT-2-small (random init, bf16) per-sequence gradients of the mean next-token log-probability for 16
    sequences of 512 uniform-random tokens (torch.func), projected to k = 8192 by ChunkedCudaProjector straight
    from the gradient dict: four parameter groups of at most 40M features (the smallest round cap that admits
    the 38.6M-feature embedding), each with its own seed, summed in the kernel's epilogue."""
    import torch
    try:
        import transformers
    except Exception as e:
        return {"unavailable": f"transformers not importable: {e}"}
    from torch.func import functional_call, grad, vmap
    from trak_b200 import fast_jl
    from trak_b200.projectors import make_chunked_projector
    torch.manual_seed(0)
    model = transformers.GPT2LMHeadModel(transformers.GPT2Config(attn_implementation="eager")).to(dev, torch.bfloat16).eval()
    params = {k: v.detach() for k, v in model.named_parameters()}
    buffers = {k: v.detach() for k, v in model.named_buffers()}
    widths = [p.numel() for p in params.values()]
    D, B, S, N = sum(widths), 16, 512, 8192
    ids = torch.randint(0, 50257, (B, S), generator=torch.Generator().manual_seed(0)).to(dev)

    def mean_next_token_logprob(p, seq):
        logits = functional_call(model, (p, buffers), (seq.unsqueeze(0),)).logits[0]
        logp = torch.log_softmax(logits[:-1].float(), dim=-1)
        return logp.gather(1, seq[1:, None]).mean()

    per_sample = vmap(grad(mean_next_token_logprob), in_dims=(None, 0), chunk_size=4)
    chunked = make_chunked_projector(widths, N, 0, B, dev, torch.bfloat16, max_chunk_size=40_000_000)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    g_ms = p_ms = 0.0
    steps = 3
    for it in range(steps + 1):   # the first pass warms up
        ev[0].record()
        grads = per_sample(params, ids)
        ev[1].record()
        out = chunked.project(grads, model_id=0)
        ev[2].record()
        torch.cuda.synchronize()
        if it > 0:
            g_ms += ev[0].elapsed_time(ev[1])
            p_ms += ev[1].elapsed_time(ev[2])
        del grads
    g_ms, p_ms = g_ms / steps, p_ms / steps
    finite = bool(torch.isfinite(out.float()).all())
    fast_jl.free_workspaces()
    del model, params, chunked
    torch.cuda.empty_cache()
    peak, _ = measured_peaks()
    return {"metric": "chunked_projection_examples_per_s", "value": B / (p_ms * 1e-3), "unit": "examples/s",
            "config": {"workload": f"C5: GPT-2-small ({D} parameters in {len(widths)} tensors, bf16), {B} x {S} tokens, "
                                   f"vmap(grad) -> ChunkedCudaProjector, 4 parameter groups <= 40M features, Rademacher k={N}"},
            "projection_ms": p_ms, "gradients_ms": g_ms, "step_examples_per_s": B / ((p_ms + g_ms) * 1e-3),
            "gradient_gb_per_s": B * D * 2 / (p_ms * 1e-3) / 1e9,
            "algorithmic_tflops": 2.0 * B * D * N / (p_ms * 1e-3) / 1e12,
            "frac_of_sustained_peak": 2.0 * B * D * N / (p_ms * 1e-3) / 1e12 / peak, "finite": finite}


def run_ours(args, D):
    import torch
    import torch.distributed as dist
    from trak_b200 import _lib, fast_jl

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); "
                         "use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        # torchrun starts every rank with OMP_NUM_THREADS=1; the host side of the end-to-end legs (adding score
        # blocks into the host accumulator, writing store rows) gets this rank's share of the host cores instead
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    lib = _lib.lib()

    ptype = _lib.TB_NORMAL if args.proj_type == "normal" else _lib.TB_RADEMACHER
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    g = (torch.randn(ROWS, D, device=dev, generator=gen) * 1e-2).half()
    out = torch.empty(ROWS, K_DIM, device=dev, dtype=torch.float32)

    def step(timed_events=None):
        if timed_events is not None:
            lib.tb_profile_events(timed_events[0].cuda_event, timed_events[1].cuda_event)
        fast_jl.project(g, K_DIM, SEED, TILES, ptype, out=out, strict=False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    _lib.device_status(local)

    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    for a, b in kev:  # create the underlying CUDA events
        a.record()
        b.record()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    props = torch.cuda.get_device_properties(local)
    try:
        pci = f"{props.pci_domain_id:08X}:{props.pci_bus_id:02X}:{props.pci_device_id:02X}.0"
    except AttributeError:
        pci = None
    sampler = ClockSampler(local, pci)
    barrier()
    sampler.start()
    ev0.record()
    for i in range(args.steps):
        step(kev[i])
    ev1.record()
    barrier()
    clocks = sampler.stop()
    _lib.device_status(local)
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    kernel_ms = torch.tensor([sum(a.elapsed_time(b) for a, b in kev) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(kernel_ms, op=dist.ReduceOp.MAX)
    ms_total, kernel_ms = ms.item(), kernel_ms.item()
    value = world * ROWS * args.steps / (ms_total * 1e-3)

    # ---- end to end through the public entry point, host buffers -------------------------
    # Every step copies its own batch from pinned host memory and reads its own result back.
    # Two device buffers: the copy of step i+1 runs on a side stream while step i projects
    # (what a featurize loop over a data loader does); all of it is inside the timed region.
    e2e_steps = max(2, min(args.steps, 20))
    host_in = torch.empty(ROWS, D, dtype=torch.float16).pin_memory()
    host_in.copy_(g)
    host_out = torch.empty(ROWS, K_DIM, dtype=torch.float32).pin_memory()
    bufs = [g, torch.empty_like(g)]
    copy_stream = torch.cuda.Stream(device=dev)

    def e2e_run(n_steps):
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        free = [torch.cuda.Event(), torch.cuda.Event()]
        main = torch.cuda.current_stream(dev)
        with torch.cuda.stream(copy_stream):
            bufs[0].copy_(host_in, non_blocking=True)
            ready[0].record(copy_stream)
        res = None
        for i in range(n_steps):
            cur, nxt = i % 2, (i + 1) % 2
            if i + 1 < n_steps:
                with torch.cuda.stream(copy_stream):
                    if i >= 1:
                        copy_stream.wait_event(free[nxt])  # step i-1 has finished reading that buffer
                    bufs[nxt].copy_(host_in, non_blocking=True)
                    ready[nxt].record(copy_stream)
            main.wait_event(ready[cur])
            res = fast_jl.project(bufs[cur], K_DIM, SEED, TILES, ptype, strict=False)
            free[cur].record(main)
            host_out.copy_(res, non_blocking=True)       # the step's result goes back to the host
        torch.cuda.synchronize()
        return res

    e2e_run(2)  # warms the pinned path
    _lib.device_status(local)
    barrier()
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    e2e_sec = (time.perf_counter() - t0) / e2e_steps
    _lib.device_status(local)
    e2e_t = torch.tensor([e2e_sec], device=dev)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_value = world * ROWS / e2e_t.item()
    assert torch.equal(host_out, out.cpu()), "end-to-end result differs from the resident-input result"
    # the host-to-device copy of one batch alone, all ranks copying at once: what the end-to-end figure is bound by
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(3):
        bufs[1].copy_(host_in, non_blocking=True)
    c1.record()
    torch.cuda.synchronize()
    h2d = torch.tensor([3 * ROWS * D * 2 / (c0.elapsed_time(c1) * 1e-3) / 1e9], device=dev)
    if world > 1:
        dist.all_reduce(h2d, op=dist.ReduceOp.MIN)
    h2d_gbs = h2d.item()
    g_stage = bufs[1]
    del host_in, g_stage, bufs
    torch.cuda.empty_cache()
    extras = not args.no_scoring and not args.no_extras
    # the other matrix type on the same batch, and the batch split over the ranks
    other = None
    if extras:
        oname, otype = ("rademacher", _lib.TB_RADEMACHER) if ptype == _lib.TB_NORMAL else ("normal", _lib.TB_NORMAL)
        barrier()
        o_ms, o_kernel = time_projection(lib, fast_jl, g, otype, calls=max(5, min(args.steps, 10)), warm=3)
        om = torch.tensor([o_ms, o_kernel], device=dev)
        if world > 1:
            dist.all_reduce(om, op=dist.ReduceOp.MAX)
        o_ms, o_kernel = om.tolist()
        other = (oname, o_ms, o_kernel)
    strong = run_scaling_strong(lib, fast_jl, _lib, g, rank, world) if (extras and world > 1) else None
    _lib.device_status(local)
    del g
    fast_jl.free_workspaces()
    torch.cuda.empty_cache()
    sweep = None
    if extras and rank == 0:
        try:
            sweep = run_rows_sweep(lib, fast_jl, _lib, dev, D)
        except Exception as e:  # an extra measurement must not take the main line down
            sweep = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    stored = None
    if extras and world == 1:
        try:
            stored = run_stored_matrix(lib, fast_jl, _lib, dev, D)
        except Exception as e:
            stored = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
    scoring = None if args.no_scoring else run_scoring(args, dev, rank, world, args.scale)

    def guarded(fn, *a):  # an extra measurement must not take the main line down
        try:
            return fn(*a)
        except Exception as e:
            return {"unavailable": f"{type(e).__name__}: {e}"[:300]}

    if scoring is not None and extras and args.scale == 1.0:
        scoring["e2e"] = guarded(run_scoring_e2e, dev, rank, world)
        if world == 1:
            scoring["reference_on_gpu"] = guarded(scoring_reference_on_gpu, dev)
    do_feat = not (args.no_scoring or args.no_featurize)
    featurize = guarded(run_featurize, dev, rank, world) if do_feat else None
    featurize_job = guarded(run_featurize_job, dev, rank, world) if (do_feat and extras) else None
    chunked = None
    if do_feat and extras:
        chunked = guarded(run_chunked, dev) if rank == 0 else None
        if world > 1:
            dist.barrier()

    if rank == 0:
        peak, peak_note = measured_peaks()
        flop = 2.0 * ROWS * D * K_DIM
        achieved = flop / (kernel_ms * 1e-3) / 1e12
        line = {
            "metric": "jl_projected_examples_per_s", "value": value, "unit": "examples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(D, args.proj_type),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "frac_burst": achieved / burst_peak(), "peak_burst": burst_peak(),
                         "traffic": NCU_TRAFFIC_BYTES_FULL["project_kernel"] * D / D_FULL,
                         "traffic_of_the_whole_call": {k: v * D / D_FULL for k, v in NCU_TRAFFIC_BYTES_FULL.items()},
                         "algorithmic_bytes_per_launch": ROWS * D * 2 + ROWS * K_DIM * 4,
                         "kernel": f"project_kernel<{args.proj_type}>", "kernel_ms": kernel_ms,
                         "algorithmic_flop_per_launch": flop, "peak_source": peak_note,
                         "note": ("generator-issue-bound: the Gaussian matrix costs ~470 instructions per "
                                  "16x32 tile, so the tensor pipe idles") if ptype == _lib.TB_NORMAL
                         else "MMA-bound under the power cap plus the restaging pass"},
            "e2e": {"value": e2e_value, "unit": "examples/s", "h2d_bytes_per_step": ROWS * D * 2,
                    "d2h_bytes_per_step": ROWS * K_DIM * 4, "h2d_gb_per_s_per_rank": h2d_gbs,
                    "h2d_bound_examples_per_s": world * h2d_gbs * 1e9 / (D * 2),
                    "note": "h2d_gb_per_s_per_rank: the pinned host-to-device copy of a batch timed alone with all "
                            "ranks copying at once (slowest rank); times the ranks and over the bytes of an example "
                            "it is the ceiling of the end-to-end figure"},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks,
        }
        if other is not None:
            oname, o_ms, o_kernel = other
            o_ach = flop / (o_kernel * 1e-3) / 1e12
            line[oname] = {"value": world * ROWS / (o_ms * 1e-3), "unit": "examples/s", "ms_per_step": o_ms,
                           "kernel_ms": o_kernel,
                           "roofline": {"bound": "tensor", "achieved": o_ach, "peak": peak, "unit": "TFLOP/s",
                                        "frac": o_ach / peak, "frac_burst": o_ach / burst_peak()},
                           "what": f"the same batch and shape with the {oname} matrix (resident input, CUDA events, "
                                   "max over ranks)"}
        if sweep is not None:
            line["rows_sweep"] = sweep
        if strong is not None:
            line["scaling_strong"] = strong
        if stored is not None:
            line["stored_matrix"] = stored
        line["strict"] = ("timed with strict=False (no device synchronisation after each call); the drop-in default "
                          "TRAK_B200_STRICT=1 adds a cudaDeviceSynchronize and a status read per call")
        if featurize is not None:
            line["featurize"] = featurize
        if featurize_job is not None:
            line["featurize_job"] = featurize_job
        if chunked is not None:
            line["chunked"] = chunked
        if scoring is not None:
            line["scoring"] = scoring
            if world == 1 and not args.no_cpu_baseline:
                scoring["cpu_baseline"], scoring["parity"] = scoring_cpu_baseline(os.cpu_count() or 1, dev)
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            sec, measured = cpu_port_sample(ROWS, D, threads, 2)
            nblocks = -(-K_DIM // BLOCK)
            who = "the reference's unmodified BasicProjector" if cpu_kind() == "reference" else "CPU port of BasicProjector"
            line["cpu_baseline"] = {
                "value": ROWS / sec, "unit": "examples/s", "cores": torch.get_num_threads(), "kind": cpu_kind(),
                "sample": f"{who} (normal, fp32): all {ROWS} rows x D={D} onto 2 of "
                          f"{nblocks} column blocks of {BLOCK} in {measured:.1f} s, scaled by {nblocks}/2"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    global ROWS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scale", type=float, default=1.0, help="fraction of D (profiler captures)")
    ap.add_argument("--proj-type", choices=["normal", "rademacher"], default="normal",
                    help="normal = the benchmark workload; rademacher for profiling the other matrix type")
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows per GPU (128 = the benchmark workload; other values for profiling other kernel shapes)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-featurize", action="store_true",
                    help="skip the featurize-step measurement (thousands of small PyTorch launches: slow under a profiler)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the secondary measurements (other matrix type, row sweep, strong scaling, scoring end to "
                         "end, featurize job, chunked projection)")
    ap.add_argument("--no-scoring", action="store_true",
                    help="skip the after-kernel scoring and the featurize-step measurements")
    args = ap.parse_args()
    ROWS = args.rows
    D = max(1024, int(D_FULL * args.scale))
    if args.impl == "reference":
        run_reference(args, D)
    else:
        run_ours(args, D)


if __name__ == "__main__":
    main()
