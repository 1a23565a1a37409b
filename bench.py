#!/usr/bin/env python
"""Benchmark of the rank-7 MLP prefill path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Metric: MLP prefill effective TFLOP/s (6*M*H*I / time for one layer:
gate_up + down, dense-equivalent FLOPs) and % speedup over the dense bf16 path.

N = 1   one "step" = one fused MLP layer of the single-layer configuration
        (4096 tokens x hidden 5120, intermediate 17408): fused residual+RMSNorm+A planes,
        chained rank-7 gate_up GEMM (SwiGLU + down's A planes in its epilogue), rank-split
        rank-7 down GEMM, residual add.  The dense arms (own tcgen05 GEMM, cuBLAS) run
        interleaved in the same process for the speedup figures (which arm goes first rotates
        step by step), and 2048 / 8192 tokens are measured beside the headline 4096.  Arms that
        alternate on one GPU share its power limiter, which flatters the hungrier rank-7 arm:
        `sustained` and --rounds are the fair comparisons (`speedup_note` says so in the line).
N > 1   the tensor-parallel configuration (8192 tokens, hidden 8192, intermediate 28672)
        split over the intermediate dimension; the ranks' partial outputs are combined by
        the package's own kernels over NVLink peer memory (--exchange peer: pushed from inside
        the down GEMM, reduced and gathered after a barrier) or by one NCCL all-reduce per
        layer (--exchange nccl); total work is fixed as N grows ("strong" scaling).  One
        process per GPU under torchrun.

Timing: CUDA events on the launching stream around every step, L2 flushed (256 MiB memset)
between steps outside the timed region, max over ranks.  `e2e` measures K steps host to host
through lcgemm.streaming.HostStreamedLayer: every step's input comes from pinned host memory
and its result goes back to the host inside the timed region, the copies of neighbouring
steps overlapping the compute; the figure with copy, compute and copy one after the other
is reported beside it (`serial_ms_per_step`).

The N = 1 line also carries `sustained` (both layer arms run back to back for seconds, in
alternating blocks, with the SM clock sampled per arm), `gemm_only` (the two GEMMs without
their seams, rank-7 against dense tcgen05), `residual_folded` (the layer with its closing add
folded into `down`, an option that is off by default) and `tp1_same_config` (the tensor-parallel
configuration on one GPU: the anchor of the strong-scaling curve); the N > 1 line carries
`parity` (the fused exchange's output against the NCCL exchange and against a dense cuBLAS
evaluation of a row sample, checked before anything is timed), `phases_ms` and the same anchor,
measured on rank 0 after the timed steps.

--impl reference times the reference's own CPU evaluation of the scheme on the host cores
(its torch functions from the unmodified install under baseline/_ref when that is present,
else the oracle port of them), on a bounded row sample of the workload, and evaluates the
fp32 CPU configuration (2048 x 4096 x 4096) at its stated size.

--rounds R runs the single-layer comparison as R matched rounds of fresh processes (one
process per arm, order alternating) and reports the median and quartiles of the per-round
speedups, the reference's protocol for making numbers comparable.
--ref-kernels times the reference's own sm_100 kernels (from baseline/_ref, one GPU) beside
this library's, or prints why they are unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT / "writes-that-matter_b200"), str(ROOT)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "MLP prefill effective TFLOP/s (6*M*H*I/t per layer) & % speedup vs dense bf16"
SINGLE = dict(tokens=4096, hidden=5120, inter=17408)
TP = dict(tokens=8192, hidden=8192, inter=28672)
EPS = 1e-6
CPU_SAMPLE_TOKENS = 256
FLUSH_BYTES = 256 << 20
# dram__bytes_read.sum + dram__bytes_write.sum of one gate_up launch at the headline shape,
# from the ncu capture summarised in profiles/k_gemm_gate_up_chain.md (4096 tokens).
GATE_UP_DRAM_TRAFFIC_BYTES = 2_218_558_208   # 1 579 047 424 read + 639 510 784 written


def layer_flops(tokens, hidden, inter):
    return 6.0 * tokens * hidden * inter


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


# ------------------------------------------------------------------ clock sampling
class ClockWatch:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
               0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------ synthetic data
def make_layer_tensors(tokens, hidden, inter, device, seed=0, inter_local=None, rank=0):
    """Seeded synthetic tensors with the benchmark's distributions: x ~ N(0,1),
    norm weight stored as w with effective scale 1 + w, w ~ N(0, 0.01), weights ~ N(0, 0.02)."""
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16
    x = torch.randn((tokens, hidden), generator=g, device=device).to(bf)
    nw = (torch.randn((hidden,), generator=g, device=device) * 0.01).to(bf)
    gw = torch.Generator(device=device).manual_seed(seed + 1000 + rank)
    il = inter if inter_local is None else inter_local
    wgu = (torch.randn((2 * il, hidden), generator=gw, device=device) * 0.02).to(bf)
    wd = (torch.randn((hidden, il), generator=gw, device=device) * 0.02).to(bf)
    return x, nw, wgu, wd


# ------------------------------------------------------------------------- timing
def timed_steps(step_fn, steps, warmup, flush, sync_all, pre_step=None):
    """Per-step CUDA-event times (ms).  `flush` is zeroed between steps, outside the events."""
    for _ in range(warmup):
        if pre_step:
            pre_step()
        step_fn()
    sync_all()
    times = []
    for _ in range(steps):
        flush.zero_()
        if pre_step:
            pre_step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step_fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    sync_all()
    return times


def streamed_e2e_ms(layer, tokens, hidden, x_host, out_host, args, sync_all, group=None, timeline=None):
    """ms per step of K host-to-host steps through HostStreamedLayer, one timed region.  With a
    dict in `timeline`, a second, untimed run records per-step events on the three streams and
    leaves their summary there."""
    from lcgemm.streaming import HostStreamedLayer

    if timeline is not None:
        tl = HostStreamedLayer(layer, tokens, hidden, group=group, timeline=True)
        tl.begin()
        for _ in range(max(8, args.steps)):
            tl.submit(x_host, out_host)
        tl.end()
        timeline.update(tl.timeline_summary())
        sync_all()
    st = HostStreamedLayer(layer, tokens, hidden, group=group)

    def run(k):
        st.begin()
        for _ in range(k):
            st.submit(x_host, out_host)
        st.end()

    run(max(args.warmup, 2))
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(args.steps)
    e1.record()
    e1.synchronize()
    sync_all()
    return e0.elapsed_time(e1) / args.steps


def _host_threads():
    """Use every host core for the CPU arm (torchrun sets OMP_NUM_THREADS=1 for its workers)."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def _import_reference():
    """The reference's own torch functions for this path, from the unmodified install under
    baseline/_ref (git-ignored; it travels with the working tree).  The reference package shares
    its name with this repository's, so it is imported with only its own directory on the path;
    callers of this function never touch this repository's package afterwards.  Returns a
    namespace, or None when the install is absent or does not import."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "lcgemm" / "scheme.py").exists():
        return None
    saved_path, saved_mods = list(sys.path), {k: v for k, v in sys.modules.items()
                                              if k == "lcgemm" or k.startswith("lcgemm.")}
    for k in saved_mods:
        del sys.modules[k]
    ours = str(ROOT / "writes-that-matter_b200")
    sys.path[:] = [str(ref)] + [q for q in sys.path if q != ours]
    try:
        import lcgemm.chain_gauge as gauge
        import lcgemm.planes as planes
        import lcgemm.scheme as scheme

        if str(ref) not in str(Path(scheme.__file__).resolve()):
            raise ImportError("lcgemm resolved outside baseline/_ref")
        try:
            from lcgemm.integrate.qwen_patch import _reference as functional
        except Exception:
            functional = None
        return type("Ref", (), dict(scheme=scheme, planes=planes, gauge=gauge,
                                    functional=staticmethod(functional) if functional else None))
    except Exception:
        for k in [k for k in sys.modules if k == "lcgemm" or k.startswith("lcgemm.")]:
            del sys.modules[k]
        sys.modules.update(saved_mods)
        sys.path[:] = saved_path
        return None


def _ref_a_planes(x, sch):
    """A planes by the reference's own pattern (lcgemm/chain_gauge.py:91-98 without SwiGLU or
    gauge): fp32 signed sums over `Scheme.a_terms`, one rounding."""
    m, k = x.shape
    m2, k2 = m // sch.p, k // sch.q
    out = torch.empty((sch.rank * m2, k2), dtype=x.dtype)
    for r, terms in enumerate(sch.a_terms):
        acc = torch.zeros(m2, k2, dtype=torch.float32)
        for bi, bk, coeff in terms:
            acc += float(coeff) * x[bi * m2:(bi + 1) * m2, bk * k2:(bk + 1) * k2].float()
        out[r * m2:(r + 1) * m2] = acc.to(x.dtype)
    return out


def _ref_combine(a_pl, b_pl, sch, m, n, out_dtype):
    """C[i][j] = sum_r c[r][i,j] * (A~_r @ B~_r^T) over `Scheme.c_terms` (lcgemm/scheme.py:160-163);
    the products in fp32 from the (rounded) planes."""
    m2, n2 = m // sch.p, n // sch.s
    c = torch.zeros((m, n), dtype=torch.float32)
    for r in range(sch.rank):
        prod = a_pl[r * m2:(r + 1) * m2].float() @ b_pl[r * n2:(r + 1) * n2].float().T
        for bi, bj, coeff in sch.c_terms[r]:
            c[bi * m2:(bi + 1) * m2, bj * n2:(bj + 1) * n2] += float(coeff) * prod
    return c.to(out_dtype)


def reference_cpu_step(ref, tokens, hidden, inter):
    """One MLP layer on the host by the reference's own functions: RMSNorm as its functional
    layer does it (lcgemm/integrate/qwen_patch.py:49-52), its `prepare_b` / `prepare_down_b`
    planes (untimed, offline in the reference too), the scheme evaluation composed from
    `Scheme.a_terms` / `c_terms`, and its `chain_a_planes` for the SwiGLU seam."""
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    x = torch.randn((tokens, hidden), generator=g).to(bf)
    nw = (torch.randn((hidden,), generator=g) * 0.01).to(bf)
    wgu = (torch.randn((2 * inter, hidden), generator=g) * 0.02).to(bf)
    wd = (torch.randn((hidden, inter), generator=g) * 0.02).to(bf)
    gs, ds = ref.scheme.load("2x2_postsum_cse"), ref.scheme.load("2x2_locality_ordered")
    gate_b = ref.planes.prepare_b(wgu, gs)
    down_b = ref.gauge.prepare_down_b(wd, ds)

    def step():
        hf = x.float()
        y = (hf * torch.rsqrt(hf.square().mean(-1, keepdim=True) + EPS) * (nw.float() + 1.0)).to(bf)
        z = _ref_combine(_ref_a_planes(y, gs), gate_b, gs, tokens, 2 * inter, bf)
        d_pl = ref.gauge.chain_a_planes(z, ds)
        out = _ref_combine(d_pl, down_b, ds, tokens, hidden, bf)
        return (x.float() + out.float()).to(bf)

    return step, layer_flops(tokens, hidden, inter)


def run_cpu_sample(tokens, hidden, inter, threads=None):
    """The oracle's chained rank-7 layer on a row sample, host cores; returns (step, flops)."""
    from oracle import lc_oracle as O

    if threads:
        torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    x = torch.randn((tokens, hidden), generator=g).to(bf)
    nw = (torch.randn((hidden,), generator=g) * 0.01).to(bf)
    wgu = (torch.randn((2 * inter, hidden), generator=g) * 0.02).to(bf)
    wd = (torch.randn((hidden, inter), generator=g) * 0.02).to(bf)
    gt, dt = O.Tables("2x2_postsum_cse"), O.Tables("2x2_locality_ordered")
    gate_b = O.prepare_b(wgu, gt).float()          # offline in the reference: not timed
    down_b = O.prepare_down_b(wd, dt).float()
    zero = torch.zeros_like(x)

    def step():
        a_pl, h = O.norm_planes(zero, x, nw, EPS, gt)
        prods = O.products(a_pl, gate_b, gt.rank)
        z = O.combine_as_kernel(prods, gt, tokens, 2 * inter).to(bf)
        d_pl = O.chain_a_planes(z, dt)
        prods = O.products(d_pl, down_b, dt.rank)
        out = O.combine_as_kernel(prods, dt, tokens, hidden, rank_split=True)
        return (h.float() + out).to(bf)

    return step, layer_flops(tokens, hidden, inter)


def cpu_baseline(hidden, inter, reps=3):
    """The oracle port on a row sample.  (Inside the GPU arm's process this repository's own
    package is loaded, so the reference install, which shares its name, is left to
    `--impl reference`.)"""
    cores = _host_threads()
    step, flops = run_cpu_sample(CPU_SAMPLE_TOKENS, hidden, inter)
    step()
    best = min(_wall(step) for _ in range(reps))
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": cores,
            "kind": "port",
            "sample": f"{CPU_SAMPLE_TOKENS} of the tokens, full hidden {hidden} / intermediate {inter}; "
                      f"oracle chained rank-7 layer (torch fp32 matmul on bf16-rounded planes), "
                      f"B planes prepared untimed, best of {reps}, {best * 1e3:.1f} ms"}


def _wall(fn):
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def cpu_config_fp32(ref, reps=5):
    """The CPU configuration at its stated size: C = A @ B through the one-level rank-7 scheme in
    fp32, A (2048 x 4096) ~ N(0, 1), B (4096 x 4096) ~ N(0, 0.02), seed 0, against dense A @ B."""
    torch.manual_seed(0)
    m, k, n = 2048, 4096, 4096
    a = torch.randn(m, k)
    b = torch.randn(k, n) * 0.02
    w = b.T.contiguous()                       # weights are (N, K), K-major
    dense = a @ b
    t_dense = min(_wall(lambda: a @ b) for _ in range(reps))
    out = {"shape": [m, k, n], "dtype": "f32", "seed": 0, "dense_ms": t_dense * 1e3, "schemes": {}}
    for name in ("2x2_postsum_cse", "2x2_locality_ordered"):
        if ref is not None:
            sch = ref.scheme.load(name)
            b_pl = ref.planes.prepare_b(w, sch)
            fn = lambda: _ref_combine(_ref_a_planes(a, sch), b_pl, sch, m, n, torch.float32)
        else:
            from oracle import lc_oracle as O

            tb = O.Tables(name)
            fn = lambda: O.scheme_matmul(a, w, tb, mode="fp32")
        c = fn()
        best = min(_wall(fn) for _ in range(reps))
        out["schemes"][name] = {
            "rel_fro_vs_dense": float(((c - dense).norm() / dense.norm()).item()),
            "max_abs_vs_dense": float((c - dense).abs().max().item()),
            "ms": best * 1e3, "b_planes": "prepared untimed"}
    return out


# ------------------------------------------------------------------ reference arm
def run_reference_arm(args, rank):
    if rank != 0:
        return
    cores = _host_threads()
    cfg = SINGLE if args.gpus == 1 else TP
    ref = _import_reference()
    if ref is not None:
        kind = "reference"
        step, flops = reference_cpu_step(ref, CPU_SAMPLE_TOKENS, cfg["hidden"], cfg["inter"])
        what = ("the reference's own torch functions from the unmodified install under baseline/_ref "
                "(Scheme tables, prepare_b, prepare_down_b, chain_a_planes; the scheme evaluation "
                "composed from Scheme.a_terms / c_terms)")
    else:
        kind = "port"
        step, flops = run_cpu_sample(CPU_SAMPLE_TOKENS, cfg["hidden"], cfg["inter"])
        what = "oracle port of the reference's torch scheme evaluation (baseline/_ref absent)"
    for _ in range(min(args.warmup, 2)):
        step()
    steps = max(1, min(args.steps, 100))
    times = [_wall(step) for _ in range(steps)]
    ms = statistics.mean(times) * 1e3
    val = flops / (ms * 1e-3) / 1e12
    sample = (f"{CPU_SAMPLE_TOKENS}-token row sample of the {cfg['tokens']}-token layer per step, "
              f"{steps} timed steps on the host cores; {what}")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": _workload_name(args.gpus), **cfg, "cpu_sample_tokens": CPU_SAMPLE_TOKENS},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "what": "CPU evaluation of the path; the reference's sm_100 device kernels are timed by "
                "`bench.py --ref-kernels` (one GPU)",
        "cpu_config_fp32": cpu_config_fp32(ref) if args.gpus == 1 else None,
    }))


def _workload_name(gpus):
    if gpus == 1:
        return "single fused MLP layer, 4096 tokens x 5120, intermediate 17408 (the single-layer configuration)"
    return f"tensor-parallel MLP tp={gpus}, 8192 tokens x 8192, intermediate 28672 (the tensor-parallel configuration)"


# --------------------------------------------------------------------- our arm
def bench_layer_arms(tokens, hidden, inter, steps, warmup, flush, device, with_parts=False, graphs=True):
    """Rank-7 layer and the two dense arms, interleaved step by step.  Returns a dict of
    median / mean ms per arm, and (optionally) the gate_up GEMM's own duration."""
    from lcgemm import ops
    from lcgemm.layer import DenseMlpLayer, Rank7MlpLayer

    x, nw, wgu, wd = make_layer_tensors(tokens, hidden, inter, device)
    r7 = Rank7MlpLayer(tokens, nw, wgu, wd, EPS)
    dn = DenseMlpLayer(tokens, nw, wgu, wd, EPS, gemm="tcgen05")
    cb = DenseMlpLayer(tokens, nw, wgu, wd, EPS, gemm="cublas")
    part_events = []

    def r7_step():                      # r7(x) kernel by kernel, so that events can sit around the gate_up GEMM
        gp, dp = r7.gate_plan, r7.down_plan
        a = gp.a_planes(x, None, nw, EPS)
        if with_parts and collecting[0]:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gp.gemm(a, r7.gate_bw)
            e1.record()
            part_events.append((e0, e1))
        else:
            gp.gemm(a, r7.gate_bw)
        d = dp(prepared_w=r7.down_bw)
        ops.add(x, d, out=r7.out)

    collecting = [False]
    arms = {"rank7": r7_step, "dense_tcgen05": lambda: dn(x), "dense_cublas": lambda: cb(x)}
    for fn in arms.values():
        for _ in range(warmup):
            fn()
    torch.cuda.synchronize()
    launches_per_step = 0
    if graphs:
        # Every arm as one CUDA graph replay per step (the same kernels, launched once); the
        # gate_up GEMM's own duration comes from a few eager steps, where events can sit inside.
        from lcgemm.layer import CapturedLayer

        if with_parts:
            collecting[0] = True
            for _ in range(max(3, steps // 2)):
                flush.zero_()
                r7_step()
            collecting[0] = False
            torch.cuda.synchronize()
        before = ops.launch_count()
        r7(x), dn(x)
        launches_per_step = ops.launch_count() - before
        arms = {"rank7": CapturedLayer(r7, x), "dense_tcgen05": CapturedLayer(dn, x),
                "dense_cublas": CapturedLayer(cb, x)}
    else:
        collecting[0] = True
    launches0 = ops.launch_count()
    times = {k: [] for k in arms}
    names = list(arms)
    for s in range(steps):
        # the arm that goes first rotates: an arm that always ran behind the other two would always
        # start from the hottest, most power-limited GPU
        for name in names[s % len(names):] + names[:s % len(names)]:
            fn = arms[name]
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            times[name].append(e0.elapsed_time(e1))
    torch.cuda.synchronize()
    ops.check_status()
    res = {k: {"mean_ms": statistics.mean(v), "median_ms": statistics.median(v)} for k, v in times.items()}
    res["launches"] = launches_per_step * steps if graphs else ops.launch_count() - launches0
    if with_parts:
        res["gate_up_ms"] = statistics.mean(e0.elapsed_time(e1) for e0, e1 in part_events)
    res["objects"] = (r7, x)
    res["arms"] = arms
    return res


def run_ours(args, rank, world, device):
    import torch.distributed as dist
    from lcgemm import ops

    flush = torch.empty(FLUSH_BYTES, dtype=torch.int8, device=device)
    peak_burst, peak_sustained, peak_kind = measured_peaks()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if world == 1:
        cfg = SINGLE
        with ClockWatch(torch.cuda.current_device()) as cw:
            head = bench_layer_arms(cfg["tokens"], cfg["hidden"], cfg["inter"], args.steps, args.warmup,
                                    flush, device, with_parts=True, graphs=args.graphs)
        clocks = cw.summary()
        r7, x = head.pop("objects")
        head_arms = head.pop("arms")
        sustained = None
        if args.sustain_seconds > 0:
            sustained = sustained_block(head_arms, args.sustain_seconds, torch.cuda.current_device())
            sr, sd_, sc = (sustained[k] for k in ("rank7", "dense_tcgen05", "dense_cublas"))
            sustained = {
                "seconds_per_arm": args.sustain_seconds, "arms": sustained,
                "how": "alternating blocks of ~0.4 s per arm, steps back to back (one step's operands exceed "
                       "L2), SM clock sampled through NVML while each block runs",
                "speedup_vs_dense_tcgen05_pct": (sd_["ms_per_step"] / sr["ms_per_step"] - 1) * 100,
                "speedup_vs_cublas_pct": (sc["ms_per_step"] / sr["ms_per_step"] - 1) * 100,
                "cycles_speedup_vs_dense_tcgen05_pct":
                    (sd_["mcycles_per_step"] / sr["mcycles_per_step"] - 1) * 100 if sr["mcycles_per_step"] else None,
                "rank7_effective_tflops": layer_flops(**cfg) / (sr["ms_per_step"] * 1e-3) / 1e12,
            }
        del head_arms
        ms = head["rank7"]["mean_ms"]
        flops = layer_flops(**cfg)
        value = flops / (ms * 1e-3) / 1e12

        # end to end through the public layer call: input from pinned host memory, result back
        x_host = x.cpu().pin_memory()
        out_host = torch.empty_like(x_host).pin_memory()
        x_dev = torch.empty_like(x)

        def e2e_step():
            x_dev.copy_(x_host, non_blocking=True)
            out_host.copy_(r7(x_dev), non_blocking=True)

        e2e_serial_ms = statistics.mean(timed_steps(e2e_step, args.steps, args.warmup, flush, sync_all))
        e2e_ms = streamed_e2e_ms(r7, cfg["tokens"], cfg["hidden"], x_host, out_host, args, sync_all)
        ops.check_status()

        by_tokens = {}
        for tokens in (2048, 8192):
            del r7, x
            torch.cuda.empty_cache()
            sub = bench_layer_arms(tokens, cfg["hidden"], cfg["inter"], max(5, args.steps // 2),
                                   args.warmup, flush, device, graphs=args.graphs)
            r7, x = sub.pop("objects")
            by_tokens[str(tokens)] = _arm_summary(sub, layer_flops(tokens, cfg["hidden"], cfg["inter"]))
        by_tokens[str(cfg["tokens"])] = _arm_summary(head, flops)
        del r7, x
        torch.cuda.empty_cache()
        sub_steps = max(5, args.steps // 2)
        gemm_only = gemm_only_block(cfg["tokens"], cfg["hidden"], cfg["inter"], sub_steps, args.warmup, flush, device)
        torch.cuda.empty_cache()
        folded = residual_folded_block(cfg["tokens"], cfg["hidden"], cfg["inter"], sub_steps, args.warmup, flush, device)
        torch.cuda.empty_cache()
        anchor = tp1_same_config(max(5, args.steps // 3), args.warmup, flush, device)

        gate_flops = 2.0 * cfg["tokens"] * cfg["hidden"] * 2 * cfg["inter"]
        gate_ms = head["gate_up_ms"]
        executed = 0.875 * gate_flops / (gate_ms * 1e-3) / 1e12
        roofline = {
            "bound": "tensor", "kernel": "k_gemm<2, planes> (chained rank-7 gate_up, 4096x5120x34816)",
            "achieved": executed, "peak": peak_burst, "unit": "TFLOP/s", "frac": executed / peak_burst,
            "peak_kind": f"{peak_kind} cuBLAS bf16 burst; sustained {peak_sustained}",
            "flops_per_launch": 0.875 * gate_flops, "effective_tflops": gate_flops / (gate_ms * 1e-3) / 1e12,
            "ms_per_launch": gate_ms, "traffic": GATE_UP_DRAM_TRAFFIC_BYTES,
            "traffic_from": "profiles/k_gemm_gate_up_chain.md (one ncu capture of this launch; not re-measured by this run)",
        }
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": _workload_name(1), **cfg, "l2": "flushed between steps (256 MiB memset)",
                       "launch": ("one CUDA graph replay per step, every arm" if args.graphs
                                  else "eager kernel launches"),
                       "schemes": {"gate_up": "2x2_postsum_cse", "down": "2x2_locality_ordered"}},
            "clocks": clocks,
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2,
                    "how": "lcgemm.streaming.HostStreamedLayer: every step copies its batch from pinned "
                           "host memory and its result back; the copies of neighbouring steps overlap "
                           "the compute (three streams, double buffers); per-step weights + activations "
                           "(0.9 GB) exceed L2, no flush",
                    "serial_ms_per_step": e2e_serial_ms},
            "gpu_launches": head["launches"],
            "speedup_vs_dense_tcgen05_pct": by_tokens[str(cfg["tokens"])]["speedup_vs_dense_tcgen05_pct"],
            "speedup_vs_cublas_pct": by_tokens[str(cfg["tokens"])]["speedup_vs_cublas_pct"],
            "speedup_note": "arms alternate step by step on one GPU under one power limiter, which flatters "
                            "the hungrier rank-7 arm; `sustained` (blocks per arm) and `bench.py --rounds R` "
                            "(a fresh process per arm) are the fair comparisons",
            "by_tokens": by_tokens, "roofline": roofline,
            "sustained": sustained, "gemm_only": gemm_only, "residual_folded": folded,
            "tp1_same_config": anchor,
            "cpu_baseline": cpu_baseline(cfg["hidden"], cfg["inter"]),
        }
        print(json.dumps(line))
        return

    # ------------------------------------------------------------- tensor parallel
    from lcgemm.tp import TensorParallelMlp

    cfg = TP
    il = cfg["inter"] // world
    x, nw, wgu, wd = make_layer_tensors(cfg["tokens"], cfg["hidden"], cfg["inter"], device,
                                        inter_local=il, rank=rank)
    layer = TensorParallelMlp(cfg["tokens"], nw, wgu, wd, EPS, slabs=args.slabs,
                              fused=args.exchange == "peer")
    parity = None
    if args.exchange == "peer":
        parity = tp_parity(layer, x, nw, wgu, wd, cfg, rank, world, device)
        ops.check_status()
        bad = [k for k, bound in parity["bounds"].items() if not parity[k] <= bound]
        if bad or not parity["ranks_bit_identical"]:
            if rank == 0:
                print(json.dumps({"error": "tensor-parallel output failed its parity check", "parity": parity}))
            raise SystemExit(3)
    launches0 = ops.launch_count()
    layer(x)
    launches = (ops.launch_count() - launches0) * args.steps
    step = lambda: layer(x)
    graphed = args.graphs and args.exchange == "peer"
    if graphed:      # the whole layer, exchange included, as one CUDA graph replay per step
        from lcgemm.tp import CapturedTensorParallel

        step = CapturedTensorParallel(layer, x)
    with ClockWatch(torch.cuda.current_device()) as cw:
        times = timed_steps(step, args.steps, args.warmup, flush, sync_all,
                            pre_step=(lambda: dist.barrier()))
    ops.check_status()
    x_host = x.cpu().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    x_dev = torch.empty_like(x)

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        out = layer(x_dev)
        if rank == 0:
            out_host.copy_(out, non_blocking=True)

    e2e_times = timed_steps(e2e_step, args.steps, args.warmup, flush, sync_all,
                            pre_step=(lambda: dist.barrier()))
    rows = cfg["tokens"] // world
    x_slice = x_host[rank * rows:(rank + 1) * rows].clone().pin_memory()
    out_slice = torch.empty_like(x_slice).pin_memory()
    dist.barrier()
    timeline = {}
    e2e_stream_ms = streamed_e2e_ms(layer, cfg["tokens"], cfg["hidden"], x_slice, out_slice, args,
                                    sync_all, group=dist.group.WORLD, timeline=timeline)
    phases = tp_phase_times(layer, x, args.steps, flush, sync_all) if args.exchange == "peer" else None
    # The one-GPU anchor comes last: run in front of the timed steps it leaves rank 0's GPU hot and
    # power-limited while the others are cool, and every step then waits for rank 0.
    anchor = None
    if args.tp1_anchor:
        if rank == 0:
            torch.cuda.synchronize()
            time.sleep(2.0)      # let the GPU leave the power-limited state the runs above put it in
            anchor = tp1_same_config(max(5, args.steps // 3), args.warmup, flush, device)
            anchor["when"] = "after the timed steps and a 2 s pause, on rank 0 alone"
        dist.barrier()
    t = torch.tensor([statistics.mean(times), e2e_stream_ms, statistics.mean(e2e_times)], device=device,
                     dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, e2e_serial_ms = t.tolist()
    if rank == 0:
        flops = layer_flops(**cfg)
        print(json.dumps({
            "metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": _workload_name(world), **cfg, "parallelism": f"tp{world}",
                       "down_slabs": args.slabs, "exchange": args.exchange,
                       "launch": "one CUDA graph replay per step" if graphed else "eager kernel launches",
                       "all_reduce_bytes": cfg["tokens"] * cfg["hidden"] * 2,
                       "l2": "flushed between steps (256 MiB memset)"},
            "clocks": cw.summary(),
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2,
                    "how": "lcgemm.streaming.HostStreamedLayer: each rank copies its tokens/tp rows of "
                           "the batch from pinned host memory, stores them into every peer's input buffer "
                           "with DMA copies over NVLink on the copy-in stream (a barrier between the ranks "
                           "on the compute stream follows), and copies its rows of the result back; "
                           "copies overlapped with compute",
                    "serial_ms_per_step": e2e_serial_ms, "timeline_rank0": timeline},
            "phases_ms": phases,
            "gpu_launches": launches * world,
            "roofline": {"bound": "tensor", "kernel": "whole step (per-rank rank-7 chain + exchange)",
                         "achieved": 0.875 * flops / (ms * 1e-3) / 1e12 / world, "peak": peak_burst,
                         "unit": "TFLOP/s per GPU", "frac": 0.875 * flops / (ms * 1e-3) / 1e12 / world / peak_burst,
                         "peak_kind": f"{peak_kind} cuBLAS bf16 burst",
                         "flops_per_launch": 0.875 * flops / world,
                         "flops_per_launch_is": "executed FLOPs of one rank's whole step (gate_up + down), "
                                                "the quantity `achieved` divides by the step time",
                         "traffic": None},
            "parity": parity, "tp1_same_config": anchor,
            "strong_scaling_vs_tp1": (anchor["ms_per_step"] / ms / world) if anchor else None,
        }))


def _arm_summary(res, flops):
    r7, dt, cb = (res[k]["mean_ms"] for k in ("rank7", "dense_tcgen05", "dense_cublas"))
    return {"rank7_ms": r7, "dense_tcgen05_ms": dt, "dense_cublas_ms": cb,
            "rank7_effective_tflops": flops / (r7 * 1e-3) / 1e12,
            "rank7_executed_tflops": 0.875 * flops / (r7 * 1e-3) / 1e12,
            "dense_tcgen05_tflops": flops / (dt * 1e-3) / 1e12,
            "dense_cublas_tflops": flops / (cb * 1e-3) / 1e12,
            "speedup_vs_dense_tcgen05_pct": (dt / r7 - 1.0) * 100.0,
            "speedup_vs_cublas_pct": (cb / r7 - 1.0) * 100.0}


# --------------------------------------------- blocks beside the headline (same run)
def sustained_block(arms, seconds, device_index, block_s=0.4):
    """Every arm back to back for `seconds` in total, in alternating blocks of about `block_s`,
    the SM clock sampled while each block runs.  No flush inside a block: one step's weights and
    planes (1.5 GB) exceed L2.  Returns per arm the ms per step, the median SM clock of its own
    blocks and their product (cycles per step, the clock-independent figure)."""
    reps = {}
    for name, fn in arms.items():
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            fn()
        e1.record()
        e1.synchronize()
        reps[name] = max(5, int(block_s * 1e3 / (e0.elapsed_time(e1) / 5)))
    acc = {name: {"ms": 0.0, "steps": 0, "mhz": []} for name in arms}
    while min(a["ms"] for a in acc.values()) < seconds * 1e3:
        for name, fn in arms.items():
            with ClockWatch(device_index) as cw:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps[name]):
                    fn()
                e1.record()
                e1.synchronize()
            acc[name]["ms"] += e0.elapsed_time(e1)
            acc[name]["steps"] += reps[name]
            acc[name]["mhz"] += cw.samples
    out = {}
    for name, a in acc.items():
        ms = a["ms"] / a["steps"]
        mhz = statistics.median(a["mhz"]) if a["mhz"] else None
        out[name] = {"ms_per_step": ms, "steps": a["steps"], "seconds": a["ms"] / 1e3, "sm_mhz_median": mhz,
                     "mcycles_per_step": ms * mhz / 1e3 if mhz else None}
    return out


def gemm_only_block(tokens, hidden, inter, steps, warmup, flush, device):
    """The two GEMMs of the layer without their seams: the rank-7 GEMM from operands that are
    already in place (gate_up: A planes written beforehand; down: planes written beforehand, and
    the form whose plane warps build the A planes inside the kernel from the activation matrix) against
    the dense tcgen05 GEMM on the same inputs.  Cold L2, arms interleaved."""
    from lcgemm import ops, scheme as S

    bf = torch.bfloat16
    x, _, wgu, wd = make_layer_tensors(tokens, hidden, inter, device)
    cse, loc = S.load("2x2_postsum_cse"), S.load("2x2_locality_ordered")
    lead = S.load("2x2_locality_lead_single")
    s_act = torch.randn((tokens, inter), device=device).to(bf)
    a_pl, d_pl = ops.a_planes(x, cse), ops.a_planes(s_act, loc)
    bp_g, bp_d, bp_l = ops.prepare_b(wgu, cse), ops.prepare_b(wd, loc), ops.prepare_b(wd, lead)
    scr = torch.empty(ops.ahead_scratch_bytes(lead, tokens, inter), dtype=torch.uint8, device=device)
    z = torch.empty((tokens, 2 * inter), device=device, dtype=bf)
    o = torch.empty((tokens, hidden), device=device, dtype=bf)
    arms = {
        "gate_up_rank7": lambda: ops.gemm_r7_planes(cse, a_pl, bp_g, tokens, 2 * inter, hidden, out=z),
        "gate_up_dense_tcgen05": lambda: ops.gemm_dense(x, wgu, out=z),
        "down_rank7_planes": lambda: ops.gemm_r7_planes(loc, d_pl, bp_d, tokens, hidden, inter, out=o),
        "down_rank7_ahead": lambda: ops.gemm_r7_ahead(s_act, bp_l, hidden, lead, out=o, scratch=scr),
        "down_dense_tcgen05": lambda: ops.gemm_dense(s_act, wd, out=o),
    }
    for fn in arms.values():
        for _ in range(warmup):
            fn()
    torch.cuda.synchronize()
    times = {k: [] for k in arms}
    for _ in range(steps):
        for name, fn in arms.items():
            times[name] += _event_times(fn, 1, 0, flush)
    ops.check_status()
    t = {k: statistics.mean(v) for k, v in times.items()}
    return {"tokens": tokens, "ms": t, "note": "operands in place, no seams; hybrid schedule",
            "gate_up_speedup_pct": (t["gate_up_dense_tcgen05"] / t["gate_up_rank7"] - 1) * 100,
            "down_planes_speedup_pct": (t["down_dense_tcgen05"] / t["down_rank7_planes"] - 1) * 100,
            "down_ahead_speedup_pct": (t["down_dense_tcgen05"] / t["down_rank7_ahead"] - 1) * 100}


def residual_folded_block(tokens, hidden, inter, steps, warmup, flush, device):
    """The layer with its closing `x + mlp` folded into `down` (`Rank7MlpLayer(fuse_residual=True)`:
    the gate_up kernel fills down's output with x instead of zeros and down reduce-adds onto it)
    against the default layer, one graph replay per step, interleaved, cold L2; and what it costs:
    both outputs against x + a dense cuBLAS evaluation of the MLP on 256 sampled rows."""
    from lcgemm.layer import CapturedLayer, Rank7MlpLayer

    x, nw, wgu, wd = make_layer_tensors(tokens, hidden, inter, device)
    plain = Rank7MlpLayer(tokens, nw, wgu, wd, EPS)
    try:
        folded = Rank7MlpLayer(tokens, nw, wgu, wd, EPS, fuse_residual=True)
    except ValueError as e:
        return {"tokens": tokens, "unavailable": str(e)}
    rows = torch.arange(0, tokens, max(1, tokens // 256), device=device)[:256]
    xs = x[rows].float()
    xn = (xs * torch.rsqrt(xs.square().mean(-1, keepdim=True) + EPS) * (nw.float() + 1)).to(torch.bfloat16)
    zz = (xn @ wgu.t()).float()
    sw = (torch.nn.functional.silu(zz[:, :inter]) * zz[:, inter:]).to(torch.bfloat16)
    want = xs + (sw @ wd.t()).float()
    rel = lambda o: ((o[rows].float() - want).norm() / want.norm()).item()
    branch = lambda o: ((o[rows].float() - xs - (want - xs)).norm() / (want - xs).norm()).item()
    err = {"plain_out_rel": rel(plain(x)), "folded_out_rel": rel(folded(x)),
           "plain_branch_rel": branch(plain(x)), "folded_branch_rel": branch(folded(x))}
    arms = {"plain": CapturedLayer(plain, x), "folded": CapturedLayer(folded, x)}
    times = {k: [] for k in arms}
    for _ in range(steps):
        for name, fn in arms.items():
            times[name] += _event_times(fn, 1, 0, flush)
    from lcgemm import ops

    ops.check_status()
    t = {k: statistics.median(v) for k, v in times.items()}
    return {"tokens": tokens, "ms": t, "saves_pct": (t["plain"] / t["folded"] - 1) * 100, **err,
            "note": "off by default: every contribution of down is rounded at the magnitude of x"}


def tp1_same_config(steps, warmup, flush, device):
    """The tensor-parallel configuration (8192 x 8192, intermediate 28672) on ONE GPU with the
    single-GPU layer: the like-for-like anchor of the strong-scaling curve."""
    from lcgemm import ops
    from lcgemm.layer import CapturedLayer, Rank7MlpLayer

    x, nw, wgu, wd = make_layer_tensors(TP["tokens"], TP["hidden"], TP["inter"], device)
    layer = Rank7MlpLayer(TP["tokens"], nw, wgu, wd, EPS)
    step = CapturedLayer(layer, x)
    ms = statistics.mean(timed_steps(step, steps, warmup, flush, torch.cuda.synchronize))
    ops.check_status()
    del layer, step, x, nw, wgu, wd
    torch.cuda.empty_cache()
    return {"ms_per_step": ms, "tflops": layer_flops(**TP) / (ms * 1e-3) / 1e12, **TP}


def tp_phase_times(layer, x, steps, flush, sync_all):
    """The fused tensor-parallel layer launched kernel by kernel with events between its phases:
    mean ms per phase over `steps` cold-L2 steps, max over ranks.  (The timed headline replays
    the same kernels as one CUDA graph, which removes the launch gaps these figures include.)"""
    import torch.distributed as dist
    from lcgemm import ops

    lay, ex = layer.layer, layer.exchange
    gate, down = lay.gate_plan, lay.down_plan
    m, k, n = down.shape
    names = ("norm_planes", "gate_up", "down_push", "barrier_1", "reduce_gather", "barrier_2")
    acc = {name: 0.0 for name in names}
    for it in range(steps + 2):
        flush.zero_()
        dist.barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        b = ex.turn
        ex.turn ^= 1
        ev[0].record()
        a = gate.a_planes(x, None, lay.norm_weight, lay.eps)      # the layer call of this bench has no delta
        ev[1].record()
        gate.gemm(a, lay.gate_bw)
        ev[2].record()
        ops.gemm_r7_push(down.scheme, down.a_planes(), lay.down_bw, m, n, k, down.c, ex.slot_ptrs[b],
                         ex.rank, ex.rows, cta_group=down.cta_group)
        ev[3].record()
        ex.barrier()
        ev[4].record()
        ops.reduce_gather(ex.slots[b], x, ex.out_ptrs, ex.rows, ex.rank)
        ev[5].record()
        ex.barrier()
        ev[6].record()
        ev[6].synchronize()
        if it >= 2:
            for j, name in enumerate(names):
                acc[name] += ev[j].elapsed_time(ev[j + 1])
    sync_all()
    ops.check_status()
    t = torch.tensor([acc[name] / steps for name in names], device=x.device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = dict(zip(names, t.tolist()))
    out["sum"] = sum(out.values())
    return out


def tp_parity(fused_layer, x, nw, wgu, wd, cfg, rank, world, device):
    """Checked before anything is timed: the fused exchange's output against the same layer
    with one NCCL all-reduce, against a dense cuBLAS evaluation of a row sample (each rank its
    shard's partial, summed over the ranks in fp32), and bit-equality of the ranks' copies."""
    import torch.distributed as dist
    import torch.nn.functional as F
    from lcgemm.tp import TensorParallelMlp

    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()
    out_f = fused_layer(x).clone()
    ref = TensorParallelMlp(cfg["tokens"], nw, wgu, wd, EPS, fused=False)
    out_n = ref(x).clone()
    rows = torch.arange(0, cfg["tokens"], max(1, cfg["tokens"] // 256), device=device)[:256]
    xs = x[rows]
    h = xs.float()
    y = (h * torch.rsqrt(h.square().mean(-1, keepdim=True) + EPS) * (nw.float() + 1.0)).to(torch.bfloat16)
    gate_z, up_z = F.linear(y, wgu).chunk(2, dim=-1)
    part = F.linear(F.silu(gate_z.float()).to(torch.bfloat16) * up_z, wd).float()
    dist.all_reduce(part)
    first = out_f.clone()
    dist.broadcast(first, src=0)
    same = torch.tensor([1 if torch.equal(first, out_f) else 0], device=device)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    res = torch.tensor([rel(out_f, out_n), rel(out_f.float() - x.float(), out_n.float() - x.float()),
                        rel(out_f[rows].float() - xs.float(), part)], device=device, dtype=torch.float64)
    dist.all_reduce(res, op=dist.ReduceOp.MAX)
    del ref, out_n, first
    torch.cuda.empty_cache()
    vs_nccl, vs_nccl_branch, vs_dense_branch = res.tolist()
    return {"vs_nccl_rel": vs_nccl, "vs_nccl_branch_rel": vs_nccl_branch, "vs_dense_rel": vs_dense_branch,
            "ranks_bit_identical": bool(same.item()), "dense_rows": int(rows.numel()),
            "bounds": {"vs_nccl_rel": 2e-2, "vs_nccl_branch_rel": 4e-2, "vs_dense_rel": 5e-2},
            "note": "the run stops if a bound is exceeded or the ranks' copies differ.  vs_dense_rel (the "
                    "MLP branch out - x on sampled rows against a dense cuBLAS evaluation summed over the "
                    "ranks in fp32) is the accuracy check; vs_nccl_rel compares two rank-7 evaluations whose "
                    "bf16 adds land in hardware order, one of them reduced by a bf16 all-reduce whose own "
                    "rounding grows with the rank count (measured 4.5e-3 at 2 GPUs), so its bound is loose; "
                    "max over ranks"}


# ------------------------------------------------- kernel-level cases and the shape sweep
SWEEP_KN = ((5120, 34816), (17408, 5120), (6144, 32768), (16384, 6144), (5000, 13999))


def _event_times(fn, steps, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def run_case(args, device):
    """One kernel of the layer on its own (few launches: the form used for ncu captures)."""
    from lcgemm import ops, scheme as S
    from lcgemm.seams import build_chain

    m, h, i = args.tokens, args.hidden, args.inter
    flush = torch.empty(FLUSH_BYTES, dtype=torch.int8, device=device)
    if args.case == "layer":
        # the whole layer in its three arms at any (tokens, hidden, intermediate), e.g. the
        # reference's second model family: --hidden 6656 --inter 19968
        res = bench_layer_arms(m, h, i, args.steps, args.warmup, flush, device, graphs=args.graphs)
        res.pop("objects"), res.pop("arms")
        print(json.dumps({"case": "layer", "tokens": m, "hidden": h, "inter": i, "steps": args.steps,
                          "warmup": args.warmup, **_arm_summary(res, layer_flops(m, h, i))}))
        return
    x, nw, wgu, wd = make_layer_tensors(m, h, i, device)
    gate, down = build_chain((m, h, 2 * i), (m, i, h))
    zero = torch.zeros_like(x)
    if args.case == "norm_planes_single":
        # the norm + A-plane kernel as the single-layer call runs it: no delta, no residual stream
        fn, flops = (lambda: gate.a_planes(x, None, nw, EPS)), 0.0
    elif args.case in ("gate_up", "norm_planes", "down"):
        gate_bw = gate.prepare_weight(wgu)
        a = gate.a_planes(x, zero, nw, EPS)
        gate.gemm(a, gate_bw)
        if args.case == "gate_up":
            fn, flops = (lambda: gate.gemm(a, gate_bw)), 2.0 * m * h * 2 * i
        elif args.case == "norm_planes":
            fn, flops = (lambda: gate.a_planes(x, zero, nw, EPS)), 0.0
        else:
            down_bw = down.prepare_weight(wd)
            fn, flops = (lambda: down(prepared_w=down_bw)), 2.0 * m * i * h
    elif args.case == "a_planes":
        s_tok = torch.randn((m, i), device=device).to(torch.bfloat16)       # a down-shaped activation
        ws = torch.empty(ops.a_plane_shape(down.scheme, m, i), device=device, dtype=torch.bfloat16)
        fn, flops = (lambda: ops.a_planes(s_tok, down.scheme, out=ws)), 0.0
    elif args.case == "bare_ahead":
        # the down-shaped bare GEMM with its A planes formed inside the kernel, one product ahead
        lead = S.load("2x2_locality_lead_single")
        s_tok = torch.randn((m, i), device=device).to(torch.bfloat16)
        bp = ops.prepare_b(wd, lead)
        scr = torch.empty(ops.ahead_scratch_bytes(lead, m, i), dtype=torch.uint8, device=device)
        out = torch.empty((m, h), device=device, dtype=torch.bfloat16)
        fn, flops = (lambda: ops.gemm_r7_ahead(s_tok, bp, h, lead, out=out, scratch=scr)), 2.0 * m * i * h
    elif args.case == "down_push_local":
        # one rank's row-parallel `down` of the tensor-parallel layer (K = --inter is the rank's shard)
        # with the push to the owners' slots, every slot in this GPU's memory: the kernel without the link
        world = 8
        loc = S.load("2x2_locality_ordered")
        s_tok = torch.randn((m, i), device=device).to(torch.bfloat16)
        ap, bp = ops.a_planes(s_tok, loc), ops.prepare_b(wd, loc)
        out = torch.empty((m, h), device=device, dtype=torch.bfloat16)
        slots = [torch.empty((m // world, h), device=device, dtype=torch.bfloat16) for _ in range(world)]
        ptrs = [t.data_ptr() for t in slots]
        fn, flops = (lambda: ops.gemm_r7_push(loc, ap, bp, m, h, i, out, ptrs, 3, m // world)), 2.0 * m * i * h
    elif args.case == "dense_gate_up":
        out = torch.empty((m, 2 * i), device=device, dtype=torch.bfloat16)
        fn, flops = (lambda: ops.gemm_dense(x, wgu, out=out)), 2.0 * m * h * 2 * i
    else:
        raise SystemExit(f"unknown case {args.case}")
    times = _event_times(fn, args.steps, args.warmup, flush)
    ops.check_status()
    ms = statistics.mean(times)
    print(json.dumps({"case": args.case, "tokens": m, "hidden": h, "inter": i, "ms": ms,
                      "effective_tflops": flops / (ms * 1e-3) / 1e12 if flops else None,
                      "steps": args.steps, "warmup": args.warmup}))


def run_sweep(args, device):
    """The bare-GEMM sweep: the rank-7 GEMM in its forms -- A planes written by a pass in front
    of the GEMM (postsum-CSE scheme); A planes formed by the GEMM kernel's own plane warps one
    product ahead of the MMAs (locality-ordered products, single-block ones first; both unit
    lists); with --sweep-fused also the form that builds the A operand tiles in shared memory --
    against the dense tcgen05 GEMM and cuBLAS, odd shapes included; B planes prepared offline.
    One JSON line per shape; `rank7_ms` is the form `lcgemm.ops.bare_gemm_form` dispatches that
    shape to."""
    from lcgemm import _native as nat, ops, scheme as S

    flush = torch.empty(FLUSH_BYTES, dtype=torch.int8, device=device)
    kn_list = [kn for kn in SWEEP_KN if args.sweep_kn is None or f"{kn[0]}x{kn[1]}" in args.sweep_kn.split(",")]
    for m in (2048, 4096, 8192):
        for k, n in kn_list:
            sch, sch_a = S.load("2x2_postsum_cse"), S.load("2x2_locality_lead_single")
            g = torch.Generator(device=device).manual_seed(m + k + n)
            a = torch.randn((m, k), generator=g, device=device).to(torch.bfloat16)
            w = (torch.randn((n, k), generator=g, device=device) * 0.02).to(torch.bfloat16)
            bp = ops.prepare_b(w, sch)
            ws = torch.empty(ops.a_plane_shape(sch, m, k), device=device, dtype=torch.bfloat16)
            ld = (n + 7) // 8 * 8
            out = torch.empty((m, ld), device=device, dtype=torch.bfloat16)[:, :n]
            cb_out = torch.empty((m, n), device=device, dtype=torch.bfloat16)
            arms = {
                "rank7_planes": lambda: ops.gemm_r7(a, bp, n, sch, out=out, a_workspace=ws, form="planes"),
                "dense_tcgen05": lambda: ops.gemm_dense(a, w, out=out),
                "dense_cublas": lambda: torch.matmul(a, w.t(), out=cb_out),
            }
            need = ops.ahead_scratch_bytes(sch_a, m, k)
            if need > 0:
                bp_a = ops.prepare_b(w, sch_a)
                scr = torch.empty(need, dtype=torch.uint8, device=device)
                arms["rank7_ahead_hybrid"] = lambda: ops.gemm_r7_ahead(a, bp_a, n, sch_a, out=out, scratch=scr)
                arms["rank7_ahead_split"] = lambda: ops.gemm_r7_ahead(a, bp_a, n, sch_a, out=out, scratch=scr,
                                                                      schedule=nat.SCHEDULE_RANK_SPLIT)
                if args.sweep_fused:
                    arms["rank7_fused"] = lambda: ops.gemm_r7_fused(a, bp_a, n, sch_a, out=out)
            for fn in arms.values():
                for _ in range(args.warmup):
                    fn()
            torch.cuda.synchronize()
            times = {name: [] for name in arms}
            for _ in range(args.steps):
                for name, fn in arms.items():
                    times[name] += _event_times(fn, 1, 0, flush)
            ops.check_status()
            t = {name: statistics.mean(v) for name, v in times.items()}
            name, form, schedule = ops.bare_gemm_form(m, n, k)
            if form == "ahead" and need > 0:
                r7 = t["rank7_ahead_split" if schedule == nat.SCHEDULE_RANK_SPLIT else "rank7_ahead_hybrid"]
            else:
                form, r7 = "planes", t["rank7_planes"]
            dn, cb = t["dense_tcgen05"], t["dense_cublas"]
            fl = 2.0 * m * n * k
            pct = lambda key: (dn / t[key] - 1) * 100 if key in t else None
            print(json.dumps({
                "sweep": "bare_gemm", "M": m, "K": k, "N": n,
                "dispatch": {"scheme": name, "form": form,
                             "schedule": {0: "all_ranks", 1: "rank_split", 2: "hybrid"}[schedule]},
                "rank7_ms": r7, "ms": t,
                "rank7_effective_tflops": fl / r7 / 1e9, "rank7_executed_tflops": 0.875 * fl / r7 / 1e9,
                "dense_tcgen05_tflops": fl / dn / 1e9, "dense_cublas_tflops": fl / cb / 1e9,
                "speedup_vs_dense_tcgen05_pct": (dn / r7 - 1) * 100, "speedup_vs_cublas_pct": (cb / r7 - 1) * 100,
                "vs_dense_tcgen05_pct": {key: pct(key) for key in t if key.startswith("rank7_")},
                "note": "rank7_planes includes the plane-forming pass; L2 flushed between timed launches"}),
                flush=True)
            del a, w, bp, ws, out, cb_out, arms
            if need > 0:
                del bp_a, scr
            torch.cuda.empty_cache()


def _compare_with_reference_kernels(d, gate, down, gate_bw, down_bw, x, zero, nw):
    """This library's kernels against the outputs the reference's kernels left for the same seeded
    inputs: each of ours is fed the REFERENCE's output of the stage before it, so that a
    difference belongs to one kernel.  gate_up runs the all-ranks schedule here (one writer per C
    block, fixed order: the reference's schedule for this shape)."""
    from lcgemm import ops
    from lcgemm._native import SCHEDULE_ALL_RANKS

    dev = x.device
    mism = lambda a, b: float((a.view(torch.int16) != b.view(torch.int16)).float().mean().item())
    rel = lambda a, b: float(((a.float() - b.float()).norm() / b.float().norm()).item())
    ref = {k: v.to(dev) for k, v in d.items()}
    out = {"b_planes_equal": bool(torch.equal(gate_bw[:4096], ref["gate_bw"])
                                  and torch.equal(down_bw[:4096], ref["down_bw"]))}
    a = gate.a_planes(x, zero, nw, EPS)
    out["residual_out_equal"] = bool(torch.equal(gate.residual_out, ref["residual_out"]))
    out["a_planes_mismatch_fraction"] = mism(a, ref["a_planes"])
    out["a_planes_rel"] = rel(a, ref["a_planes"])
    saved = gate.schedule
    gate.schedule = SCHEDULE_ALL_RANKS
    try:
        z = gate.gemm(ref["a_planes"], gate_bw)
        out["z_equal_given_reference_a_planes"] = bool(torch.equal(z, ref["z"]))
        out["z_mismatch_fraction"] = mism(z, ref["z"])
        out["down_planes_equal"] = bool(torch.equal(gate.planes, ref["planes"]))
        out["down_planes_mismatch_fraction"] = mism(gate.planes, ref["planes"])
    finally:
        gate.schedule = saved
    z_h = gate.gemm(ref["a_planes"], gate_bw)
    out["z_rel_hybrid_schedule"] = rel(z_h, ref["z"])
    o = down.gemm(ref["planes"], down_bw)
    out["out_rel_given_reference_planes"] = rel(o, ref["out"])
    out["out_mismatch_fraction"] = mism(o, ref["out"])
    ops.check_status()
    return out


def run_ref_kernels(args, device):
    """The reference's own sm_100 kernels beside this library's, same GPU, same call: the fused
    norm + A-plane kernel, the chained gate_up GEMM and the rank-split down GEMM of one layer at
    `--tokens`.  The reference runs in a child process (baseline/ref_kernels.py: its package
    shares this one's name) between two timings of this library's kernels; if it cannot import,
    JIT-compile or run here, the line says so with the error text."""
    import subprocess

    from lcgemm import ops
    from lcgemm.seams import build_chain

    m, h, i = args.tokens, args.hidden, args.inter
    flush = torch.empty(FLUSH_BYTES, dtype=torch.int8, device=device)
    x, nw, wgu, wd = make_layer_tensors(m, h, i, device)
    gate, down = build_chain((m, h, 2 * i), (m, i, h))
    gate_bw, down_bw = gate.prepare_weight(wgu), down.prepare_weight(wd)
    zero = torch.zeros_like(x)
    a = gate.a_planes(x, zero, nw, EPS)
    stages = {"norm_planes": lambda: gate.a_planes(x, zero, nw, EPS),
              "gate_up": lambda: gate.gemm(a, gate_bw),
              "down": lambda: down(prepared_w=down_bw)}

    def ours():
        out = {}
        for name, fn in stages.items():
            t = _event_times(fn, args.steps, args.warmup, flush)
            out[name] = {"mean_us": statistics.mean(t) * 1e3, "median_us": statistics.median(t) * 1e3,
                         "min_us": min(t) * 1e3}
        ops.check_status()
        return out

    before = ours()
    torch.cuda.synchronize()
    child = ROOT / "baseline" / "ref_kernels.py"
    ref = None
    import tempfile

    dump = Path(tempfile.gettempdir()) / f"lcg_ref_kernels_{os.getpid()}.pt"
    try:
        proc = subprocess.run([sys.executable, str(child), str(m), str(args.steps), str(args.warmup), str(dump),
                               str(h), str(i)], capture_output=True, text=True, timeout=args.ref_timeout)
        for ln in reversed(proc.stdout.strip().splitlines()):
            if ln.startswith("{"):
                ref = json.loads(ln)
                break
        if ref is None:
            ref = {"unavailable": f"child exited {proc.returncode} without a result: "
                                  + (proc.stderr.strip().splitlines() or ["(no output)"])[-1][-400:]}
    except subprocess.TimeoutExpired:
        ref = {"unavailable": f"child did not finish within {args.ref_timeout} s"}
    after = ours()
    bits = None
    if dump.exists():
        try:
            bits = _compare_with_reference_kernels(torch.load(dump), gate, down, gate_bw, down_bw, x, zero, nw)
        finally:
            dump.unlink()
    print(json.dumps({"ref_kernels": True, "tokens": m, "hidden": h, "inter": i, "steps": args.steps,
                      "warmup": args.warmup, "l2": "flushed between timed launches",
                      "ours_before": before, "reference": ref, "ours_after": after,
                      "bits_vs_reference_kernels": bits,
                      "describe": {"gate_up": gate.describe(), "down": down.describe()}}))


def run_round_arm(args, device):
    """One arm of one matched round, in a process of its own: median of `--steps` cold-L2 passes
    of one layer (the reference's `cold_passes`, lcgemm/bench/common.py:116-127, with CUDA events
    in place of the host clock)."""
    from lcgemm import ops
    from lcgemm.layer import CapturedLayer, DenseMlpLayer, Rank7MlpLayer

    cfg = dict(SINGLE, tokens=args.tokens)
    flush = torch.empty(FLUSH_BYTES, dtype=torch.int8, device=device)
    x, nw, wgu, wd = make_layer_tensors(cfg["tokens"], cfg["hidden"], cfg["inter"], device)
    if args.round_arm == "rank7":
        layer = Rank7MlpLayer(cfg["tokens"], nw, wgu, wd, EPS)
    else:
        layer = DenseMlpLayer(cfg["tokens"], nw, wgu, wd, EPS,
                              gemm="cublas" if args.round_arm == "dense_cublas" else "tcgen05")
    step = CapturedLayer(layer, x)
    with ClockWatch(torch.cuda.current_device()) as cw:
        times = []
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        for _ in range(args.steps):
            time.sleep(0.02)
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
    ops.check_status()
    print("RESULT_JSON " + json.dumps({"arm": args.round_arm, "tokens": cfg["tokens"], "runs": len(times),
                                       "median_us": statistics.median(times), "mean_us": statistics.mean(times),
                                       "samples_us": times, "clocks": cw.summary()}))


def _quantile(values, q):
    """Linear interpolation at (n - 1) * q (lcgemm/bench/headline.py:27-35)."""
    v = sorted(values)
    pos = (len(v) - 1) * q
    lo = int(pos)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def run_rounds(args):
    """R matched rounds: every round runs each arm in a fresh process, the order alternating from
    round to round (lcgemm/bench/headline.py:66-67); a round's speedup compares the arms' medians;
    the result is the median and quartiles of the rounds' speedups, with a sign guard: every
    round must fall on the side of zero the median does."""
    import subprocess

    arms = ("dense_tcgen05", "dense_cublas", "rank7")
    rows = []
    for r in range(1, args.rounds + 1):
        order = arms if r % 2 else tuple(reversed(arms))
        got = {}
        for arm in order:
            proc = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--round-arm", arm,
                                   "--tokens", str(args.tokens), "--steps", str(args.steps),
                                   "--warmup", str(args.warmup)], capture_output=True, text=True)
            line = next((ln for ln in proc.stdout.splitlines() if ln.startswith("RESULT_JSON ")), None)
            if proc.returncode != 0 or line is None:
                raise SystemExit(f"round {r} arm {arm} failed: {proc.stderr[-500:]}")
            got[arm] = json.loads(line[len("RESULT_JSON "):])
        rows.append({
            "round": r, "order": list(order),
            "median_us": {a: got[a]["median_us"] for a in arms},
            "sm_mhz": {a: got[a]["clocks"]["sm_mhz"] for a in arms},
            "speedup_vs_dense_tcgen05_pct": 100 * (got["dense_tcgen05"]["median_us"] / got["rank7"]["median_us"] - 1),
            "speedup_vs_cublas_pct": 100 * (got["dense_cublas"]["median_us"] / got["rank7"]["median_us"] - 1)})

    def dist(key):
        vals = [row[key] for row in rows]
        med = _quantile(vals, 0.5)
        return {"n": len(vals), "q1": _quantile(vals, 0.25), "median": med, "q3": _quantile(vals, 0.75),
                "values": vals, "sign_consistent": all((v > 0) == (med > 0) for v in vals)}

    print(json.dumps({"rounds": args.rounds, "tokens": args.tokens, "runs_per_arm": args.steps,
                      "protocol": "fresh process per arm, arm order alternating by round, cold L2 before every "
                                  "pass, one CUDA graph replay per pass, median of passes per arm, median of "
                                  "rounds (quartiles beside it)",
                      "speedup_vs_dense_tcgen05_pct": dist("speedup_vs_dense_tcgen05_pct"),
                      "speedup_vs_cublas_pct": dist("speedup_vs_cublas_pct"), "rows": rows}))


def run_model(args, device):
    """The end-to-end configuration: batch-1 prefill of a random-init 64-layer dense decoder, stock MLP vs
    rank-7 MLP, on seeded uniform-random prompts of 2048 / 4096 / 8192 tokens.  Times come from the
    first prompt of a length; agreement (equal top-1, tie-aware top-20 count, final hidden state)
    is taken over `--prompts` seeded prompts per length and reported as rates, for the rank-7 arm,
    for its bit-reproducible all-ranks form, and for the calibration pair `eager` vs `stock` (two
    implementations of the same stock layer that differ only in where SwiGLU rounds)."""
    from lcgemm import ops
    from lcgemm.model import DecoderConfig, RandomInitDecoder, compare_arms

    cfg = DecoderConfig(layers=args.layers)
    model = RandomInitDecoder(cfg, device)
    flush = torch.empty(FLUSH_BYTES, dtype=torch.int8, device=device)
    lengths = [int(t) for t in args.model_tokens.split(",")]
    for tokens in lengths:
        info = model.install(tokens)
        prompts = [torch.randint(0, cfg.vocab, (tokens,),
                                 generator=torch.Generator().manual_seed(tokens + 7919 * j)).to(device)
                   for j in range(args.prompts)]
        ids = prompts[0]
        times = {"stock": [], "rank7": [], "dense": []}
        for arm in times:
            for _ in range(max(1, args.warmup - 2)):
                model.prefill(ids, arm=arm)
        torch.cuda.synchronize()
        before = dict(model.calls)
        for _ in range(args.steps):
            for arm in times:
                times[arm] += _event_times(lambda: model.prefill(ids, arm=arm), 1, 0, flush)
        ops.check_status()
        fused = model.calls["fused"] - before["fused"]
        st, r7, dn = (statistics.median(times[a]) for a in ("stock", "rank7", "dense"))
        pairs = {"rank7": [], "rank7_allranks": [], "eager": [], "dense": []}
        repeat_equal = []
        for ids_j in prompts:
            ref = model.prefill(ids_j, arm="stock")
            for arm in pairs:
                got = model.prefill(ids_j, arm=arm)
                pairs[arm].append(compare_arms(ref[0], got[0], ref[1], got[1]))
                if arm == "rank7_allranks":
                    again = model.prefill(ids_j, arm=arm)
                    repeat_equal.append(bool(torch.equal(got[0], again[0]) and torch.equal(got[1], again[1])))
        ops.check_status()

        def rates(rows):
            n = len(rows)
            return {"prompts": n, "top1_equal_rate": sum(r["top1_equal"] for r in rows) / n,
                    "tie_aware_top20_min": min(r["tie_aware_top20"] for r in rows),
                    "tie_aware_top20_mean": sum(r["tie_aware_top20"] for r in rows) / n,
                    "passes_gate_rate": sum(r["top1_equal"] and r["tie_aware_top20"] >= 19 for r in rows) / n,
                    "hidden_rel_fro_mean": sum(r["hidden_rel_fro"] for r in rows) / n,
                    "max_abs_logit_diff_max": max(r["max_abs_logit_diff"] for r in rows),
                    "top1_gap_of_stock_median": statistics.median(r["top1_gap"] for r in rows),
                    "logit_std": rows[0]["logit_std"]}

        print(json.dumps({
            "model": "random-init dense decoder", "layers": cfg.layers, "hidden": cfg.hidden,
            "inter": cfg.inter, "heads": [cfg.q_heads, cfg.kv_heads, cfg.head_dim], "vocab": cfg.vocab,
            "tokens": tokens, "passes": args.steps, "stock_ms": st, "rank7_ms": r7, "dense_tcgen05_ms": dn,
            "speedup_pct": (st / r7 - 1.0) * 100.0, "speedup_vs_dense_tcgen05_pct": (dn / r7 - 1.0) * 100.0,
            "fused_calls": fused,
            "expected_fused_calls": args.steps * cfg.layers, "planes_gib": info["planes_gib"],
            "gate": "equal top-1 and >= 19 of 20 tie-aware (lcgemm/bench/headline.py:195-200)",
            "agreement_rank7_vs_stock": rates(pairs["rank7"]),
            "agreement_rank7_allranks_vs_stock": rates(pairs["rank7_allranks"]),
            "agreement_dense_tcgen05_vs_stock": rates(pairs["dense"]),
            "agreement_eager_vs_stock": rates(pairs["eager"]),
            "rank7_allranks_repeat_bit_equal_rate": sum(repeat_equal) / len(repeat_equal),
            "data": "synthetic: random-init weights (seed 0), uniform-random token ids"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", action="store_true",
                    help="end-to-end prefill of the random-init decoder")
    ap.add_argument("--layers", type=int, default=64, help="decoder layers for --model")
    ap.add_argument("--prompts", type=int, default=8, help="seeded prompts per length for --model's agreement rates")
    ap.add_argument("--model-tokens", default="2048,4096,8192", help="prompt lengths for --model")
    ap.add_argument("--case", default=None,
                    help="time one kernel alone: gate_up | down | norm_planes | norm_planes_single | a_planes | bare_ahead | down_push_local | dense_gate_up; "
                         "or `layer`: the whole layer's three arms at --tokens / --hidden / --inter")
    ap.add_argument("--tokens", type=int, default=4096, help="token count for --case")
    ap.add_argument("--hidden", type=int, default=SINGLE["hidden"], help="hidden size for --case")
    ap.add_argument("--inter", type=int, default=SINGLE["inter"], help="intermediate size for --case")
    ap.add_argument("--sweep", action="store_true", help="bare-GEMM shape sweep, odd shapes included")
    ap.add_argument("--sweep-fused", action="store_true",
                    help="--sweep: also time the form that builds the A operand tiles in shared memory (slow)")
    ap.add_argument("--sweep-kn", default=None,
                    help="restrict --sweep to these KxN pairs, comma separated (e.g. 17408x5120,16384x6144)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-graphs", dest="graphs", action="store_false",
                    help="launch the layer's kernels one by one instead of replaying a CUDA graph")
    ap.add_argument("--exchange", choices=("peer", "nccl"), default="peer",
                    help="N > 1: how the ranks' partial outputs are combined: 'peer' = pushed from inside "
                         "the down GEMM over NVLink, then reduce + gather in this package's kernels; "
                         "'nccl' = one library all-reduce")
    ap.add_argument("--ref-kernels", action="store_true",
                    help="time the reference's own sm_100 kernels (baseline/_ref) beside this library's, one GPU")
    ap.add_argument("--ref-timeout", type=int, default=420, help="seconds the --ref-kernels child may take")
    ap.add_argument("--rounds", type=int, default=0,
                    help="matched rounds of fresh processes, one per arm (single layer at --tokens)")
    ap.add_argument("--round-arm", default=None, choices=("rank7", "dense_tcgen05", "dense_cublas"),
                    help="(used by --rounds) run one arm in this process and print its RESULT_JSON line")
    ap.add_argument("--sustain-seconds", type=float, default=2.0,
                    help="N = 1: seconds per arm of the back-to-back `sustained` block (0 = skip)")
    ap.add_argument("--no-tp1-anchor", dest="tp1_anchor", action="store_false",
                    help="N > 1: skip timing the tensor-parallel configuration on rank 0 alone")
    ap.add_argument("--slabs", type=int, default=1,
                    help="N > 1: slabs of the down GEMM pipelined with the all-reduce (1 = no overlap)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.rounds > 0:
        if world != 1:
            raise SystemExit("--rounds runs on one GPU")
        return run_rounds(args)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch under torchrun); got {world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rank-7 path has no CPU implementation")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if args.case or args.sweep or args.model or args.ref_kernels or args.round_arm:
        if world != 1:
            raise SystemExit("--case / --sweep / --model / --ref-kernels / --rounds run on one GPU")
        if args.ref_kernels:
            return run_ref_kernels(args, device)
        if args.round_arm:
            return run_round_arm(args, device)
        if args.model:
            return run_model(args, device)
        return run_case(args, device) if args.case else run_sweep(args, device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner on stdout at NCCL_DEBUG=VERSION; stdout carries the one
        # JSON line of this run, so keep NCCL to warnings unless the caller asked for more.
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        run_ours(args, rank, world, device)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
