#!/usr/bin/env python
"""Benchmark of the MEXT hot path (online NVFP4 quantiser + folded FP4 GEMM) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): the NVFP4 MEXT sweep over the four Qwen3-32B-shaped projections
(K->N: qkv 5120->10240, o 8192->5120, gate_up 5120->51200, down 25600->5120) and tokens
M in {1,2,4,8,16,32,64,128}.  One pass over all 32 (shape, M) cases is captured in a CUDA graph (the
reference measures under CUDA graphs as well); each case is two kernels of this library (quantiser,
GEMM).  One *step* replays that graph SWEEPS_PER_STEP times, so that the timed region of the default
run lasts about half a second, and is timed with CUDA events on the launching stream.  Successive
cases stream different weights (274 MB per pass over the four shapes, more than the 126 MB L2), so
every weight read comes from HBM.

Printed JSON (one line, rank 0):
  value / ms_per_step   mean microseconds per linear op over the sweep (lower is better)
  roofline              the GEMM kernel: algorithmic bytes per launch / mean launch time, against the
                        measured HBM copy bandwidth (MEASURED_PEAKS.json)
  e2e                   the same sweep through the public op ``residue::nvfp4_linear`` with pinned host
                        buffers: H2D of x and D2H of y inside the timed region
  cpu_baseline          the reference's torch-eager quantise/dequantise/matmul path on the host cores
                        for a bounded sample (N = 1 only)
  detail                per-case microseconds, TFLOP/s, fraction of roofline; ResAttn decode numbers

N > 1 (torchrun): tensor parallel on one node.  qkv / gate_up are column-parallel (N/tp per rank),
o / down row-parallel (K/tp per rank) followed by an NCCL all-reduce of the BF16 output; time is the
maximum over ranks.  ``--impl reference`` times the CPU restatement of the reference's eager path.
"""
from __future__ import annotations

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

SHAPES = [("qkv", 5120, 10240, "col"), ("o", 8192, 5120, "row"), ("gate_up", 5120, 51200, "col"),
          ("down", 25600, 5120, "row")]
MS = [1, 2, 4, 8, 16, 32, 64, 128]
L2_BYTES = 126 * 1024 * 1024
SWEEPS_PER_STEP = 40                 # replays of the 32-case sweep graph per step
CPU_MS = (1, 16, 128)                # token counts the CPU arm runs (4 shapes each)
# DRAM traffic of the GEMM kernel / its algorithmic bytes, from one ncu capture per shape (see roofline.traffic_source)
NCU_TRAFFIC_RATIO = 281.31 / 277.36


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run_nvml(self):
        """Read-only NVML polling every 2 ms (SM clock, max SM clock, clock event reasons)."""
        import pynvml as N
        N.nvmlInit()
        h = N.nvmlDeviceGetHandleByIndex(self.index)
        mx = N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM)
        get_reasons = getattr(N, "nvmlDeviceGetCurrentClocksEventReasons", None) or N.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = (0x8, 0x40, 0x20, 0x4)        # hw_slowdown, hw_thermal_slowdown, sw_thermal_slowdown, sw_power_cap
        while not self._stop.is_set():
            r = int(get_reasons(h))
            self.samples.append([str(N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM)), str(mx)] +
                                ["Active" if r & b else "Not Active" for b in bits])
            self._stop.wait(0.002)

    def _run(self):
        try:
            return self._run_nvml()
        except Exception:
            pass
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# algorithmic work
# ------------------------------------------------------------------------------------------------
SCALE_BLOCK = 16                     # elements per block scale: 16 (NVFP4) or 32 (MXFP4, set by --format)


def mext_bytes(m, k, n):
    """x (bf16) + W codes and block scales + y (bf16): the bytes a fused MEXT linear must move."""
    return 2 * m * k + n * k * (0.5 + 1.0 / SCALE_BLOCK) + 2 * m * n


def gemm_bytes(m, k, n):
    """GEMM kernel alone: activation codes+scales (base and residue), W codes+scales, y."""
    return 2 * m * k * (0.5 + 1.0 / SCALE_BLOCK) + n * k * (0.5 + 1.0 / SCALE_BLOCK) + 2 * m * n


def mext_flops(m, k, n):
    return 2.0 * m * n * (2 * k)


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the torch-eager path on host cores
# ------------------------------------------------------------------------------------------------
_CPU_INPUTS = {}


FORMAT = "nvfp4"                     # set by --format


def cpu_eager_step(ms=CPU_MS):
    """One bounded CPU step of the metric: the eager quantise/dequantise/matmul path (oracle port of the
    reference's ResidueQuantLinear._forward_residue_qdq) for the four sweep shapes at the token counts
    `ms` on all host threads.  Returns the mean microseconds per linear op and the thread count.  The CPU
    time hardly depends on M (the weight is re-quantised on every call, as in the reference's eager path),
    so 12 of the 32 cases (M = 1, 16, 128) stand for the sweep."""
    import torch
    import oracle
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    total, n = 0.0, 0
    for m in ms:
        for name, k, nn, _ in SHAPES:
            if (name, m) not in _CPU_INPUTS:
                _CPU_INPUTS[(name, m)] = (torch.from_numpy(oracle.make_activation(m, k, seed=0)).to(torch.bfloat16),
                                          torch.from_numpy(oracle.make_weight(nn, k, seed=1)).to(torch.bfloat16))
            x, w = _CPU_INPUTS[(name, m)]
            t0 = time.perf_counter()
            oracle.eager_residue_linear(x, w, fmt=FORMAT)
            total += (time.perf_counter() - t0) * 1e6
            n += 1
    return total / n, cores


_CPU_SAMPLE = "12 of 32 sweep cases per step: qkv, o, gate_up, down at M in {1, 16, 128}, ratio 1.0"


def cpu_eager_sample():
    """cpu_baseline of the GPU arm: a warm-up over the four shapes at M = 16, then one step (12 cases)."""
    cpu_eager_step((16,))
    v, cores = cpu_eager_step()
    return {"value": v, "unit": "us", "cores": cores, "kind": "port",
            "sample": _CPU_SAMPLE + ", one step after a warm-up pass over the four shapes"}


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU path (oracle port) for the same metric and config, on rank 0."""
    global FORMAT
    FORMAT = args.format
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu_eager_step((16,))                                    # warm-up: thread pool, allocator, one pass over the shapes
    for _ in range(max(0, args.warmup - 1)):
        cpu_eager_step()
    ts = []
    cores = 0
    t_begin = time.perf_counter()
    for _ in range(max(1, args.steps)):
        v, cores = cpu_eager_step()
        ts.append(v)
        if time.perf_counter() - t_begin > 240:            # keep the whole run within a few minutes
            break
    v = statistics.mean(ts)
    line = {
        "impl": "reference", "metric": "mext_%s_linear_latency" % args.format, "value": v, "unit": "us", "n_gpus": args.gpus,
        "steps": len(ts), "warmup": max(1, args.warmup), "ms_per_step": v * len(SHAPES) * len(CPU_MS) / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None,
        "dtype": ("mxfp4 (E2M1 x E8M0 block scales)" if args.format == "mxfp4" else "nvfp4 (E2M1 x E4M3 block scales)") + ", fp32 accumulate",
        "data": "synthetic", "config": workload_config(args.gpus, args.format),
        "cpu_baseline": {"value": v, "unit": "us", "cores": cores, "kind": "port", "sample": _CPU_SAMPLE},
        "e2e": {"value": v, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus, fmt="nvfp4"):
    return {"workload": "MEXT " + fmt.upper() + " sweep: qkv 5120->10240, o 8192->5120, gate_up 5120->51200, down 25600->5120; "
                        "M in {1,2,4,8,16,32,64,128}; online quantiser + folded GEMM per case",
            "step": "%d replays of the 32-case sweep graph (GPU arm); the CPU arm runs 12 of the 32 cases per step, "
                    "M in {1, 16, 128}" % SWEEPS_PER_STEP,
            "l2": "inputs larger than L2: 274 MB of weights stream per pass over the four shapes, rotating copies",
            "parallelism": "tp%d" % n_gpus if n_gpus > 1 else "single GPU", "cuda_graph": True}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class Layer:
    """One projection on one rank: prequantised weight copies + activation buffers."""

    def __init__(self, name, k, n, par, tp, rank, dev, copies_bytes=2 * L2_BYTES, fmt="nvfp4"):
        import torch
        from resinfer_b200.quant import weight_prep
        self.name, self.par = name, par
        self.k_full, self.n_full = k, n
        self.k = k // tp if par == "row" else k
        self.n = n // tp if par == "col" else n
        g = torch.Generator(device=dev).manual_seed(1 + rank)
        w = (torch.randn(self.n, self.k, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        prep = weight_prep.quantize_weight_mxfp4(w) if fmt == "mxfp4" else weight_prep.quantize_weight_nvfp4(w)
        del w
        wbytes = prep["weight"].numel() + prep["weight_scale"].numel()
        self.copies = max(1, min(8, -(-copies_bytes // wbytes)))
        self.w = [prep["weight"].clone() for _ in range(self.copies)]
        self.w_sf = [prep["weight_scale"].clone() for _ in range(self.copies)]
        self.w_gs = prep.get("weight_global_scale", torch.ones(1, device=dev))   # MXFP4 has no global scale
        self.x, self.gs_inv, self.alpha = {}, {}, {}
        for m in MS:
            gx = torch.Generator(device=dev).manual_seed(0)
            x = torch.randn(m, k, generator=gx, device=dev, dtype=torch.float32)
            out_ch = torch.randperm(k, generator=gx, device=dev)[: max(1, k // 100)]
            x[:, out_ch] *= 20.0
            x = x.to(torch.bfloat16)
            gs = float(x.float().abs().max()) / (6.0 * 448.0)
            if par == "row":
                x = x[:, rank * self.k:(rank + 1) * self.k].contiguous()
            self.x[m] = x
            self.gs_inv[m] = torch.tensor([1.0 / gs], dtype=torch.float32, device=dev)
            self.alpha[m] = (self.w_gs * gs).float().reshape(1)
        self.use = 0

    def next_copy(self):
        c = self.use % self.copies
        self.use += 1
        return c


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-detail", action="store_true", help="skip the per-case and ResAttn detail measurements")
    ap.add_argument("--format", default="nvfp4", choices=["nvfp4", "mxfp4"],
                    help="number format of the headline sweep (NVFP4 MEXT is the headline configuration, MXFP4 MEXT "
                         "the second one)")
    ap.add_argument("--allreduce", choices=("peer", "fused", "auto", "nccl"), default="peer",
                    help="N > 1: how the row-parallel partials are summed: by this library's stand-alone one-shot "
                         "kernel over peer memory (the default: fastest inside the sweep, 10.7 us per reduction on two "
                         "GPUs against 20.1 for the epilogue), in the GEMM's epilogue over peer memory "
                         "(ri_fp4_gemm_allreduce), auto = the epilogue up to 16 tokens and the stand-alone kernel "
                         "above, or NCCL")
    ap.add_argument("--attn-format", default="fp16", choices=["fp16", "e4m3"],
                    help="number format of V and P in the ResAttn measurements (ops.resattn_pv_format)")
    ap.add_argument("--sweeps", action="store_true",
                    help="measure the other sweeps of the three hot paths (MXFP4 MEXT, KEXT, ResAttn batch sizes) "
                         "and print them as a second JSON line {\"sweeps\": ...}; N = 1 only")
    ap.add_argument("--only", default=None,
                    help="profiling aid: 'gemm:<shape>:<M>' times that single (shape, M) case, 'resattn:<index>' "
                         "that single ResAttn point, 'kext:<shape>:<M>:<ratio>' one KEXT case (ratio 1.0 = K-concat "
                         "MEXT), 'quant:<M>:<K>' the NVFP4 MEXT quantiser alone; plain launches, no e2e, no CPU "
                         "baseline, not a bench value")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    tp = world

    def note(msg):                                          # progress on stderr (rank 0), never on the JSON line
        if rank == 0 and (world > 1 or os.environ.get("BENCH_VERBOSE")):
            print(f"[bench] {msg}", file=sys.stderr, flush=True)

    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.quant import mxfp4_linear  # noqa: F401  (registers residue::mxfp4_linear)
    from resinfer_b200.quant.vllm_integration import residue_linear_op  # noqa: F401
    nvfp4.ensure_loaded()

    global SHAPES, MS, SCALE_BLOCK, FORMAT, ATTN_FORMAT
    FORMAT = args.format
    ATTN_FORMAT = args.attn_format
    SCALE_BLOCK = 32 if args.format == "mxfp4" else 16
    if args.only:
        kind, _, rest = args.only.partition(":")
        if kind == "resattn":
            hbm_gbs, _ = load_peaks()
            res = measure_resattn(torch, dev, ops, None, None, hbm_gbs, only=int(rest), steps=args.steps,
                                  warmup=args.warmup)
            print(json.dumps({"only": args.only, "resattn": res}), flush=True)
            return
        if kind in ("kext", "quant"):
            print(json.dumps({"only": args.only, "result": run_single_case(torch, dev, kind, rest, args.steps, args.warmup)}),
                  flush=True)
            return
        shape, _, m_only = rest.partition(":")
        SHAPES = [s for s in SHAPES if s[0] == shape]
        MS = [int(m_only)]
        args.no_detail = True
    note("process group up; building layers")
    layers = [Layer(nm, k, n, par, tp, rank, dev, fmt=args.format) for nm, k, n, par in SHAPES]
    note("layers built")
    mx = args.format == "mxfp4"
    if mx:
        from resinfer_b200.nvfp4 import mxfp4
    outs = {(L.name, m): torch.empty(m, L.n, dtype=torch.bfloat16, device=dev) for L in layers for m in MS}
    launches = {"n": 0}
    # N > 1: the partial outputs of the row-parallel layers are summed by this library's one-shot all-reduce
    # over peer memory (a kernel per rank, plain NVLink loads); NCCL if the peers cannot be mapped or
    # --allreduce nccl is given.  The GEMM writes its partial straight into the exported buffer.
    peer_ar = None
    if tp > 1 and args.allreduce in ("auto", "fused", "peer"):
        # the constructor exchanges its outcome among the ranks: it raises on all of them or on none
        try:
            from resinfer_b200.quant.tp import PeerAllReduce
            peer_ar = PeerAllReduce(max(MS) * max(L.n for L in layers if L.par == "row"), slots=2)
        except Exception as e:
            note(f"peer all-reduce unavailable ({type(e).__name__}: {e}); using NCCL")
    ar_status = torch.zeros(1, dtype=torch.int32, device=dev)

    FUSED_MAX_M = 16                                         # --allreduce auto: the epilogue reduction up to here

    def fused_for(L, reduce, m=None):
        if peer_ar is None or L.par != "row" or not reduce:
            return None
        if args.allreduce == "fused" or (args.allreduce == "auto" and m is not None and m <= FUSED_MAX_M):
            return peer_ar
        return None

    def red_ctx(L, m):
        # how the public op of a row-parallel layer gets its sum: in the epilogue or by the stand-alone kernel
        if peer_ar is None or L.par != "row":
            return ops.row_parallel_reduction(None)
        return ops.row_parallel_reduction(peer_ar, epilogue=fused_for(L, True, m) is not None)

    def gemm_out(L, m, reduce):
        if peer_ar is not None and L.par == "row" and reduce and fused_for(L, reduce, m) is None:
            return peer_ar.partial((m, L.n))
        return outs[(L.name, m)]

    def finish(L, m, y, reduce):
        if tp > 1 and L.par == "row" and reduce and fused_for(L, reduce, m) is None:
            if peer_ar is not None:
                launches["n"] += 1
                return peer_ar.reduce(y, outs[(L.name, m)], status=ar_status)
            dist.all_reduce(y)
        return y

    def mext_layout(L, m):
        # the operand layout the public op picks for the fold route (same arithmetic either way)
        from resinfer_b200.quant.vllm_integration.residue_linear_op import fold_prefers_concat_k
        return "concat_k" if (not mx and fold_prefers_concat_k(m, L.k)) else "row_pair"

    def run_case(L, m, quant=True, pre=None, reduce=True):
        c = L.next_copy()
        lay = mext_layout(L, m)
        if quant:
            if mx:
                codes, sf = mxfp4.quantize_mext(L.x[m], pdl_mode="early")
            else:
                codes, sf = nvfp4.scaled_fp4_quant_mext_r1(L.x[m], L.gs_inv[m], layout_mode=3 if lay == "concat_k" else 1,
                                                           enable_pdl=True)
            launches["n"] += 1
        else:
            codes, sf = pre
        y = ops.fp4_gemm(codes, sf, L.w[c], L.w_sf[c], None if mx else L.alpha[m], m=m, fmt=args.format,
                         layout=lay, out=gemm_out(L, m, reduce), allreduce=fused_for(L, reduce, m))
        launches["n"] += 1
        return finish(L, m, y, reduce)

    def sweep(quant=True, pre=None, reduce=True):
        for m in MS:
            for L in layers:
                run_case(L, m, quant, None if pre is None else pre[(L.name, m)], reduce)

    if peer_ar is not None:
        # Self-check before anything is timed: one eager sweep, then every row-parallel layer's reduction
        # against the rank-ordered FP32 sum of the same partials (gathered with NCCL), which the kernel must
        # reproduce bit for bit.  Every rank runs the same sequence of collectives whatever it observes; the
        # verdicts are combined once at the end, and a failure on any rank sends all of them to NCCL.
        torch.cuda.synchronize()
        dist.barrier()
        sweep()
        bad = False
        for L in layers:
            if L.par != "row":
                continue
            m = MS[-1]
            part = run_case(L, m, reduce=False).clone()
            parts = [torch.empty_like(part) for _ in range(tp)]
            dist.all_gather(parts, part)
            want = torch.zeros_like(part, dtype=torch.float32)
            for q in parts:                                  # rank order, FP32: the kernel's own order
                want += q.float()
            want = want.to(torch.bfloat16)
            if args.allreduce in ("auto", "fused"):
                # (auto: the largest M goes through the stand-alone kernel below, the smallest through the epilogue)
                ms = MS[0] if args.allreduce == "auto" else m
                ps = [torch.empty(ms, L.n, dtype=torch.bfloat16, device=dev) for _ in range(tp)]
                dist.all_gather(ps, run_case(L, ms, reduce=False).clone())
                ws_ = torch.zeros(ms, L.n, dtype=torch.float32, device=dev)
                for q in ps:
                    ws_ += q.float()
                got_s = run_case(L, ms).clone()
                run_case(L, ms)                              # keep the inboxes alternating in pairs
                torch.cuda.synchronize()
                bad = bad or not torch.equal(got_s, ws_.to(torch.bfloat16))
            if args.allreduce == "fused":
                got = want
            else:
                pbuf = peer_ar.partial((m, L.n))
                pbuf.copy_(part)
                got = peer_ar.reduce(pbuf, status=ar_status)
                pbuf2 = peer_ar.partial((m, L.n))
                pbuf2.copy_(part)
                peer_ar.reduce(pbuf2, status=ar_status)
            torch.cuda.synchronize()
            bad = bad or not torch.equal(got, want)
        bad = bad or int(ar_status.item()) != 0 or int(peer_ar.status.item()) != 0
        flag = torch.tensor([1 if bad else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        if int(flag.item()):
            note("peer all-reduce failed its self-check; using NCCL")
            peer_ar = None
            ar_status.zero_()
    graphs = []

    def capture(fn):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()                                           # warm-up: workspaces, attributes
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(g):
                fn()
            graphs.append(g)
            return g.replay
        except Exception as e:                             # e.g. a collective that cannot be captured
            if rank == 0:
                print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); timing eagerly", file=sys.stderr)
            torch.cuda.synchronize()
            return fn

    def timed(replay, steps, warmup):
        for _ in range(warmup):
            replay()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            replay()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    n_cases = len(MS) * len(layers)
    inner = 1 if args.only else SWEEPS_PER_STEP            # sweep-graph replays per step

    def step_of(replay_one):
        def step():
            for _ in range(inner):
                replay_one()
        return step

    # ---- headline: quantiser + GEMM over the sweep
    launches["n"] = 0
    note("capturing the sweep")
    replay = capture(lambda: sweep(True))
    note("captured; timing")
    per_sweep_launches = launches["n"] // 2                 # warm-up + capture both counted
    with ClockSampler(local) as clk:
        ms_step = timed(step_of(replay), args.steps, args.warmup)
    ops.check_status(dev)
    note(f"timed: {ms_step:.3f} ms per step")
    us_per_op = ms_step * 1e3 / (n_cases * inner)

    # ---- N > 1: the same sweep without the all-reduce of the row-parallel layers, for the cost of one reduction
    allreduce_us = None
    if tp > 1:
        replay_nr = capture(lambda: sweep(True, reduce=False))
        ms_nr = timed(step_of(replay_nr), args.steps, args.warmup)
        n_row_ops = len(MS) * sum(1 for L in layers if L.par == "row")
        allreduce_us = (ms_step - ms_nr) * 1e3 / (inner * max(1, n_row_ops))

    # ---- GEMM kernel alone (pre-quantised activations) for the roofline of the dominant kernel
    pre = {(L.name, m): (mxfp4.quantize_mext(L.x[m]) if mx else
                         nvfp4.scaled_fp4_quant_mext_r1(L.x[m], L.gs_inv[m],
                                                        layout_mode=3 if mext_layout(L, m) == "concat_k" else 1))
           for L in layers for m in MS}
    replay_g = capture(lambda: sweep(False, pre, reduce=False))
    hbm_gbs, peak_kind = load_peaks()
    roofline = None
    if replay_g is not None:
        ms_gemm = timed(step_of(replay_g), args.steps, args.warmup) / inner     # one sweep of GEMM launches
        gbytes = sum(gemm_bytes(m, L.k, L.n) for L in layers for m in MS) / n_cases
        achieved = gbytes / (ms_gemm * 1e-3 / n_cases) / 1e9
        roofline = {"kernel": "fp4_gemm_kernel (tcgen05 block-scaled, %d launches per step" % (n_cases * inner)
                              + (", this rank's shard, no all-reduce)" if tp > 1 else ")"), "bound": "hbm",
                    "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                    "peak_source": peak_kind, "traffic": gbytes * NCU_TRAFFIC_RATIO,
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of single launches of the four "
                                      "shapes at M=16 (the weights dominate at every M <= 128, so traffic grows in "
                                      "proportion), scaled to the sweep's mean launch",
                    "us_per_launch": ms_gemm * 1e3 / n_cases, "algorithmic_bytes_per_launch": gbytes}

    # ---- e2e through the public op with pinned host buffers
    e2e = None
    if not args.only:
        hx = {(L.name, m): L.x[m].cpu().pin_memory() for L in layers for m in MS}
        hy = {(L.name, m): torch.empty(m, L.n, dtype=torch.bfloat16).pin_memory() for L in layers for m in MS}
        zero_mask = torch.zeros(1, dtype=torch.uint8, device=dev)

        out_stream = torch.cuda.Stream()                    # results go home on their own stream, under the next op
        done = [torch.cuda.Event() for _ in range(n_cases)]

        def e2e_sweep():
            keep = []                                       # device results stay alive until their copy has run
            i = 0
            for m in MS:
                for L in layers:
                    c = L.next_copy()
                    xd = hx[(L.name, m)].to(dev, non_blocking=True)
                    with red_ctx(L, m):                         # row-parallel layers: the sum over the ranks
                        if mx:
                            y = torch.ops.residue.mxfp4_linear(xd, L.w[c], L.w_sf[c], zero_mask, zero_mask, "mext_r1",
                                                               torch.bfloat16, None)
                        else:
                            y = torch.ops.residue.nvfp4_linear(xd, L.w[c], L.gs_inv[m], L.w_sf[c], L.w_sf[c], zero_mask,
                                                               L.alpha[m], L.k, 0, 0, L.n, True, False, True)
                    if tp > 1 and L.par == "row" and peer_ar is None:
                        dist.all_reduce(y)
                    done[i].record()
                    out_stream.wait_event(done[i])
                    with torch.cuda.stream(out_stream):
                        hy[(L.name, m)].copy_(y, non_blocking=True)
                    keep.append(y)
                    i += 1
            torch.cuda.synchronize()

        def wall_us(fn, reps):
            for _ in range(2):
                fn()
            t0 = time.perf_counter()
            for _ in range(reps):
                fn()
            us = (time.perf_counter() - t0) / reps * 1e6 / n_cases
            if world > 1:
                tt = torch.tensor([us], device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                us = float(tt.item())
            return us

        reps = max(3, min(args.steps, 10)) * 4             # sweeps per wall-clock measurement
        eager_us = wall_us(e2e_sweep, reps)
        e2e_us, how = eager_us, "eager"
        if tp == 1 or peer_ar is not None:                  # (NCCL collectives stay out of this graph)
            # The way a serving stack drives decode: the whole sweep (every H2D copy of x from pinned memory,
            # every call of the public op, every D2H copy of y on a second stream) captured once in a CUDA
            # graph and replayed per step; the wall clock covers replay + synchronize.
            xs = {k: torch.empty_like(v, device=dev) for k, v in hx.items()}
            side, inbound = torch.cuda.Stream(), torch.cuda.Stream()

            def graphed_body():
                cur = torch.cuda.current_stream()
                keep = []
                # inputs travel on their own stream, ahead of the ops; each op waits for its own x only
                inbound.wait_stream(cur)
                arrived = {}
                order = sorted(MS, reverse=True)          # large results first: their trip home hides under later ops
                with torch.cuda.stream(inbound):
                    for m in order:
                        for L in layers:
                            xs[(L.name, m)].copy_(hx[(L.name, m)], non_blocking=True)
                            ev = torch.cuda.Event()
                            ev.record(inbound)
                            arrived[(L.name, m)] = ev
                for m in order:
                    for L in layers:
                        c = L.next_copy()
                        xd = xs[(L.name, m)]
                        cur.wait_event(arrived[(L.name, m)])
                        with red_ctx(L, m):
                            if mx:
                                y = torch.ops.residue.mxfp4_linear(xd, L.w[c], L.w_sf[c], zero_mask, zero_mask, "mext_r1",
                                                                   torch.bfloat16, None)
                            else:
                                y = torch.ops.residue.nvfp4_linear(xd, L.w[c], L.gs_inv[m], L.w_sf[c], L.w_sf[c],
                                                                   zero_mask, L.alpha[m], L.k, 0, 0, L.n, True, False, True)
                        side.wait_stream(cur)
                        with torch.cuda.stream(side):
                            hy[(L.name, m)].copy_(y, non_blocking=True)
                        keep.append(y)                      # no reuse of a result's memory inside the graph
                cur.wait_stream(inbound)
                cur.wait_stream(side)
                return keep

            n_before = len(graphs)
            replay = capture(graphed_body)
            if len(graphs) > n_before:                      # captured (otherwise capture() fell back to eager)
                def graphed_step():
                    replay()
                    torch.cuda.synchronize()
                ref_y = {k: v.clone() for k, v in hy.items()}      # eager results, for a sanity check
                if world > 1:                               # the peers' kernels wait for each other (bounded): start together
                    torch.cuda.synchronize()
                    dist.barrier()
                graphed_step()
                same = all(torch.equal(ref_y[k], hy[k]) for k in hy)
                if world > 1:                               # one decision for all ranks
                    flag = torch.tensor([1 if same else 0], device=dev)
                    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                    same = bool(flag.item())
                if same:
                    e2e_us, how = wall_us(graphed_step, reps), "graph"
                elif rank == 0:
                    print("[bench] graphed e2e results differ from the eager ones; reporting the eager time", file=sys.stderr)
        e2e = {"value": e2e_us, "unit": "us",
               "h2d_bytes_per_step": inner * world * sum(2 * m * L.k for L in layers for m in MS),
               "d2h_bytes_per_step": inner * world * sum(2 * m * L.n for L in layers for m in MS),
               "sweeps_timed": reps,
               "eager_us": eager_us, "mode": how,
               "note": ("residue::%s_linear from pinned host buffers: H2D of x, the op, D2H of y on a second stream. "
                        "mode=graph: the whole sweep captured once in a CUDA graph (inputs on an inbound stream, results on an "
                        "outbound stream, ops on a third) and replayed per step, as a serving stack runs decode; wall clock "
                        "over replay + synchronize; eager_us: the same calls issued "
                        "one by one from Python (dispatch-bound)") % args.format}

    detail = None
    if not args.no_detail and tp == 1 and not mx:
        detail = measure_detail(torch, dev, layers, outs, nvfp4, ops, capture, timed, hbm_gbs)
    elif not args.no_detail and tp > 1 and 8 % tp == 0:
        # ResAttn shards by KV head (8 / tp KV heads and 64 / tp query heads per rank, no collective);
        # the time is the maximum over ranks, the bytes are those of all ranks
        try:
            ra = measure_resattn(torch, dev, ops, capture, timed, hbm_gbs, custom=(128, 64, 16), heads=(64 // tp, 8 // tp))
            for r in ra:
                r["tbs"] = round(r["tbs"] * tp, 3)
                r["frac_hbm"] = round(r["frac_hbm"], 3)
                r["note"] = "KV heads sharded over %d GPUs; TB/s summed over ranks, frac_hbm per GPU" % tp
            detail = {"resattn": ra}
        except Exception as e:
            detail = {"resattn": [{"error": f"{type(e).__name__}: {e}"}]}

    cpu = None
    if rank == 0 and tp == 1 and not args.only:
        try:
            cpu = cpu_eager_sample()
        except Exception as e:                              # the oracle is optional equipment
            cpu = {"value": None, "unit": "us", "cores": len(os.sched_getaffinity(0)), "kind": "port",
                   "sample": f"failed: {type(e).__name__}: {e}"}

    if rank == 0:
        flops = sum(mext_flops(m, L.k_full, L.n_full) for L in layers for m in MS)
        # the ResAttn point that the documents quote, as a top-level key (records may cut the detail short)
        attn_key = {}
        for r in (detail or {}).get("resattn", []):
            if r.get("head_dim") == 128 and r.get("batch") == 64 and r.get("page") == 16:
                attn_key = {"resattn_d128_b64_page16": {k: r[k] for k in ("us", "tbs", "frac_hbm", "splits") if k in r}}
        line = {
            "metric": "mext_%s_linear_latency" % args.format, "value": us_per_op, "unit": "us", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None,
            "dtype": ("mxfp4 (E2M1 x E8M0 block scales)" if mx else "nvfp4 (E2M1 x E4M3 block scales)") + ", fp32 accumulate",
            "data": "synthetic",
            "config": dict(workload_config(world, args.format),
                           **({"allreduce": {"fused": "in the GEMM's epilogue over peer memory (ri_fp4_gemm_allreduce)",
                                             "auto": "M <= 16: in the GEMM's epilogue over peer memory "
                                                     "(ri_fp4_gemm_allreduce); above: one-shot kernel over peer memory "
                                                     "(ri_peer_allreduce_bf16)"}.get(
                                                 args.allreduce, "one-shot over peer memory (ri_peer_allreduce_bf16)")
                               if peer_ar is not None
                               else "NCCL"} if tp > 1 else {})),
            "clocks": clk.summary(),
            **({"allreduce_status": int(ar_status.item()) | (int(peer_ar.status.item()) if peer_ar is not None else 0),
                "allreduce_us": allreduce_us} if tp > 1 else {}),
            "gpu_launches": per_sweep_launches * inner * args.steps,
            "tflops": flops * inner / (ms_step * 1e-3) / 1e12, "fp4_peak_frac": flops * inner / (ms_step * 1e-3) / 9.0e15,
            "hbm_gbs_algorithmic": sum(mext_bytes(m, L.k_full, L.n_full) for L in layers for m in MS) * inner / (ms_step * 1e-3) / 1e9,
            "e2e": e2e, "roofline": roofline, "cpu_baseline": cpu, **attn_key, "detail": detail,
        }
        if args.only:
            line["only"] = args.only
        print(json.dumps(line), flush=True)
    if args.sweeps and tp == 1 and not args.only:
        hbm_gbs2, _ = load_peaks()
        print(json.dumps({"sweeps": measure_sweeps(torch, dev, capture, timed, hbm_gbs2)}), flush=True)
    if world > 1:
        # captured graphs hold NCCL kernels: release them before the communicator goes away, and do not
        # let a slow communicator teardown keep the finished benchmark alive
        graphs.clear()
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        threading.Timer(20.0, lambda: os._exit(0)).start()
        dist.destroy_process_group()
        os._exit(0)


def run_single_case(torch, dev, kind, rest, steps, warmup):
    """`--only kext:<shape>:<M>:<ratio>` / `--only quant:<M>:<K>`: plain launches of one case on the current
    stream (what a profiler is pointed at), timed with CUDA events.  Weights rotate over copies larger than L2."""
    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.nvfp4.quant import indices_to_channel_masks
    from resinfer_b200.quant import weight_prep
    parts = rest.split(":")
    g = torch.Generator(device=dev).manual_seed(0)

    def act(m, k):
        x = torch.randn(m, k, generator=g, device=dev, dtype=torch.float32)
        x[:, torch.randperm(k, generator=g, device=dev)[: max(1, k // 100)]] *= 20.0
        return x.to(torch.bfloat16)

    if kind == "quant":
        m, k = int(parts[0]), int(parts[1])
        x = act(m, k)
        gi = torch.tensor([100.0], dtype=torch.float32, device=dev)
        xs = [x.clone() for _ in range(max(2, min(8, (2 * L2_BYTES) // (2 * m * k) + 1)))]
        fn = lambda i: nvfp4.scaled_fp4_quant_mext_r1(xs[i % len(xs)], gi, layout_mode=1)    # noqa: E731
        nbytes = 2 * m * k + 2 * m * k * (0.5 + 1.0 / 16)
        flops = 0.0
    else:
        name, m, ratio = parts[0], int(parts[1]), float(parts[2])
        k, n = next((kk, nn) for nm, kk, nn, _ in SHAPES if nm == name)
        per8 = {0.125: 1, 0.25: 2, 0.5: 4, 1.0: 8}[ratio]
        idx = None if per8 == 8 else weight_prep.salient_indices_per8(k, per8, device=dev)
        w = (torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        prep = weight_prep.quantize_weight_nvfp4(w, idx)
        del w
        nb = prep["weight"].numel() + prep["weight_scale"].numel()
        copies = max(2, min(8, -(-2 * L2_BYTES // nb)))
        ws = [prep["weight"].clone() for _ in range(copies)]
        sfs = [prep["weight_scale"].clone() for _ in range(copies)]
        s = 0 if idx is None else idx.numel()
        mask = None if idx is None else indices_to_channel_masks(idx, k)
        x = act(m, k)
        gs = float(x.float().abs().max()) / (6.0 * 448.0)
        gi = torch.tensor([1.0 / gs], dtype=torch.float32, device=dev)
        alpha = (prep["weight_global_scale"] * gs).float().reshape(1)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)

        def fn(i):
            c = i % copies
            if per8 == 8:
                codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=3)
                return ops.fp4_gemm(codes, sf, ws[c], sfs[c], alpha, m=m, fmt="nvfp4", layout="concat_k", out=y)
            codes, sf = nvfp4.scaled_fp4_quant_with_mask(x, gi, mask, s, use_swapped_residue=False)
            return ops.fp4_gemm(codes, sf, ws[c], sfs[c], alpha, m=m, fmt="nvfp4", layout="plain", out=y)
        k_eff = 2 * k if per8 == 8 else k + s
        nbytes = 2 * m * k + k / 8 + n * (k if per8 == 8 else k + s) * 0.5625 + 2 * m * n
        flops = 2.0 * m * n * k_eff
    for i in range(max(1, warmup)):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(max(1, steps)):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / max(1, steps) * 1e3
    return {"us": round(us, 2), "gbs": round(nbytes / us / 1e3), "tflops": round(flops / us / 1e6, 1)}


def measure_detail(torch, dev, layers, outs, nvfp4, ops, capture, timed, hbm_gbs):
    """Per-case latency (cold weights: rotating copies larger than L2) and a ResAttn decode point."""
    from resinfer_b200.quant.vllm_integration.residue_linear_op import fold_prefers_concat_k
    cases = []
    for L in layers:
        for m in MS:
            def one(L=L, m=m):
                for _ in range(L.copies):
                    c = L.next_copy()
                    lay = "concat_k" if fold_prefers_concat_k(m, L.k) else "row_pair"     # as the public op picks it
                    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(L.x[m], L.gs_inv[m], layout_mode=3 if lay == "concat_k" else 1,
                                                               enable_pdl=True)
                    ops.fp4_gemm(codes, sf, L.w[c], L.w_sf[c], L.alpha[m], m=m, fmt="nvfp4", layout=lay,
                                 out=outs[(L.name, m)])
            rp = capture(one)
            us = timed(rp, 10, 3) * 1e3 / L.copies
            t_bound = mext_bytes(m, L.k, L.n) / (hbm_gbs * 1e9) * 1e6
            cases.append({"shape": L.name, "m": m, "us": round(us, 2), "tflops": round(mext_flops(m, L.k, L.n) / us / 1e6, 1),
                          "gbs": round(mext_bytes(m, L.k, L.n) / us / 1e3, 0), "frac_hbm_roofline": round(t_bound / us, 3)})
    attn = []
    try:
        attn = measure_resattn(torch, dev, ops, capture, timed, hbm_gbs)
    except Exception as e:
        attn = [{"error": f"{type(e).__name__}: {e}"}]
    return {"mext_nvfp4_cases": cases, "resattn": attn}


def measure_sweeps(torch, dev, capture, timed, hbm_gbs):
    """The sweeps beside the headline: MXFP4 MEXT (4 shapes x M), NVFP4 KEXT (4 shapes x M x ratio) and
    ResAttn over batch sizes.  Every linear case is timed as quantiser + GEMM under a CUDA graph with
    rotating weight copies (more than L2 in total), like the headline sweep."""
    from resinfer_b200 import nvfp4, ops
    from resinfer_b200.nvfp4 import mxfp4
    from resinfer_b200.nvfp4.quant import indices_to_channel_masks
    from resinfer_b200.quant import weight_prep
    out = {"mxfp4_mext": [], "kext_nvfp4": [], "resattn": [], "stock_mm_fp4": []}

    def weights(k, n, fmt, idx=None):
        g = torch.Generator(device=dev).manual_seed(5)
        w = (torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        prep = (weight_prep.quantize_weight_mxfp4 if fmt == "mxfp4" else weight_prep.quantize_weight_nvfp4)(w, idx)
        del w
        nbytes = prep["weight"].numel() + prep["weight_scale"].numel()
        copies = max(2, min(8, -(-2 * L2_BYTES // nbytes)))
        return prep, [prep["weight"].clone() for _ in range(copies)], [prep["weight_scale"].clone() for _ in range(copies)]

    def act(m, k):
        gx = torch.Generator(device=dev).manual_seed(0)
        x = torch.randn(m, k, generator=gx, device=dev, dtype=torch.float32)
        x[:, torch.randperm(k, generator=gx, device=dev)[: max(1, k // 100)]] *= 20.0
        return x.to(torch.bfloat16)

    def time_case(fn, copies):
        rp = capture(lambda: [fn(c) for c in range(copies)])
        return timed(rp, 10, 3) * 1e3 / copies

    # ---- ResAttn: batch sizes of the configuration, page 16, both head sizes.  Measured first: after the
    # long tensor-bound KEXT cases the part sits at its power cap and the same kernel reads 8-15 % slower.
    for d, batches in ((128, (1, 8, 32, 128, 256)), (256, (1, 8, 32, 128))):
        for b in batches:
            try:
                out["resattn"] += measure_resattn(torch, dev, ops, capture, timed, hbm_gbs, custom=(d, b, 16))
            except Exception as e:                          # e.g. out of memory on a smaller part
                out["resattn"].append({"head_dim": d, "batch": b, "error": f"{type(e).__name__}: {e}"})
            torch.cuda.empty_cache()
    # ---- stock anchor: FlashInfer's plain NVFP4 W4A4 GEMM (no residue) behind this library's plain
    # quantiser, on the four shapes.  A comparison kernel, never part of the product path: the reference
    # publishes its MEXT latency as a ratio to this stock kernel.
    try:
        from flashinfer import mm_fp4
        out["stock_mm_fp4"] = []
        for name, k, n, _ in SHAPES:
            prep, ws, sfs = weights(k, n, "nvfp4")
            w_sf_v = [t.view(torch.float8_e4m3fn).view(((n + 127) // 128) * 128, (k // 64) * 4) for t in sfs]
            for m in MS:
                x = act(m, k)
                gs = float(x.float().abs().max()) / (6.0 * 448.0)
                gi = torch.tensor([1.0 / gs], dtype=torch.float32, device=dev)
                alpha = (prep["weight_global_scale"] * gs).float().reshape(1)
                codes = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
                sf = torch.zeros(((m + 127) // 128) * ((k + 63) // 64) * 512, dtype=torch.uint8, device=dev)
                sf_v = sf.view(torch.float8_e4m3fn).view(((m + 127) // 128) * 128, (k // 64) * 4)
                y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)

                def fn(c, x=x, gi=gi, alpha=alpha, codes=codes, sf=sf, sf_v=sf_v, y=y):
                    torch.ops.nvfp4.scaled_fp4_quant_mext_r1(codes, x, sf, gi, 0, 5, True)      # base codes only
                    return mm_fp4(codes, ws[c].T, sf_v, w_sf_v[c].T, alpha, torch.bfloat16, out=y, backend="cudnn")
                us = time_case(fn, len(ws))
                out["stock_mm_fp4"].append({"shape": name, "m": m, "us": round(us, 2), "backend": "cudnn",
                                            "what": "plain NVFP4 quantiser of this library + flashinfer.mm_fp4, no residue"})
            del prep, ws, sfs, w_sf_v
    except Exception as e:                                  # the comparison kernel is optional equipment
        out["stock_mm_fp4"] = [{"error": f"{type(e).__name__}: {str(e)[:300]}"}]
    # ---- MXFP4 MEXT: online E8M0 quantiser (row_pair) + block32 fold GEMM
    for name, k, n, _ in SHAPES:
        prep, ws, sfs = weights(k, n, "mxfp4")
        for m in MS:
            x = act(m, k)

            def fn(c, x=x, m=m):
                a, a_sf = mxfp4.quantize_mext(x, pdl_mode="early")
                return mxfp4.fold_gemm(a, ws[c], a_sf, sfs[c], out_dtype=torch.bfloat16)
            us = time_case(fn, len(ws))
            nbytes = 2 * m * k + n * k * (0.5 + 1 / 32) + 2 * m * n
            out["mxfp4_mext"].append({"shape": name, "m": m, "us": round(us, 2), "tflops": round(4.0 * m * n * k / us / 1e6, 1),
                                      "gbs": round(nbytes / us / 1e3), "frac_hbm_roofline": round(nbytes / us / 1e3 / hbm_gbs, 3)})
        del prep, ws, sfs
    # ---- KEXT NVFP4: masked residue along K + plain GEMM over K + S; ratio 1.0 = MEXT K-concat
    for name, k, n, _ in SHAPES:
        for ratio, per8 in ((0.125, 1), (0.25, 2), (0.5, 4), (1.0, 8)):
            idx = None if per8 == 8 else weight_prep.salient_indices_per8(k, per8, device=dev)
            prep, ws, sfs = weights(k, n, "nvfp4", idx)
            s = 0 if idx is None else idx.numel()
            mask = None if idx is None else indices_to_channel_masks(idx, k)
            for m in (16, 128, 1024, 8192):
                x = act(m, k)
                gs = float(x.float().abs().max()) / (6.0 * 448.0)
                gi = torch.tensor([1.0 / gs], dtype=torch.float32, device=dev)
                alpha = (prep["weight_global_scale"] * gs).float().reshape(1)
                y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)

                def fn(c, x=x, m=m, gi=gi, alpha=alpha, y=y):
                    if per8 == 8:
                        codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=3)
                        return ops.fp4_gemm(codes, sf, ws[c], sfs[c], alpha, m=m, fmt="nvfp4", layout="concat_k", out=y)
                    codes, sf = nvfp4.scaled_fp4_quant_with_mask(x, gi, mask, s, use_swapped_residue=False)
                    return ops.fp4_gemm(codes, sf, ws[c], sfs[c], alpha, m=m, fmt="nvfp4", layout="plain", out=y)
                us = time_case(fn, len(ws))
                k_eff = 2 * k if per8 == 8 else k + s
                w_k = k if per8 == 8 else k + s                  # weight columns that are read
                nbytes = 2 * m * k + k / 8 + n * w_k * 0.5625 + 2 * m * n
                flops = 2.0 * m * n * k_eff
                t_mem, t_tc = nbytes / (hbm_gbs * 1e9), flops / 9.0e15     # dense FP4 nominal 9 PFLOP/s
                out["kext_nvfp4"].append({"shape": name, "ratio": ratio, "m": m, "us": round(us, 2),
                                          "tflops": round(flops / us / 1e6, 1), "gbs": round(nbytes / us / 1e3),
                                          "bound": "hbm" if t_mem >= t_tc else "tensor",
                                          "frac_roofline": round(max(t_mem, t_tc) * 1e6 / us, 3)})
            del prep, ws, sfs
    return out


# ResAttn decode points of the driver-run line: (head_dim, batch, page size).  The first three are the ones
# `--only resattn:<index>` addresses.
ATTN_FORMAT = "fp16"
RESATTN_POINTS = ((128, 8, 16), (128, 64, 16), (256, 32, 16),
                  (128, 1, 16), (128, 32, 16), (128, 128, 16), (128, 256, 16),
                  (256, 1, 16), (256, 8, 16), (256, 128, 16), (256, 256, 16),
                  (128, 1, 128), (128, 8, 128), (128, 64, 128), (128, 256, 128), (256, 32, 128), (256, 128, 128),
                  # fixed context lengths, page 128: the cases of the reference's own published latency plot
                  (128, 1, 128, 8192), (128, 8, 128, 32768), (128, 32, 128, 32768), (128, 64, 128, 32768))


def measure_resattn(torch, dev, ops, capture, timed, hbm_gbs, only=None, steps=10, warmup=3, custom=None,
                    heads=(64, 8), points=RESATTN_POINTS):
    """ResAttn decode: 64 query heads, 8 KV heads, context lengths uniform in [1024, 32768], block tables a
    random permutation of the page pool.  The KV tensors are uniform random code bytes with E4M3 scale bytes
    in 0x28-0x48 (timing inputs: the kernel's work does not depend on the values); quantised N(0,1) K/V are
    what the parity tests use."""
    from resinfer_b200.nvfp4.cute_attn.plan import select_decode_plan
    res = []
    hq, hkv = heads
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    for idx, point in enumerate(points if custom is None else (custom,)):
        d, batch, page = point[:3]
        fixed_len = point[3] if len(point) > 3 else None
        if only is not None and idx != only:
            continue
        g = torch.Generator(device=dev).manual_seed(3)
        lens = torch.randint(1024, 32769, (batch,), generator=g, device=dev, dtype=torch.int32)
        if fixed_len:
            lens = torch.full((batch,), fixed_len, device=dev, dtype=torch.int32)
        pages_per = (lens + page - 1) // page
        total = int(pages_per.sum())
        pool = int(total * 1.1) + 1
        perm = torch.randperm(pool, generator=g, device=dev)[:total].to(torch.int32)
        bt = torch.zeros(batch, int(pages_per.max()), dtype=torch.int32, device=dev)
        off = 0
        for b in range(batch):
            n = int(pages_per[b])
            bt[b, :n] = perm[off:off + n]
            off += n
        kd = torch.randint(0, 256, (pool, hkv, page, d // 2), generator=g, device=dev, dtype=torch.uint8)
        vd = torch.randint(0, 256, (pool, hkv, page, d // 2), generator=g, device=dev, dtype=torch.uint8)
        ks = torch.randint(0x28, 0x48, (pool, hkv, page, d // 16), generator=g, device=dev, dtype=torch.uint8)
        vs = torch.randint(0x28, 0x48, (pool, hkv, page, d // 16), generator=g, device=dev, dtype=torch.uint8)
        q = torch.randn(batch, hq, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        out = torch.empty(batch, hq, d, dtype=torch.bfloat16, device=dev)
        # the lengths are host knowledge in a serving stack (the scheduler's), so the plan may use them
        splits, reducer = select_decode_plan(batch, hkv, int(lens.max()), sms, head_dim=d, seq_lens=lens.tolist())
        reducer = "cluster" if reducer == "cga_sharded" else "ticket"
        max_len = int(lens.max())
        def call():                                         # the format switch is a host-side setting: it is
            with ops.resattn_pv_format(ATTN_FORMAT):        # captured with the launch
                ops.resattn_decode(q, kd, ks, vd, vs, bt, lens, d ** -0.5, 1.0, out, splits=splits, reducer=reducer,
                                   max_kv_len=max_len)
        if capture is None:                                 # single-case mode: plain launches, CUDA events
            for _ in range(warmup):
                call()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                call()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / steps * 1e3
        else:
            us = timed(capture(call), 10, 3) * 1e3
        tokens = int(lens.sum())
        nbytes = tokens * hkv * d * 2 * (0.5 + 1 / 16) + 4 * batch * hq * d + 4 * total
        res.append({"head_dim": d, "batch": batch, "page": page, "context": fixed_len or "U[1024,32768]", "tokens": tokens,
                    "splits": splits, "reducer": reducer, "pv_format": ATTN_FORMAT, "us": round(us, 1),
                    "tbs": round(nbytes / us / 1e6, 3), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3),
                    "kv_bytes_gt_l2": bool(nbytes > L2_BYTES)})
        del kd, vd, ks, vs, q, out, bt
        torch.cuda.empty_cache()
    return res


if __name__ == "__main__":
    main()
