"""Benchmark of the W4A4 fused-linear hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME] [--legs a,b,..]

One step = one pass of the hot path over the workload's linears (activation
quantisation + fused dense/residual GEMM each).  The default workload is the
decode sweep: the four Llama-3-8B linear shapes (qkv 4096->6144, o 4096->4096,
gate_up 4096->28672, down 14336->4096) at M = 1, 4 and 16 tokens with a 5 %
block-sparse residual - twelve linears per step.  Inputs are seeded synthetic
tensors; weights rotate through several distinct copies so that a step never
finds its weights in L2.

Printed JSON (one line, rank 0): `value` = effective TOPS (2*M*K*N per linear,
dense ops only) with inputs resident in HBM and the step replayed as a CUDA
graph; `e2e` = the same metric through the public module call with pinned host
activations copied in and results copied out every step; `roofline` = HBM
bytes/s of the GEMM kernel launches alone; `cpu_baseline` = the reference's CPU
route (quantise -> dequantise -> fp32 matmul) on the host cores.  Every timed
figure is the median of `windows` windows, each `reps_per_window` x `steps`
steps long (at least 0.2 s), bracketed by a barrier and a device synchronise,
timed with CUDA events, maximum over ranks.

Further legs in the same line (`--legs`, default all that apply):
  cfg0     one linear 4096->4096 at 16 tokens
  prefill  many-token sweep: M in {2048, 8192} x residual density {0, 5, 15 %} on the four
           shapes, packed nibbles and prepared e4m3 bytes, against the tensor roofline
  cfg3     Llama-2-70B linears split column-parallel over the ranks (strong scaling),
           M = 1 and M = 4096, with and without the all-gather of the output
  stack    decoder-stack decode tokens per second (one GPU)
  legacy   the reference's naive mma.sync kernels recompiled for sm_100a, as a same-GPU anchor (one GPU)
and, on more than one GPU, `sharded_parity`: the gathered output of a sharded
layer equals the single-GPU output bit for bit.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]
LLAMA2_70B = [("qkv", 8192, 10240), ("o", 8192, 8192), ("gate_up", 8192, 57344), ("down", 28672, 8192)]
DENSITY = 0.05
L2_BYTES = 126 * 1024 * 1024
MIN_WINDOW_S = 0.2
WINDOWS = 3

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the dominant kernel, from
# one profiler capture per entry: (bytes, kernel instantiation, capture date).  A figure applies only
# to the workload and weight format it is keyed by; anything else reports null.
NCU_TRAFFIC = {
    ("decode", "packed"): (30.49e6, "decode_gemm_kernel<1|2,false>, mean of the 12 launches", "2026-11-25"),
    ("gate_up_m16", "packed"): (65.82e6, "decode_gemm_kernel<2,false>", "2026-11-25"),
    ("prefill_gate_up", "prepared"): (226.5e6, "prefill_gemm_kernel<false,true,true>", "2026-11-25"),
    ("prefill_gate_up", "packed"): (155.0e6, "prefill_gemm_kernel<false,false,false>", "2026-11-25"),
}


def workload_items(name):
    if name == "decode":
        return [(f"{n}_M{m}", m, k, o) for m in (1, 4, 16) for (n, k, o) in LLAMA3_8B]
    if name == "prefill":
        return [(f"{n}_M{m}", m, k, o) for m in (2048,) for (n, k, o) in LLAMA3_8B]
    if name == "cfg0":
        return [("o_M16", 16, 4096, 4096)]
    if name == "gate_up_m16":        # small single-kernel case for profiler captures
        return [("gate_up_M16", 16, 4096, 28672)]
    if name == "prefill_gate_up":    # the same for the tensor-core kernel
        return [("gate_up_M2048", 2048, 4096, 28672)]
    if name == "prefill_gate_up_8192":
        return [("gate_up_M8192", 8192, 4096, 28672)]
    raise SystemExit(f"unknown workload {name}")


WORKLOAD_DESC = {
    "decode": "Llama-3-8B linears (qkv,o,gate_up,down) x M in {1,4,16}, 5% residual blocks",
    "prefill": "Llama-3-8B linears (qkv,o,gate_up,down) x M=2048, 5% residual blocks",
    "cfg0": "single linear 4096->4096, M=16, 5% residual blocks",
    "gate_up_m16": "single linear 4096->28672, M=16, 5% residual blocks",
    "prefill_gate_up": "single linear 4096->28672, M=2048, 5% residual blocks",
    "prefill_gate_up_8192": "single linear 4096->28672, M=8192, 5% residual blocks",
}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, nm in names.items():
                    if mask & bit:
                        self.reasons.add(nm)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ----------------------------------------------------------------------------- helpers
def measured_peak(key, fallback):
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))[key]), "measured"
        except Exception:
            pass
    return fallback, "fallback"


class Timer:
    """CUDA-event timing in windows: warm-up, then WINDOWS windows of reps x steps steps each (a window
    lasts at least MIN_WINDOW_S), each bracketed by a barrier + synchronise; per window the maximum over
    ranks; the median window is reported."""

    def __init__(self, world, device):
        self.world, self.device = world, device

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def _max_over_ranks(self, v):
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([v], device=self.device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    def _window(self, run, steps, reps, start):
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        i = start
        for _ in range(reps):
            for _ in range(steps):
                run(i)
                i += 1
        e1.record()
        self.barrier()
        return self._max_over_ranks(e0.elapsed_time(e1)) / reps, i

    def time(self, run, steps, warmup, windows=WINDOWS, min_window_s=MIN_WINDOW_S):
        """Returns (median ms per `steps` steps, reps per window, all window values)."""
        i = 0
        for _ in range(warmup):
            run(i)
            i += 1
        ms, i = self._window(run, steps, 1, i)          # calibration pass (also warm)
        reps = max(1, int(math.ceil(min_window_s * 1e3 / max(ms, 1e-3))))
        vals = []
        for _ in range(windows):
            ms, i = self._window(run, steps, reps, i)
            vals.append(ms)
        return statistics.median(vals), reps, vals


def make_weights(K, N, density, device, n_sets, base=None):
    """n_sets distinct device copies of one synthetic container (so that consecutive steps never find
    their weights in L2).  `base`: a container of the same shape whose dense part is reused (only the
    residual mask and blocks are drawn again for another density)."""
    from zip_kernel_b200 import synth
    if base is None:
        W = synth.make_container(N, K, density, seed=synth.shape_seed(0, K, N))
    else:
        W = synth.make_container_like(base, density, seed=synth.shape_seed(1, K, N) + int(density * 1000))
    return W, [W.to(device) for _ in range(n_sets)]


def sets_for(bytes_per_step):
    return max(2, min(8, -(-2 * L2_BYTES // max(bytes_per_step, 1)) + 1))


def alg_bytes_gemm(M, K, N, nnz, prepared=False):
    """Bytes one GEMM launch must move: weights (half a byte per code packed, one byte
    prepared), scales/zeros, residual blocks and index, expanded activation codes (one
    byte each) with their scales and group sums, output."""
    ng, nbr = K // 128, (N + 127) // 128
    wb = 2 if prepared else 1
    b_w = wb * K * N // 2 + 4 * N * ng + wb * 8192 * nnz + 4 * (nbr + 1) + 4 * nnz
    return b_w + (M * K + 2 * M + 4 * M * ng) + 2 * M * N


def fused_call(ops, X, W, token_major=True):
    return ops.fused_dense_sparse_e2e_cuda(X, W.perm, W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets,
                                           W.hp_col_indices, W.scale_u4, W.zero_u4, W.d_out, W.d_in,
                                           token_major=token_major, prepared=W.prepared)


def gemm_call(ops, W, XE, sumxf, sx, token_major=True):
    return ops.fused_dense_sparse_expanded_cuda(W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets,
                                                W.hp_col_indices, XE, sumxf, W.scale_u4, W.zero_u4, sx,
                                                W.d_out, W.d_in, token_major=token_major, prepared=W.prepared,
                                                e4m3=W.prepared is not None)


def capture_graphs(fn, n_sets):
    """One CUDA graph per weight set of fn(r); the graphs share scratch of their own (they are replayed
    one after the other on one stream), kept alive with them."""
    from zip_kernel_b200 import _lib
    holder = _lib.WorkspaceHolder()
    graphs = []
    side = torch.cuda.Stream()
    with _lib.use_workspace(holder), torch.cuda.stream(side):
        for r in range(n_sets):
            fn(r)
            fn(r)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn(r)
            graphs.append(g)
    torch.cuda.synchronize()
    return graphs, holder


# ----------------------------------------------------------------------------- CPU arm
def reference_functions():
    """The reference's own CPU route when its pure-Python files were installed under baseline/_ref
    (baseline/install_reference.py does that where the reference tree is present), else the oracle's
    restatement of it."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if os.path.exists(os.path.join(ref_root, "kernel", "tools", "parity", "fp16_reference.py")):
        if ref_root not in sys.path:
            sys.path.insert(0, ref_root)
        try:
            from kernel.tools.parity.fp16_reference import fp16_fused_reference
            from kernel.tools.parity.quant_reference import quantize_activation_s4_reference

            def path(X, perm, Wt):
                xs4, sx, sumx = quantize_activation_s4_reference(X, perm)
                return fp16_fused_reference(Wt["W_low_packed"], Wt["W_high_blocks_packed"], Wt["hp_row_offsets"],
                                            Wt["hp_col_indices"], xs4, Wt["scale_u4"], Wt["zero_u4"], sx,
                                            Wt["d_out"], Wt["d_in"], sum_X=sumx)
            return path, "reference", "tools/parity quantize_activation_s4_reference + fp16_fused_reference (torch CPU)"
        except Exception as exc:      # fall back to the port, and say why
            why = f"reference install unusable ({type(exc).__name__}: {exc}); "
    else:
        why = ""
    from oracle import w4a4_oracle as O
    return O.cpu_reference_path, "port", why + "oracle restatement of quantise + dequantise->fp32 matmul (torch CPU)"


def cpu_pass(items, passes, warm):
    """Times `passes` passes over the linears `items` [(name, M, K, N)] on all host threads."""
    from zip_kernel_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    path, kind, how = reference_functions()
    data, wcache = [], {}
    for name, M, K, N in items:
        if (K, N) not in wcache:
            W = synth.make_container(N, K, DENSITY, seed=synth.shape_seed(0, K, N))
            wcache[(K, N)] = (W, dict(W_low_packed=W.W_low_packed, W_high_blocks_packed=W.W_high_blocks_packed,
                                      scale_u4=W.scale_u4, zero_u4=W.zero_u4, hp_row_offsets=W.hp_row_offsets,
                                      hp_col_indices=W.hp_col_indices, d_out=N, d_in=K))
        W, Wt = wcache[(K, N)]
        X = synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1)
        data.append((X, W.perm, Wt, 2 * M * K * N))
    for X, perm, Wt, _ in data[:warm]:
        path(X, perm, Wt)
    t0 = time.perf_counter()
    for _ in range(passes):
        for X, perm, Wt, _ in data:
            path(X, perm, Wt)
    dt = (time.perf_counter() - t0) / passes
    ops_pass = sum(d[3] for d in data)
    return ops_pass / dt / 1e12, dt, kind, how


def run_reference(args, items):
    """Reference arm: the reference's CPU implementation of the path on the host cores, on the same
    linears as this arm's workload; a step = one pass over them."""
    steps = max(1, min(args.steps, 2))       # bounded: a pass over the twelve decode linears takes ~10 s
    warm = 1 if args.warmup > 0 else 0
    val, dt, kind, how = cpu_pass(items, steps, warm)
    desc = f"all {len(items)} linears of the workload, {steps} timed pass(es) after {warm} warm-up linear(s)"
    return {
        "impl": "reference", "metric": "w4a4_fused_linear_effective_tops", "value": val, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s4xs4->s32",
        "data": "synthetic", "config": {"workload": WORKLOAD_DESC.get(args.workload, args.workload), "sample": desc},
        "cpu_baseline": {"value": val, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"{desc}; {how}"},
        "e2e": {"value": val, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# ----------------------------------------------------------------------------- legs
def leg_prefill(timer, device, args):
    """Many-token sweep: M in {2048, 8192} x residual density {0, 5, 15 %} x the four Llama-3-8B shapes,
    on packed nibbles and on prepared e4m3 bytes.  Per configuration the GEMM launch alone (activations
    expanded beforehand) against the tensor roofline, and quantisation + GEMM."""
    from zip_kernel_b200 import ops, synth, v9_linear
    bf16_burst, kind = measured_peak("bf16_tflops", 1590.0)
    bf16_sus, _ = measured_peak("bf16_tflops_sustained", 1400.0)
    peak_burst, peak_sus = 2.0 * bf16_burst, 2.0 * bf16_sus      # the 8-bit pipes run at twice the bf16 rate
    out = {"peak_burst": peak_burst, "peak_sustained": peak_sus,
           "peak_kind": f"{kind} bf16 cuBLAS figures x2 (no 8-bit peak was measured on this pool)", "unit": "TOP/s",
           "note": "GEMM-only launch per configuration; operands of the small shapes fit L2 (tensor-bound kernel)",
           "configs": {}}
    Ms = [int(m) for m in args.prefill_m.split(",")]
    dens = [float(d) for d in args.prefill_density.split(",")]
    for name, K, N in LLAMA3_8B:
        base = synth.make_container(N, K, DENSITY, seed=synth.shape_seed(0, K, N))
        for d in dens:
            W = base if abs(d - DENSITY) < 1e-9 else synth.make_container_like(base, d, seed=synth.shape_seed(1, K, N) + int(d * 1000))
            Wd = W.to(device)
            v9_linear.prepare_for_prefill(Wd)
            prep = Wd.prepared
            for M in Ms:
                X = synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1).to(device)
                q = ops.activation_quant_cuda(X, Wd.perm)
                for fmt in ("packed", "prepared"):
                    Wd.prepared = prep if fmt == "prepared" else None
                    XE, sumxf = ops.expand_activations_cuda(q[0], q[2], e4m3=fmt == "prepared")
                    gg, h1 = capture_graphs(lambda r: gemm_call(ops, Wd, XE, sumxf, q[1]), 1)
                    fg, h2 = capture_graphs(lambda r: fused_call(ops, X, Wd), 1)
                    ms_g, reps, _ = timer.time(lambda i: gg[0].replay(), 1, 3)
                    ms_f, _, _ = timer.time(lambda i: fg[0].replay(), 1, 3)
                    dense_ops = 2.0 * M * K * N
                    tops = dense_ops / (ms_g * 1e-3) / 1e12
                    out["configs"][f"{name}_M{M}_d{int(round(d * 100))}_{fmt}"] = {
                        "us_gemm": ms_g * 1e3, "us_quant_gemm": ms_f * 1e3, "tops_gemm": tops,
                        "tops_quant_gemm": dense_ops / (ms_f * 1e-3) / 1e12,
                        "residual_ops_frac": 2.0 * M * 16384 * W.n_hp_blocks / dense_ops,
                        "roofline": {"bound": "tensor", "achieved": tops, "frac_burst": tops / peak_burst,
                                     "frac_sustained": tops / peak_sus}, "reps_per_window": reps}
                    del gg, fg, h1, h2, XE, sumxf
                if W.n_hp_blocks == 0:
                    # the W4A16 route the reference takes for such a layer at this length (dequantise once, library
                    # fp16 GEMM; activations are NOT quantised): reported beside the W4A4 kernels, see DESIGN
                    W16 = v9_linear.dequant_u4_to_fp16(Wd)
                    ms_dq, _, _ = timer.time(lambda i: ops.dequant_u4_to_fp16_cuda(Wd.W_low_packed, Wd.scale_u4, Wd.zero_u4), 1, 2, min_window_s=0.05)
                    ms_mm, _, _ = timer.time(lambda i: torch.nn.functional.linear(X, W16), 1, 3, min_window_s=0.1)
                    out.setdefault("w4a16_route", {})[f"{name}_M{M}"] = {
                        "us_library_fp16_gemm": ms_mm * 1e3, "us_dequantise_weights": ms_dq * 1e3,
                        "tflops_library_fp16_gemm": 2.0 * M * K * N / (ms_mm * 1e-3) / 1e12}
                    del W16
                    Wd._fp16_cache = None
                del X, q
            Wd.prepared = None
            del Wd, prep
        del base
        torch.cuda.empty_cache()
    for fmt in ("packed", "prepared"):
        sel = [v for k, v in out["configs"].items() if k.endswith(fmt)]
        if sel:
            out[f"frac_burst_{fmt}_mean"] = statistics.mean(v["roofline"]["frac_burst"] for v in sel)
            out[f"frac_burst_{fmt}_min"] = min(v["roofline"]["frac_burst"] for v in sel)
    return out


def leg_sharded(timer, rank, world, device, args):
    """Llama-2-70B linears split column-parallel over the ranks (block-row granularity, activations
    replicated, every rank quantises itself), at M = 1 (graph-replayed, weights rotated past L2) and
    M = 4096, with and without the all-gather of the fp16 output shards.  Total work is fixed: strong
    scaling.  M = 1 also as one graph holding the linear AND its all-gather."""
    import torch.distributed as dist
    from zip_kernel_b200 import _lib, ops, sharding, synth, v9_linear

    hbm, hk = measured_peak("hbm_gbs", 6650.0)
    bf16, _ = measured_peak("bf16_tflops", 1590.0)
    shards, nnz_per_rank, res = {}, {}, {"per_linear_us": {}, "allgather_us": {}, "linear_plus_gather_graph_us": {},
                                         "linear_plus_peer_exchange_us": {}}
    pg = sharding.PeerGather(2 * 4096 * 57344, device=device) if world > 1 else None
    for name, K, N in LLAMA2_70B:
        W = synth.make_container(N, K, DENSITY, seed=synth.shape_seed(0, K, N))
        sh = sharding.shard_container(W, rank, world) if world > 1 else W
        if world > 1:
            sharding.check_shard_metadata(N, K, sh, rank, world)
        n_sets = sets_for(4 * sh.W_low_packed.numel())     # the four linears rotate together
        shards[name] = [sh.to(device) for _ in range(n_sets)]
        if args.prepared != "off":       # the M = 4096 leg runs on weights widened once; M = 1 streams the packed arrays
            for Wd in shards[name]:
                v9_linear.prepare_for_prefill(Wd)
        nnz_per_rank[name] = sh.n_hp_blocks
        del W
    for M in (1, 4096):
        Xs = {name: synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1).to(device) for name, K, N in LLAMA2_70B}
        ops_total = sum(2 * M * K * N for _, K, N in LLAMA2_70B)
        bytes_total = 0
        per = {}
        for name, K, N in LLAMA2_70B:
            sets = shards[name]

            def linear(r, sets=sets, name=name):
                return fused_call(ops, Xs[name], sets[r % len(sets)], token_major=False)   # (d_out_r, M): contiguous rows of the full output

            if M == 1:
                graphs, keep = capture_graphs(linear, len(sets))
                ms, _, _ = timer.time(lambda i: graphs[i % len(graphs)].replay(), 1, 3)
            else:
                ms, _, _ = timer.time(lambda i: linear(i), 1, 3, min_window_s=0.05)
            per[name] = ms * 1e3
            bytes_total += alg_bytes_gemm(M, K, N, 0)      # residual blocks left out: a lower bound
            if world > 1:
                y = linear(0)
                full = torch.empty((N, M), dtype=torch.float16, device=device)
                equal = len(set(sharding.shard_sizes(N, world))) == 1

                def gather():
                    if equal:
                        dist.all_gather_into_tensor(full, y)
                    else:
                        sharding.gather_output(y, N, token_major=False)
                ms_g, _, _ = timer.time(lambda i: gather(), 1, 3, min_window_s=0.05)
                res["allgather_us"][f"{name}_M{M}"] = ms_g * 1e3
                if M == 1 and equal:
                    # the linear and its all-gather captured together: one graph launch per step
                    try:
                        holder = _lib.WorkspaceHolder()
                        side = torch.cuda.Stream()
                        gl = []
                        with _lib.use_workspace(holder), torch.cuda.stream(side):
                            for r in range(len(sets)):
                                dist.all_gather_into_tensor(full, linear(r))
                            torch.cuda.synchronize()
                            for r in range(len(sets)):
                                g = torch.cuda.CUDAGraph()
                                with torch.cuda.graph(g, stream=side):
                                    dist.all_gather_into_tensor(full, linear(r))
                                gl.append(g)
                        torch.cuda.synchronize()
                        ms_lg, _, _ = timer.time(lambda i: gl[i % len(gl)].replay(), 1, 3)
                        res["linear_plus_gather_graph_us"][f"{name}_M{M}"] = ms_lg * 1e3
                        del gl, holder
                    except Exception as exc:   # capture of a collective refused: the eager figures stand
                        res["linear_plus_gather_graph_us"][f"{name}_M{M}"] = f"capture failed: {type(exc).__name__}"
                # the linear followed by the peer-memory exchange (one more kernel, no collective library call)
                if M == 1:
                    gp, kp = capture_graphs(lambda r: pg.gather(linear(r), N, token_major=False), len(sets) + (len(sets) & 1))
                    ms_p, _, _ = timer.time(lambda i: gp[i % len(gp)].replay(), 1, 3)
                    del gp, kp
                else:
                    # many tokens: token bands; a band's exchange runs on a side stream while the next band's GEMM runs
                    ms_p = time_banded_exchange(timer, ops, pg, Xs[name], sets, N, device)
                res["linear_plus_peer_exchange_us"][f"{name}_M{M}"] = ms_p * 1e3
            res["per_linear_us"][f"{name}_M{M}"] = per[name]
        t_lin = sum(per.values()) * 1e-6
        res[f"tops_M{M}"] = ops_total / t_lin / 1e12
        if M == 1:
            res["roofline_M1"] = {"bound": "hbm", "achieved": bytes_total / t_lin / 1e9, "peak": world * hbm,
                                  "frac": bytes_total / t_lin / 1e9 / (world * hbm), "unit": "GB/s",
                                  "peak_kind": f"{hk} copy bandwidth x {world} GPUs"}
        else:
            res[f"roofline_M{M}"] = {"bound": "tensor", "achieved": res[f"tops_M{M}"], "peak": world * 2 * bf16,
                                     "frac": res[f"tops_M{M}"] / (world * 2 * bf16), "unit": "TOP/s",
                                     "peak_kind": f"bf16 burst x2 x {world} GPUs"}
        if world > 1:
            t_g = t_lin + sum(res["allgather_us"][f"{n}_M{M}"] for n, _, _ in LLAMA2_70B) * 1e-6
            res[f"tops_M{M}_with_allgather"] = ops_total / t_g / 1e12
            lg = [res["linear_plus_gather_graph_us"].get(f"{n}_M{M}") for n, _, _ in LLAMA2_70B]
            if M == 1 and all(isinstance(v, float) for v in lg):
                res["tops_M1_linear_plus_gather_graph"] = ops_total / (sum(lg) * 1e-6) / 1e12
            lp = [res["linear_plus_peer_exchange_us"][f"{n}_M{M}"] for n, _, _ in LLAMA2_70B]
            res[f"tops_M{M}_with_peer_exchange"] = ops_total / (sum(lp) * 1e-6) / 1e12
        del Xs
    if pg is not None:
        pg.close()
    res["residual_blocks_per_rank"] = nnz_per_rank
    res["weights"] = "packed" if args.prepared == "off" else "packed; M=4096 on the prepared e4m3 copy"
    res["scaling"] = "strong"
    return res


def time_banded_exchange(timer, ops, pg, X, sets, N, device, bands=4):
    """One many-token sharded linear with its output exchanged over peer memory in token bands: band b's
    GEMM writes (T_b, N_r) token-major, its exchange runs on a side stream while band b + 1 computes."""
    T = int(X.shape[0])
    edges = [T * b // bands for b in range(bands + 1)]
    side = torch.cuda.Stream(device=device)

    def step(i):
        W = sets[i % len(sets)]
        main = torch.cuda.current_stream(device)
        outs = []
        for b in range(bands):
            y = fused_call(ops, X[edges[b]:edges[b + 1]], W, token_major=True)           # (T_b, N_r)
            y.record_stream(side)
            ev = torch.cuda.Event()
            ev.record(main)
            outs.append((y, ev))
        with torch.cuda.stream(side):
            for b, (y, ev) in enumerate(outs):
                side.wait_event(ev)
                pg.gather_band(y, N, T, edges[b])
        pg.advance()
        main.wait_stream(side)

    ms, _, _ = timer.time(step, 1, 3, min_window_s=0.05)
    return ms


def sharded_parity(rank, world, device):
    """A small layer sharded over the ranks (equal and ragged shard sizes), outputs gathered over NCCL and
    compared bit for bit with the single-GPU output every rank computes itself."""
    import torch.distributed as dist
    from zip_kernel_b200 import sharding, synth, v9_linear
    ok = True
    for (T, N, K) in ((5, 128 * 2 * world, 1024), (33, 128 * (2 * world + 1), 512), (300, 128 * world + 72, 256)):
        W = synth.make_container(N, K, 0.2, seed=synth.shape_seed(T, K, N), perm_seed=3)
        X = synth.make_activations(T, K, seed=7 + T).to(device)
        full = v9_linear.v9_linear_forward(X, W.to(device))
        sh = sharding.shard_container(W, rank, world)
        sharding.check_shard_metadata(N, K, sh, rank, world)
        got = sharding.column_parallel_forward(X, sh.to(device), N)
        ok = ok and bool(torch.equal(got, full))
        pg = sharding.PeerGather(2 * T * N, device=device)       # the library's own exchange over peer memory
        for _ in range(3):
            ok = ok and bool(torch.equal(sharding.column_parallel_forward(X, sh.to(device), N, exchange=pg), full))
        pg.close()
    flag = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def leg_legacy(timer, device):
    """Same-GPU anchor (reported, not a target): the reference's naive mma.sync s4 kernels (dense GEMM, block-sparse
    GEMM, element-wise sum), built for sm_100a from the reference tree by baseline/build_naive_reference.py, fed with
    activations quantised by this library.  None when the extension was not built."""
    from baseline import build_naive_reference
    from zip_kernel_b200 import ops, synth
    mod = build_naive_reference.load()
    if mod is None:
        return {"unavailable": "baseline/_ref/naive was not built (needs the reference tree and nvcc at build time)"}
    out = {"kernels": "reference csrc_naive dense_gemm_naive + sparse_gemm_naive + reduce_sum_naive, recompiled for sm_100a",
           "configs": {}}
    for name, M, K, N in (("o_M16", 16, 4096, 4096), ("gate_up_M16", 16, 4096, 28672), ("gate_up_M2048", 2048, 4096, 28672)):
        W = synth.make_container(N, K, DENSITY, seed=synth.shape_seed(0, K, N)).to(device)
        X = synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1).to(device)
        q4, qs, qsum = ops.activation_quant_cuda(X, W.perm)
        Yl = torch.empty((N, M), dtype=torch.float16, device=device)
        Yh = torch.zeros((N, M), dtype=torch.float16, device=device)
        Yt = torch.empty((N, M), dtype=torch.float16, device=device)

        def run(i):
            mod.dense_gemm(W.W_low_packed, q4, W.scale_u4, W.zero_u4, qsum, qs, Yl)
            mod.sparse_gemm(W.W_high_blocks_packed, W.hp_row_offsets, W.hp_col_indices, q4, W.scale_u4, qs, Yh, N, K)
            mod.reduce_sum(Yl, Yh, Yt)
        ms, _, _ = timer.time(run, 1, 3, min_window_s=0.05)
        ours = ops.fused_dense_sparse_cuda(W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets, W.hp_col_indices,
                                           q4, W.scale_u4, W.zero_u4, qsum, qs, N, K)
        ref = Yt.float()                 # the naive sparse kernel already carries the factor 16 of the residual
        dev_rel = float((ours.float() - ref).abs().max() / ref.abs().max().clamp(min=1e-6))
        g, kp = capture_graphs(lambda r: ops.fused_dense_sparse_cuda(W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets,
                                                                      W.hp_col_indices, q4, W.scale_u4, W.zero_u4, qsum, qs, N, K), 1)
        ms_ours, _, _ = timer.time(lambda i: g[0].replay(), 1, 3, min_window_s=0.05)
        out["configs"][name] = {"us_legacy": ms * 1e3, "tops_legacy": 2.0 * M * K * N / (ms * 1e-3) / 1e12,
                                "us_this_library_warm_l2": ms_ours * 1e3, "max_rel_deviation_from_this_library": dev_rel}
        del g, kp, W
    return out


def leg_stack(device):
    """Decoder-stack decode tokens per second (random-init Llama-3-8B architecture, batch 32, 1024-token
    prompt, 128 decode steps)."""
    from zip_kernel_b200 import decoder_stack as ds
    r = ds.run(ds.StackConfig(), 32, 1024, 128, device)
    return {"decode_tok_s": r["value"], "prefill_tok_s": r["prefill_tokens_per_s"],
            "ms_per_decode_step": r["ms_per_decode_step"], "config": r["config"]}


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode")
    ap.add_argument("--legs", default="auto",
                    help="comma list of cfg0,prefill,cfg3,stack; auto = all for the default workload, none otherwise")
    ap.add_argument("--prefill-m", default="2048,8192")
    ap.add_argument("--prefill-density", default="0,0.05,0.15")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prepared", default="auto", choices=["auto", "on", "off"],
                    help="many-token workloads: also hold the weights widened once to e4m3 bytes "
                         "(prepare_for_prefill, 2x the packed bytes) so the tensor-core kernel runs its "
                         "fp8 instantiation; auto = on when every M >= 256")
    args = ap.parse_args()
    if args.workload == "cfg3_sharded":       # former name of the sharded leg on its own
        args.workload, args.legs = "decode", "cfg3"
    items = workload_items(args.workload)
    legs = (["cfg0", "prefill", "cfg3", "stack", "legacy"] if args.workload == "decode" else []) if args.legs == "auto" \
        else [l for l in args.legs.split(",") if l and l != "none"]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, items)), flush=True)
        return

    import torch.distributed as dist
    from zip_kernel_b200 import _lib, backend, ops, synth, v9_linear

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    timer = Timer(world, device)
    t_start = time.perf_counter()

    parity = sharded_parity(rank, world, device) if world > 1 else None

    # ------------------------------------------------------------------ main workload
    shapes = {(k, n) for _, _, k, n in items}
    w_bytes = sum(k * n // 2 for k, n in shapes)
    n_sets = sets_for(w_bytes)
    many_tokens = min(i[1] for i in items) >= 256
    if args.prepared == "on" and not many_tokens:
        raise SystemExit("--prepared on needs a workload whose linears all take the tensor-core kernel (M >= 256)")
    use_prepared = many_tokens and args.prepared != "off"
    wsets = {}
    for K, N in shapes:
        _, wsets[(K, N)] = make_weights(K, N, DENSITY, device, n_sets)
        if use_prepared:
            for W in wsets[(K, N)]:
                v9_linear.prepare_for_prefill(W)
    data = []
    for name, M, K, N in items:
        Xh = synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1).pin_memory()
        it = dict(name=name, M=M, K=K, N=N, X_host=Xh, W=wsets[(K, N)], X_dev=Xh.to(device),
                  Y_host=torch.empty((M, N), dtype=torch.float16).pin_memory())
        it["q"] = ops.activation_quant_cuda(it["X_dev"], it["W"][0].perm)
        it["XE"], it["sumxf"] = ops.expand_activations_cuda(it["q"][0], it["q"][2], e4m3=use_prepared)
        data.append(it)

    def device_step(r):
        for it in data:
            it["Y"] = fused_call(ops, it["X_dev"], it["W"][r])

    def gemm_only_step(r):
        for it in data:
            gemm_call(ops, it["W"][r], it["XE"], it["sumxf"], it["q"][1])

    def e2e_step(i):
        # public host-staged call: pinned activations in, pinned results out.  The linears of a step are
        # independent requests with buffers of their own; the batch call captures copy in, quantisation +
        # GEMM and copy out of all of them as one graph (up to twelve parallel branches, so one request's
        # copies and kernels overlap another's; `value` chains the same linears on ONE stream) and replays it.
        # The step ends when every result is on the host.
        host_batches[i % n_sets].replay()
        torch.cuda.current_stream().synchronize()

    step_graphs, keep1 = capture_graphs(device_step, n_sets)
    gemm_graphs, keep2 = capture_graphs(gemm_only_step, n_sets)
    per_shape = {}
    warmup = max(3, args.warmup)
    with ClockSampler(local_rank) as clk:
        ms_dev, reps_dev, win_dev = timer.time(lambda i: step_graphs[i % n_sets].replay(), args.steps, warmup)
        ms_gemm, reps_gemm, _ = timer.time(lambda i: gemm_graphs[i % n_sets].replay(), args.steps, warmup)
    e2e_steps = max(5, args.steps // 5)
    # one captured batch per weight set, held like a serving loop holds it (arguments are checked at capture)
    # (submitted largest first: the long linears start at once and the short ones fill in beside them)
    by_size = sorted(data, key=lambda it: -it["K"] * it["N"] * max(it["M"], 16))
    host_batches = [backend.v9_linear_host_batch_graph([(it["X_host"], it["W"][r], it["Y_host"]) for it in by_size])
                    for r in range(n_sets)]
    ms_e2e, reps_e2e, _ = timer.time(e2e_step, e2e_steps, 3)

    # per-linear GEMM launches on their own (graph of n_sets launches of one linear, weights rotating)
    hbm_peak, hbm_kind = measured_peak("hbm_gbs", 6650.0)
    if not many_tokens and len(data) > 1:
        for it in data:
            gl, kp = capture_graphs(lambda r, it=it: [gemm_call(ops, it["W"][s], it["XE"], it["sumxf"], it["q"][1])
                                                      for s in range(n_sets)], 1)
            ms1, _, _ = timer.time(lambda i: gl[0].replay(), 1, 3, min_window_s=0.05)
            us = ms1 * 1e3 / n_sets
            b = alg_bytes_gemm(it["M"], it["K"], it["N"], it["W"][0].n_hp_blocks)
            per_shape[it["name"]] = {"us_gemm": us, "frac_hbm": b / (us * 1e-6) / 1e9 / hbm_peak}
            del gl, kp

    dev_err = _lib.device_error(device)
    ops_step = sum(2 * it["M"] * it["K"] * it["N"] for it in data)
    bytes_gemm = sum(alg_bytes_gemm(it["M"], it["K"], it["N"], it["W"][0].n_hp_blocks, use_prepared) for it in data)
    gemm_s = ms_gemm / 1e3 / args.steps
    if many_tokens:
        bf16, peak_kind = measured_peak("bf16_tflops", 1590.0)
        peak, achieved = 2.0 * bf16, ops_step / gemm_s / 1e12
        peak_kind += " bf16 burst x2 (8-bit tensor pipe)"
    else:
        peak, peak_kind = hbm_peak, hbm_kind + " copy bandwidth"
        achieved = bytes_gemm / gemm_s / 1e9
    value = world * ops_step / (ms_dev / 1e3 / args.steps) / 1e12
    e2e_val = world * ops_step / (ms_e2e / 1e3 / e2e_steps) / 1e12
    traffic = NCU_TRAFFIC.get((args.workload, "prepared" if use_prepared else "packed"))

    out = {
        "metric": "w4a4_fused_linear_effective_tops", "value": value, "unit": "TOPS",
        "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_dev / args.steps,
        "windows": WINDOWS, "reps_per_window": reps_dev, "window_ms_per_step": [w / args.steps for w in win_dev],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s4xs4->s32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_DESC[args.workload], "linears_per_step": len(data),
                   "l2": f"weights rotate through {n_sets} distinct copies (> 2x L2)",
                   "step": "CUDA-graph replay of quant+GEMM per linear", "parallelism": f"replicated x{world}",
                   "timing": f"median of {WINDOWS} windows of reps_per_window x steps steps (>= {MIN_WINDOW_S} s each), CUDA events, max over ranks",
                   "weights": ("packed nibbles + copy widened once to e4m3 bytes (opt-in prepare_for_prefill); "
                               "MMA kind::f8f6f4, bit-identical outputs") if use_prepared else "packed nibbles"},
        "us_per_linear": ms_dev / args.steps / len(data) * 1e3,
        "e2e": {"value": e2e_val, "unit": "TOPS",
                "h2d_bytes_per_step": sum(it["X_host"].numel() * 2 for it in data),
                "d2h_bytes_per_step": sum(it["Y_host"].numel() * 2 for it in data),
                "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps, "reps_per_window": reps_e2e,
                "schedule": "the step's linears as independent host-staged requests on parallel graph branches "
                            "(copies and kernels of different requests overlap; `value` chains them on one stream)"},
        "gpu_launches": args.steps * len(data) * 2,
        "roofline": {"bound": "tensor" if many_tokens else "hbm", "achieved": achieved, "peak": peak,
                     "unit": "TOP/s" if many_tokens else "GB/s", "frac": achieved / peak,
                     "traffic": traffic[0] if traffic else None,
                     "traffic_source": f"{traffic[1]}, captured {traffic[2]}" if traffic else None,
                     "peak_kind": peak_kind,
                     "kernel": "prefill_gemm_kernel" if many_tokens else "decode_gemm_kernel",
                     "us_per_launch": gemm_s / len(data) * 1e6, "bytes_per_launch": bytes_gemm / len(data),
                     "per_shape": per_shape or None},
        "clocks": clk.summary(),
        "device_error_word": dev_err,
    }
    if parity is not None:
        out["sharded_parity"] = parity
    del step_graphs, gemm_graphs, keep1, keep2, host_batches, data, wsets
    backend.clear_cuda_graph_cache()
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ further legs
    for leg in legs:
        try:
            if leg in ("cfg0", "prefill") and world > 1:
                continue                      # single-GPU legs: the N = 1 line carries them
            if leg == "cfg0":
                K = N = 4096
                _, ws = make_weights(K, N, DENSITY, device, sets_for(K * N // 2))
                X = synth.make_activations(16, K, seed=synth.shape_seed(16, K, N) + 1).to(device)
                g, kp = capture_graphs(lambda r: [fused_call(ops, X, W) for W in ws], 1)
                ms0, _, _ = timer.time(lambda i: g[0].replay(), 1, 3, min_window_s=0.05)
                us = ms0 * 1e3 / len(ws)
                out["cfg0"] = {"workload": WORKLOAD_DESC["cfg0"], "us_per_linear": us, "tops": 2 * 16 * K * N / (us * 1e-6) / 1e12}
                del g, kp, ws
            elif leg == "prefill":
                out["prefill"] = leg_prefill(timer, device, args)
            elif leg == "cfg3":
                out["cfg3"] = leg_sharded(timer, rank, world, device, args)
            elif leg == "legacy" and world == 1:
                out["legacy_gpu_baseline"] = leg_legacy(timer, device)
            elif leg == "stack" and world == 1:
                out["stack"] = leg_stack(device)
                out["decode_tok_s"] = out["stack"]["decode_tok_s"]
        except Exception as exc:      # a leg never takes the headline down with it
            out[leg] = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.empty_cache()
    out["device_error_word_after_legs"] = _lib.device_error(device)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        val, dt, kind, how = cpu_pass(items, 1, 1)
        out["cpu_baseline"] = {"value": val, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": kind,
                               "sample": f"one pass over all {len(items)} linears of the workload ({dt:.1f} s) after one warm-up linear; {how}"}
    out["wall_s"] = time.perf_counter() - t_start
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
