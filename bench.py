"""Benchmark of the W4A4 fused-linear hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload decode|prefill]

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
bytes/s of the GEMM kernel launches alone; `cpu_baseline` = the CPU oracle's
dequantise->matmul route on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA3_8B = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]
DENSITY = 0.05
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum per GEMM launch (mean over the
# workload's launches) from the profiler capture summarised under profiles/
NCU_TRAFFIC_BYTES = {
    "decode": 30.49e6,            # profiles/decode_gemm_kernel_dram_traffic.md
    "gate_up_m16": 65.82e6,       # profiles/decode_gemm_kernel_gate_up_m16.md
    "prefill_gate_up": 225.9e6,   # profiles/prefill_gemm_kernel_gate_up_m2048.md (prepared weights)
    "prefill_gate_up/packed": 153.2e6,
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
    raise SystemExit(f"unknown workload {name}")


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


def build_inputs(items, device, n_sets):
    """Per item: host activations (pinned), and n_sets distinct device copies of the weights."""
    from zip_kernel_b200 import synth
    cache, out = {}, []
    for name, M, K, N in items:
        if (K, N) not in cache:
            W = synth.make_container(N, K, DENSITY, seed=synth.shape_seed(0, K, N))
            cache[(K, N)] = [W.to(device)] + [None] * (n_sets - 1)
            for r in range(1, n_sets):
                cache[(K, N)][r] = W.to(device)      # a distinct allocation per set
        X = synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1).pin_memory()
        out.append(dict(name=name, M=M, K=K, N=N, X_host=X, W=cache[(K, N)]))
    return out


def alg_bytes_gemm(it, prepared=False):
    """Bytes one GEMM launch must move: weights (half a byte per code packed, one byte
    prepared), scales/zeros, residual blocks and index, expanded activation codes (one
    byte each) with their scales and group sums, output."""
    M, K, N = it["M"], it["K"], it["N"]
    nnz = it["W"][0].n_hp_blocks
    ng, nbr = K // 128, (N + 127) // 128
    wb = 2 if prepared else 1
    b_w = wb * K * N // 2 + 4 * N * ng + wb * 8192 * nnz + 4 * (nbr + 1) + 4 * nnz
    return b_w + (M * K + 2 * M + 4 * M * ng) + 2 * M * N


# ----------------------------------------------------------------------------- reference arm
def run_reference(args, items):
    """CPU arm: the oracle's restatement of the reference's dequantise -> fp32
    matmul route, all host threads, on a bounded sample of the workload."""
    from oracle import w4a4_oracle as O
    from zip_kernel_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    # bounded sample: the M=16 linears of the two smaller shapes
    sample = [it for it in items if it[1] == max(i[1] for i in items)][:2]
    data = []
    for name, M, K, N in sample:
        W = synth.make_container(N, K, DENSITY, seed=synth.shape_seed(0, K, N))
        X = synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1)
        Wt = dict(W_low_packed=W.W_low_packed, W_high_blocks_packed=W.W_high_blocks_packed,
                  scale_u4=W.scale_u4, zero_u4=W.zero_u4, hp_row_offsets=W.hp_row_offsets,
                  hp_col_indices=W.hp_col_indices, d_out=N, d_in=K)
        data.append((X, W.perm, Wt, 2 * M * K * N))
    def step():
        for X, perm, Wt, _ in data:
            O.cpu_reference_path(X, perm, Wt)
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    ops = sum(d[3] for d in data)
    val = ops / dt / 1e12
    desc = "+".join(n for n, *_ in sample)
    return {
        "impl": "reference", "metric": "w4a4_fused_linear_effective_tops", "value": val, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s4xs4->s32",
        "data": "synthetic", "config": {"workload": args.workload_desc, "sample": desc},
        "cpu_baseline": {"value": val, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{desc}: quantise + dequantise->fp32 matmul, {steps} passes"},
        "e2e": {"value": val, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# ----------------------------------------------------------------------------- sharded 70B linears
LLAMA2_70B = [("qkv", 8192, 10240), ("o", 8192, 8192), ("gate_up", 8192, 57344), ("down", 28672, 8192)]


def run_sharded(args, rank, world, device):
    """Llama-2-70B linears split column-parallel over the ranks (block-row
    granularity, activations replicated, every rank quantises itself), at M = 1
    (graph-replayed, weights rotated past L2) and M = 4096, each with and without
    the all-gather of the fp16 output shards.  Total work is fixed: strong scaling."""
    import torch.distributed as dist
    from zip_kernel_b200 import ops, sharding, synth, v9_linear

    def ev_time(fn, reps, warm):
        for _ in range(warm):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms * 1e3     # us

    shards, nnz_per_rank = {}, {}
    for name, K, N in LLAMA2_70B:
        W = synth.make_container(N, K, DENSITY, seed=synth.shape_seed(0, K, N))
        sh = sharding.shard_container(W, rank, world) if world > 1 else W
        sharding.check_shard_metadata(N, K, sh, rank, world) if world > 1 else None
        shard_bytes = sh.W_low_packed.numel()
        n_sets = max(2, -(-2 * L2_BYTES // max(4 * shard_bytes, 1)) + 1)     # the four linears rotate together
        shards[name] = [sh.to(device) for _ in range(min(n_sets, 8))]
        if args.prepared != "off":       # the M = 4096 leg runs on weights widened once; M = 1 streams the packed arrays
            for Wd in shards[name]:
                v9_linear.prepare_for_prefill(Wd)
        nnz_per_rank[name] = sh.n_hp_blocks
        del W
    res = {"per_linear_us": {}, "allgather_us": {}}
    ops_total = {}
    for M in (1, 4096):
        Xs = {name: synth.make_activations(M, K, seed=synth.shape_seed(M, K, N) + 1).to(device) for name, K, N in LLAMA2_70B}
        for name, K, N in LLAMA2_70B:
            ops.reserve_workspace(device, M, K, shards[name][0].d_out, shards[name][0].n_hp_blocks)

        def linear(name, r):
            W = shards[name][r % len(shards[name])]
            return ops.fused_dense_sparse_e2e_cuda(Xs[name], W.perm, W.W_low_packed, W.W_high_blocks_packed,
                                                   W.hp_row_offsets, W.hp_col_indices, W.scale_u4, W.zero_u4,
                                                   W.d_out, W.d_in, prepared=W.prepared)   # (d_out_r, M): contiguous rows of the full output
        ops_total[M] = sum(2 * M * K * N for _, K, N in LLAMA2_70B)
        per = {}
        for name, K, N in LLAMA2_70B:
            n_sets = len(shards[name])
            if M == 1:
                side = torch.cuda.Stream()
                with torch.cuda.stream(side):
                    ops.reserve_workspace(device, M, K, shards[name][0].d_out, shards[name][0].n_hp_blocks)
                    for r in range(n_sets):
                        linear(name, r)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        for r in range(n_sets):
                            linear(name, r)
                torch.cuda.synchronize()
                per[name] = ev_time(g.replay, 30, 3) / n_sets
            else:
                cnt = [0]
                def one():
                    cnt[0] += 1
                    linear(name, cnt[0])
                per[name] = ev_time(one, 10, 3)
            if world > 1:
                y = linear(name, 0)
                full = torch.empty((N, M), dtype=torch.float16, device=device)
                equal = len(set(sharding.shard_sizes(N, world))) == 1
                def gather():
                    if equal:
                        dist.all_gather_into_tensor(full, y)
                    else:
                        sharding.gather_output(y, N, token_major=False)
                res["allgather_us"][f"{name}_M{M}"] = ev_time(gather, 20, 3)
            res["per_linear_us"][f"{name}_M{M}"] = per[name]
        res[f"tops_M{M}"] = ops_total[M] / (sum(per.values()) * 1e-6) / 1e12
        if world > 1:
            t_g = sum(per.values()) + sum(res["allgather_us"][f"{n}_M{M}"] for n, _, _ in LLAMA2_70B)
            res[f"tops_M{M}_with_allgather"] = ops_total[M] / (t_g * 1e-6) / 1e12
    res["residual_blocks_per_rank"] = nnz_per_rank
    return res


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prepared", default="auto", choices=["auto", "on", "off"],
                    help="many-token workloads: also hold the weights widened once to e4m3 bytes "
                         "(prepare_for_prefill, 2x the packed bytes) so the tensor-core kernel runs its "
                         "fp8 instantiation; auto = on when every M >= 256")
    args = ap.parse_args()
    items = workload_items(args.workload) if args.workload != "cfg3_sharded" else []
    args.workload_desc = {
        "decode": "Llama-3-8B linears (qkv,o,gate_up,down) x M in {1,4,16}, 5% residual blocks",
        "prefill": "Llama-3-8B linears (qkv,o,gate_up,down) x M=2048, 5% residual blocks",
        "cfg0": "single linear 4096->4096, M=16, 5% residual blocks",
        "gate_up_m16": "single linear 4096->28672, M=16, 5% residual blocks",
        "prefill_gate_up": "single linear 4096->28672, M=2048, 5% residual blocks",
        "cfg3_sharded": "Llama-2-70B linears (qkv,o,gate_up,down), M in {1,4096}, column-parallel shards, 5% residual blocks",
    }[args.workload]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, items)), flush=True)
        return

    import torch.distributed as dist
    from zip_kernel_b200 import backend, ops, v9_linear

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if args.workload == "cfg3_sharded":
        res = run_sharded(args, rank, world, device)
        if rank == 0:
            print(json.dumps({"metric": "w4a4_fused_linear_effective_tops", "value": res["tops_M1"], "unit": "TOPS",
                              "n_gpus": world, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                              "dtype": "s4xs4->s32", "data": "synthetic",
                              "config": {"workload": args.workload_desc, "parallelism": f"column-parallel x{world}",
                                         "weights": "packed" if args.prepared == "off" else "packed + prepared e4m3 copy for M=4096"},
                              **res}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    w_bytes = sum(k * n // 2 for _, k, n in {(i[2], i[3]): (0, i[2], i[3]) for i in items}.values())
    n_sets = max(2, -(-2 * L2_BYTES // max(w_bytes, 1)) + 1)
    data = build_inputs(items, device, n_sets)
    many_tokens = min(i[1] for i in items) >= 256
    if args.prepared == "on" and not many_tokens:
        raise SystemExit("--prepared on needs a workload whose linears all take the tensor-core kernel (M >= 256)")
    use_prepared = many_tokens and args.prepared != "off"
    if use_prepared:
        for W in {id(W): W for it in data for W in it["W"]}.values():
            v9_linear.prepare_for_prefill(W)
    for it in data:
        it["X_dev"] = it["X_host"].to(device)
        it["Y_host"] = torch.empty((it["M"], it["N"]), dtype=torch.float16).pin_memory()
        ops.reserve_workspace(device, it["M"], it["K"], it["N"], it["W"][0].n_hp_blocks)

    def device_step(r):
        for it in data:
            W = it["W"][r]
            it["Y"] = ops.fused_dense_sparse_e2e_cuda(
                it["X_dev"], W.perm, W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets,
                W.hp_col_indices, W.scale_u4, W.zero_u4, W.d_out, W.d_in, token_major=True, prepared=W.prepared)

    def gemm_only_step(r):
        for it in data:
            W = it["W"][r]
            q = it["q"]
            ops.fused_dense_sparse_expanded_cuda(W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets,
                                                 W.hp_col_indices, it["XE"], it["sumxf"], W.scale_u4,
                                                 W.zero_u4, q[1], W.d_out, W.d_in, token_major=True,
                                                 prepared=W.prepared, e4m3=W.prepared is not None)

    def e2e_step(r):
        # public host-staged call: pinned activations in, pinned results out.  The twelve linears of a
        # step are independent requests with buffers of their own; the batch call captures copy in,
        # quantisation + GEMM and copy out of all of them as one graph (three parallel branches, so one
        # linear's copies overlap another's kernels) and replays it.  The step ends when every result is
        # on the host.
        backend.v9_linear_forward_host_graph_many([(it["X_host"], it["W"][r], it["Y_host"]) for it in data])
        torch.cuda.current_stream().synchronize()

    # eager warm-up (also sizes every workspace before capture)
    for it in data:
        it["q"] = ops.activation_quant_cuda(it["X_dev"], it["W"][0].perm)
        it["XE"], it["sumxf"] = ops.expand_activations_cuda(it["q"][0], it["q"][2], e4m3=use_prepared)
    for r in range(n_sets):
        device_step(r)
        gemm_only_step(r)
    torch.cuda.synchronize()

    def capture(fn):
        graphs = []
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for r in range(n_sets):
                from zip_kernel_b200 import _lib
                for it in data:   # the workspace is keyed by stream: allocate on the capture stream
                    ops.reserve_workspace(device, it["M"], it["K"], it["N"], it["W"][0].n_hp_blocks)
                fn(r)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    fn(r)
                graphs.append(g)
        torch.cuda.synchronize()
        return graphs

    step_graphs = capture(device_step)
    gemm_graphs = capture(gemm_only_step)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run, steps, warmup):
        for i in range(warmup):
            run(i % n_sets)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            run((warmup + i) % n_sets)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    warmup = max(3, args.warmup)
    with ClockSampler(local_rank) as clk:
        ms_dev = timed(lambda r: step_graphs[r].replay(), args.steps, warmup)
        ms_gemm = timed(lambda r: gemm_graphs[r].replay(), args.steps, warmup)
    for r in range(n_sets):
        e2e_step(r)           # captures
    ms_e2e = timed(e2e_step, max(10, args.steps // 5), 3)
    e2e_steps = max(10, args.steps // 5)

    from zip_kernel_b200 import _lib
    dev_err = _lib.device_error(device)

    ops_step = sum(2 * it["M"] * it["K"] * it["N"] for it in data)
    bytes_gemm = sum(alg_bytes_gemm(it, use_prepared) for it in data)
    gemm_s = ms_gemm / 1e3 / args.steps
    tensor_bound = min(it["M"] for it in data) >= 256
    if tensor_bound:
        # s8 tensor-core work: the int8 pipe runs at twice the bf16 rate, so the
        # denominator is twice the measured bf16 GEMM burst figure
        bf16, peak_kind = measured_peak("bf16_tflops", 1590.0)
        peak, achieved = 2.0 * bf16, ops_step / gemm_s / 1e12
        peak_kind += " bf16 burst x2 (int8 pipe)"
    else:
        peak, peak_kind = measured_peak("hbm_gbs", 6650.0)
        achieved = bytes_gemm / gemm_s / 1e9
    value = world * ops_step / (ms_dev / 1e3 / args.steps) / 1e12
    e2e_val = world * ops_step / (ms_e2e / 1e3 / e2e_steps) / 1e12

    out = {
        "metric": "w4a4_fused_linear_effective_tops", "value": value, "unit": "TOPS",
        "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_dev / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s4xs4->s32",
        "data": "synthetic",
        "config": {"workload": args.workload_desc, "linears_per_step": len(data),
                   "l2": f"weights rotate through {n_sets} distinct copies (> 2x L2)",
                   "step": "CUDA-graph replay of quant+GEMM per linear", "parallelism": f"replicated x{world}",
                   "weights": ("packed nibbles + copy widened once to e4m3 bytes (opt-in prepare_for_prefill); "
                               "MMA kind::f8f6f4, bit-identical outputs") if use_prepared else "packed nibbles"},
        "us_per_linear": ms_dev / args.steps / len(data) * 1e3,
        "e2e": {"value": e2e_val, "unit": "TOPS",
                "h2d_bytes_per_step": sum(it["X_host"].numel() * 2 for it in data),
                "d2h_bytes_per_step": sum(it["Y_host"].numel() * 2 for it in data),
                "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": args.steps * len(data) * 2,
        "roofline": {"bound": "tensor" if tensor_bound else "hbm", "achieved": achieved, "peak": peak,
                     "unit": "TOP/s" if tensor_bound else "GB/s",
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(args.workload if (use_prepared or not many_tokens)
                                                                else args.workload + "/packed"), "peak_kind": peak_kind,
                     "kernel": "prefill_gemm_kernel" if tensor_bound else "decode_gemm_kernel",
                     "us_per_launch": gemm_s / len(data) * 1e6,
                     "bytes_per_launch": bytes_gemm / len(data)},
        "clocks": clk.summary(),
        "device_error_word": dev_err,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ref = run_reference(argparse.Namespace(**{**vars(args), "steps": 3, "warmup": 1}), items)
        out["cpu_baseline"] = ref["cpu_baseline"]
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
