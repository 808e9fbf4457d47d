"""Benchmark of the low-bit matmul hot path.

Headline workload (N = 1 GPU): decode-size A16W4 GEMV, M = 1, bf16, 8192 x 8192, group_size 128,
with bias, over 32 DISTINCT layers per step (1.1 GB of packed weights, far larger than the 126 MB L2,
so every launch streams its weights from HBM).  metric = algorithmic HBM GB/s.

  value     kernel-only: the 32 gl_matmul launches of a step replayed as one CUDA graph, inputs resident
  e2e       the public API (GemLiteLinear.forward) with host buffers: pinned-host x -> device, 32 chained
            layer forwards, result -> host, every step (also as a CUDA graph; eager Python numbers beside it)
  roofline  algorithmic bytes per launch / average launch time, against the measured HBM copy peak
  cpu_baseline   the reference's CPU-capable torch path (unpack -> (W_q - z) * s -> matmul) on host cores
  sweep     other batch sizes / formats of the benchmark configurations (GB/s for M <= 16, TFLOP/s above)

`--impl reference` times that CPU path alone (the reference has no GPU-free way to run its Triton kernels;
its CPU implementation is what can run without them).  With --gpus N > 1 (torchrun) every rank runs the
same per-GPU workload (weak scaling, no data-path collective) and rank 0 reports the aggregate.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_FEAT = K_FEAT = 8192
GROUP = 128
LAYERS = 32


def bench_reference():
    """Figures measured outside this script and kept beside it in bench_reference.json: the DRAM bytes of one launch
    of the headline kernel from an ncu capture, and the reference's own Triton kernels timed on a B200."""
    try:
        return json.load(open(os.path.join(ROOT, "bench_reference.json")))
    except Exception:
        return {}


def algorithmic_bytes(M, N, K, nbits, group, itemsize=2, bias=True):
    """Bytes each operand is read / written once: packed W + scales + zeros + x + out (+ bias)."""
    G = K // group
    return N * K * nbits // 8 + G * N * 2 * itemsize + M * K * itemsize + M * N * itemsize + (N * itemsize if bias else 0)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1585.3)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "samples": len(sm), "reasons": sorted(reasons)}


# -------------------------------------------------------------------------------------------------
def cpu_path_sample(seconds=12.0, N=N_FEAT, K=K_FEAT, nbits=4, group=GROUP):
    """Time the reference's CPU path (oracle port, torch ops, all host threads) for about `seconds`."""
    from oracle import oracle
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(2000)
    e = 32 // nbits
    Wp = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // e), generator=g, dtype=torch.int64).to(torch.int32)
    s = (torch.randn(N * K // group, 1, generator=g).abs() * 0.02)
    z = torch.rand(N * K // group, 1, generator=g) * (2 ** nbits - 1)
    x = torch.randn(1, K, generator=g)
    oracle.cpu_reference_forward(x, Wp, s, z, nbits, group)     # warm-up
    times, t_end = [], time.perf_counter() + seconds
    while time.perf_counter() < t_end or len(times) < 3:
        t0 = time.perf_counter()
        oracle.cpu_reference_forward(x, Wp, s, z, nbits, group)
        times.append(time.perf_counter() - t0)
        if len(times) >= 50:
            break
    times.sort()
    med = times[len(times) // 2]
    gbs = algorithmic_bytes(1, N, K, nbits, group, bias=False) / med / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "%d forward passes of one %dx%d A16W%d layer (M=1, gs=%d): unpack + dequant + matmul in fp32 torch ops, median %.1f ms"
                      % (len(times), N, K, nbits, group, med * 1e3), "ms_per_layer": med * 1e3}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per = max(2.0, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_path_sample(seconds=per / 4)
    vals = [cpu_path_sample(seconds=per) for _ in range(max(1, args.steps))]
    v = sum(r["value"] for r in vals) / len(vals)
    ms = sum(r["ms_per_layer"] for r in vals) / len(vals) * LAYERS
    base = dict(vals[-1]); base["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": "A16W4 GEMV HBM GB/s (M=1, 8192x8192, gs=128, bf16)", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg2 A16W4 M=1 8192x8192 gs128: reference CPU path (torch unpack + dequant + matmul), one layer per sample", "l2": "n/a (CPU)"},
        "cpu_baseline": base, "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


# -------------------------------------------------------------------------------------------------
def build_layers(device, n_layers, M_max, nbits=4, group=GROUP, N=N_FEAT, K=K_FEAT, seed=1234):
    from gemlite_b200 import helper
    g = torch.Generator(device=device).manual_seed(seed)
    proc = helper.A16Wn_HQQ_INT(device=str(device), dtype=torch.bfloat16, W_nbits=nbits)
    layers = []
    for _ in range(n_layers):
        W_q = torch.randint(0, 2 ** nbits, (N, K), generator=g, device=device, dtype=torch.int32).to(torch.uint8)
        s = (torch.randn(N * K // group, 1, generator=g, device=device).abs() * 0.02).to(torch.bfloat16)
        # scales of the benchmark distribution make activations grow ~7x per chained layer; they are
        # divided by that factor so that 32 chained layers stay finite (timing does not depend on it)
        s = s / 6.7
        z = (torch.rand(N * K // group, 1, generator=g, device=device) * (2 ** nbits - 1)).to(torch.bfloat16)
        b = (torch.randn(N, generator=g, device=device) * 0.01).to(torch.bfloat16)
        layers.append(proc.from_weights(W_q, s, z, bias=b))
        del W_q
    return layers


def time_graph(fn, steps, warmup, stream):
    """Run fn() twice eagerly, capture it once in a CUDA graph on `stream`, replay it `warmup` times and return
    the graph; the caller times `steps` replays with CUDA events on the same stream."""
    with torch.cuda.stream(stream):
        for _ in range(2):
            fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        return graph


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel decoder-layer step")
    ap.add_argument("--case", default=None, help="run one format:M case of the sweep a few times and print its time (for profiling), e.g. MXFP4:4096")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.case:
        fmt, M = args.case.split(":")
        print(json.dumps(sweep_gemm(torch.device("cuda", 0), only=(fmt, int(M)))))
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=180))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)

    from gemlite_b200 import _lib, core
    L = _lib.lib()
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    M = 1
    layers = build_layers(device, LAYERS, M)
    stream = torch.cuda.Stream(device)
    bytes_per_launch = algorithmic_bytes(M, N_FEAT, K_FEAT, 4, GROUP)

    # ---- kernel-only: 32 gl_matmul launches per step through the C ABI, inputs resident ----------
    x_dev = torch.randn(M, K_FEAT, device=device, dtype=torch.bfloat16)
    outs = [torch.empty(M, N_FEAT, device=device, dtype=torch.bfloat16) for _ in range(LAYERS)]
    arg_structs = []
    with torch.cuda.stream(stream):
        for lyr, out in zip(layers, outs):
            a = core._fill_args(x_dev, lyr.bias, lyr.W_q, lyr.scales, lyr.zeros, None, None, out, lyr.get_meta_args(), -1)
            ws = core._workspace(device, int(L.gl_matmul_workspace_bytes(ctypes.byref(a))))
            if ws is not None:
                a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            arg_structs.append(a)
    kernel_name = L.gl_matmul_kernel_name(ctypes.byref(arg_structs[0])).decode()

    def step_kernels():
        sp = torch.cuda.current_stream(device).cuda_stream
        for a in arg_structs:
            st = L.gl_matmul(ctypes.byref(a), sp)
            if st != 0:
                raise RuntimeError(L.gl_last_error().decode())

    graph = time_graph(step_kernels, args.steps, args.warmup, stream)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
    barrier()
    ms_kernel = e0.elapsed_time(e1) / args.steps

    # ---- end to end: pinned host x -> device, 32 chained GemLiteLinear.forward, result -> host ---
    x_host = torch.randn(M, K_FEAT, dtype=torch.bfloat16).pin_memory()
    y_host = torch.empty(M, N_FEAT, dtype=torch.bfloat16).pin_memory()
    x_in = torch.empty(M, K_FEAT, device=device, dtype=torch.bfloat16)

    def step_e2e():
        x_in.copy_(x_host, non_blocking=True)
        h = x_in
        for lyr in layers:
            h = lyr(h)
        y_host.copy_(h, non_blocking=True)

    graph_e2e = time_graph(step_e2e, args.steps, args.warmup, stream)
    barrier()
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(args.steps):
            graph_e2e.replay()
        e1.record(stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    finite = bool(torch.isfinite(y_host.float()).all())
    # eager Python path (no graph), wall-bounded by host launch overhead
    with torch.cuda.stream(stream):
        for _ in range(3):
            step_e2e()
        stream.synchronize()
        e0.record(stream)
        for _ in range(max(5, args.steps // 5)):
            step_e2e()
        e1.record(stream)
        stream.synchronize()
    ms_eager = e0.elapsed_time(e1) / max(5, args.steps // 5)
    clocks = sampler.stop()

    # ---- max over ranks ------------------------------------------------------------------------
    if dist is not None:
        t = torch.tensor([ms_kernel, ms_e2e, ms_eager], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_kernel, ms_e2e, ms_eager = t.tolist()
    total_bytes = bytes_per_launch * LAYERS * world
    value = total_bytes / (ms_kernel * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e * 1e-3) / 1e9
    achieved = bytes_per_launch * LAYERS / (ms_kernel * 1e-3) / 1e9     # per GPU, per launch average

    result = {
        "metric": "A16W4 GEMV HBM GB/s (M=1, 8192x8192, gs=128, bf16)", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_kernel, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg2 A16W4 M=1 bf16 8192x8192 gs128 +bias: %d distinct layers per step, CUDA-graph replay" % LAYERS,
                   "l2": "inputs larger than L2 (%.2f GB of packed weights per step cycle through 126 MB)" % (LAYERS * bytes_per_launch / 1e9),
                   "kernel": kernel_name, "parallelism": "replicas x%d" % world, "us_per_launch": ms_kernel * 1e3 / LAYERS},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                "ms_per_step": ms_e2e, "mode": "GemLiteLinear.forward x%d chained, CUDA-graph replay incl. H2D/D2H copies" % LAYERS,
                "eager_ms_per_step": ms_eager, "eager_value": total_bytes / (ms_eager * 1e-3) / 1e9, "finite": finite},
        "gpu_launches": args.steps * LAYERS,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": bench_reference().get("ncu_dram_bytes_per_launch", {}).get(kernel_name), "peak_kind": peak_kind, "frac_of_nominal_8000": achieved / 8000.0,
                     "bytes_per_launch": bytes_per_launch},
        "clocks": clocks,
    }

    if rank == 0 and not args.no_sweep:
        result["sweep"] = sweep(device, layers, stream, hbm_peak, bf16_peak)
        del layers, arg_structs, outs
        torch.cuda.empty_cache()
        try:
            result["measured_mma_peak_tflops"] = measure_mma_peaks(device)
        except Exception as e:
            result["measured_mma_peak_tflops"] = {"error": str(e)[:200]}
        try:
            result["sweep_gemm"] = sweep_gemm(device, mma_peaks=result.get("measured_mma_peak_tflops"))
        except Exception as e:  # the extra formats must not lose the headline numbers
            result["sweep_gemm"] = [{"error": str(e)[:200]}]
    if rank == 0 and not args.no_cpu and world >= 1:
        try:
            result["cpu_baseline"] = cpu_path_sample(seconds=12.0)
        except Exception as e:  # the CPU sample must not lose the GPU numbers
            result["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": "failed: %s" % e}
    if not args.no_tp:
        try:
            torch.cuda.empty_cache()
            tp = tensor_parallel_step(device, rank, world, dist)
            if rank == 0:
                result["tensor_parallel"] = tp
        except Exception as e:  # the weak-scaling line above stands on its own
            if rank == 0:
                result["tensor_parallel"] = {"error": str(e)[:300]}
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))


def tensor_parallel_step(device, rank, world, dist, Ms=(1, 8, 32, 64, 2048), steps=30):
    """The seven A16W4 linears of one Llama-70B decoder layer (hidden 8192, intermediate 28672, 64 q / 8 kv heads of
    128), tensor-parallel over all ranks: column-parallel fused qkv and gate/up, row-parallel o_proj and down_proj
    with an all-reduce each -- the one-shot peer-memory kernel while the result fits its receive slots (decode
    sizes), NCCL above.  For every M: device time per step as a CUDA-graph replay (max over ranks) and the relative
    Frobenius error of the sharded result against the same layers unsharded on one GPU (rank 0 holds both)."""
    from gemlite_b200 import tp
    hidden, inter, heads, kv_heads, head_dim = 8192, 28672, 64, 8, 128
    comm = tp.PeerComm(device, slot_bytes=2 << 20) if world > 1 else None
    blk = tp.LlamaLinears(hidden, inter, heads, kv_heads, head_dim, world, rank, device, seed=11, comm=comm)
    full = tp.LlamaLinears(hidden, inter, heads, kv_heads, head_dim, 1, 0, device, seed=11) if (world > 1 and rank == 0) else None
    weights = (heads + 2 * kv_heads) * head_dim * hidden + hidden * heads * head_dim + 3 * inter * hidden   # elements
    rows = []
    side = torch.cuda.Stream(device)
    for M in Ms:
        gx = torch.Generator(device=device).manual_seed(500 + M)             # the same activations on every rank
        x = (torch.randn(M, hidden, generator=gx, device=device) * 0.1).to(torch.bfloat16)
        n_steps = steps if M <= 64 else 5
        for _ in range(3):
            y = blk(x)
        rel = None
        if full is not None:
            y1 = full(x).float()
            rel = float((y.float() - y1).norm() / y1.norm())
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            y = blk(x)
        e1.record()
        torch.cuda.synchronize(device)
        ms_eager = e0.elapsed_time(e1) / n_steps
        # the same step captured once in a CUDA graph (all-reduces included) and replayed: device-bound time
        ms_graph, graph = None, None
        try:
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    y = blk(x)
            side.synchronize()
        except Exception:
            graph = None
        ok = torch.tensor([0.0 if graph is None else 1.0], device=device, dtype=torch.float64)
        if dist is not None:   # replay only if every rank captured: a rank replaying all-reduces alone would wait
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 1.0:
            with torch.cuda.stream(side):
                for _ in range(3):
                    graph.replay()
                side.synchronize()
                if dist is not None:
                    dist.barrier()
                e0.record(side)
                for _ in range(n_steps):
                    graph.replay()
                e1.record(side)
                side.synchronize()
            ms_graph = e0.elapsed_time(e1) / n_steps
        t = torch.tensor([ms_eager, ms_graph if ms_graph is not None else 0.0], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        one_shot = comm is not None and M * hidden * 2 <= comm.slot_bytes
        rows.append({"M": M, "ms_per_step": t[1].item() if ms_graph is not None else t[0].item(), "ms_per_step_eager": t[0].item(),
                     "timing": "CUDA graph replay" if ms_graph is not None else "eager",
                     "all_reduce": "none (one GPU)" if world == 1 else ("one-shot peer-memory kernel" if one_shot else "NCCL"),
                     "rel_fro_vs_unsharded": rel, "finite": bool(torch.isfinite(y.float()).all())})
        del graph
    status = comm.status()[0] if comm is not None else 0
    if comm is not None:
        comm.close()
    return {"workload": "Llama-70B decoder-layer linears, A16W4 gs128, tp%d" % world, "all_reduces_per_step": 0 if world == 1 else 2,
            "packed_weight_GB_per_step_all_ranks": weights / 2 / 1e9, "parity_tolerance": 1e-2, "wait_status": status, "per_M": rows,
            "ms_per_step": rows[0]["ms_per_step"]}


# -------------------------------------------------------------------------------------------------
# Output checks of the sweeps (outside every timed region): a plain torch fp32 product of the same quantised
# operands, decoded with torch ops, on up to 256 sampled rows.  No library matmul kernel is involved.
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def _decode_fp4(q_bytes, scale_bytes, group, e8m0):
    R, K2 = q_bytes.shape
    lut = torch.tensor(_E2M1, dtype=torch.float32, device=q_bytes.device)
    vals = torch.stack((lut[(q_bytes & 0xF).long()], lut[(q_bytes >> 4).long()]), dim=-1).view(R, K2 * 2)
    sb = scale_bytes.view(torch.uint8)[:R]
    sc = torch.pow(2.0, sb.float() - 127.0) if e8m0 else sb.view(torch.float8_e4m3fn).float()
    return (vals.view(R, -1, group) * sc.view(R, -1, 1)).view(R, K2 * 2)


def _decode_mxfp8(q, scale_bytes):
    """fp32 [R, K] of e4m3 values with one e8m0 scale per 32."""
    R, K = q.shape
    sc = torch.pow(2.0, scale_bytes.view(torch.uint8)[:R].float() - 127.0)
    return (q.view(torch.float8_e4m3fn).float().view(R, -1, 32) * sc.view(R, -1, 1)).view(R, K)


def _dequant_packed_int(layer):
    """fp32 [K, N] weights of a packed A16Wn layer from its stored tensors: codes * s + z' (fma mode) or (codes - z) * s."""
    nbits, e, gs = layer.W_nbits, layer.elements_per_sample, layer.group_size
    Wp = layer.W_q                                         # int32 [K/e, N]
    shifts = (torch.arange(e, device=Wp.device, dtype=torch.int32) * nbits).view(1, e, 1)
    codes = ((Wp.unsqueeze(1) >> shifts) & (2 ** nbits - 1)).reshape(-1, Wp.shape[1]).float()      # [K, N]
    sc = layer.scales.float().repeat_interleave(gs, 0)
    z = layer.zeros.float().repeat_interleave(gs, 0)
    return codes * sc + z if layer.W_group_mode == 4 else (codes - z) * sc


def check_output(layer, fmt, x, y, W_ref=None):
    """Relative Frobenius error of y = layer(x) against the torch product of the identical quantised operands."""
    from gemlite_b200 import quant_utils as qu
    M = x.shape[0]
    idx = torch.arange(0, M, max(1, M // 256), device=x.device)[:256]
    if fmt.startswith("A16"):
        W = W_ref if W_ref is not None else _dequant_packed_int(layer)
        ref = x[idx].float() @ W + (layer.bias.float() if layer.bias is not None else 0.0)
    elif fmt in ("FP8", "INT8"):
        xq, sx = qu.scale_activations_per_token(x, torch.float8_e4m3fn if fmt == "FP8" else torch.int8)
        ref = (xq[idx].float() @ layer.W_q.float()) * sx[idx].view(-1, 1) * layer.scales.float().view(1, -1)
    elif fmt == "FP8blk":          # 128 x 128 block scales: per-block partial products scaled by s_x[m, kb] * s_w[kb, nb]
        xq, sx = qu.scale_activations_per_block(x, torch.float8_e4m3fn)
        Kb = xq.shape[1] // 128
        xs = (xq[idx].float().view(len(idx), Kb, 128) * sx[idx].view(len(idx), Kb, 1)).view(len(idx), -1)
        sw = layer.scales.float().repeat_interleave(128, 0)[:xq.shape[1]].repeat_interleave(128, 1)[:, :layer.out_features]
        ref = xs @ (layer.W_q.float() * sw)
    elif fmt == "MXFP8":
        xq, sx = qu.scale_activations_mxfp8(x, scale_layout=0)
        Wd = W_ref if W_ref is not None else _decode_mxfp8(layer.W_q.t().contiguous(), layer.scales.contiguous())
        ref = _decode_mxfp8(xq[idx].contiguous(), sx[idx].contiguous()) @ Wd.T
    else:
        gs, e8 = (32, True) if fmt == "MXFP4" else (16, False)
        wq, sw = layer.W_q.t().contiguous(), layer.scales.contiguous().view(torch.uint8)
        if fmt == "MXFP4":
            xq, sx = qu.scale_activations_mxfp4(x, scale_layout=0)
            meta = 1.0
        else:
            xq, sx, mx = qu.scale_activations_nvfp4(x, scale_layout=0)
            meta = 1.0 / (float(layer.meta_scale.item()) * float(mx.item()))
        Wd = W_ref if W_ref is not None else _decode_fp4(wq, sw, gs, e8)
        ref = (_decode_fp4(xq[idx], sx[idx], gs, e8) @ Wd.T) * meta
    got = y[idx].float()
    return float((got - ref).norm() / ref.norm())


def sweep(device, layers, stream, hbm_peak, bf16_peak):
    """Other batch sizes of the A16W4 configuration on the same 32 layers (graph replay, 10 steps)."""
    from gemlite_b200 import _lib, core
    L = _lib.lib()
    res = []
    W_last = _dequant_packed_int(layers[-1])               # reference weights of the layer whose output is checked
    for M in (1, 2, 4, 8, 16):
        x = torch.randn(M, K_FEAT, device=device, dtype=torch.bfloat16)
        outs = [torch.empty(M, N_FEAT, device=device, dtype=torch.bfloat16) for _ in layers]
        structs = []
        with torch.cuda.stream(stream):
            for lyr, out in zip(layers, outs):
                a = core._fill_args(x, lyr.bias, lyr.W_q, lyr.scales, lyr.zeros, None, None, out, lyr.get_meta_args(), -1)
                ws = core._workspace(device, int(L.gl_matmul_workspace_bytes(ctypes.byref(a))))
                if ws is not None:
                    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
                structs.append(a)

        def fn():
            sp = torch.cuda.current_stream(device).cuda_stream
            for a in structs:
                if L.gl_matmul(ctypes.byref(a), sp) != 0:
                    raise RuntimeError(L.gl_last_error().decode())
        try:
            graph = time_graph(fn, 10, 3, stream)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                e0.record(stream)
                for _ in range(10):
                    graph.replay()
                e1.record(stream)
                stream.synchronize()
            us = e0.elapsed_time(e1) / 10 / len(layers) * 1e3
            b = algorithmic_bytes(M, N_FEAT, K_FEAT, 4, GROUP)
            flops = 2.0 * M * N_FEAT * K_FEAT
            torch.cuda.synchronize(device)
            rel = check_output(layers[-1], "A16W4", x, outs[-1], W_ref=W_last)
            res.append({"format": "A16W4", "M": M, "us_per_launch": us, "GBps": b / us / 1e3, "frac_hbm": b / us / 1e3 / hbm_peak,
                        "TFLOPs": flops / us / 1e6, "kernel": L.gl_matmul_kernel_name(ctypes.byref(structs[0])).decode(),
                        "checked": rel < 1e-2, "rel_fro": rel})
        except Exception as e:
            res.append({"format": "A16W4", "M": M, "error": str(e)[:200]})
    return res


def measure_mma_peaks(device, iters=4000, reps=6):
    """Tensor-pipe ceiling of this GPU per MMA kind: `reps` back-to-back launches of the library's resident-tile
    tcgen05.mma kernel (no loads, no epilogue), TFLOP/s over the whole set, i.e. under the power cap the GEMMs see."""
    from gemlite_b200 import _lib
    from gemlite_b200.dtypes import DType
    L = _lib.lib()
    status = torch.zeros(1, dtype=torch.int32, device=device)
    out = {}
    for name, kind in (("bf16", DType.BF16), ("fp8", DType.FP8), ("int8", DType.INT8), ("mxfp4", DType.MXFP4), ("nvfp4", DType.NVFP4)):
        flops = ctypes.c_double(0.0)
        sp = torch.cuda.current_stream(device).cuda_stream
        for _ in range(2):
            if L.gl_mma_peak(kind.value, iters, status.data_ptr(), ctypes.byref(flops), sp) != 0:
                raise RuntimeError(L.gl_last_error().decode())
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            L.gl_mma_peak(kind.value, iters, status.data_ptr(), ctypes.byref(flops), sp)
        e1.record()
        torch.cuda.synchronize(device)
        out[name] = flops.value * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12
    out["wait_status"] = int(status.item())
    return out


def sweep_gemm(device, only=None, mma_peaks=None):
    """The other benchmark configurations through the public API (GemLiteLinear.forward incl. the fused
    activation quantiser): FP8 4096->14336, MXFP4 / NVFP4 16384x16384, A16W4 8192x8192 at prefill size.
    L2 is flushed between timed calls; min of 10 calls; TFLOP/s = 2 M N K / time.  `ref_triton_ms` is the
    reference's own Triton kernel timed on a B200 when the golden fixtures were captured."""
    from gemlite_b200 import helper
    ref = bench_reference().get("reference_triton_timings", {}).get("timings", {})
    ref_graph = bench_reference().get("reference_triton_timings_graph", {}).get("timings", {})
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device=device)
    dense_peak = {"A16W4": 2250.0, "A16W2": 2250.0, "A16W8": 2250.0, "FP8": 4500.0, "MXFP4": 9000.0, "NVFP4": 9000.0,
                  "A16W8c": 2250.0, "A16W4MX": 2250.0, "MXFP8": 4500.0, "FP8blk": 4500.0, "INT8": 4500.0}     # nominal dense TFLOP/s

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(device)
        best = 1e9
        for _ in range(reps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize(device)
            best = min(best, a.elapsed_time(b))
        return best

    def make(fmt):
        g = torch.Generator(device=device).manual_seed(7)
        if fmt in ("A16W4", "A16W2", "A16W8"):
            N = K = 8192
            nbits, gs = {"A16W4": (4, 128), "A16W2": (2, 64), "A16W8": (8, 128)}[fmt]
            W_q = torch.randint(0, 2 ** nbits, (N, K), generator=g, device=device, dtype=torch.int32).to(torch.uint8)
            sc = (torch.randn(N * K // gs, 1, generator=g, device=device).abs() * 0.02).to(torch.bfloat16)
            z = (torch.rand(N * K // gs, 1, generator=g, device=device) * (2 ** nbits - 1)).to(torch.bfloat16)
            b = (torch.randn(N, generator=g, device=device) * 0.01).to(torch.bfloat16)
            return helper.A16Wn_HQQ_INT(device=str(device), dtype=torch.bfloat16, W_nbits=nbits).from_weights(W_q, sc, z, bias=b), K, N
        K, N = (4096, 14336) if fmt in ("FP8", "INT8") else ((8192, 8192) if fmt in ("A16W8c", "A16W4MX", "MXFP8", "FP8blk") else (16384, 16384))
        lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16, device=device)
        lin.weight.data.normal_(0, 0.02, generator=g)
        # A16W8c: weight-only INT8 with one scale per channel; A16W4MX: weight-only MXFP4 (16-bit activations)
        P = {"FP8": helper.A8W8_FP8_dynamic, "MXFP4": helper.A4W4_MXFP_dynamic, "NVFP4": helper.A4W4_NVFP_dynamic,
             "A16W8c": helper.A16W8_INT8, "A16W4MX": helper.A16W4_MXFP, "MXFP8": helper.A8W8_MXFP_dynamic, "FP8blk": helper.A8W8_FP8_dynamic, "INT8": helper.A8W8_INT8_dynamic}[fmt]
        if fmt == "FP8blk":      # one fp32 scale per 128 x 128 weight block, activations per row and 128 k
            return P(device=str(device), dtype=torch.bfloat16, block_quant=True).from_linear(lin), K, N
        if fmt == "MXFP8":       # block scales on both operands
            return P(device=str(device), dtype=torch.bfloat16, post_scale=False).from_linear(lin), K, N
        return P(device=str(device), dtype=torch.bfloat16).from_linear(lin), K, N

    res = []
    stream = torch.cuda.Stream(device)
    cases = (("A16W4", (32, 64, 256, 1024, 4096, 8192)), ("A16W2", (1, 16, 64, 256, 1024, 4096, 8192)), ("A16W8", (1, 16, 1024)), ("FP8", (1, 16, 128, 1024, 4096)),
             ("MXFP4", (1, 64, 512, 4096, 16384)), ("NVFP4", (1, 64, 512, 4096, 16384)), ("A16W8c", (1, 4)), ("A16W4MX", (1, 4)), ("MXFP8", (1, 4096)), ("FP8blk", (1024, 4096)), ("INT8", (1, 4096)))
    if only is not None:
        cases = ((only[0], (only[1],)),)
    for fmt, Ms in cases:
        try:
            layer, K, N = make(fmt)
            wbytes = N * K // {"FP8": 1, "INT8": 1, "A16W8": 1, "A16W8c": 1, "MXFP8": 1, "FP8blk": 1, "A16W2": 4}.get(fmt, 2)
            W_ref = (layer.W_q.float() * layer.scales.float().view(1, -1)) if fmt == "A16W8c" else (
                _decode_fp4(layer.W_q.t().contiguous(), layer.scales.contiguous().view(torch.uint8), 32, True).t().contiguous()) if fmt == "A16W4MX" else (
                _dequant_packed_int(layer)) if fmt.startswith("A16") else (
                None if fmt in ("FP8", "INT8", "MXFP8", "FP8blk") else _decode_fp4(layer.W_q.t().contiguous(), layer.scales.contiguous().view(torch.uint8),
                                                      32 if fmt == "MXFP4" else 16, fmt == "MXFP4"))
            for M in Ms:
                x = torch.randn(M, K, dtype=torch.bfloat16, device=device)
                row = {"format": fmt, "M": M, "N": N, "K": K}
                rel = check_output(layer, fmt, x, layer(x), W_ref=W_ref)      # once, outside the timed region
                row.update({"checked": rel < (1e-2 if fmt.startswith("A16") else 5e-3), "rel_fro": rel})
                if fmt == "NVFP4":
                    row["reference_parity"] = "oracle only: the reference's NVFP4 Triton kernels do not compile on sm_100 with Triton 3.6"
                if M <= 512:
                    # small batch: host launch overhead would hide the kernels, so the forwards of several distinct
                    # layers (together larger than L2) are captured in one CUDA graph and replayed
                    n_layers = max(2, -(-160 * 1024 * 1024 // wbytes))
                    layers = [layer] + [make(fmt)[0] for _ in range(n_layers - 1)]
                    graph = time_graph(lambda: [l(x) for l in layers], 10, 3, stream)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    with torch.cuda.stream(stream):
                        e0.record(stream)
                        for _ in range(10):
                            graph.replay()
                        e1.record(stream)
                        stream.synchronize()
                    ms = e0.elapsed_time(e1) / 10 / n_layers
                    row.update({"ms": ms, "GBps": wbytes / ms / 1e6, "timing": "CUDA graph over %d distinct layers" % n_layers})
                    del layers, graph
                else:
                    ms = timed(lambda: layer(x))
                    row["ms"] = ms
                tf = 2.0 * M * N * K / ms / 1e9
                row.update({"TFLOPs": tf, "frac_dense_nominal": tf / dense_peak[fmt]})
                pk = (mma_peaks or {}).get({"FP8": "fp8", "INT8": "int8", "MXFP8": "fp8", "FP8blk": "fp8", "MXFP4": "mxfp4", "NVFP4": "nvfp4"}.get(fmt, "bf16"))
                if pk:
                    row["frac_measured_mma_peak"] = tf / pk
                key = "%s_%dx%d_M%d" % (fmt, K if fmt in ("FP8", "INT8") else N, N if fmt in ("FP8", "INT8") else K, M)
                r, rg = ref.get(key), ref_graph.get(key)
                if rg and M <= 512:          # same protocol as this row: graph replay over distinct layers
                    row["ref_triton_ms"] = rg["ms_per_layer"]
                    row["ref_triton_protocol"] = "CUDA-graph replay over %d distinct layers (separate capture)" % rg["layers"]
                elif r:
                    row["ref_triton_ms"] = r["min_ms"]
                    row["ref_triton_protocol"] = "eager call, L2 flushed (separate capture)"
                res.append(row)
            del layer, W_ref
            torch.cuda.empty_cache()
        except Exception as e:
            res.append({"format": fmt, "error": str(e)[:200]})
    return res


if __name__ == "__main__":
    main()
