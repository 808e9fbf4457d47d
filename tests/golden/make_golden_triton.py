"""Captures outputs of the REFERENCE's own Triton kernels and torch quantisers on a CUDA GPU, on the
seeded inputs the parity tests regenerate, into tests/golden/triton_golden.npz.

Run on a GPU machine with a checkout of the reference (it is not part of this repository):
    python tests/golden/make_golden_triton.py --ref /path/to/gemlite-checkout --out <file.npz> [--time]
The reference package is imported from --ref; nothing of this repository's kernels is used.
With --time the reference's kernels are also timed, eager and as a CUDA-graph replay over distinct layers (CUDA events, 256 MB L2 flush between calls, the
protocol of the reference's examples/benchmark_triton.py:48-64) on the headline shapes and the numbers
are written next to the fixture as JSON.
With --baseline only the benchmark configurations at their own sizes (tests/golden_inputs.py BASELINE_CASES) are
captured, as sampled rows and columns, into tests/golden/triton_golden_baseline.npz.
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests.util import make_a16wn  # noqa: E402

A16_CASES = [  # (seed, N, K, nbits, group_size, dtype, Ms)
    (2001, 2032, 3968, 4, 128, "bf16", (1, 3, 16, 65)),
    (2002, 2032, 3968, 2, 64, "bf16", (1, 4, 30)),
    (2003, 1024, 2048, 4, 64, "fp16", (1, 5, 100)),
    (2004, 512, 1024, 8, 128, "fp16", (2, 16)),
]
DT = {"bf16": torch.bfloat16, "fp16": torch.float16}


def families_for(M):
    return ["GEMV", "GEMV_REVSPLITK", "GEMV_SPLITK", "GEMM_SPLITK", "GEMM"] if M <= 4 else ["GEMM_SPLITK", "GEMM"]


def bench(fn, reps=50):
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device="cuda")
    for _ in range(5):
        fn()
    ts = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return {"min_ms": ts[0], "median_ms": ts[len(ts) // 2]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--baseline", action="store_true", help="capture only the benchmark configurations at their own sizes (sampled rows / columns)")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    import gemlite                                   # the reference
    from gemlite import helper as rh
    from gemlite import quant_utils as rq
    assert os.path.abspath(os.path.dirname(gemlite.__file__)).startswith(os.path.abspath(args.ref))
    gemlite.set_autotune(False)
    out, log = {}, {"errors": []}

    def guard(name, fn):
        try:
            fn()
        except Exception as e:  # record and go on: one broken reference kernel must not lose the rest
            log["errors"].append("%s: %s: %s" % (name, type(e).__name__, str(e)[:300]))

    # ---- the benchmark configurations at their own sizes: sampled rows / columns of the reference's outputs ----
    if args.baseline:
        from tests import golden_inputs as gi
        for tag, kind, N, K, nbits, gs, fams_by_M in gi.BASELINE_CASES:
            layer = None
            for M, fams in fams_by_M.items():
                ops = gi.baseline_inputs(tag, M)
                x = ops[0]
                if layer is None:
                    if kind == "a16":
                        layer = rh.A16Wn_HQQ_INT(device="cuda:0", dtype=torch.bfloat16, W_nbits=nbits).from_weights(ops[1].cuda(), ops[2].cuda(), ops[3].cuda())
                    else:
                        lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
                        lin.weight.data = ops[1].clone()
                        proc = rh.A8W8_FP8_dynamic if kind == "fp8" else rh.A4W4_MXFP_dynamic
                        layer = proc(device="cuda:0", dtype=torch.bfloat16).from_linear(lin.cuda())
                out["%s_M%d_x_sum" % (tag, M)] = np.array([float(x.double().sum())])
                rows, cols = gi.kept_rows(M), gi.kept_cols(N)
                for fam in fams:
                    def run(fam=fam, M=M, x=x, tag=tag):
                        y = layer.forward_manual(x.cuda(), fam)
                        torch.cuda.synchronize()
                        out["%s_M%d_%s" % (tag, M, fam)] = y.float().cpu().numpy()[rows][:, cols].astype(np.float32)
                    guard("%s M%d %s" % (tag, M, fam), run)
            del layer
            torch.cuda.empty_cache()
        out["reference_errors"] = np.array(log["errors"])
        out["reference_env"] = np.array([torch.cuda.get_device_name(0), "triton " + __import__("triton").__version__])
        np.savez_compressed(args.out, **out)
        print("baseline fixture:", len(out), "arrays,", os.path.getsize(args.out), "bytes, errors:", log["errors"])
        return

    # ---- A16Wn, every family ----
    for seed, N, K, nbits, gs, dt, Ms in A16_CASES:
        for M in Ms:
            x, W_q, s, z, b = make_a16wn(N, K, nbits, gs, DT[dt], seed + M, M=M, with_bias=False)
            layer = rh.A16Wn_HQQ_INT(device="cuda:0", dtype=DT[dt], W_nbits=nbits).from_weights(W_q.cuda(), s.cuda(), z.cuda())
            for fam in families_for(M):
                def run(fam=fam, M=M):
                    y = layer.forward_manual(x.cuda(), fam)
                    torch.cuda.synchronize()
                    out["a16_s%d_M%d_%s" % (seed, M, fam)] = y.float().cpu().numpy().astype(np.float32)
                guard("a16 %d M%d %s" % (seed, M, fam), run)

    # ---- activation quantisers (Triton) and weight quantisers (torch) ----
    g = torch.Generator().manual_seed(3001)
    for M, K in ((1, 4096), (5, 4224), (33, 2048)):
        x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16)
        out["xq_M%d_K%d_x" % (M, K)] = x.float().numpy()
        def per_token(M=M, K=K, x=x):
            q, s = rq.scale_activations_per_token(x.cuda(), w_dtype=torch.float8_e4m3fn)
            out["xq_M%d_K%d_fp8_q" % (M, K)] = q.view(torch.uint8).cpu().numpy(); out["xq_M%d_K%d_fp8_s" % (M, K)] = s.float().cpu().numpy()
            q, s = rq.scale_activations_per_token(x.cuda(), w_dtype=torch.int8)
            out["xq_M%d_K%d_int8_q" % (M, K)] = q.cpu().numpy(); out["xq_M%d_K%d_int8_s" % (M, K)] = s.float().cpu().numpy()
        guard("per_token", per_token)
        def mx4(M=M, K=K, x=x):
            q, s = rq.scale_activations_mxfp4(x.cuda())
            out["xq_M%d_K%d_mxfp4_q" % (M, K)] = q.cpu().numpy(); out["xq_M%d_K%d_mxfp4_s" % (M, K)] = s.view(torch.uint8).cpu().numpy()
        guard("mxfp4", mx4)
        def mx8(M=M, K=K, x=x):
            q, s = rq.scale_activations_mxfp8(x.cuda())
            out["xq_M%d_K%d_mxfp8_q" % (M, K)] = q.view(torch.uint8).cpu().numpy(); out["xq_M%d_K%d_mxfp8_s" % (M, K)] = s.view(torch.uint8).cpu().numpy()
        guard("mxfp8", mx8)
        def nv4(M=M, K=K, x=x):
            q, s, m = rq.scale_activations_nvfp4(x.cuda())
            out["xq_M%d_K%d_nvfp4_q" % (M, K)] = q.cpu().numpy(); out["xq_M%d_K%d_nvfp4_s" % (M, K)] = s.view(torch.uint8).cpu().numpy()
            out["xq_M%d_K%d_nvfp4_meta" % (M, K)] = m.float().cpu().numpy().reshape(-1)
        guard("nvfp4", nv4)
    W = (torch.randn(256, 1024, generator=g) * 0.02).to(torch.bfloat16)
    out["wq_W"] = W.float().numpy()
    def wquant():
        wqz = rq.WeightQuantizerMXFP(compute_dtype=torch.bfloat16, device="cuda:0")
        c, s = wqz.quantize_mxfp4(W.cuda(), index=True)
        out["wq_mxfp4_codes"] = c.view(256, 1024).cpu().numpy(); out["wq_mxfp4_scales"] = s.view(torch.uint8).view(256, -1).cpu().numpy()
        c, s, m = wqz.quantize_nvfp4(W.cuda(), index=True)
        out["wq_nvfp4_codes"] = c.view(256, 1024).cpu().numpy(); out["wq_nvfp4_scales"] = s.view(torch.uint8).view(256, -1).cpu().numpy()
        out["wq_nvfp4_meta"] = m.float().cpu().numpy().reshape(-1)
    guard("weight quantisers", wquant)

    # ---- A8W8 FP8 / INT8 dynamic, A4W4 MXFP4 / NVFP4 dynamic ----
    for name, proc_name, N, K, Ms in (("fp8", "A8W8_FP8_dynamic", 1024, 2048, (1, 16, 130)),
                                      ("int8", "A8W8_INT8_dynamic", 1024, 2048, (2, 65)),
                                      ("mxfp4", "A4W4_MXFP_dynamic", 2048, 4224, (1, 16, 100)),
                                      ("nvfp4", "A4W4_NVFP_dynamic", 2048, 4224, (1, 16, 100))):
        gg = torch.Generator().manual_seed(4000 + N)
        Wl = (torch.randn(N, K, generator=gg) * 0.02).to(torch.bfloat16)
        def build(proc_name=proc_name, Wl=Wl, N=N, K=K):
            lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
            lin.weight.data = Wl.clone()
            return getattr(rh, proc_name)(device="cuda:0", dtype=torch.bfloat16).from_linear(lin.cuda())
        try:
            layer = build()
        except Exception as e:
            log["errors"].append("build %s: %s" % (name, str(e)[:300]))
            continue
        for M in Ms:
            xm = torch.randn(M, K, generator=gg).to(torch.bfloat16)
            out["lin_%s_M%d_x" % (name, M)] = xm.float().numpy()
            fams = ["GEMM_SPLITK", "GEMM"] if name in ("mxfp4", "nvfp4") or M > 2 else ["GEMV_SPLITK", "GEMM_SPLITK", "GEMM"]
            for fam in fams:
                def run(fam=fam, M=M, xm=xm, name=name):
                    y = layer.forward_manual(xm.cuda(), fam)
                    torch.cuda.synchronize()
                    out["lin_%s_M%d_%s" % (name, M, fam)] = y.float().cpu().numpy()
                guard("lin %s M%d %s" % (name, M, fam), run)
        out["lin_%s_W" % name] = Wl.float().numpy().astype(np.float16)

    np.savez_compressed(args.out, **out)
    log["keys"] = len(out)
    log["triton"] = __import__("triton").__version__
    log["gpu"] = torch.cuda.get_device_name(0)

    # ---- timings of the reference kernels on the headline shapes ----
    if args.time:
        timings = {}
        gemlite.set_autotune("fast")
        def time_case(tag, layer, K, M, dtype=torch.bfloat16):
            x = torch.randn(M, K, dtype=dtype, device="cuda")
            t0 = time.time()
            for _ in range(3):
                layer(x)
            torch.cuda.synchronize()
            r = bench(lambda: layer(x))
            r["warmup_s"] = time.time() - t0
            timings[tag] = r
        for M in (1, 4096):
            def a16(M=M):
                x, W_q, s, z, b = make_a16wn(8192, 8192, 4, 128, torch.bfloat16, 1, M=1, with_bias=False)
                layer = rh.A16W4_HQQ_INT(device="cuda:0", dtype=torch.bfloat16).from_weights(W_q.cuda(), s.cuda(), z.cuda())
                time_case("A16W4_8192x8192_M%d" % M, layer, 8192, M)
            guard("time a16 M%d" % M, a16)
        for name, proc_name in (("MXFP4", "A4W4_MXFP_dynamic"), ("NVFP4", "A4W4_NVFP_dynamic")):
            def fp4(name=name, proc_name=proc_name):
                lin = torch.nn.Linear(16384, 16384, bias=False, dtype=torch.bfloat16, device="cuda")
                lin.weight.data.normal_(0, 0.02)
                layer = getattr(rh, proc_name)(device="cuda:0", dtype=torch.bfloat16).from_linear(lin)
                for M in (1, 4096):
                    time_case("%s_16384x16384_M%d" % (name, M), layer, 16384, M)
            guard("time " + name, fp4)
        def fp8():
            lin = torch.nn.Linear(4096, 14336, bias=False, dtype=torch.bfloat16, device="cuda")
            lin.weight.data.normal_(0, 0.02)
            layer = rh.A8W8_FP8_dynamic(device="cuda:0", dtype=torch.bfloat16).from_linear(lin)
            for M in (1, 4096):
                time_case("FP8_4096x14336_M%d" % M, layer, 4096, M)
        guard("time fp8", fp8)
        log["timings"] = timings

        # ---- the same kernels as a CUDA-graph replay over distinct layers (together larger than L2): the protocol
        # bench.py uses for decode sizes, so that both sides of a comparison are measured the same way ----
        timings_graph = {}
        def graph_case(tag, make_layer, K, M, n_layers, reps=20):
            layers = [make_layer(i) for i in range(n_layers)]
            x = torch.randn(M, K, dtype=torch.bfloat16, device="cuda")
            for _ in range(2):
                for l in layers:
                    l(x)                                   # JIT + autotune before the capture
            torch.cuda.synchronize()
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for l in layers:
                    l(x)
                st.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    for l in layers:
                        l(x)
                for _ in range(3):
                    g.replay()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(st)
                for _ in range(reps):
                    g.replay()
                b.record(st)
                st.synchronize()
            timings_graph[tag] = {"ms_per_layer": a.elapsed_time(b) / reps / n_layers, "layers": n_layers, "replays": reps}
            del layers, g
            torch.cuda.empty_cache()
        def a16_layer(i):
            gen = torch.Generator(device="cuda").manual_seed(100 + i)
            N = K = 8192
            W_q = torch.randint(0, 16, (N, K), generator=gen, device="cuda", dtype=torch.int32).to(torch.uint8)
            s = (torch.randn(N * K // 128, 1, generator=gen, device="cuda").abs() * 0.02).to(torch.bfloat16)
            z = (torch.rand(N * K // 128, 1, generator=gen, device="cuda") * 15).to(torch.bfloat16)
            return rh.A16W4_HQQ_INT(device="cuda:0", dtype=torch.bfloat16).from_weights(W_q, s, z)
        for M, n in ((1, 32), (16, 8), (64, 8), (256, 8)):
            guard("graph a16 M%d" % M, lambda M=M, n=n: graph_case("A16W4_8192x8192_M%d" % M, a16_layer, 8192, M, n))
        def fp8_layer(i):
            lin = torch.nn.Linear(4096, 14336, bias=False, dtype=torch.bfloat16, device="cuda")
            lin.weight.data.normal_(0, 0.02)
            return rh.A8W8_FP8_dynamic(device="cuda:0", dtype=torch.bfloat16).from_linear(lin)
        guard("graph fp8 M1", lambda: graph_case("FP8_4096x14336_M1", fp8_layer, 4096, 1, 4))
        def mx_layer(i):
            lin = torch.nn.Linear(16384, 16384, bias=False, dtype=torch.bfloat16, device="cuda")
            lin.weight.data.normal_(0, 0.02)
            return rh.A4W4_MXFP_dynamic(device="cuda:0", dtype=torch.bfloat16).from_linear(lin)
        guard("graph mxfp4 M1", lambda: graph_case("MXFP4_16384x16384_M1", mx_layer, 16384, 1, 2))
        log["timings_graph"] = timings_graph
        log["timings_graph_protocol"] = "CUDA-graph replay of layer(x) over distinct layers, CUDA events around 20 replays"
        log["date"] = time.strftime("%Y-%m-%d")
        try:
            import subprocess
            log["clocks"] = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active", "--format=csv,noheader"],
                                           capture_output=True, text=True, timeout=20).stdout.strip()
        except Exception as e:
            log["clocks"] = "unavailable: %s" % e
    with open(os.path.splitext(args.out)[0] + ".json", "w") as fh:
        json.dump(log, fh, indent=1)
    print(json.dumps(log)[:2000])


if __name__ == "__main__":
    main()
