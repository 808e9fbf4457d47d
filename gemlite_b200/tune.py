"""Tuner of the tile-config cache: measures the decode kernel's CTA shapes on the GPU at hand and writes the file the
library picks up at first use (``gemlite_b200/configs/<gpu tag>.json``).

The reference ships such tables per GPU (gemlite/configs/*.json), fills them with Triton's autotuner as kernels run
and saves them with ``GemLiteLinear.cache_config`` (gemlite/core.py:80-89, 838-877, 913-933).  Here the tunable
kernels are the decode-size ones: for every (M bucket, N, K, group size, bit width) the candidates
``{"s_in", "c_in", "cluster_k"}`` (K slices and 32-column groups per CTA, CTAs per cluster along K) are timed as a
CUDA-graph replay over enough distinct layers to exceed the L2 cache, and the fastest is stored under the
reference's signature ``(Mb, N, K, group_size, e, type_id)`` in the ``GEMV_REVSPLITK`` family.  Entries equal to what
the built-in planner would pick anyway are left out, so the file only carries what measurement changed.

    python -m gemlite_b200.tune                  # the benchmark shapes, writes configs/<tag>.json
    python -m gemlite_b200.tune --shapes 8192x8192x4x128 --ms 1 4 16 --out my.json
"""
import argparse
import ctypes
import json
import os

import torch

from . import _lib, core, helper

HERE = os.path.dirname(os.path.abspath(__file__))

# (N, K, bits, group): cfg2 (square 8192, W4 / W2) and the Llama-70B decoder linears at tensor-parallel degrees 1..8
DEFAULT_SHAPES = [(8192, 8192, 4, 128), (8192, 8192, 2, 64)] + [
    s for tp in (1, 2, 4, 8) for s in (((64 + 16) * 128 // tp, 8192, 4, 128), (8192, 8192 // tp, 4, 128),
                                      (2 * 28672 // tp, 8192, 4, 128), (8192, 28672 // tp, 4, 128))]
# (K slices per CTA, 32-column groups per CTA, CTAs per cluster along K): every shape of at most 16 warps; the planner
# rejects the ones a problem cannot use (slice length, shared memory)
CANDIDATES = [(s, c, cl) for s in (1, 2, 4, 8, 16) for c in (1, 2, 4, 8) for cl in (1, 2, 4, 8) if s * c <= 16]


def gpu_tag(device=0):
    return torch.cuda.get_device_properties(device).name.lower().replace("nvidia", "").strip().replace(" ", "_")


def _time_layers(layers, x, stream, reps=20):
    L = _lib.lib()
    dev = x.device
    outs = [torch.empty((x.shape[0], l.out_features), dtype=x.dtype, device=dev) for l in layers]
    structs = []
    with torch.cuda.stream(stream):
        for lyr, out in zip(layers, outs):
            a = core._fill_args(x, lyr.bias, lyr.W_q, lyr.scales, lyr.zeros, None, None, out, lyr.get_meta_args(), -1)
            ws = core._workspace(dev, int(L.gl_matmul_workspace_bytes(ctypes.byref(a))))
            if ws is not None:
                a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            structs.append(a)
    name = L.gl_matmul_kernel_name(ctypes.byref(structs[0])).decode()

    def fn():
        sp = torch.cuda.current_stream(dev).cuda_stream
        for a in structs:
            if L.gl_matmul(ctypes.byref(a), sp) != 0:
                raise RuntimeError(L.gl_last_error().decode())

    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) / reps / len(layers) * 1e3, name


def tune(shapes=DEFAULT_SHAPES, Ms=(1, 2, 4, 8, 16), device="cuda:0", verbose=True):
    """Returns {signature: (best entry or None, built-in us, best us)} and leaves the winners in the library's cache."""
    L = _lib.lib()
    dev = torch.device(device)
    stream = torch.cuda.Stream(dev)
    results = {}
    for (N, K, nbits, group) in shapes:
        wbytes = N * K * nbits // 8
        n_layers = max(2, min(32, -(-200 * 1024 * 1024 // wbytes)))
        g = torch.Generator(device=dev).manual_seed(N + K)
        proc = helper.A16Wn_HQQ_INT(device=str(dev), dtype=torch.bfloat16, W_nbits=nbits)
        layers = []
        for _ in range(n_layers):
            W_q = torch.randint(0, 2 ** nbits, (N, K), generator=g, device=dev, dtype=torch.int32).to(torch.uint8)
            s = (torch.randn(N * K // group, 1, generator=g, device=dev).abs() * 0.02).to(torch.bfloat16)
            z = (torch.rand(N * K // group, 1, generator=g, device=dev) * (2 ** nbits - 1)).to(torch.bfloat16)
            layers.append(proc.from_weights(W_q, s, z))
        for M in Ms:
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            sig = "(%d, %d, %d, %d, %d, %d)" % (L.gl_get_closest_m(M), N, K, group, 32 // nbits, 100 + nbits)
            L.gl_cfg_set(b"GEMV_REVSPLITK", sig.encode(), b"{}")
            base_us, name = _time_layers(layers, x, stream)
            best = (base_us, None)
            if name in ("gl_gemv_warp_kernel", "gl_gemv_stream_kernel"):
                for (s_in, c_in, cl) in CANDIDATES:
                    entry = {"s_in": s_in, "c_in": c_in, "cluster_k": cl}
                    L.gl_cfg_set(b"GEMV_REVSPLITK", sig.encode(), json.dumps(entry).encode())
                    try:
                        us, nm = _time_layers(layers, x, stream)
                    except Exception:
                        continue
                    if nm == "gl_gemv_warp_kernel" and us < best[0] * 0.97:      # keep the built-in choice unless 3 % faster
                        best = (us, entry)
            L.gl_cfg_set(b"GEMV_REVSPLITK", sig.encode(), json.dumps(best[1] or {}).encode())
            results[sig] = (best[1], base_us, best[0])
            if verbose:
                print("%-38s M=%-2d built-in %.2f us -> %.2f us %s" % (sig, M, base_us, best[0], best[1] or "(built-in)"), flush=True)
        del layers
        torch.cuda.empty_cache()
    return results


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", nargs="*", default=None, help="NxKxBITSxGROUP ...")
    ap.add_argument("--ms", nargs="*", type=int, default=[1, 2, 4, 8, 16])
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    shapes = DEFAULT_SHAPES if not args.shapes else [tuple(int(v) for v in s.split("x")) for s in args.shapes]
    res = tune(shapes, args.ms)
    table = {"GEMV_REVSPLITK": {sig: entry for sig, (entry, _, _) in res.items() if entry}}
    out = args.out or os.path.join(HERE, "configs", gpu_tag() + ".json")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    with open(out, "w") as fh:
        json.dump(table, fh, indent=1, sort_keys=True)
    print("wrote %s (%d entries)" % (out, len(table["GEMV_REVSPLITK"])))


if __name__ == "__main__":
    main()
