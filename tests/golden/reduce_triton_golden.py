"""Shrinks the raw capture of tests/golden/make_golden_triton.py to the committed fixture
tests/golden/triton_golden.npz: inputs that the tests regenerate from their seeds are dropped (a checksum is
kept instead), matmul outputs keep their first 4 rows, quantiser outputs keep at most 64 rows.
Usage: python tests/golden/reduce_triton_golden.py <raw.npz> [<raw.json>]"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    raw = np.load(sys.argv[1])
    out = {}
    for k in raw.files:
        a = raw[k]
        if k.endswith("_x") or k in ("wq_W",) or (k.startswith("lin_") and k.endswith("_W")):
            out[k + "_sum"] = np.array([np.asarray(a, dtype=np.float64).sum()])      # regenerate from the seed, verify by sum
        elif k.startswith("a16_") or (k.startswith("lin_") and not k.endswith("_x")):
            out[k] = np.asarray(a[:4], dtype=np.float32)
        elif k.startswith("wq_") and a.ndim == 2:
            out[k] = a[:64]
        else:
            out[k] = a
    if len(sys.argv) > 2:
        meta = json.load(open(sys.argv[2]))
        out["reference_errors"] = np.array(meta.get("errors", []))
        out["reference_env"] = np.array([str(meta.get("gpu")), "triton " + str(meta.get("triton"))])
        with open(os.path.join(HERE, "triton_timings.json"), "w") as fh:
            json.dump({"gpu": meta.get("gpu"), "triton": meta.get("triton"), "timings": meta.get("timings", {}),
                       "errors": meta.get("errors", [])}, fh, indent=1)
    dst = os.path.join(HERE, "triton_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
