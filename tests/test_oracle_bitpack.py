"""CPU: the oracle's bit packing against golden vectors made by the reference's own torch
functions (tests/golden/make_golden_bitpack.py), plus the defining formula for the 64-bit case."""
import os

import numpy as np
import torch

from oracle import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "bitpack_golden.npz")


def make_input(seed, rows, cols, nbits):
    g = torch.Generator().manual_seed(int(seed))
    return torch.randint(0, 2 ** int(nbits), (int(rows), int(cols)), generator=g, dtype=torch.int32).to(torch.uint8).numpy()


def test_oracle_pack_matches_reference_golden():
    gold = np.load(GOLDEN)
    assert len(gold["cases"]) >= 10
    for seed, rows, cols, nbits, pb in gold["cases"]:
        W = make_input(seed, rows, cols, nbits)
        pc, e = oracle.pack_over_cols(W, int(nbits), int(pb))
        key = "s%d" % seed
        assert pc.dtype == gold[key + "_cols"].dtype
        assert np.array_equal(pc, gold[key + "_cols"]), (seed, nbits, pb)
        pr, _ = oracle.pack_over_rows(W[: (rows // e) * e], int(nbits), int(pb))
        assert np.array_equal(pr, gold[key + "_rows"]), (seed, nbits, pb)
        assert np.array_equal(oracle.unpack_over_cols(pc, int(nbits), int(cols)), gold[key + "_ucols"])
        assert np.array_equal(oracle.unpack_over_rows(pr, int(nbits), int((rows // e) * e)), gold[key + "_urows"])


def test_oracle_pack_64bit_formula_and_roundtrip():
    for nbits in (1, 2, 4, 8):
        W = make_input(99 + nbits, 128, 128, nbits)
        e = 64 // nbits
        pc, _ = oracle.pack_over_cols(W, nbits, 64)
        want = np.zeros((128, 128 // e), dtype=np.uint64)
        for r in range(128):
            for c in range(128 // e):
                for j in range(e):
                    want[r, c] |= np.uint64(int(W[r, c * e + j]) << (j * nbits))
        assert np.array_equal(pc.view(np.uint64), want)
        assert np.array_equal(oracle.unpack_over_cols(pc, nbits, 128), W)
        pr, _ = oracle.pack_over_rows(W, nbits, 64)
        assert np.array_equal(oracle.unpack_over_rows(pr, nbits, 128), W)


def test_oracle_unpack_partial_fields():
    # the reference takes num_output_cols // cols fields per word, whatever the word width
    W = make_input(5, 8, 64, 4)
    pc, _ = oracle.pack_over_cols(W, 4, 32)
    part = oracle.unpack_over_cols(pc, 4, pc.shape[1] * 4)
    assert np.array_equal(part.reshape(8, -1, 4), W.reshape(8, -1, 8)[:, :, :4])
