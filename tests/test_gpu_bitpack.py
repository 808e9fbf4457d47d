"""GPU: the CUDA bit-packing kernels, through the C ABI, bit-exact against the reference-made golden
vectors and the oracle (including ragged / empty shapes and every packing width)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "bitpack_golden.npz")


def make_input(seed, rows, cols, nbits):
    g = torch.Generator().manual_seed(int(seed))
    return torch.randint(0, 2 ** int(nbits), (int(rows), int(cols)), generator=g, dtype=torch.int32).to(torch.uint8)


def test_pack_unpack_match_reference_golden(lib):
    from gemlite_b200 import bitpack
    gold = np.load(GOLDEN)
    for seed, rows, cols, nbits, pb in gold["cases"]:
        seed, rows, cols, nbits, pb = int(seed), int(rows), int(cols), int(nbits), int(pb)
        W = make_input(seed, rows, cols, nbits).cuda()
        key = "s%d" % seed
        pc, e = bitpack.pack_weights_over_cols(W, nbits, pb, transpose=False)
        assert np.array_equal(pc.cpu().numpy(), gold[key + "_cols"]), (seed, nbits, pb)
        pt, _ = bitpack.pack_weights_over_cols(W, nbits, pb, transpose=True)
        assert pt.shape == (cols // e, rows) and torch.equal(pt.t(), pc)
        pr, _ = bitpack.pack_weights_over_rows(W[: (rows // e) * e], nbits, pb, transpose=False)
        assert np.array_equal(pr.cpu().numpy(), gold[key + "_rows"]), (seed, nbits, pb)
        assert np.array_equal(bitpack.unpack_over_cols(pc, nbits, cols, torch.uint8).cpu().numpy(), gold[key + "_ucols"])
        assert np.array_equal(bitpack.unpack_over_rows(pr, nbits, (rows // e) * e, torch.uint8).cpu().numpy(), gold[key + "_urows"])


@pytest.mark.parametrize("nbits", [1, 2, 4, 8])
@pytest.mark.parametrize("pb", [8, 16, 32, 64])
def test_pack_matches_oracle_all_widths(lib, nbits, pb):
    from gemlite_b200 import bitpack
    W = make_input(100 * nbits + pb, 192, 256, nbits)
    pc, e = bitpack.pack_weights_over_cols(W.cuda(), nbits, pb, transpose=False)
    oc, oe = oracle.pack_over_cols(W.numpy(), nbits, pb)
    assert e == oe and np.array_equal(pc.cpu().numpy(), oc)
    pr, _ = bitpack.pack_weights_over_rows(W.cuda(), nbits, pb, transpose=False)
    assert np.array_equal(pr.cpu().numpy(), oracle.pack_over_rows(W.numpy(), nbits, pb)[0])
    for dt in (torch.uint8, torch.int32, torch.float16, torch.bfloat16, torch.float32):
        u = bitpack.unpack_over_cols(pc, nbits, 256, dt)
        assert u.dtype == dt and torch.equal(u.cpu().to(torch.uint8), W)
    assert torch.equal(bitpack.unpack_over_rows(pr, nbits, 192, torch.uint8).cpu(), W)


def test_full_size_roundtrip_and_checksum(lib):
    # 8192 x 8192 4-bit codes (the benchmark layer): pack -> unpack is the identity and the packed
    # words sum to the value the codes define (a checksum independent of any kernel).
    from gemlite_b200 import bitpack
    g = torch.Generator(device="cuda").manual_seed(7)
    W = torch.randint(0, 16, (8192, 8192), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    p, e = bitpack.pack_weights_over_cols(W, 4, 32, transpose=False)
    assert torch.equal(bitpack.unpack_over_cols(p, 4, 8192, torch.uint8), W)
    want = (W.view(8192, -1, 8).to(torch.int64) << (4 * torch.arange(8, device="cuda"))).sum(-1)
    assert torch.equal(p.to(torch.int64) & 0xFFFFFFFF, want)


def test_empty_and_invalid(lib):
    from gemlite_b200 import bitpack
    empty = torch.empty((0, 64), dtype=torch.uint8, device="cuda")
    p, e = bitpack.pack_weights_over_cols(empty, 4, 32, transpose=False)
    assert p.shape == (0, 8)
    with pytest.raises(AssertionError):
        bitpack.pack_weights_over_cols(torch.zeros((4, 64), dtype=torch.uint8, device="cuda"), 3, 32, False)
    with pytest.raises(RuntimeError):
        bitpack.pack_weights_over_cols(torch.zeros((4, 64), dtype=torch.uint8), 4, 32, False)   # CPU tensor: no CPU path
