"""Shared fixtures for the GPU parity tests: seeded synthetic layers in the shapes and value
distributions of the benchmark configurations (x ~ N(0,1); W_q uniform codes; scales
|N(0,1)|*0.02; zeros uniform in the code range; bias N(0, 0.01))."""
import numpy as np
import torch


def make_a16wn(N, K, nbits, group_size, dtype, seed, M=1, with_bias=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    W_q = torch.randint(0, 2 ** nbits, (N, K), generator=g, dtype=torch.int32).to(torch.uint8)
    G = K // group_size
    scales = (torch.randn(N * G, 1, generator=g).abs() * 0.02).to(dtype)
    zeros = (torch.rand(N * G, 1, generator=g) * (2 ** nbits - 1)).to(dtype)
    bias = (torch.randn(N, generator=g) * 0.01).to(dtype) if with_bias else None
    return x, W_q, scales, zeros, bias


def exact_a16wn(x, W_q, scales, zeros, bias, group_size):
    """fp64 truth of the layer: x @ ((W_q - z) * s).T + bias from the unrounded formula."""
    N, K = W_q.shape
    W = ((W_q.double().view(N, -1, group_size) - zeros.double().view(N, -1, 1)) * scales.double().view(N, -1, 1)).view(N, K)
    y = x.double() @ W.T
    if bias is not None:
        y = y + bias.double()
    return y.numpy()


def rel_fro(y, ref):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30))
