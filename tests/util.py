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


# ---- plain-torch references on the GPU (fp32 matmul, no TF32) for sizes the CPU oracle cannot finish in seconds.
# They take the QUANTISED operands (codes and scales as the kernels and the oracle-pinned quantisers produce them),
# decode them to fp32 and multiply with torch; nothing of the library's matmul kernels is involved.
E2M1_TABLE = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def torch_ref_a16wn(x, W_q, scales, zeros, bias, group_size):
    """x [M, K] fp16/bf16, W_q codes [N, K] uint8, scales / zeros [N*G, 1]; fp32 result of x @ ((W_q - z) * s).T + bias."""
    N, K = W_q.shape
    W = ((W_q.float().view(N, -1, group_size) - zeros.float().view(N, -1, 1)) * scales.float().view(N, -1, 1)).view(N, K)
    y = x.float() @ W.T
    return y if bias is None else y + bias.float()


def torch_decode_fp4(q_bytes, scale_bytes, group_size, e8m0):
    """q_bytes uint8 [R, K/2] (even k in the low nibble), scale_bytes [R', K/group] (R' >= R; e8m0 or e4m3 bytes) -> fp32 [R, K]."""
    R, K2 = q_bytes.shape
    lut = torch.tensor(E2M1_TABLE, dtype=torch.float32, device=q_bytes.device)
    lo, hi = (q_bytes & 0xF).long(), (q_bytes >> 4).long()
    vals = torch.stack((lut[lo], lut[hi]), dim=-1).view(R, K2 * 2)
    sb = scale_bytes.view(torch.uint8)[:R]
    if e8m0:
        s = torch.pow(2.0, sb.float() - 127.0)
    else:
        s = sb.view(torch.float8_e4m3fn).float()
    return (vals.view(R, -1, group_size) * s.view(R, -1, 1)).view(R, K2 * 2)


def sample_index(n, count, seed):
    """`count` distinct indices in [0, n) that always include the first and the last."""
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(n, generator=g)[:max(count - 2, 0)].tolist() + [0, n - 1]
    return sorted(set(idx))
