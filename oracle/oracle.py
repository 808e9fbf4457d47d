"""CPU restatement of GemLite's low-bit matmul path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference arm may
import this file; the product (``gemlite_b200``) never does and has no CPU path.

Every function restates one piece of the reference and cites it (paths inside the reference
project).  Parity pins:
  * bit packing: pinned bit-for-bit against the reference's own torch functions, run on CPU
    (fixtures in ``tests/golden/bitpack_golden.npz`` made by ``tests/golden/make_golden_bitpack.py``).
  * dequantise + matmul, activation quantisation, MX / NV weight quantisation: the reference
    has no golden vectors for them (its tests are tolerance checks against ``torch.matmul``,
    tests/test_int.py:96-97, tests/test_mxfp.py:74-104); they are pinned against outputs of the
    reference's Triton kernels and torch functions captured on a B200
    (``tests/golden/triton_golden.npz`` made by ``tests/golden/make_golden_triton.py``) where that
    file is present; without it these parts are "parity unpinned".

numpy for integer / byte work, torch-on-CPU for fp8 casts and for the timed baseline matmul
(the reference's CPU-capable path is torch: unpack_over_cols_torch -> (W_q - z) * s -> matmul).
"""
import numpy as np
import torch

# ---------------------------------------------------------------------------------------------
# bit packing  (gemlite/bitpack.py)
# ---------------------------------------------------------------------------------------------
_WORD = {8: np.uint8, 16: np.int16, 32: np.int32, 64: np.int64}   # gemlite/dtypes.py:95-100
_UWORD = {8: np.uint8, 16: np.uint16, 32: np.uint32, 64: np.uint64}


def pack_over_cols(W_q, nbits, packing_bitwidth):
    """gemlite/bitpack.py:36-60: out[r, c] = OR_j W_q[r, c*e + j] << (j * nbits), field 0 lowest."""
    e = packing_bitwidth // nbits
    W = np.asarray(W_q).astype(np.uint64)
    rows, cols = W.shape
    out = np.zeros((rows, cols // e), dtype=np.uint64)
    for j in range(e):
        out |= W[:, j:(cols // e) * e:e] << np.uint64(j * nbits)
    return out.astype(_UWORD[packing_bitwidth]).view(_WORD[packing_bitwidth]), e


def pack_over_rows(W_q, nbits, packing_bitwidth):
    """gemlite/bitpack.py:10-34: out[r, c] = OR_j W_q[r*e + j, c] << (j * nbits)."""
    e = packing_bitwidth // nbits
    W = np.asarray(W_q).astype(np.uint64)
    rows, cols = W.shape
    out = np.zeros((rows // e, cols), dtype=np.uint64)
    for j in range(e):
        out |= W[j:(rows // e) * e:e, :] << np.uint64(j * nbits)
    return out.astype(_UWORD[packing_bitwidth]).view(_WORD[packing_bitwidth]), e


def unpack_over_cols(packed, nbits, num_output_cols):
    """gemlite/bitpack.py:146-163: e = num_output_cols // cols; (word >> j*nbits) & mask."""
    p = np.asarray(packed)
    u = p.view(_UWORD[p.dtype.itemsize * 8]).astype(np.uint64)
    rows, cols = u.shape
    e = num_output_cols // cols
    out = np.zeros((rows, cols, e), dtype=np.uint8)
    for j in range(e):
        out[:, :, j] = ((u >> np.uint64(j * nbits)) & np.uint64((1 << nbits) - 1)).astype(np.uint8)
    return out.reshape(rows, num_output_cols)


def unpack_over_rows(packed, nbits, num_output_rows):
    """gemlite/bitpack.py:320-336."""
    p = np.asarray(packed)
    u = p.view(_UWORD[p.dtype.itemsize * 8]).astype(np.uint64)
    rows, cols = u.shape
    e = num_output_rows // rows
    out = np.zeros((rows, e, cols), dtype=np.uint8)
    for j in range(e):
        out[:, j, :] = ((u >> np.uint64(j * nbits)) & np.uint64((1 << nbits) - 1)).astype(np.uint8)
    return out.reshape(num_output_rows, cols)


# ---------------------------------------------------------------------------------------------
# helpers: rounding to a storage dtype, fp8 / fp4 / e8m0 codecs
# ---------------------------------------------------------------------------------------------
def _round_to(t, dtype):
    """Round an fp32 / fp64 torch tensor to ``dtype`` precision and return it as fp32."""
    if dtype in (torch.float16, torch.bfloat16):
        return t.to(torch.float32).to(dtype).to(torch.float32)
    return t.to(torch.float32)


FP4_VALUES = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)
FP4_THRESHOLDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def e2m1_decode(codes):
    """E2M1 code -> value, sign in bit 3 (gemlite/quant_utils.py:36-41)."""
    return FP4_VALUES[np.asarray(codes).astype(np.int64) & 15]


def e2m1_encode_thresholds(v):
    """Activation-side rounding of the Triton kernels: count of thresholds exceeded, +8 when
    negative (gemlite/quant_utils.py:2081-2087). Ties go to the smaller magnitude; values
    in (-0.25, 0) give code 8 (negative zero)."""
    v = np.asarray(v, dtype=np.float32)
    idx = (np.abs(v)[..., None] > FP4_THRESHOLDS).sum(-1).astype(np.uint8)
    return np.where(v >= 0, idx, idx + 8).astype(np.uint8)


def e8m0_decode(b):
    """e8m0 byte -> 2^(b-127) (b = 0 -> 2^-127, b = 255 -> NaN)."""
    return torch.from_numpy(np.asarray(b, dtype=np.uint8).copy()).view(torch.float8_e8m0fnu).to(torch.float32).numpy()


def e4m3_decode(b):
    return torch.from_numpy(np.asarray(b, dtype=np.uint8).copy()).view(torch.float8_e4m3fn).to(torch.float32).numpy()


def e4m3_encode(v):
    """fp32 -> e4m3 bytes, round to nearest even (inputs are clamped to +-448 by the callers)."""
    return torch.from_numpy(np.asarray(v, dtype=np.float32).copy()).to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def pow2_ceil_exp(v, eps_exp=-30):
    """gemlite/quant_utils.py:697-705 (next_power_of_2_bitwise_triton): biased exponent of
    2^ceil(log2 v), clamped to [127+eps_exp, 254]."""
    bits = np.asarray(v, dtype=np.float32).view(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int64) + ((bits & 0x7FFFFF) != 0)
    return np.clip(exp, 127 + eps_exp, 254).astype(np.uint8)


# ---------------------------------------------------------------------------------------------
# dequantise + matmul for integer / fp8 / fp16 weights
# ---------------------------------------------------------------------------------------------
def dequantize(W_int, scales, zeros, W_group_mode, group_size, meta_dtype=torch.float32, exact=False):
    """gemlite/triton_kernels/utils.py:73-105 on a whole [K, N] matrix.

    W_int [K, N] (integer codes or raw weights, torch); scales / zeros [G, N] or scalar; the
    arithmetic runs in ``meta_dtype`` with one rounding per operation as Triton does, or in fp64
    when ``exact`` (the tie-breaking truth)."""
    K, N = W_int.shape
    f = torch.float64 if exact else torch.float32
    b = W_int.to(f)

    def expand(t):
        if t is None:
            return None
        t = t.to(f)
        if t.numel() == 1:
            return t.reshape(1, 1)
        return t.reshape(-1, N).repeat_interleave(group_size, dim=0)[:K]

    s, z = expand(scales), expand(zeros)
    rnd = (lambda t: t) if exact else (lambda t: _round_to(t, meta_dtype))
    if W_group_mode == 1:
        return rnd(b - z)
    if W_group_mode == 2:
        return rnd(b * s)
    if W_group_mode == 3:
        if zeros is not None and zeros.numel() == 1:
            return rnd((b - z) * s)
        return rnd(rnd(b - z) * s)
    if W_group_mode == 4:
        return rnd(b * s + z) if exact else _round_to((b.double() * s.double() + z.double()), meta_dtype)
    return b


def matmul_int(x, W_int, scales, zeros, W_group_mode, channel_scale_mode, group_size, x_dtype=torch.bfloat16,
               meta_dtype=None, out_dtype=None, scales_x=None, bias=None, exact=False):
    """Forward of the integer-weight kernels (gemlite/triton_kernels/gemm_kernels.py:285-496):
    y = x @ dequantize(W) with fp32 accumulation, then channel scales (:472-484), then the
    separate bias add of gemlite/core.py:271-272.  ``exact`` computes everything in fp64 from the
    unrounded formula (the tie-breaking truth)."""
    meta_dtype = meta_dtype or x_dtype
    out_dtype = out_dtype or x_dtype
    gs = None if W_group_mode in (0,) else scales
    W = dequantize(W_int, gs if W_group_mode >= 2 else None, zeros if W_group_mode in (1, 3, 4) else None,
                   W_group_mode, group_size, meta_dtype, exact)
    if exact:
        y = x.double() @ W.double()
    else:
        if x_dtype in (torch.float16, torch.bfloat16):
            W = _round_to(W, x_dtype)                      # tl.dot(a, b.to(input_dtype))
        y = (x.to(torch.float32).double() @ W.double()).to(torch.float32)   # fp32 accumulate, order-free
    if channel_scale_mode == 1:
        y = y * scales.reshape(1, -1).to(y.dtype)
    elif channel_scale_mode == 2:
        y = y * scales_x.reshape(-1, 1).to(y.dtype)
    elif channel_scale_mode == 3:
        y = y * (scales_x.reshape(-1, 1).to(y.dtype) * scales.reshape(1, -1).to(y.dtype))
    if bias is not None:
        y = y + bias.to(y.dtype).reshape(1, -1)
    return y if exact else _round_to(y, out_dtype)


def cpu_reference_forward(x, W_q_packed, scales, zeros, W_nbits, group_size, compute_dtype=torch.float32):
    """The reference's CPU-runnable path, used as the timed CPU baseline: unpack with the torch
    shift/mask of gemlite/bitpack.py:146-163, dequantise per group ``(W_q - zeros) * scales``
    (README.md:84, tests/test_int.py:43-57), then ``torch.matmul(x, W.T)``
    (examples/benchmark_triton.py:67-72).  W_q_packed int32 [N, K/e]; scales, zeros [N*G, 1]."""
    N, Kp = W_q_packed.shape
    e = 32 // W_nbits
    shifts = torch.arange(e, dtype=W_q_packed.dtype) * W_nbits
    W_q = ((W_q_packed.unsqueeze(-1) >> shifts) & ((1 << W_nbits) - 1)).to(compute_dtype).view(N, Kp * e)
    W = ((W_q.view(-1, group_size) - zeros.view(-1, 1).to(compute_dtype)) * scales.view(-1, 1).to(compute_dtype)).view(N, Kp * e)
    return torch.matmul(x.to(compute_dtype), W.T)


# ---------------------------------------------------------------------------------------------
# activation quantisation
# ---------------------------------------------------------------------------------------------
def scale_activations_per_token(x, qdtype="fp8"):
    """gemlite/quant_utils.py:467-508: s = max(amax/qmax, 1e-6); q = clamp(x / s); int8 rounds
    half away from zero (libdevice.round).  x [M, K] fp32 numpy.  Returns (q bytes / int8, s [M,1])."""
    x = np.asarray(x, dtype=np.float32)
    qmax, qmin = (np.float32(448.0), np.float32(-448.0)) if qdtype == "fp8" else (np.float32(127.0), np.float32(-128.0))
    s = np.maximum(np.abs(x).max(axis=1, keepdims=True) / qmax, np.float32(1e-6)).astype(np.float32)
    t = np.clip((x / s).astype(np.float32), qmin, qmax)
    if qdtype == "fp8":
        return e4m3_encode(t), s
    r = np.where(t >= 0, np.floor(t + np.float32(0.5)), np.ceil(t - np.float32(0.5)))
    return r.astype(np.int8), s


def scale_activations_per_block(x, qdtype="fp8", block=128):
    """gemlite/quant_utils.py:2504-2522 / 2613-2675: one scale per row and per `block` consecutive k,
    s = max(amax/qmax, 1e-6); q = clamp(x / s); int8 rounds half away from zero (libdevice.round in the active kernel).
    x [M, K] fp32 numpy, K % block == 0.  Returns (q bytes / int8 [M, K], s fp32 [M, K/block])."""
    x = np.asarray(x, dtype=np.float32)
    M, K = x.shape
    assert K % block == 0
    qmax, qmin = (np.float32(448.0), np.float32(-448.0)) if qdtype == "fp8" else (np.float32(127.0), np.float32(-128.0))
    g = x.reshape(M, K // block, block)
    s = np.maximum(np.abs(g).max(axis=-1) / qmax, np.float32(1e-6)).astype(np.float32)
    t = np.clip((g / s[..., None]).astype(np.float32), qmin, qmax).reshape(M, K)
    if qdtype == "fp8":
        return e4m3_encode(t), s
    r = np.where(t >= 0, np.floor(t + np.float32(0.5)), np.ceil(t - np.float32(0.5)))
    return r.astype(np.int8), s


def quantize_block_weights(W, qdtype="fp8", block=128):
    """gemlite/helper.py:556-575: 128 x 128 blocks of W [N, K] (zero-padded at the edges), one fp32 scale per block,
    s = max(amax/qmax, 1e-6), q = clamp(W / s) cast (fp8) or rounded half to even (int8, torch.round).
    Returns (q bytes / int8 [N, K], s fp32 [ceil(N/block), ceil(K/block)])."""
    W = np.asarray(W, dtype=np.float32)
    N, K = W.shape
    nb, kb = -(-N // block), -(-K // block)
    Wp = np.zeros((nb * block, kb * block), dtype=np.float32)
    Wp[:N, :K] = W
    g = Wp.reshape(nb, block, kb, block)
    qmax, qmin = (np.float32(448.0), np.float32(-448.0)) if qdtype == "fp8" else (np.float32(127.0), np.float32(-128.0))
    s = np.maximum(np.abs(g).max(axis=(1, 3)) / qmax, np.float32(1e-6)).astype(np.float32)
    t = np.clip((g / s[:, None, :, None]).astype(np.float32), qmin, qmax).reshape(nb * block, kb * block)[:N, :K]
    if qdtype == "fp8":
        return e4m3_encode(t), s
    return np.rint(t).astype(np.int8), s


def matmul_block_quant(xq, sx, wq, sw, qdtype="fp8", block=128, bias=None):
    """channel_scale_mode 5 (gemlite/triton_kernels/gemm_kernels.py:396-450): for every block kb of `block` k,
    out[m, n] += (sum_{k in kb} x[m, k] * w[n, k]) * sx[m, kb] * sw[n // block, kb].  float64 accumulation."""
    X = e4m3_decode(xq).astype(np.float64) if qdtype == "fp8" else np.asarray(xq, dtype=np.float64)
    W = e4m3_decode(wq).astype(np.float64) if qdtype == "fp8" else np.asarray(wq, dtype=np.float64)
    M, K = X.shape
    N = W.shape[0]
    out = np.zeros((M, N), dtype=np.float64)
    sw_n = np.repeat(np.asarray(sw, dtype=np.float64), block, axis=0)[:N]           # [N, K/block]
    for kb in range(K // block):
        part = X[:, kb * block:(kb + 1) * block] @ W[:, kb * block:(kb + 1) * block].T
        out += part * np.asarray(sx, dtype=np.float64)[:, kb:kb + 1] * sw_n[:, kb][None, :]
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float64)
    return out


def scale_activations_mxfp4(x):
    """gemlite/quant_utils.py:2005-2105.  Returns (q uint8 [M, K/2], e8m0 bytes [ceil32(M), K/32])."""
    x = np.asarray(x, dtype=np.float32)
    M, K = x.shape
    Mpad = (M + 31) // 32 * 32
    g = x.reshape(M, K // 32, 32)
    exp = pow2_ceil_exp((np.abs(g).max(-1) / np.float32(6.0)).astype(np.float32))
    scale = (exp.astype(np.uint32) << 23).view(np.float32)
    codes = e2m1_encode_thresholds((g / scale[..., None]).astype(np.float32)).reshape(M, K)
    q = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    scales = np.full((Mpad, K // 32), 127, dtype=np.uint8)
    scales[:M] = exp
    return q, scales


def scale_activations_mxfp8(x):
    """gemlite/quant_utils.py:1024-1093.  Returns (q e4m3 bytes [M, K], e8m0 bytes [ceil32(M), K/32])."""
    x = np.asarray(x, dtype=np.float32)
    M, K = x.shape
    Mpad = (M + 31) // 32 * 32
    g = x.reshape(M, K // 32, 32)
    exp = pow2_ceil_exp((np.abs(g).max(-1) / np.float32(448.0)).astype(np.float32))
    scale = (exp.astype(np.uint32) << 23).view(np.float32)
    t = np.clip((g * (np.float32(1.0) / scale)[..., None]).astype(np.float32), -448.0, 448.0)
    scales = np.full((Mpad, K // 32), 127, dtype=np.uint8)
    scales[:M] = exp
    return e4m3_encode(t.reshape(M, K)), scales


def scale_activations_nvfp4(x, meta_scale=None):
    """gemlite/quant_utils.py:2161-2311 (dynamic) / :2329-2431 (given meta_scale).
    Returns (q uint8 [M, K/2], e4m3 bytes [ceil16(M), K/16], meta fp32)."""
    x = np.asarray(x, dtype=np.float32)
    M, K = x.shape
    Mpad = (M + 15) // 16 * 16
    if meta_scale is None:
        meta = np.float32(448.0 * 6.0) / np.maximum(np.abs(x).max().astype(np.float32), np.float32(1e-6))
    else:
        meta = np.float32(meta_scale)
    meta = np.float32(meta)
    g = x.reshape(M, K // 16, 16)
    amax = np.abs(g).max(-1).astype(np.float32)
    sraw = np.minimum(((amax * meta).astype(np.float32) / np.float32(6.0)).astype(np.float32), np.float32(448.0))
    s8 = e4m3_encode(sraw)
    sfull = np.maximum((e4m3_decode(s8) / meta).astype(np.float32), np.float32(1e-6))
    codes = e2m1_encode_thresholds((g / sfull[..., None]).astype(np.float32)).reshape(M, K)
    q = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    scales = np.full((Mpad, K // 16), 0x38, dtype=np.uint8)   # 1.0 in e4m3
    scales[:M] = s8
    return q, scales, meta


# ---------------------------------------------------------------------------------------------
# MX / NV block-scaled matmul (gemlite/triton_kernels/gemm_kernels.py:509-737)
# ---------------------------------------------------------------------------------------------
def unpack_fp4(q):
    """uint8 [R, K/2] -> fp32 [R, K]; even k in the low nibble (gemlite/quant_utils.py:2089-2090)."""
    q = np.asarray(q, dtype=np.uint8)
    out = np.empty((q.shape[0], q.shape[1] * 2), dtype=np.float32)
    out[:, 0::2] = e2m1_decode(q & 15)
    out[:, 1::2] = e2m1_decode(q >> 4)
    return out


def matmul_mx(xq, sx, wq, sw, group_size, meta_scale=None, x_is_fp4=True, w_is_fp4=True, scales_x_token=None):
    """y[m, n] = sum_g (sum_{k in g} x[m,k] w[n,k]) * sx[m,g] * sw[n,g]  (* meta_scale for group 16,
    * per-token scale for channel_scale_mode 2).  xq: fp4 bytes [M, K/2], e4m3 bytes [M, K] or
    float [M, K] (weight-only); wq: fp4 bytes [N, K/2] or e4m3 bytes [N, K]; sx [>=M, K/g] bytes or
    None; sw [N, K/g] bytes.  fp64 accumulation."""
    dec = e4m3_decode if group_size == 16 else e8m0_decode
    W = unpack_fp4(wq) if w_is_fp4 else e4m3_decode(wq)
    N, K = W.shape
    Wd = (W.reshape(N, K // group_size, group_size).astype(np.float64) * dec(sw).astype(np.float64)[:N, :, None]).reshape(N, K)
    if sx is not None:
        X = unpack_fp4(xq) if x_is_fp4 else e4m3_decode(xq)
        M = X.shape[0]
        Xd = (X.reshape(M, K // group_size, group_size).astype(np.float64) * dec(sx).astype(np.float64)[:M, :, None]).reshape(M, K)
    else:
        Xd = np.asarray(xq, dtype=np.float64)
    y = Xd @ Wd.T
    if meta_scale is not None:
        y = y * np.float64(meta_scale)
    if scales_x_token is not None:
        y = y * np.asarray(scales_x_token, dtype=np.float64).reshape(-1, 1)
    return y


# ---------------------------------------------------------------------------------------------
# offline MX / NV weight quantisation (gemlite/quant_utils.py:130-219, window_size = 0)
# ---------------------------------------------------------------------------------------------
def _round_fp4_weights(v):
    """torch.searchsorted(thresholds, |v|) (left bisect): ties to the smaller magnitude; to_index()
    maps -0.0 to code 0 (gemlite/quant_utils.py:80-99)."""
    v = np.asarray(v, dtype=np.float32)
    idx = np.searchsorted(FP4_THRESHOLDS, np.abs(v), side="left").astype(np.uint8)
    neg = (v < 0) & (idx > 0)
    return np.where(neg, idx + 8, idx).astype(np.uint8)


def quantize_mxfp4_weights(W):
    """gemlite/quant_utils.py:130-168.  W fp32 [N, K] -> (codes uint8 [N, K], e8m0 bytes [N, K/32])."""
    W = np.asarray(W, dtype=np.float32)
    N, K = W.shape
    g = W.reshape(-1, 32)
    ideal = (np.abs(g).max(1, keepdims=True) / np.float32(6.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        scales = np.maximum(np.exp2(np.ceil(np.log2(ideal))).astype(np.float32), np.float32(2.0 ** -30))
    codes = _round_fp4_weights((g / scales).astype(np.float32)).reshape(N, K)
    sb = torch.from_numpy(scales.copy()).to(torch.float8_e8m0fnu).view(torch.uint8).numpy().reshape(N, K // 32)
    return codes, sb


def quantize_nvfp4_weights(W, meta=None):
    """gemlite/quant_utils.py:171-219.  -> (codes [N, K], e4m3 bytes [N, K/16], meta fp32).

    The tensor scale 448 / max(amax/6) is written `448 / tensor` in the reference, which torch evaluates
    as tensor.reciprocal() * 448; the last bit of that product differs between torch's CPU and CUDA
    kernels, so a caller comparing against a layer quantised on a GPU passes the layer's `meta`."""
    W = np.asarray(W, dtype=np.float32)
    N, K = W.shape
    g = W.reshape(-1, 16)
    ideal = (np.abs(g).max(1, keepdims=True) / np.float32(6.0)).astype(np.float32)
    if meta is None:
        meta = np.float32((np.float32(1.0) / np.maximum(ideal.max(), np.float32(1e-6))) * np.float32(448.0))
    meta = np.float32(meta)
    s8 = e4m3_encode(np.minimum((ideal * meta).astype(np.float32), np.float32(448.0)))
    sfull = np.maximum((e4m3_decode(s8) / meta).astype(np.float32), np.float32(1e-6))
    codes = _round_fp4_weights((g / sfull).astype(np.float32)).reshape(N, K)
    return codes, s8.reshape(N, K // 16), np.float32(meta)


def pack_fp4_codes(codes):
    """codes uint8 [N, K] -> bytes [N, K/2], even k in the low nibble (pack_over_cols, 4 bits in 8)."""
    return pack_over_cols(codes, 4, 8)[0]


def rel_frobenius(y, y_ref):
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    return float(np.linalg.norm(y - y_ref) / max(np.linalg.norm(y_ref), 1e-30))
