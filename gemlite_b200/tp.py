"""Tensor-parallel sharding of GemLite linears across the GPUs of one node (one process per GPU).

The reference has no multi-GPU code: under vLLM the host shards the weights and performs the all-reduce
(gemlite/vllm/onthefly.py:83-99).  This module is that host role for the low-bit layers here:

* column-parallel (q/k/v, gate/up): the output features N are split; x is replicated; no exchange.
* row-parallel (o_proj, down_proj): the input features K are split on group boundaries; every rank holds a
  partial sum of the full output and one `all_reduce(SUM)` over NCCL (NVLink / NVSwitch) completes it.  The
  bias is added on rank 0 only, before the reduction.

`LlamaLinears` strings the seven linears of one Llama decoder layer together (fused qkv, o, fused gate/up, down)
with the two all-reduces, which is the communication pattern of a tensor-parallel decoder step; attention
itself and the norms are not part of the low-bit matmul path and are not modelled.
"""
import ctypes

import torch
import torch.distributed as dist

from . import _lib
from .dtypes import TORCH_TO_DTYPE


def quantize_affine_minmax(W, nbits=4, group_size=128):
    """Per-group min/max affine quantisation W ~ (W_q - zero) * scale (uint codes, float zero): what an
    HQQ layer with optimize=False holds.  Returns (W_q uint8 [N, K], scales [N*G, 1], zeros [N*G, 1])."""
    N, K = W.shape
    Wg = W.float().reshape(-1, group_size)
    mn, mx = Wg.amin(1, keepdim=True), Wg.amax(1, keepdim=True)
    qmax = 2 ** nbits - 1
    scale = ((mx - mn) / qmax).clamp_(min=1e-8)
    zero = -mn / scale
    W_q = torch.round(Wg / scale + zero).clamp_(0, qmax).to(torch.uint8).reshape(N, K)
    return W_q, scale.to(W.dtype), zero.to(W.dtype)


def shard_bounds(total, world, rank, multiple=1):
    """[begin, end) of `rank`'s share of `total` items split into `world` equal parts of a multiple of `multiple`."""
    if total % (world * multiple) != 0:
        raise ValueError("cannot split %d into %d shards of a multiple of %d" % (total, world, multiple))
    per = total // world
    return rank * per, (rank + 1) * per


def shard_column(W_q, scales, zeros, bias, world, rank, group_size):
    """Split the output features.  W_q [N, K]; scales / zeros [N*G, 1] (or [N, G]); bias [N] or None."""
    N, K = W_q.shape
    G = K // group_size
    a, b = shard_bounds(N, world, rank)
    s = scales.reshape(N, G)[a:b].reshape(-1, 1) if scales is not None else None
    z = zeros.reshape(N, G)[a:b].reshape(-1, 1) if zeros is not None else None
    return W_q[a:b].contiguous(), s, z, (bias[a:b].contiguous() if bias is not None else None)


def shard_row(W_q, scales, zeros, bias, world, rank, group_size):
    """Split the input features on group boundaries.  The bias stays on rank 0 (added once, before the reduce)."""
    N, K = W_q.shape
    G = K // group_size
    a, b = shard_bounds(K, world, rank, multiple=group_size)
    ga, gb = a // group_size, b // group_size
    s = scales.reshape(N, G)[:, ga:gb].reshape(-1, 1).contiguous() if scales is not None else None
    z = zeros.reshape(N, G)[:, ga:gb].reshape(-1, 1).contiguous() if zeros is not None else None
    return W_q[:, a:b].contiguous(), s, z, (bias if (bias is not None and rank == 0) else None)


class PeerComm:
    """One-shot all-reduce over peer memory for decode-size results (`gl_tp_allreduce` of the C ABI).

    Every rank creates one receive buffer with the library, the 64-byte handles travel through the process group
    (a host-side all-gather at set-up), and each rank maps the buffers of the others.  `all_reduce(x)` then is ONE
    kernel: push the local partial result into every rank's receive area, publish a flag per chunk, wait (bounded)
    for the other ranks' flags, add the chunks in rank order.  Results are bit-identical on all ranks.  Tensors
    larger than `slot_bytes` do not fit and are the caller's business (NCCL)."""

    def __init__(self, device, group=None, slot_bytes=2 << 20, wait_cycles=0):
        self.device = torch.device(device)
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("PeerComm supports at most 8 ranks")
        L = _lib.lib()
        self.slot_bytes = int(slot_bytes)
        nbytes = int(L.gl_tp_buffer_bytes(self.world, self.slot_bytes))
        own, handle = ctypes.c_void_p(), (ctypes.c_uint8 * 64)()
        with torch.cuda.device(self.device):
            _lib.check(L.gl_tp_buffer_create(nbytes, ctypes.byref(own), handle))
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._opened = []
        self.comm = _lib.GLTpComm()
        self.comm.rank, self.comm.world = self.rank, self.world
        self.comm.slot_bytes, self.comm.wait_cycles = self.slot_bytes, int(wait_cycles)
        with torch.cuda.device(self.device):
            for r in range(self.world):
                if r == self.rank:
                    self.comm.buffers[r] = self._own
                    continue
                ptr = ctypes.c_void_p()
                h = (ctypes.c_uint8 * 64).from_buffer_copy(handles[r])
                _lib.check(L.gl_tp_buffer_open(h, ctypes.byref(ptr)))
                self._opened.append(ptr.value)
                self.comm.buffers[r] = ptr.value
        dist.barrier(group=group)

    def fits(self, t):
        return t.is_contiguous() and t.numel() * t.element_size() <= self.slot_bytes and (t.numel() * t.element_size()) % 16 == 0

    def all_reduce(self, x, out=None):
        _lib.require_cuda(x, "x")
        if out is None:
            out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().gl_tp_allreduce(ctypes.byref(self.comm), x.data_ptr(), out.data_ptr(), x.numel(),
                                                  TORCH_TO_DTYPE[x.dtype].value, TORCH_TO_DTYPE[out.dtype].value,
                                                  _lib.current_stream_ptr(x.device)))
        return out

    def status(self):
        """(status word, completed all-reduces); a non-zero status means a flag wait ran out of its cycle budget."""
        st, ep = ctypes.c_int32(), ctypes.c_uint32()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().gl_tp_status(ctypes.byref(self.comm), ctypes.byref(st), ctypes.byref(ep)))
        return st.value, ep.value

    def close(self):
        """Collective: every rank must have finished its last all-reduce before any buffer goes away."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        L = _lib.lib()
        with torch.cuda.device(self.device):
            for ptr in self._opened:
                L.gl_tp_buffer_close(ptr)
            dist.barrier(group=self.group)
            L.gl_tp_buffer_destroy(self._own)
        self._own, self._opened = None, []


def silu_mul(gate_up):
    """silu(gate) * up for a fused [.., 2 * inter] gate/up projection output, as one kernel."""
    _lib.require_cuda(gate_up, "gate_up")
    gu = gate_up.contiguous().view(-1, gate_up.shape[-1])
    inter = gu.shape[1] // 2
    out = torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device)
    with torch.cuda.device(gu.device):
        _lib.check(_lib.lib().gl_silu_mul(gu.data_ptr(), out.data_ptr(), gu.shape[0], inter, TORCH_TO_DTYPE[gu.dtype].value,
                                          _lib.current_stream_ptr(gu.device)))
    return out.view(gate_up.shape[:-1] + (inter,))


class TPLinear(torch.nn.Module):
    """A sharded layer plus its collective.  `layer` is any callable x -> y (a GemLiteLinear on a GPU).  With a
    `PeerComm`, results that fit its receive slots are reduced by the one-shot kernel, larger ones by NCCL."""

    def __init__(self, layer, mode, group=None, comm=None, world=None):
        super().__init__()
        assert mode in ("column", "row")
        self.layer, self.mode, self.group, self.comm = layer, mode, group, comm
        # number of shards the layer was cut into (None: the size of the process group); an unsharded layer never reduces
        self.world = world

    def forward(self, x):
        y = self.layer(x)
        world = self.world if self.world is not None else (dist.get_world_size(self.group) if dist.is_initialized() else 1)
        if self.mode == "row" and world > 1:
            if self.comm is not None and self.comm.fits(y):
                return self.comm.all_reduce(y)
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y


def build_a16w4_tp_linear(W, bias, mode, world, rank, device, dtype=torch.bfloat16, nbits=4, group_size=128, comm=None):
    """Quantise a full-precision weight [N, K] and build this rank's shard as a packed GemLiteLinear."""
    from .helper import A16Wn_HQQ_INT
    W_q, s, z = quantize_affine_minmax(W, nbits, group_size)
    shard = shard_column if mode == "column" else shard_row
    W_q, s, z, b = shard(W_q, s, z, bias, world, rank, group_size)
    proc = A16Wn_HQQ_INT(device=str(device), dtype=dtype, W_nbits=nbits)
    layer = proc.from_weights(W_q.to(device), s.to(device), z.to(device), bias=None if b is None else b.to(device))
    return TPLinear(layer, mode, comm=comm, world=world)


class LlamaLinears(torch.nn.Module):
    """The seven linears of one Llama decoder layer, tensor-parallel: fused qkv (column) -> o_proj (row,
    all-reduce) -> fused gate/up (column) -> down_proj (row, all-reduce)."""

    def __init__(self, hidden, intermediate, n_heads, n_kv_heads, head_dim, world, rank, device, dtype=torch.bfloat16,
                 seed=0, group_size=128, comm=None):
        super().__init__()
        self.world, self.rank, self.comm = world, rank, comm
        self.q_local = n_heads * head_dim // world
        self.kv_local = n_kv_heads * head_dim // world
        self.inter_local = intermediate // world
        gen_dev = torch.device(device)
        g = torch.Generator(device=gen_dev).manual_seed(seed)   # same seed on every rank: all ranks shard the same matrices

        def w(n, k):
            return (torch.randn(n, k, generator=g, device=gen_dev) * 0.02).to(dtype)

        def col(*mats):   # each matrix is column-sharded on its own, the shards are fused per rank
            parts = [quantize_affine_minmax(m, 4, group_size) for m in mats]
            shards = [shard_column(p[0], p[1], p[2], None, world, rank, group_size) for p in parts]
            W_q = torch.cat([s[0] for s in shards], 0)
            sc = torch.cat([s[1].reshape(s[0].shape[0], -1) for s in shards], 0).reshape(-1, 1)
            zz = torch.cat([s[2].reshape(s[0].shape[0], -1) for s in shards], 0).reshape(-1, 1)
            from .helper import A16W4_HQQ_INT
            layer = A16W4_HQQ_INT(device=str(device), dtype=dtype).from_weights(W_q.to(device), sc.to(device), zz.to(device))
            return TPLinear(layer, "column", world=world)

        self.qkv = col(w(n_heads * head_dim, hidden), w(n_kv_heads * head_dim, hidden), w(n_kv_heads * head_dim, hidden))
        self.o = build_a16w4_tp_linear(w(hidden, n_heads * head_dim), None, "row", world, rank, device, dtype, 4, group_size, comm)
        self.gate_up = col(w(intermediate, hidden), w(intermediate, hidden))
        self.down = build_a16w4_tp_linear(w(hidden, intermediate), None, "row", world, rank, device, dtype, 4, group_size, comm)

    def forward(self, x):
        qkv = self.qkv(x)
        attn = qkv[..., : self.q_local].contiguous()          # stand-in for the attention output of the local heads
        h = self.o(attn)
        gu = self.gate_up(h)
        return self.down(silu_mul(gu))
