"""Sequence-parallel tensor parallelism with the collectives inside the kernels
(``methods(tensor="fused")``, GPUs of one NVLink domain).

Two primitives over symmetric memory, each one compute step and one exchange that
overlap tile by tile:

* `gather_matmul`  y = all_gather_seq(x_l) · W^T: every rank stores its rows into every
  peer's gather buffer (P2P stores on a few SMs) and raises its flag there; the tcgen05
  GEMM starts on its own rows at once and its TMA producer waits, per tile, only for
  the flag of the rank whose rows the tile reads.
* `matmul_scatter` y_l = reduce_scatter_seq(x · W^T): the GEMM writes its partial sums
  into a symmetric buffer and raises its flag; each rank then sums its own row block out
  of every peer's buffer by P2P loads (fp32), optionally adding the residual stream.

Each is the other's backward (the gradient of a gather is a scatter of partial sums),
so attention (qkv = gather, o = scatter) and the MLP (gate/up = gather, down = scatter)
need nothing else. Buffers are reused by every layer; "free" flags keep a rank from
overwriting a buffer its peers still read. Reference: the chunked method of
``parallel/tensor.py:114-340`` overlaps the same pairs with chained XLA collectives.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

CH_READY, CH_FREE = 0, 1


class Fabric:
    """One symmetric buffer [world · rows, width] with its ready / free flags on the
    tensor group. `role` tells gather buffers (peers write, this rank's GEMM reads) from
    partial-sum buffers (this rank's GEMM writes, peers read)."""

    def __init__(self, group, device, rows_local: int, width: int):
        import torch.distributed._symmetric_memory as symm

        self.group, self.device = group, device
        self.world, self.me = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.width = rows_local, width
        name = group.group_name
        self.buf = symm.empty(self.world * rows_local, width, dtype=torch.bfloat16, device=device)
        bh = symm.rendezvous(self.buf, name)
        flags = symm.empty(2 * self.world, dtype=torch.int32, device=device)
        fh = symm.rendezvous(flags, name)
        flags.zero_()
        self.flags = flags.view(2, self.world)
        self.ptrs = torch.tensor([int(p) for p in bh.buffer_ptrs], dtype=torch.int64, device=device)
        self.flag_ptrs = torch.tensor([int(p) for p in fh.buffer_ptrs], dtype=torch.int64, device=device)
        self.epoch = [0, 0]
        self.rotate = (self.me * rows_local) // 128 if rows_local % 128 == 0 else 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def signal(self, ch: int) -> int:
        from ..ops import kernels as K

        self.epoch[ch] += 1
        K.ep_signal(self.flag_ptrs, ch, self.world, self.me, self.epoch[ch])
        return self.epoch[ch]

    def wait_free(self) -> None:
        """Until every peer is done with the buffer's previous contents."""
        from ..ops import kernels as K

        if self.epoch[CH_FREE] > 0:
            K.ep_wait(self.flags[CH_FREE], self.epoch[CH_FREE])


_FABRICS: dict = {}


def fabric(role: str, group, device, rows_local: int, width: int) -> Fabric:
    key = (role, id(group), rows_local, width)
    if key not in _FABRICS:
        _FABRICS[key] = Fabric(group, device, rows_local, width)
    return _FABRICS[key]


_SIDE: dict = {}


def _side(device) -> torch.cuda.Stream:
    key = torch.device(device).index
    if key not in _SIDE:
        _SIDE[key] = torch.cuda.Stream(device=device)
    return _SIDE[key]


def _gather(group, x_l: torch.Tensor):
    """Starts the exchange of this rank's rows on a side stream, so the GEMM that follows on
    the main stream runs beside it (its tiles wait for their senders' flags); returns
    (fabric, epoch the GEMM waits for). This rank's own block is copied and flagged
    first: the GEMM starts on it."""
    from ..ops import kernels as K

    f = fabric("gather", group, x_l.device, x_l.shape[0], x_l.shape[1])
    main, side = torch.cuda.current_stream(x_l.device), _side(x_l.device)
    f.wait_free()
    side.wait_stream(main)
    with torch.cuda.stream(side):
        K.tp_push_block(x_l, f.ptrs, f.me)
        epoch = f.signal(CH_READY)
    x_l.record_stream(side)
    # own rows: a local copy, flagged at once
    f.buf[f.me * f.rows:(f.me + 1) * f.rows].copy_(x_l)
    f.flags[CH_READY, f.me].fill_(epoch)
    return f, epoch


def _scatter(group, device, rows_local: int, width: int, gemm_into, residual=None):
    """`gemm_into(buffer)` writes this rank's partial sums [world · rows_local, width]; returns
    this rank's rows of their sum over the ranks."""
    from ..ops import kernels as K

    f = fabric("partial", group, device, rows_local, width)
    f.wait_free()
    gemm_into(f.buf)
    e = f.signal(CH_READY)
    out = torch.empty(rows_local, width, dtype=torch.bfloat16, device=device)
    K.tp_pull_reduce(f.ptrs, f.me, out, residual, f.flags[CH_READY], e)
    f.signal(CH_FREE)
    return out


class GatherMatmul(torch.autograd.Function):
    """x_l [rows_l, k] (this rank's positions), w [n_local, k] → y [world·rows_l, n_local]."""

    @staticmethod
    def forward(ctx, x_l, w, group):
        from ..ops import kernels as K

        x_l = x_l.contiguous()
        f, epoch = _gather(group, x_l)
        y = K.gemm_bf16(f.buf, w, wait_flags=f.flags[CH_READY], wait_epoch=epoch, wait_rows=f.rows,
                        m_rotate=f.rotate)
        f.signal(CH_FREE)
        ctx.save_for_backward(x_l, w)
        ctx.group = group
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import kernels as K

        x_l, w = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        dx_l = dw = None
        if ctx.needs_input_grad[1]:
            # dW = dy^T · gather(x): the rows of x arrive again; the contraction waits per sender
            f, epoch = _gather(group, x_l)
            dw = K.gemm_bf16(dy, f.buf, a_mn=True, b_mn=True, wait_flags=f.flags[CH_READY], wait_epoch=epoch,
                             wait_rows=f.rows, wait_on_k=True)
            f.signal(CH_FREE)
        if ctx.needs_input_grad[0]:
            # dx = scatter(dy · W): partial sums over this rank's output columns
            dx_l = _scatter(group, dy.device, x_l.shape[0], w.shape[1],
                            lambda buf: K.gemm_bf16(dy, w, b_mn=True, out=buf))
        return dx_l, dw, None


class MatmulScatter(torch.autograd.Function):
    """x [world·rows_l, k_local], w [n, k_local] → y_l [rows_l, n]: this rank's rows of Σ_ranks x·W^T."""

    @staticmethod
    def forward(ctx, x, w, group, rows_local):
        from ..ops import kernels as K

        x = x.contiguous()
        y_l = _scatter(group, x.device, rows_local, w.shape[0], lambda buf: K.gemm_bf16(x, w, out=buf))
        ctx.save_for_backward(x, w)
        ctx.group = group
        return y_l

    @staticmethod
    def backward(ctx, dy_l):
        from ..ops import kernels as K

        x, w = ctx.saved_tensors
        f, epoch = _gather(ctx.group, dy_l.contiguous())
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm_bf16(f.buf, w, b_mn=True, wait_flags=f.flags[CH_READY], wait_epoch=epoch,
                             wait_rows=f.rows, m_rotate=f.rotate)
        if ctx.needs_input_grad[1]:
            dw = K.gemm_bf16(f.buf, x, a_mn=True, b_mn=True, wait_flags=f.flags[CH_READY], wait_epoch=epoch,
                             wait_rows=f.rows, wait_on_k=True)
        f.signal(CH_FREE)
        return dx, dw, None, None


def gather_matmul(x_l: torch.Tensor, w: torch.Tensor, group, reorder: bool = True) -> torch.Tensor:
    """[b, t/n, k] → [b, t, n_local]. The kernel's rows come in (rank, batch, position)
    order; `reorder` puts them back into [batch, position] (attention needs it, an MLP
    whose output goes straight into `matmul_scatter` does not)."""
    b, tl, k = x_l.shape
    world = dist.get_world_size(group)
    y = GatherMatmul.apply(x_l.reshape(b * tl, k), w, group)
    y = y.view(world, b, tl, -1)
    return y.permute(1, 0, 2, 3).reshape(b, world * tl, -1) if reorder else y.reshape(1, world * b * tl, -1)


def matmul_scatter(x: torch.Tensor, w: torch.Tensor, group, batch: int, reorder: bool = True) -> torch.Tensor:
    """[b, t, k_local] (or rows already in (rank, batch, position) order) → [b, t/n, n]."""
    world = dist.get_world_size(group)
    k = x.shape[-1]
    if reorder:
        b, t, _ = x.shape
        x = x.view(b, world, t // world, k).permute(1, 0, 2, 3)
    rows = x.numel() // k
    y_l = MatmulScatter.apply(x.reshape(rows, k), w, group, rows // world)
    return y_l.view(batch, rows // world // batch, -1)
