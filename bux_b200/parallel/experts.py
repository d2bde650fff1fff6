"""Expert parallelism: experts split over the ``expert`` mesh axis, tokens exchanged.

Two methods (``methods(moe=...)``):

* ``fused_ep``: the exchange is done by this library's own kernels over NVLink peer
  memory (symmetric buffers). Dispatch = P2P stores of token rows straight into the
  owner's expert-sorted receive buffer + epoch flags; the owner's first grouped GEMM
  waits for the flags in its TMA producer warp; combine = P2P loads of the expert
  outputs where they were produced, weighted and summed per token. The backward
  mirrors it: dout rows are pushed to the owners with their weights beside them, each
  owner takes the dot products of its dy and y rows for the router weights' gradient
  (only those scalars cross NVLink again) and applies the weights as it quantises; dx is
  pulled. No NCCL call moves a token; one tiny all-gather moves the per-expert counts.
* ``all_to_all`` (also ``nccl_ep`` / ``ragged_all_to_all``, which keep their meaning of
  "library collective"): the same layout through ``torch.distributed.all_to_all_single``,
  the measured baseline and the CPU/gloo path of the tests.

Layout on the owner: expert-major, source-rank-major inside an expert, every expert
padded to 128 rows; `capacity` bounds the buffer (rows past it are dropped and counted).

Reference: ``parallel/experts.py:75-741`` and ``parallel/nccl_ep.py``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import fused

ALIGN = 128
CH_X, CH_Y, CH_DY, CH_DX, CH_DOT = 0, 1, 2, 3, 4


@dataclass
class Route:
    src_token: torch.Tensor   # int32[P] token of each pick, in expert-sorted order
    dst_rank: torch.Tensor    # int32[P]
    dst_row: torch.Tensor     # int32[P] row in the owner's buffer, -1 = dropped
    rank_of: torch.Tensor     # int32[T,k] the same, by (token, slot)
    row_of: torch.Tensor      # int32[T,k]
    offsets: torch.Tensor     # int32[El+1] padded starts of my local experts
    counts: torch.Tensor      # int32[El] real rows of my local experts
    order: torch.Tensor       # int64[P] sorted position -> flat pick
    dropped: torch.Tensor     # scalar


def route(idx: torch.Tensor, num_experts: int, group, cap_rows: int) -> Route:
    """Where each pick goes. One small all-gather (the per-expert counts of every rank)
    is the only collective; everything else is local integer work on the device."""
    world, me = dist.get_world_size(group), dist.get_rank(group)
    el = num_experts // world
    t, k = idx.shape
    dev = idx.device
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts).to(torch.int32)
    allc = torch.empty(world * num_experts, dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(allc, counts, group=group)
    allc64 = allc.view(world, num_experts).long()
    before_me = allc64[:me].sum(0)                       # rows of earlier sources, per expert
    total = allc64.sum(0)
    padded = (total + ALIGN - 1) // ALIGN * ALIGN
    base = (padded.view(world, el).cumsum(1) - padded.view(world, el)).reshape(-1)  # start on its owner
    my_start = counts.long().cumsum(0) - counts.long()
    sorted_e = flat[order]
    rank_within = torch.arange(t * k, device=dev) - my_start[sorted_e]
    dst_row = base[sorted_e] + before_me[sorted_e] + rank_within
    dropped = (dst_row >= cap_rows)
    dst_row = torch.where(dropped, torch.full_like(dst_row, -1), dst_row)
    dst_rank = sorted_e // el
    row_of = torch.empty(t * k, dtype=torch.int32, device=dev)
    rank_of = torch.empty(t * k, dtype=torch.int32, device=dev)
    row_of[order] = dst_row.to(torch.int32)
    rank_of[order] = dst_rank.to(torch.int32)
    mine = slice(me * el, (me + 1) * el)
    offsets = torch.zeros(el + 1, dtype=torch.int64, device=dev)
    offsets[:-1] = base[mine]
    offsets[-1] = base[mine][-1] + padded[mine][-1]
    offsets = offsets.clamp(max=cap_rows // ALIGN * ALIGN)
    local_counts = torch.minimum(total[mine], (offsets[1:] - offsets[:-1]))
    return Route((order // k).to(torch.int32), dst_rank.to(torch.int32), dst_row.to(torch.int32),
                 rank_of.view(t, k), row_of.view(t, k), offsets.to(torch.int32),
                 local_counts.to(torch.int32), order, dropped.sum())


# ====================================================================== fused (peer memory)
class FusedEP:
    """State of the in-kernel exchange for one MoE shape: symmetric buffers, the peers'
    base addresses, flag rows and epoch counters."""

    def __init__(self, group, device, d: int, cap_rows: int, dtype=torch.bfloat16):
        import torch.distributed._symmetric_memory as symm

        self.group, self.device, self.d, self.cap = group, device, d, cap_rows
        self.world, self.me = dist.get_world_size(group), dist.get_rank(group)
        name = group.group_name
        self.bufs, self.tables = {}, {}
        for key in ("x", "y", "dy", "dx"):
            buf = symm.empty(cap_rows, d, dtype=dtype, device=device)
            hdl = symm.rendezvous(buf, name)
            buf.zero_()
            self.bufs[key] = buf
            self.tables[key] = torch.tensor([int(p) for p in hdl.buffer_ptrs], dtype=torch.int64, device=device)
        for key in ("dys", "dots"):  # per-row fp32: the weight of a pushed dy row, and <dy, y> of a row
            buf = symm.empty(cap_rows, dtype=torch.float32, device=device)
            hdl = symm.rendezvous(buf, name)
            buf.zero_()
            self.bufs[key] = buf
            self.tables[key] = torch.tensor([int(p) for p in hdl.buffer_ptrs], dtype=torch.int64, device=device)
        flags = symm.empty(8 * self.world, dtype=torch.int32, device=device)
        fh = symm.rendezvous(flags, name)
        flags.zero_()
        self.flags = flags.view(8, self.world)
        self.peer_flags = torch.tensor([int(p) for p in fh.buffer_ptrs], dtype=torch.int64, device=device)
        self.epoch = [0, 0, 0, 0, 0]
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def bump(self, ch: int) -> int:
        self.epoch[ch] += 1
        return self.epoch[ch]

    def signal(self, ch: int) -> int:
        from ..ops import kernels as K

        e = self.bump(ch)
        K.ep_signal(self.peer_flags, ch, self.world, self.me, e)
        return e


class _IO:
    """What `_ExpertsOnSorted` needs from the exchange (see its docstring)."""

    def __init__(self, ep: FusedEP, x_epoch: int):
        self.ep, self.x_epoch = ep, x_epoch
        self.dy_epoch = None

    def before_forward(self, in_kernel: bool):
        from ..ops import kernels as K

        if in_kernel:
            return self.ep.flags[CH_X], self.x_epoch
        K.ep_wait(self.ep.flags[CH_X], self.x_epoch)
        return None

    def y_out(self, rows, d):
        return self.ep.bufs["y"][:rows]

    def after_forward(self):
        self.y_epoch = self.ep.signal(CH_Y)

    def before_backward(self, dy):
        from ..ops import kernels as K

        K.ep_wait(self.ep.flags[CH_DY], self.ep.epoch[CH_DY])
        return dy

    def dy_scale(self, rows):
        """The weights of the dy rows, which arrived unscaled: the expert stack applies them."""
        return self.ep.bufs["dys"][:rows]

    def dx_out(self, rows, d):
        return self.ep.bufs["dx"][:rows]

    def after_backward(self):
        self.ep.signal(CH_DX)


class _Dispatch(torch.autograd.Function):
    """Forward: push my rows into the owners' buffers, flag them. Backward: pull the
    owners' dx rows of my picks and sum them per token."""

    @staticmethod
    def forward(ctx, x, ep: FusedEP, r: Route):
        from ..ops import kernels as K

        K.ep_push_rows(x, r.src_token, r.dst_rank, r.dst_row, ep.tables["x"])
        ctx.x_epoch = ep.signal(CH_X)
        ctx.ep, ctx.r, ctx.shape, ctx.dtype = ep, r, x.shape, x.dtype
        rows = int(ep.cap)
        return ep.bufs["x"][:rows]

    @staticmethod
    def backward(ctx, dxs):
        from ..ops import kernels as K

        ep, r = ctx.ep, ctx.r
        dx = K.ep_pull_combine(ep.tables["dx"], r.rank_of, r.row_of, None, ctx.shape[0], ctx.shape[1],
                               ctx.dtype, flags=ep.flags[CH_DX], epoch=ep.epoch[CH_DX])
        return dx, None, None


class _Combine(torch.autograd.Function):
    """Forward: out[t] = Σ_j w[t,j]·y_owner[row(t,j)] read from the owners. Backward:
    dw by a pulled dot product, and w·dout pushed into the owners' dy buffers."""

    @staticmethod
    def forward(ctx, y, weights, ep: FusedEP, r: Route, tokens: int, values_unused: bool = False,
                y_stays: bool = False):
        from ..ops import kernels as K

        w = weights.float().contiguous()
        # the backward takes <dout row, y row> on this rank: y lives in the shared exchange
        # buffer, which the next MoE layer overwrites, so it is copied unless the caller says
        # that the backward runs before anything else uses the buffer (a checkpointed replay)
        ctx.y_rows = None
        if any(ctx.needs_input_grad) and not y_stays:
            ctx.y_rows = y.detach().clone()
        ctx.y_epoch = ep.epoch[CH_Y]
        if values_unused:
            # the replay of a checkpointed block whose last op this is: only the graph is
            # needed, so the rows stay where they are (nothing crosses NVLink)
            out = torch.empty(tokens, ep.d, dtype=y.dtype, device=y.device)
        else:
            out = K.ep_pull_combine(ep.tables["y"], r.rank_of, r.row_of, w, tokens, ep.d, y.dtype,
                                    flags=ep.flags[CH_Y], epoch=ctx.y_epoch)
        ctx.save_for_backward(w)
        ctx.ep, ctx.r, ctx.rows, ctx.wdtype = ep, r, y.shape[0], weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import kernels as K

        (w,) = ctx.saved_tensors
        ep, r = ctx.ep, ctx.r
        dout = dout.contiguous()
        # dout rows go to the owners as they are, each with its weight beside it
        scale = w.reshape(-1)[r.order].contiguous()
        K.ep_push_rows(dout, r.src_token, r.dst_rank, r.dst_row, ep.tables["dy"], row_scale=scale,
                       peer_scale=ep.tables["dys"])
        e_dy = ep.signal(CH_DY)
        # as an owner: <dout row, y row> of every row that arrived here (y is this rank's own
        # output), so that only one scalar per pick crosses NVLink for the router's gradient
        K.ep_wait(ep.flags[CH_DY], e_dy)
        y_rows = ctx.y_rows if ctx.y_rows is not None else ep.bufs["y"][:ctx.rows]
        K.row_dots(ep.bufs["dy"][:ctx.rows], y_rows, ep.bufs["dots"])
        ctx.y_rows = None
        e_dot = ep.signal(CH_DOT)
        dw = K.ep_pull_scalar(ep.tables["dots"], r.rank_of, r.row_of, flags=ep.flags[CH_DOT], epoch=e_dot)
        return ep.bufs["dy"][:ctx.rows], dw.to(ctx.wdtype), None, None, None, None, None


# ====================================================================== library all-to-all
class _A2A(torch.autograd.Function):
    """rows[i] of rank s lands at row dst_row[i] of rank dst_rank[i] (zeros elsewhere);
    the backward sends the gradient rows back. Sizes are read on the host (a sync): this
    is the baseline path."""

    @staticmethod
    def forward(ctx, rows, dst_rank, dst_row, group, cap):
        world = dist.get_world_size(group)
        keep = dst_row >= 0
        send_counts = torch.bincount(dst_rank[keep].long(), minlength=world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        order = torch.argsort(torch.where(keep, dst_rank, torch.full_like(dst_rank, world)).long(), stable=True)
        order = order[: int(keep.sum())]
        send_rows = rows[order].contiguous()
        send_idx = dst_row[order].long().contiguous()
        recv_rows = rows.new_empty(sum(rc), rows.shape[1])
        recv_idx = torch.empty(sum(rc), dtype=torch.long, device=rows.device)
        dist.all_to_all_single(recv_rows, send_rows, rc, sc, group=group)
        dist.all_to_all_single(recv_idx, send_idx, rc, sc, group=group)
        out = rows.new_zeros(cap, rows.shape[1])
        out.index_copy_(0, recv_idx, recv_rows)
        ctx.save_for_backward(order, recv_idx)
        ctx.meta = (group, sc, rc, rows.shape)
        return out

    @staticmethod
    def backward(ctx, dout):
        order, recv_idx = ctx.saved_tensors
        group, sc, rc, shape = ctx.meta
        back = dout[recv_idx].contiguous()
        got = dout.new_empty(sum(sc), shape[1])
        dist.all_to_all_single(got, back, sc, rc, group=group)
        dx = dout.new_zeros(shape)
        dx.index_copy_(0, order, got)
        return dx, None, None, None, None


class _A2ABack(torch.autograd.Function):
    """The inverse exchange: fetch row dst_row[i] of rank dst_rank[i] for each of my picks."""

    @staticmethod
    def forward(ctx, y, dst_rank, dst_row, group, n_picks):
        world = dist.get_world_size(group)
        keep = dst_row >= 0
        send_counts = torch.bincount(dst_rank[keep].long(), minlength=world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        order = torch.argsort(torch.where(keep, dst_rank, torch.full_like(dst_rank, world)).long(), stable=True)
        order = order[: int(keep.sum())]
        want = dst_row[order].long().contiguous()
        asked = torch.empty(sum(rc), dtype=torch.long, device=y.device)
        dist.all_to_all_single(asked, want, rc, sc, group=group)
        reply = y[asked].contiguous()
        got = y.new_empty(sum(sc), y.shape[1])
        dist.all_to_all_single(got, reply, sc, rc, group=group)
        out = y.new_zeros(n_picks, y.shape[1])
        out.index_copy_(0, order, got)
        ctx.save_for_backward(order, asked)
        ctx.meta = (group, sc, rc, y.shape)
        return out

    @staticmethod
    def backward(ctx, dout):
        order, asked = ctx.saved_tensors
        group, sc, rc, shape = ctx.meta
        send = dout[order].contiguous()
        got = dout.new_empty(sum(rc), shape[1])
        dist.all_to_all_single(got, send, rc, sc, group=group)
        dy = dout.new_zeros(shape)
        dy.index_add_(0, asked, got)
        return dy, None, None, None, None


# ====================================================================== the MoE hook
class ExpertParallel:
    """Installed as ``moe.ep``: runs a MoE layer's routed experts across the group."""

    def __init__(self, group, method: str = "fused_ep", capacity: Optional[float] = None):
        self.group = group
        self.method = method if method in ("fused_ep",) else "all_to_all"
        self.capacity = capacity or 1.25
        self.world = dist.get_world_size(group)
        self.fused: dict = {}
        self.dropped = None

    def cap_rows(self, tokens: int, k: int, el: int) -> int:
        rows = int(self.capacity * tokens * k) + el * (ALIGN - 1)
        return -(-rows // ALIGN) * ALIGN

    def __call__(self, moe, x, weights, idx, ctx, fmt):
        c = moe.c
        t, d = x.shape
        k = idx.shape[1]
        el = c.num_experts // self.world
        cap = self.cap_rows(t, k, el)
        r = route(idx, c.num_experts, self.group, cap)
        self.dropped = r.dropped
        ec = c.expert
        kw = dict(act=ec.activation, limit=ec.limit, up_offset=ec.up_offset, fmt=fmt)
        if self.method == "fused_ep" and x.is_cuda:
            key = (d, cap)
            if key not in self.fused:
                self.fused[key] = FusedEP(self.group, x.device, d, cap, x.dtype)
            ep = self.fused[key]
            xs = _Dispatch.apply(x.contiguous(), ep, r)
            io = _IO(ep, ep.epoch[CH_X])
            y = fused.experts_on_sorted(xs, r.offsets, r.counts, moe.experts_gate_up, moe.experts_down,
                                        io=io, **kw)
            return _Combine.apply(y, weights, ep, r, t, bool(getattr(ctx, "tail_values_unused", False)),
                                  bool(getattr(ctx, "exchange_buffers_stay", False)))
        rows = x[r.src_token.long()]
        xs = _A2A.apply(rows, r.dst_rank, r.dst_row, self.group, cap)
        y = fused.experts_on_sorted(xs, r.offsets, r.counts, moe.experts_gate_up, moe.experts_down, **kw)
        picked = _A2ABack.apply(y, r.dst_rank, r.dst_row, self.group, t * k)
        wsorted = weights.reshape(-1)[r.order].unsqueeze(-1)
        out = torch.zeros(t, d, dtype=torch.float32, device=x.device)
        out = out.index_add(0, r.src_token.long(), picked.float() * wsorted.float())
        return out.to(x.dtype)
