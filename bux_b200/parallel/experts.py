"""Expert parallelism: experts split over the ``expert`` mesh axis, tokens exchanged.

Two methods (``methods(moe=...)``):

* ``fused_ep``: the exchange is done by this library's own kernels over NVLink peer
  memory (symmetric buffers). Dispatch = P2P stores of token rows straight into the
  owner's expert-sorted receive buffer + epoch flags; with MXFP8 experts the rows are
  quantised as they are sent (d e4m3 bytes + d/32 scale bytes per row, the reference's
  wire format, ``parallel/experts.py:326-349`` there) and land as the owner's GEMM operand,
  scale tiles included. Each row's router weight travels beside it and multiplies the
  activation, so the combine = P2P loads of the expert outputs where they were produced,
  summed per token. The backward mirrors it: dout rows are pushed (MXFP8 again), the
  owner's activation backward yields dx rows and one scalar per row for the router weights'
  gradient, and both are pulled. Tokens go in ``methods(moe_chunks=...)`` ranges, each
  range's transfers on a side stream (``methods(moe_stream=true)``) beside the GEMMs of the
  range before it. No NCCL call moves a token; one small all-gather moves the per-expert
  counts.
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
SLOTS = 2  # exchange buffers per kind: a chunk's rows travel while the chunk before it computes


class FusedEP:
    """State of the in-kernel exchange for one MoE shape: symmetric buffers (two slots of
    each kind, so that consecutive token chunks overlap), the peers' base addresses, flag
    rows, epoch counters and the side stream the transfers run on."""

    KINDS = (("x", 2), ("y", 2), ("dy", 2), ("dx", 2))   # [cap, d] bf16 (x, dy: e4m3 bytes in the MXFP8 exchange)
    SCALES = ("xsf", "dysf")                               # [cap, d/32] E8M0 scales of x and dy rows that travel as MXFP8
    SCALARS = ("xw", "dots")                               # [cap] fp32: a row's router weight; its gradient

    def __init__(self, group, device, d: int, cap_rows: int, dtype=torch.bfloat16):
        import torch.distributed._symmetric_memory as symm

        from ..ops import kernels as K

        self.group, self.device, self.d, self.cap = group, device, d, cap_rows
        self.world, self.me = dist.get_world_size(group), dist.get_rank(group)
        name = group.group_name
        # one symmetric allocation, carved into the pieces (every piece starts 256-byte aligned)
        pieces, at = {}, 0
        for key, width in self.KINDS:
            for slot in range(SLOTS):
                pieces[(key, slot)] = (at, cap_rows * d * width)
                at += -(-cap_rows * d * width // 256) * 256
        for key in self.SCALARS:
            for slot in range(SLOTS):
                pieces[(key, slot)] = (at, cap_rows * 4)
                at += -(-cap_rows * 4 // 256) * 256
        sf_size = cap_rows * (d // 32) if d % 128 == 0 else 0   # row-major, as the senders write them
        for key in self.SCALES:
            for slot in range(SLOTS):
                pieces[(key, slot)] = (at, sf_size)
                at += -(-sf_size // 256) * 256
        flags_at = at
        at += 8 * self.world * 4
        heap = symm.empty(at, dtype=torch.uint8, device=device)
        hdl = symm.rendezvous(heap, name)
        heap.zero_()
        bases = [int(p) for p in hdl.buffer_ptrs]
        self.heap = heap
        self.bufs, self.tables = {}, {}
        for (key, slot), (off, size) in pieces.items():
            view = heap[off:off + size]
            if key in self.SCALARS:
                self.bufs[(key, slot)] = view.view(torch.float32)
            elif key in self.SCALES:
                self.bufs[(key, slot)] = view.view(cap_rows, d // 32) if sf_size else view
            else:
                self.bufs[(key, slot)] = view.view(dtype).view(cap_rows, d)
                if key in ("x", "dy"):  # the same memory as the e4m3 rows of the MXFP8 exchange
                    self.bufs[(key + "q", slot)] = view[:cap_rows * d].view(cap_rows, d)
                    self.tables[(key + "q", slot)] = torch.tensor([b + off for b in bases], dtype=torch.int64,
                                                                  device=device)
            self.tables[(key, slot)] = torch.tensor([b + off for b in bases], dtype=torch.int64, device=device)
        # the scale tiles the GEMMs read, made on this rank from the row-major scales that arrived
        self.tiles = {(key, slot): torch.zeros(K.sf_bytes(cap_rows, d), dtype=torch.uint8, device=device)
                      for key in self.SCALES for slot in range(SLOTS)} if sf_size else {}
        self.flags = heap[flags_at:flags_at + 8 * self.world * 4].view(torch.int32).view(8, self.world)
        self.peer_flags = torch.tensor([b + flags_at for b in bases], dtype=torch.int64, device=device)
        self.epoch = [0, 0, 0, 0, 0]
        # Pushes and pulls share one side stream: with a stream each, a chunk's push and the pull of
        # the chunk two before it ran at once and each went slower; two GPUs measured 5.51 s a step
        # on one stream against 5.66 s on two.
        self.send = torch.cuda.Stream(device=device)
        self.recv = self.send
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def signal(self, ch: int) -> int:
        """Publish the channel's next epoch to every peer, after the current stream's work."""
        from ..ops import kernels as K

        self.epoch[ch] += 1
        K.ep_signal(self.peer_flags, ch, self.world, self.me, self.epoch[ch])
        return self.epoch[ch]

    def wait(self, ch: int, epoch: int) -> None:
        """Make the current stream wait (bounded) until every peer has published `epoch`."""
        from ..ops import kernels as K

        K.ep_wait(self.flags[ch], epoch)


def route_chunks(idx: torch.Tensor, num_experts: int, group, cap_rows: int, chunks: int) -> list:
    """`route` for `chunks` equal token ranges at once: one all-gather of every range's
    per-expert counts, then local integer work. Returns one `Route` per range, its token
    indices relative to the range."""
    t = idx.shape[0]
    tc = t // chunks
    world, me = dist.get_world_size(group), dist.get_rank(group)
    el = num_experts // world
    k = idx.shape[1]
    dev = idx.device
    p = tc * k
    flat = idx.reshape(chunks, p)
    order = torch.argsort(flat, dim=1, stable=True)
    counts = torch.zeros(chunks, num_experts, dtype=torch.int32, device=dev)
    counts.scatter_add_(1, flat, torch.ones_like(flat, dtype=torch.int32))
    allc = torch.empty(world, chunks, num_experts, dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(allc.view(-1), counts.view(-1), group=group)
    allc64 = allc.long()
    before_me = allc64[:me].sum(0)                                 # [C, E] rows of earlier sources
    total = allc64.sum(0)                                          # [C, E]
    padded = (total + ALIGN - 1) // ALIGN * ALIGN
    by_owner = padded.view(chunks, world, el)
    base = (by_owner.cumsum(2) - by_owner).reshape(chunks, num_experts)   # start on its owner
    counts64 = counts.long()
    my_start = counts64.cumsum(1) - counts64
    sorted_e = flat.gather(1, order)
    rank_within = torch.arange(p, device=dev).unsqueeze(0) - my_start.gather(1, sorted_e)
    dst_row = base.gather(1, sorted_e) + before_me.gather(1, sorted_e) + rank_within
    dropped = dst_row >= cap_rows
    dst_row = torch.where(dropped, torch.full_like(dst_row, -1), dst_row).to(torch.int32)
    dst_rank = (sorted_e // el).to(torch.int32)
    row_of = torch.empty(chunks, p, dtype=torch.int32, device=dev).scatter_(1, order, dst_row)
    rank_of = torch.empty(chunks, p, dtype=torch.int32, device=dev).scatter_(1, order, dst_rank)
    mine = slice(me * el, (me + 1) * el)
    offsets = torch.zeros(chunks, el + 1, dtype=torch.int64, device=dev)
    offsets[:, :-1] = base[:, mine]
    offsets[:, -1] = base[:, mine][:, -1] + padded[:, mine][:, -1]
    offsets = offsets.clamp(max=cap_rows // ALIGN * ALIGN)
    local_counts = torch.minimum(total[:, mine], offsets[:, 1:] - offsets[:, :-1]).to(torch.int32)
    offsets = offsets.to(torch.int32)
    src_token = (order // k).to(torch.int32)
    n_dropped = dropped.sum(1)
    return [Route(src_token[c], dst_rank[c], dst_row[c], rank_of[c].view(tc, k), row_of[c].view(tc, k),
                  offsets[c], local_counts[c], order[c], n_dropped[c]) for c in range(chunks)]


class _FusedExperts(torch.autograd.Function):
    """One MoE layer's routed experts across the ranks, token chunk by token chunk, the
    exchange on a side stream beside the GEMMs.

    Per chunk: push my rows (and each row's router weight) into the owners' slot, flag;
    the owner waits for every sender's flag, runs up/gate GEMM → weighted activation →
    down GEMM into its output slot, flags; I sum my picks' rows out of the owners' slots.
    The weight multiplies the activation, so the combine is a plain sum and the weight's
    gradient comes out of the activation's backward on the owner (one scalar per row,
    pulled back with dx). The backward mirrors it with the dy / dx slots.

    Pushes and pulls run on one side stream. Slot reuse is safe by construction: before a rank pushes chunk c + 2 into the input
    slot that chunk c used, the side stream waits for *every* owner's "output ready" flag of
    chunk c, which an owner raises after it has read the slot's input rows; and the flag of
    that push is raised only after the rank's own pull of chunk c has finished, so an owner,
    which overwrites an output slot only once every sender's next push into the matching
    input slot is flagged, never writes over rows that are still being pulled."""

    @staticmethod
    def forward(ctx, x, weights, w_gu, w_down, ep: FusedEP, routes, act, limit, up_offset, mx,
                values_unused, side_stream):
        from ..ops import kernels as K

        t, d = x.shape
        e, f2, _ = w_gu.shape
        f = f2 // 2
        chunks = len(routes)
        tc = t // chunks
        kind = K.KIND_MXFP8 if mx else K.KIND_BF16
        grad = any(ctx.needs_input_grad)
        main = torch.cuda.current_stream(x.device)
        send, recv = (ep.send, ep.recv) if side_stream else (main, main)
        wts = weights.float().contiguous()
        out = torch.empty(t, d, dtype=x.dtype, device=x.device)
        cap = ep.cap
        if mx:
            gq, gsf, gtq, gtsf = K.quant_mxfp8_batched(w_gu.detach(), rowwise=True, colwise=grad)
            dq, dsf, dtq, dtsf = K.quant_mxfp8_batched(w_down.detach(), rowwise=True, colwise=grad)
        send.wait_stream(main)
        recv.wait_stream(main)
        x_epoch, y_epoch, pulled, saved = {}, {}, {}, []

        def push(c):
            r = routes[c]
            with torch.cuda.stream(send):
                slot = c % SLOTS
                if c >= SLOTS:  # every owner has read what the input slot held
                    ep.wait(CH_Y, y_epoch[c - SLOTS])
                if mx:  # rows leave as e4m3 bytes + E8M0 scales, straight into the owner's GEMM operand
                    K.ep_push_rows_mx(x[c * tc:(c + 1) * tc], r.rank_of, r.row_of, ep.tables[("xq", slot)],
                                      ep.tables[("xsf", slot)], weights=wts[c * tc:(c + 1) * tc],
                                      peer_scale=ep.tables[("xw", slot)])
                else:
                    scale = wts[c * tc:(c + 1) * tc].reshape(-1)[r.order].contiguous()
                    K.ep_push_rows(x[c * tc:(c + 1) * tc], r.src_token, r.dst_rank, r.dst_row, ep.tables[("x", slot)],
                                   row_scale=scale, peer_scale=ep.tables[("xw", slot)])
                if c >= SLOTS and side_stream:  # my own pull of the output slot's old rows is done
                    send.wait_event(pulled[c - SLOTS])
                x_epoch[c] = ep.signal(CH_X)

        def compute(c):
            r, slot = routes[c], c % SLOTS
            ep.wait(CH_X, x_epoch[c])
            w_row = ep.bufs[("xw", slot)][:cap]
            y_out = ep.bufs[("y", slot)]
            xtq = xtsf = None
            if mx:
                # what arrived is the GEMM's operand already; padding rows are cleared (zero bytes)
                xq = ep.bufs[("xq", slot)]
                xsf = K.sf_rows_to_tiles(ep.bufs[("xsf", slot)], out=ep.tiles[("xsf", slot)])
                K.zero_pad_rows(xq.view(torch.bfloat16), r.offsets, r.counts)
                h = K.grouped_gemm(xq, gq, r.offsets, f2, d, kind=kind, asf=xsf, bsf=gsf)
                if grad:  # the transposed copy for the weight gradient, before the slot is reused
                    xtq, xtsf = K.requant_mxfp8_cols(xq, xsf, cap, d)
                aq, asf, _, _ = K.quant_mxfp8_glu(h, None, act, limit=limit, up_offset=up_offset, row_scale=w_row)
                K.grouped_gemm(aq, dq, r.offsets, d, f, kind=kind, asf=asf, bsf=dsf, out=y_out)
            else:
                xs = ep.bufs[("x", slot)]
                K.zero_pad_rows(xs, r.offsets, r.counts)
                h = K.grouped_gemm(xs, w_gu.view(e * f2, d), r.offsets, f2, d)
                a = K.glu_fwd(h, act, w_row, limit, up_offset)
                K.grouped_gemm(a, w_down.view(e * d, f), r.offsets, d, f, out=y_out)
            y_epoch[c] = ep.signal(CH_Y)
            if grad:
                saved.append((h, xtq if mx else xs.clone(), xtsf, w_row.clone()))

        def pull(c):
            r = routes[c]
            with torch.cuda.stream(recv):
                ep.wait(CH_Y, y_epoch[c])
                if not values_unused:
                    K.ep_pull_combine(ep.tables[("y", c % SLOTS)], r.rank_of, r.row_of, None, tc, d, x.dtype,
                                      out=out[c * tc:(c + 1) * tc])
                if side_stream:
                    pulled[c] = torch.cuda.Event()
                    pulled[c].record(recv)

        for c in range(min(SLOTS, chunks)):
            push(c)
        for c in range(chunks):
            compute(c)
            pull(c)
            if c + SLOTS < chunks:
                push(c + SLOTS)
        main.wait_stream(send)
        main.wait_stream(recv)
        ctx.save_for_backward(x, w_gu, w_down)
        ctx.held = (saved, (gtq, gtsf, dtq, dtsf) if mx and grad else None)
        ctx.cfg = (ep, routes, act, limit, up_offset, mx, side_stream, weights.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import kernels as K

        x, w_gu, w_down = ctx.saved_tensors
        ep, routes, act, limit, up_offset, mx, side_stream, w_dtype = ctx.cfg
        saved, wq = ctx.held
        ctx.held = None
        t, d = x.shape
        e, f2, _ = w_gu.shape
        f = f2 // 2
        chunks = len(routes)
        tc = t // chunks
        k = routes[0].row_of.shape[1]
        kind = K.KIND_MXFP8 if mx else K.KIND_BF16
        main = torch.cuda.current_stream(x.device)
        send, recv = (ep.send, ep.recv) if side_stream else (main, main)
        dout = dout.contiguous()
        cap = ep.cap
        g_gu = getattr(w_gu, "main_grad", None)
        g_down = getattr(w_down, "main_grad", None)
        # the first chunk's GEMMs write the weight gradients in the dtype they are kept in; the
        # later chunks' add into them
        acc = {"gu": g_gu, "down": g_down}
        if mx:
            gtq, gtsf, dtq, dtsf = wq
        dx = torch.empty_like(x)
        dw = torch.empty(t, k, dtype=torch.float32, device=x.device)
        send.wait_stream(main)
        recv.wait_stream(main)
        dy_epoch, dx_epoch, pulled = {}, {}, {}
        result = {}

        def push(c):
            r = routes[c]
            with torch.cuda.stream(send):
                if c >= SLOTS:  # every owner has read what the dy slot held
                    ep.wait(CH_DX, dx_epoch[c - SLOTS])
                if mx:
                    K.ep_push_rows_mx(dout[c * tc:(c + 1) * tc], r.rank_of, r.row_of, ep.tables[("dyq", c % SLOTS)],
                                      ep.tables[("dysf", c % SLOTS)])
                else:
                    K.ep_push_rows(dout[c * tc:(c + 1) * tc], r.src_token, r.dst_rank, r.dst_row,
                                   ep.tables[("dy", c % SLOTS)])
                if c >= SLOTS and side_stream:  # my own pull of the dx slot's old rows is done
                    send.wait_event(pulled[c - SLOTS])
                dy_epoch[c] = ep.signal(CH_DY)

        def compute(c):
            r, slot = routes[c], c % SLOTS
            h, xsave, xtsf, w_row = saved[c]
            saved[c] = None
            ep.wait(CH_DY, dy_epoch[c])
            dots = ep.bufs[("dots", slot)][:cap]
            dx_out = ep.bufs[("dx", slot)]
            if mx:
                dyq = ep.bufs[("dyq", slot)]
                dysf = K.sf_rows_to_tiles(ep.bufs[("dysf", slot)], out=ep.tiles[("dysf", slot)])
                K.zero_pad_rows(dyq.view(torch.bfloat16), r.offsets, r.counts)
                dytq, dytsf = K.requant_mxfp8_cols(dyq, dysf, cap, d)
                _, _, atq, atsf = K.quant_mxfp8_glu(h, None, act, rowwise=False, colwise=True, limit=limit,
                                                    up_offset=up_offset, row_scale=w_row)
                result["down"] = acc["down"] = K.grouped_gemm_k(
                    dytq, atq, r.offsets, d, f, kind=kind, asf=dytsf, bsf=atsf, out=acc["down"],
                    accumulate=acc["down"] is not None, out_dtype=fused._grad_dtype(w_down))
                del dytq, dytsf, atq, atsf
                da = K.grouped_gemm(dyq, dtq, r.offsets, f, d, kind=kind, asf=dysf, bsf=dtsf)
            else:
                dy = ep.bufs[("dy", slot)]
                K.zero_pad_rows(dy, r.offsets, r.counts)
                a = K.glu_fwd(h, act, w_row, limit, up_offset)
                result["down"] = acc["down"] = K.grouped_gemm_k(
                    dy, a, r.offsets, d, f, a_mn=True, b_mn=True, out=acc["down"],
                    accumulate=acc["down"] is not None, out_dtype=fused._grad_dtype(w_down))
                da = K.grouped_gemm(dy, w_down.view(e * d, f), r.offsets, f, d, b_mn=True)
                del a
            # dh, and <da', glu(h)> per row (the router weight's gradient) straight into the slot
            dh = K.glu_bwd_into(h, da, act, w_row, dots, limit, up_offset)
            del da, h
            if mx:
                hq, hsf, htq, htsf = K.quant_mxfp8(dh, rowwise=True, colwise=True)
                del dh
                result["gu"] = acc["gu"] = K.grouped_gemm_k(
                    htq, xsave, r.offsets, f2, d, kind=kind, asf=htsf, bsf=xtsf, out=acc["gu"],
                    accumulate=acc["gu"] is not None, out_dtype=fused._grad_dtype(w_gu))
                del htq, htsf
                K.grouped_gemm(hq, gtq, r.offsets, d, f2, kind=kind, asf=hsf, bsf=gtsf, out=dx_out)
            else:
                result["gu"] = acc["gu"] = K.grouped_gemm_k(
                    dh, xsave, r.offsets, f2, d, a_mn=True, b_mn=True, out=acc["gu"],
                    accumulate=acc["gu"] is not None, out_dtype=fused._grad_dtype(w_gu))
                K.grouped_gemm(dh, w_gu.view(e * f2, d), r.offsets, d, f2, b_mn=True, out=dx_out)
            dx_epoch[c] = ep.signal(CH_DX)

        def pull(c):
            r = routes[c]
            with torch.cuda.stream(recv):
                ep.wait(CH_DX, dx_epoch[c])
                K.ep_pull_combine(ep.tables[("dx", c % SLOTS)], r.rank_of, r.row_of, None, tc, d, x.dtype,
                                  out=dx[c * tc:(c + 1) * tc])
                K.ep_pull_scalar(ep.tables[("dots", c % SLOTS)], r.rank_of, r.row_of, out=dw[c * tc:(c + 1) * tc])
                if side_stream:
                    pulled[c] = torch.cuda.Event()
                    pulled[c].record(recv)

        for c in range(min(SLOTS, chunks)):
            push(c)
        for c in range(chunks):
            compute(c)
            pull(c)
            if c + SLOTS < chunks:
                push(c + SLOTS)
        main.wait_stream(send)
        main.wait_stream(recv)
        gw_gu = None if g_gu is not None else result["gu"].to(w_gu.dtype)
        gw_down = None if g_down is not None else result["down"].to(w_down.dtype)
        return dx, dw.to(w_dtype), gw_gu, gw_down, None, None, None, None, None, None, None, None


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
        # `nccl_ep` is the reference's name for its in-kernel exchange: a file written for it takes
        # this package's counterpart; every other method over the expert axis takes the library all-to-all
        self.method = "fused_ep" if method in ("fused_ep", "nccl_ep") else "all_to_all"
        if self.method == "fused_ep":
            from .. import runtime

            if not runtime.on_one_node(group):
                # the in-kernel exchange stores into the peers' memory over NVLink: one machine only
                import warnings

                warnings.warn("methods(moe=fused_ep): the expert axis spans machines; taking moe=all_to_all (NCCL)")
                self.method = "all_to_all"
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
        ec = c.expert
        kw = dict(act=ec.activation, limit=ec.limit, up_offset=ec.up_offset, fmt=fmt)
        if self.method == "fused_ep" and x.is_cuda:
            return self._fused(moe, x, weights, idx, ctx, kw)
        r = route(idx, c.num_experts, self.group, cap)
        self.dropped = r.dropped
        rows = x[r.src_token.long()]
        xs = _A2A.apply(rows, r.dst_rank, r.dst_row, self.group, cap)
        y = fused.experts_on_sorted(xs, r.offsets, r.counts, moe.experts_gate_up, moe.experts_down, **kw)
        picked = _A2ABack.apply(y, r.dst_rank, r.dst_row, self.group, t * k)
        wsorted = weights.reshape(-1)[r.order].unsqueeze(-1)
        out = torch.zeros(t, d, dtype=torch.float32, device=x.device)
        out = out.index_add(0, r.src_token.long(), picked.float() * wsorted.float())
        return out.to(x.dtype)

    def _fused(self, moe, x, weights, idx, ctx, kw):
        """The in-kernel exchange: tokens in ``methods(moe_chunks=...)`` equal ranges, the
        transfers on a side stream with ``methods(moe_stream=true)``."""
        c = moe.c
        t, d = x.shape
        k = idx.shape[1]
        el = c.num_experts // self.world
        methods = getattr(ctx, "methods", None)
        chunks = max(1, int(getattr(methods, "moe_chunks", 1) or 1))
        if t % chunks:
            chunks = 1
        cap = self.cap_rows(t // chunks, k, el)
        key = (d, cap)
        if key not in self.fused:
            self.fused[key] = FusedEP(self.group, x.device, d, cap, x.dtype)
        ep = self.fused[key]
        routes = route_chunks(idx, c.num_experts, self.group, cap, chunks)
        self.dropped = sum(r.dropped for r in routes)
        f = moe.experts_down.shape[-1]
        mx = kw["fmt"] in ("mxfp8", "mxfp8_2d") and d % 128 == 0 and f % 128 == 0
        return _FusedExperts.apply(x.contiguous(), weights, moe.experts_gate_up, moe.experts_down, ep, routes,
                                   kw["act"], float(kw["limit"] or 0.0), float(kw["up_offset"]), mx,
                                   bool(getattr(ctx, "tail_values_unused", False)),
                                   bool(getattr(methods, "moe_stream", False)))
