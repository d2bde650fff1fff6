"""Context (sequence) parallelism of softmax attention over the ``context`` axis.

Every rank holds ``t / c`` consecutive positions of each row; everything per-position
(norms, MLPs, experts, the loss) runs on those alone. Attention is where positions
meet, by one of (``methods(attention=...)``; reference ``parallel/context.py:406-600``,
``parallel/ring.py:58-190``):

* ``ulysses``: all-to-all [b, t/c, h, d] → [b, t, h/c, d] around a whole-row kernel call
  and back (needs c | kv heads); 4 all-to-alls forward, 4 backward.
* ``gathered``: K and V are all-gathered once; rank r's queries see the keys of chunks
  0..r in one kernel call (the kernel's causal mask with more keys than queries), and the
  backward reduce-scatters dK, dV.
* ``ring``: the blockwise form. K and V blocks are all-gathered once; the queries are
  exchanged into the *zigzag* placement (rank r works on half-chunks r and 2c-1-r, so every
  rank has the same number of (query, key) block pairs under the causal mask); each
  (query half, key block) pair is one kernel call and the partial outputs are merged by
  their log-sum-exp. The backward runs the pairs again with the merged log-sum-exp, which
  makes every pair's dQ, dK, dV exact parts of the whole, then un-zigzags dQ and
  reduce-scatters dK, dV.
* ``auto``: ulysses when c divides the kv heads, else gathered.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out


class _ToHeads(torch.autograd.Function):
    """[b, t/c, h, d] → [b, t, h/c, d]"""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _to_heads(x, group)

    @staticmethod
    def backward(ctx, g):
        return _to_positions(g.contiguous(), ctx.group), None


class _ToPositions(torch.autograd.Function):
    """[b, t, h/c, d] → [b, t/c, h, d]"""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _to_positions(x, group)

    @staticmethod
    def backward(ctx, g):
        return _to_heads(g.contiguous(), ctx.group), None


def _to_heads(x, group):
    c = dist.get_world_size(group)
    b, tl, h, d = x.shape
    # send head-group j to rank j: [c, b, tl, h/c, d]
    send = x.reshape(b, tl, c, h // c, d).permute(2, 0, 1, 3, 4).contiguous()
    got = _a2a(send, group)
    # got[i] = rank i's positions of my heads → concatenate along t
    return got.permute(1, 0, 2, 3, 4).reshape(b, c * tl, h // c, d)


def _to_positions(x, group):
    c = dist.get_world_size(group)
    b, t, hl, d = x.shape
    send = x.reshape(b, c, t // c, hl, d).permute(1, 0, 2, 3, 4).contiguous()
    got = _a2a(send, group)
    # got[j] = my positions of head-group j → concatenate along heads
    return got.permute(1, 2, 0, 3, 4).reshape(b, t // c, c * hl, d)


class _GatherKV(torch.autograd.Function):
    """Local [b, t/c, g, d] → the first (r+1) chunks [b, (r+1)·t/c, g, d]; the backward
    sums every rank's gradient of this rank's chunk (reduce-scatter)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        c, r = dist.get_world_size(group), dist.get_rank(group)
        parts = [torch.empty_like(x) for _ in range(c)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.shape = x.shape
        return torch.cat(parts[: r + 1], dim=1)

    @staticmethod
    def backward(ctx, g):
        c, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        tl = ctx.shape[1]
        full = g.new_zeros(c, *ctx.shape)
        full[: r + 1] = g.reshape(g.shape[0], r + 1, tl, *g.shape[2:]).transpose(0, 1)
        if g.is_cuda:
            mine = torch.empty(ctx.shape, dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(mine, full, group=ctx.group)
        else:
            dist.all_reduce(full, group=ctx.group)
            mine = full[r]
        return mine.contiguous(), None


def method_for(name: str, kv_heads: int, heads: int, world: int) -> str:
    if name in ("auto", "cudnn", "fa4", "tokamax", "xla"):
        return "ulysses" if kv_heads % world == 0 and heads % world == 0 else "gathered"
    if name == "ring":
        return "ring"
    if name in ("gathered", "allgather"):
        return "gathered"
    if name == "ulysses":
        if kv_heads % world or heads % world:
            raise ValueError(f"ulysses needs the context size {world} to divide the heads ({heads}/{kv_heads})")
        return "ulysses"
    raise ValueError(f"methods(attention={name!r}) is not a context-parallel method")


def attend(attention, q, k, v, group, method: str, **kw):
    """`attention(q, k, v, **kw)` is the whole-row kernel call; this wraps it for rows
    split by position over `group`."""
    c = dist.get_world_size(group)
    how = method_for(method, k.shape[2], q.shape[2], c)
    segments = kw.get("segments")
    whole = None
    if segments is not None:
        # packed rows: the document ids of the whole row (every rank holds a run of positions)
        parts = [torch.empty_like(segments) for _ in range(c)]
        dist.all_gather(parts, segments.contiguous(), group=group)
        whole = torch.cat(parts, dim=1)
    if how == "ulysses":
        qh, kh, vh = (_ToHeads.apply(x.contiguous(), group) for x in (q, k, v))
        sinks = kw.get("sinks")
        if sinks is not None:  # this rank's heads
            r, per = dist.get_rank(group), q.shape[2] // c
            kw = dict(kw, sinks=sinks[r * per:(r + 1) * per])
        if whole is not None:  # whole rows of this rank's heads: the kernels' document masks apply as they are
            kw = dict(kw, segments=whole)
        out = attention(qh, kh, vh, **kw)
        return _ToPositions.apply(out.contiguous(), group)
    plain = all(kw.get(name) is None for name in ("window", "sinks", "softcap", "segments"))
    if how == "ring" and plain and q.shape[1] % 2 == 0:
        return _Ring.apply(q.contiguous(), k.contiguous(), v.contiguous(), group, kw.get("scale"))
    kg, vg = _GatherKV.apply(k, group), _GatherKV.apply(v, group)
    if whole is not None:
        # my queries against the gathered keys (those up to my last position): the document ids
        # of my positions and of the keys'
        kw = dict(kw, segments=(segments, whole[:, :kg.shape[1]]))
    return attention(q, kg, vg, **kw)


# ---------------------------------------------------------------------- blockwise ("ring")
def merge_by_lse(outs: list, lses: list) -> tuple:
    """Partial attention outputs over disjoint key sets → the output over their union.
    outs[i]: [b, t, h, d]; lses[i]: [b, h, t] (−inf where a part saw no key)."""
    lse = torch.logsumexp(torch.stack(lses), dim=0)
    out = torch.zeros_like(outs[0], dtype=torch.float32)
    for o, l in zip(outs, lses):
        w = torch.exp(l - lse)
        w = torch.nan_to_num(w, nan=0.0)          # −inf − −inf
        out += o.float() * w.transpose(1, 2).unsqueeze(-1)
    return out.to(outs[0].dtype), lse


def _zigzag_plan(c: int, r: int) -> tuple:
    """Half-chunks are numbered 0..2c-1 along the row; rank r *holds* (2r, 2r+1) and *works
    on* (r, 2c-1-r). Returns (destinations of my two halves, sources of my two work halves)."""
    def worker(g: int) -> int:
        return g if g < c else 2 * c - 1 - g

    return (worker(2 * r), worker(2 * r + 1)), (r // 2, (2 * c - 1 - r) // 2)


def _exchange_halves(x: torch.Tensor, group, to_work: bool) -> torch.Tensor:
    """[b, 2·half, ...] held (contiguous placement) ↔ worked on (zigzag placement)."""
    c, r = dist.get_world_size(group), dist.get_rank(group)
    b, t = x.shape[0], x.shape[1]
    half = t // 2
    dests, sources = _zigzag_plan(c, r)
    lo, hi = x[:, :half].contiguous(), x[:, half:].contiguous()
    got = [None, None]
    if to_work:
        # I send held half i to dests[i]; I receive work half j from sources[j]
        send = [(dests[0], lo, 2 * r), (dests[1], hi, 2 * r + 1)]
        want = [(sources[0], r), (sources[1], 2 * c - 1 - r)]
    else:
        # the inverse: I send work half j back to sources[j]; I receive held half i from dests[i]
        send = [(sources[0], lo, r), (sources[1], hi, 2 * c - 1 - r)]
        want = [(dests[0], 2 * r), (dests[1], 2 * r + 1)]
    # one all-to-all with per-peer piece counts: pieces to a peer go in ascending half-chunk id
    outgoing = {p: [] for p in range(c)}
    for peer, piece, gid in send:
        outgoing[peer].append((gid, piece))
    incoming = {p: [] for p in range(c)}
    for slot, (peer, gid) in enumerate(want):
        incoming[peer].append((gid, slot))
    piece_numel = lo.numel()
    send_buf = torch.cat([piece.reshape(-1) for p in range(c) for _, piece in sorted(outgoing[p], key=lambda e: e[0])])
    in_split = [len(outgoing[p]) * piece_numel for p in range(c)]
    out_split = [len(incoming[p]) * piece_numel for p in range(c)]
    recv_buf = torch.empty(sum(out_split), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv_buf, send_buf, out_split, in_split, group=group)
    at = 0
    for p in range(c):
        for gid, slot in sorted(incoming[p], key=lambda e: e[0]):
            got[slot] = recv_buf[at:at + piece_numel].view(lo.shape)
            at += piece_numel
    return torch.cat(got, dim=1)


def _pair_forward(q, k, v, causal: bool, scale):
    """(out, lse) of one (query half, key block) pair."""
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128):
        from ..ops import kernels as K

        return K.attn_fwd(q, k, v, causal=causal, scale=scale)
    from ..ops import reference as ref

    return ref.attention(q, k, v, causal=causal, scale=scale)


def _pair_backward(q, k, v, o, do, lse, causal: bool, scale):
    """(dq, dk, dv) of one pair given the *merged* output and log-sum-exp of the whole row."""
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128):
        from ..ops import kernels as K

        dq, dk, dv, _ = K.attn_bwd(q, k, v, o, do, lse, causal=causal, scale=scale)
        return dq, dk.float(), dv.float()
    b, t, h, d = q.shape
    s, g = k.shape[1], k.shape[2]
    sc = d ** -0.5 if scale is None else scale
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(h // g, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(h // g, dim=1)
    dof = do.float().transpose(1, 2)
    logits = (qf @ kf.transpose(-1, -2)) * sc
    if causal:
        keep = torch.ones(t, s, dtype=torch.bool, device=q.device).tril(diagonal=s - t)
        logits = logits.masked_fill(~keep, float("-inf"))
    p = torch.nan_to_num(torch.exp(logits - lse.unsqueeze(-1)), nan=0.0)
    delta = (o.float() * do.float()).sum(-1).transpose(1, 2)          # [b, h, t]
    dv = p.transpose(-1, -2) @ dof
    ds = p * (dof @ vf.transpose(-1, -2) - delta.unsqueeze(-1)) * sc
    dq = (ds @ kf).transpose(1, 2)
    dk = ds.transpose(-1, -2) @ qf
    fold = lambda x: x.reshape(b, g, h // g, s, d).sum(2).transpose(1, 2)  # noqa: E731
    return dq, fold(dk), fold(dv)


class _Ring(torch.autograd.Function):
    """Causal attention of rows split by position, blockwise with zigzag placement."""

    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        c, r = dist.get_world_size(group), dist.get_rank(group)
        b, tl, h, d = q.shape
        half = tl // 2
        ks = [torch.empty_like(k) for _ in range(c)]
        vs = [torch.empty_like(v) for _ in range(c)]
        dist.all_gather(ks, k, group=group)
        dist.all_gather(vs, v, group=group)
        # key blocks are half-chunks, in row order
        kb = [part[:, i * half:(i + 1) * half] for part in ks for i in range(2)]
        vb = [part[:, i * half:(i + 1) * half] for part in vs for i in range(2)]
        qz = _exchange_halves(q, group, to_work=True)
        work = (r, 2 * c - 1 - r)
        outs, lses = [], []
        for slot, gid in enumerate(work):
            qh = qz[:, slot * half:(slot + 1) * half].contiguous()
            po, pl = [], []
            for j in range(gid + 1):
                o, lse = _pair_forward(qh, kb[j].contiguous(), vb[j].contiguous(), j == gid, scale)
                po.append(o)
                pl.append(lse)
            o, lse = merge_by_lse(po, pl)
            outs.append(o)
            lses.append(lse)
        oz = torch.cat(outs, dim=1)
        ctx.save_for_backward(qz, torch.stack(kb), torch.stack(vb), oz, torch.stack(lses))
        ctx.group, ctx.scale = group, scale
        return _exchange_halves(oz, group, to_work=False)

    @staticmethod
    def backward(ctx, dout):
        qz, kb, vb, oz, lses = ctx.saved_tensors
        group, scale = ctx.group, ctx.scale
        c, r = dist.get_world_size(group), dist.get_rank(group)
        half = qz.shape[1] // 2
        doz = _exchange_halves(dout.contiguous(), group, to_work=True)
        dk_all = torch.zeros(kb.shape, dtype=torch.float32, device=kb.device)
        dv_all = torch.zeros(vb.shape, dtype=torch.float32, device=vb.device)
        dqs = []
        for slot, gid in enumerate((r, 2 * c - 1 - r)):
            sl = slice(slot * half, (slot + 1) * half)
            qh, oh, doh = qz[:, sl].contiguous(), oz[:, sl].contiguous(), doz[:, sl].contiguous()
            dq = torch.zeros(qh.shape, dtype=torch.float32, device=qh.device)
            for j in range(gid + 1):
                dqj, dkj, dvj = _pair_backward(qh, kb[j].contiguous(), vb[j].contiguous(), oh, doh, lses[slot],
                                               j == gid, scale)
                dq += dqj.float()
                dk_all[j] += dkj
                dv_all[j] += dvj
            dqs.append(dq)
        dq = _exchange_halves(torch.cat(dqs, dim=1).to(qz.dtype), group, to_work=False)
        # key block 2p and 2p+1 belong to rank p: sum over ranks, keep mine
        def mine(full):
            full = full.to(kb.dtype).contiguous()              # [2c, b, half, g, d]
            if full.is_cuda:
                out = torch.empty(2, *full.shape[1:], dtype=full.dtype, device=full.device)
                dist.reduce_scatter_tensor(out, full, group=group)
            else:
                dist.all_reduce(full, group=group)
                out = full[2 * r:2 * r + 2]
            return torch.cat([out[0], out[1]], dim=1)

        return dq, mine(dk_all), mine(dv_all), None, None
