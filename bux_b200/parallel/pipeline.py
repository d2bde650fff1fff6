"""Pipeline parallelism over the ``stage`` axis.

Only the architecture's top-level repeat pipelines: its blocks are split into
contiguous, FLOP-balanced shares (``methods(stages=[...])`` overrides them); what comes
before the repeat (embedding) runs on the first stage, what comes after (final norm,
head, loss) on the last (reference: ``parallel/pipeline.py:87-203``,
``train/stages.py:40``). A rank drops the parameters of the stages it does not run.
A step follows a schedule table (`schedule.TABLES`: gpipe, 1f1b, zbh1): activations go
to the next stage and gradients to the previous one by point-to-point sends on the
``stage`` group (NCCL send/recv on GPUs), sends asynchronous so a forward send never
blocks against the neighbour's backward send.
"""

from __future__ import annotations


import torch
import torch.distributed as dist
from torch import nn

from . import schedule as S


def shares(weights: list, stages: int, first_extra: float = 0.0, last_extra: float = 0.0) -> list:
    """Contiguous split of `weights` (cost per block) into `stages` parts whose largest
    cost, counting the extras of the first and last stage, is smallest."""
    n = len(weights)
    if stages > n:
        raise ValueError(f"{stages} stages need at least {stages} blocks, the repeat has {n}")
    prefix = [0.0]
    for w in weights:
        prefix.append(prefix[-1] + w)

    def cost(i, j, s):
        c = prefix[j] - prefix[i]
        if s == 0:
            c += first_extra
        if s == stages - 1:
            c += last_extra
        return c

    best = {(0, 0): (0.0, [])}
    for s in range(stages):
        nxt = {}
        for (i, _), (worst, cuts) in best.items():
            for j in range(i + 1, n - (stages - 1 - s) + 1):
                if s == stages - 1 and j != n:
                    continue
                w = max(worst, cost(i, j, s))
                if (j, 0) not in nxt or w < nxt[(j, 0)][0]:
                    nxt[(j, 0)] = (w, cuts + [j - i])
        best = nxt
    return best[(n, 0)][1]


class _Skip(nn.Module):
    """Stands where another stage's module was."""

    def forward(self, x, ctx=None):
        return x


class Pipeline:
    def __init__(self, model: nn.Module, par):
        from ..models.graph import Repeated, Sequence
        from ..models.layers.basic import Head

        self.par = par
        self.group = par.stage_group
        self.stages = par.shape["stage"]
        self.stage = par.coords["stage"]
        t = par.train
        graph = model.graph
        if not isinstance(graph, Sequence):
            raise ValueError("pipeline: the model must be a sequence with a repeated block")
        where = [i for i, m in enumerate(graph.items) if isinstance(m, Repeated)]
        if len(where) != 1:
            raise ValueError("pipeline: exactly one repeat outside any branch can pipeline")
        (r,) = where
        self.pre, self.repeat, self.post = list(graph.items[:r]), graph.items[r], list(graph.items[r + 1:])
        for m in model.modules():
            if isinstance(m, Head) and getattr(m, "tied_to", None) is not None:
                raise NotImplementedError("pipeline: a tied head would share a table between the first "
                                          "and the last stage; use head(tied=false)")
        blocks = list(self.repeat.items)
        if t.methods.stages:
            split = list(t.methods.stages)
            if len(split) != self.stages or sum(split) != len(blocks):
                raise ValueError(f"methods(stages={split}) must list {self.stages} shares of {len(blocks)} blocks")
        else:
            cost = [float(sum(p.numel() for p in b.parameters())) for b in blocks]
            first = float(sum(p.numel() for m in self.pre for p in m.parameters())) * 0.0
            last = float(sum(p.numel() for m in self.post for p in m.parameters()))
            split = shares(cost, self.stages, first, last)
        self.split = split
        lo = sum(split[: self.stage])
        self.mine = blocks[lo: lo + split[self.stage]]
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        # what other stages run becomes a parameterless pass-through, so the parameters
        # this stage keeps have the same paths as in the whole model
        keep = set(range(lo, lo + split[self.stage]))
        for i in range(len(blocks)):
            if i not in keep:
                self.repeat.items[i] = _Skip()
        for i in range(len(graph.items)):
            if (i < r and not self.first) or (i > r and not self.last):
                graph.items[i] = _Skip()
        self.table = S.TABLES[t.methods.pipeline](self.stages, max(1, t.methods.microbatches))[self.stage]
        self.ranks = [dist.get_global_rank(self.group, i) for i in range(self.stages)]
        self._pair_groups()

    def _pair_groups(self) -> None:
        """One communicator per pair of neighbouring stages and per direction. NCCL matches
        the point-to-point operations of a pair in the order each side issued them, and a
        send waits on the device for its receive: with activations and gradients on one
        communicator, 1F1B makes both stages send at once (stage s its next activation,
        stage s+1 its first input gradient) and neither receive is ever posted. On their own
        communicators each direction is a plain sequence of sends on one side and receives
        on the other, in the same order. Every rank creates every group (a collective)."""
        everyone = [None] * dist.get_world_size()
        dist.all_gather_object(everyone, tuple(self.ranks))
        self.fwd_next = self.fwd_prev = self.bwd_next = self.bwd_prev = None
        me = dist.get_rank()
        for ranks in sorted(set(everyone)):
            for a, b in zip(ranks[:-1], ranks[1:]):
                fwd = dist.new_group([a, b])
                bwd = dist.new_group([a, b])
                if me == a:
                    self.fwd_next, self.bwd_next = fwd, bwd
                if me == b:
                    self.fwd_prev, self.bwd_prev = fwd, bwd

    # ------------------------------------------------------------------ one step
    def run(self, trainer, micro: list, inv_count, n_micro: int, world: int):
        """Run the schedule over `micro` (every stage holds the same rows). Returns
        (sum of the cross-entropy parts, terms) on the last stage, zeros elsewhere."""
        from ..models.registry import Context
        from ..train import objective

        model, dev = trainer.model, trainer.device
        d = trainer.run.arch.d_model
        dtype = trainer.compute
        held: dict = {}
        sends: list = []
        loss_sum = torch.zeros((), dtype=torch.float32, device=dev)
        terms: dict = {}
        nxt = self.ranks[self.stage + 1] if not self.last else None
        prv = self.ranks[self.stage - 1] if not self.first else None
        for op, m in self.table:
            ids, pos, mask = micro[m]
            if op == "F":
                segments = None
                if getattr(micro[m], "packed", False):
                    from ..train.trainer import segments_of

                    segments = segments_of(pos)
                ctx = Context(ids, pos, segments, training=True, precision=trainer.precision,
                              methods=trainer.train.methods, parallel=trainer.parallel, step=trainer.step)
                if self.first:
                    x = ids
                    for layer in self.pre:
                        x = layer(x, ctx)
                    x_in = None
                else:
                    x_in = torch.empty(ids.shape[0], ids.shape[1], d, dtype=dtype, device=dev)
                    dist.recv(x_in, src=prv, group=self.fwd_prev)
                    x_in.requires_grad_(True)
                    x = x_in
                x = self.repeat(x, ctx)
                if self.last:
                    for layer in self.post:
                        x = layer(x, ctx)
                    parts = objective.compute(ctx, micro[m], trainer.train.loss)
                    loss = parts.total_sum * inv_count + parts.per_batch / (n_micro * world)
                    loss_sum += (parts.ce_sum * inv_count.squeeze()).detach()
                    for name, v in parts.terms.items():
                        terms[name] = terms.get(name, 0) + v.float().detach() / n_micro
                    held[m] = (x_in, loss, None)
                else:
                    y = x.contiguous()
                    sends.append(dist.isend(y.detach(), dst=nxt, group=self.fwd_next))
                    aux = [v for v in ctx.losses.values()]
                    held[m] = (x_in, y, aux)
            elif op == "B":
                x_in, out, aux = held.pop(m)
                if self.last:
                    out.backward()
                else:
                    dy = torch.empty_like(out)
                    dist.recv(dy, src=nxt, group=self.bwd_next)
                    outs, grads = [out], [dy]
                    for a in aux or ():
                        if a.requires_grad:  # auxiliary losses of this stage's layers
                            outs.append(a / (n_micro * world))
                            grads.append(torch.ones_like(a))
                    torch.autograd.backward(outs, grads)
                if x_in is not None:
                    sends.append(dist.isend(x_in.grad.contiguous(), dst=prv, group=self.bwd_prev))
            # "W": the weight gradients were produced with the input gradients (autograd
            # does not split a block's backward), so the slot is a no-op here
        for h in sends:
            h.wait()
        return loss_sum, terms

    # ------------------------------------------------------------------ checkpoints
    def gather_tree(self, tree: dict) -> dict:
        """The union of the stages' trees on the first stage (paths are the whole model's)."""
        cpu = {k: {n: (v.cpu() if isinstance(v, torch.Tensor) else v) for n, v in part.items()}
               for k, part in tree.items()}
        got = [None] * self.stages if self.first else None
        dist.gather_object(cpu, got, dst=self.ranks[0], group=self.group)
        if not self.first:
            return tree
        for other in got[1:]:
            for k, part in other.items():
                for n, v in part.items():
                    tree[k].setdefault(n, v)
        return tree
