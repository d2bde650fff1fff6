"""Microbatches that overlap: each one's forward runs beside the backward of the one before
it, a piece of the model at a time (``methods(interleave=true)``), as a combined 1F1B runs
them without a pipeline.

One after another, a microbatch's collectives each wait on the compute just before them and
nothing runs beside them. Here the model is cut into pieces (the items of its graph, every
pass of a repeat a piece of its own) and a step runs::

    forward of microbatch 0
    for i in 0 .. n-2:
        tick t, for t in 0 .. r-1:   piece t's forward of i+1, piece r-1-t's backward of i
        the loss of i+1
    backward of microbatch n-1

PyTorch is eager, so the schedule is made of two coroutines per pair of microbatches instead
of a traced program: the forward of i+1 pauses in a forward pre-hook at every piece, the
backward of i pauses in a gradient hook at every piece's input, and the scheduler resumes
them in turn, one piece each per tick. The autograd graph is left whole (taps, ports and
auxiliary losses cross pieces as they always do); only the order in which the host issues
the work changes, and it is the same on every rank, so collectives still meet in one order.
On a GPU each microbatch's forward is issued on one of two streams by its parity and
autograd runs a backward op on its forward's stream: the two halves of a tick are queued on
different streams and the device overlaps them. The gradients are the ones a plain
accumulation gives (each parameter receives the microbatches' terms in the same order).

What it does not combine with, and then runs the microbatches one after another with a
warning: parameters gathered by the peer-memory kernels (one staging buffer per unit; the NCCL
gathers run under it), the in-kernel expert exchange (one set of exchange buffers per layer),
block inputs kept in host memory (their prefetch follows one backward at a time), a
pipeline, and the update fused into the backward. Reference: ``train/interleave.py:1-30,209``.
"""

from __future__ import annotations

import threading
from typing import Callable, Optional

import torch
from torch import nn


class Coroutine:
    """`fn` run on a thread that only ever runs while the caller waits for it: `resume` lets
    it run to its next `pause` (or its end) and returns whether it is still alive. What it
    raised is raised by the `resume` that saw it end."""

    def __init__(self, fn: Callable, name: str):
        self.fn = fn
        self.go, self.back = threading.Semaphore(0), threading.Semaphore(0)
        self.alive, self.error, self.result = True, None, None
        self.thread = threading.Thread(target=self._run, name=name, daemon=True)
        self.started = False

    def _run(self) -> None:
        self.go.acquire()
        try:
            self.result = self.fn()
        except BaseException as err:  # noqa: BLE001 - handed to the scheduler
            self.error = err
        finally:
            self.alive = False
            self.back.release()

    def resume(self) -> bool:
        if not self.alive:
            return False
        if not self.started:
            self.started = True
            self.thread.start()
        self.go.release()
        self.back.acquire()
        if self.error is not None:
            error, self.error = self.error, None
            raise error
        return self.alive

    def pause(self) -> None:
        """Called from inside `fn` (on whatever thread runs its hooks): hand the turn back."""
        self.back.release()
        self.go.acquire()

    def finish(self):
        while self.resume():
            pass
        return self.result


def pieces_of(model) -> list:
    """The modules a step is cut at: the items of the model's graph in order, every pass of a
    repeat that sits among them a piece of its own."""
    from ..models.graph import Repeated, Sequence

    graph = model.graph
    if not isinstance(graph, Sequence):
        raise TypeError(f"methods(interleave=true) cuts a model into the items of its graph, which is a "
                        f"{type(graph).__name__}, not a sequence")
    out: list = []
    for item in graph.items:
        out += list(item.items) if isinstance(item, Repeated) else [item]
    return out


def unsupported(trainer) -> Optional[str]:
    """Why this trainer's step cannot be interleaved, or None."""
    par, m = trainer.parallel, trainer.train.methods
    if getattr(trainer, "fuse_optimizer", False):
        return "the update fused into the backward changes parameters a forward in flight reads"
    if par is not None:
        if getattr(par, "pipeline", None) is not None:
            return "a pipeline has its own schedule"
        if par.fsdp is not None and getattr(par.fsdp, "fused_comm", None) is not None:
            return "the peer-memory all-gather keeps one staging buffer per unit"
        if par.expert_group is not None and getattr(m, "moe", "") in ("fused_ep", "nccl_ep"):
            return "the in-kernel expert exchange has one set of buffers per layer"
    from ..models.graph import Repeated

    if any(isinstance(x, Repeated) and x.offload for x in trainer.model.modules()):
        return "block inputs kept in host memory are prefetched for one backward at a time"
    return None


class Interleaved:
    """The schedule of one trainer: hooks on the model's pieces, installed once."""

    def __init__(self, trainer):
        self.trainer = trainer
        self.pieces = pieces_of(trainer.model)
        self.index = {id(m): t for t, m in enumerate(self.pieces)}
        self.forward: Optional[Coroutine] = None      # the forward coroutine that is being gated
        self.forward_thread: Optional[int] = None
        self.marking = None                            # the backward gate of the microbatch whose forward runs
        self.ticks = 0                                 # ticks that ran both halves (for tests and logs)
        for m in self.pieces:
            m.register_forward_pre_hook(self._before_piece)
        self.streams = None
        if trainer.device.type == "cuda":
            self.streams = [torch.cuda.Stream(device=trainer.device) for _ in range(2)]

    # ------------------------------------------------------------------ hooks
    def _before_piece(self, module: nn.Module, args):
        gate = self.marking
        if gate is None or threading.get_ident() != self.forward_thread:
            return None          # not a scheduled forward (an eval, a replay inside a backward)
        t = self.index[id(module)]
        x = args[0] if args else None
        if isinstance(x, torch.Tensor) and x.requires_grad and t > 0:
            # the gradient of a piece's input is ready when the piece's backward is done
            x.register_hook(lambda g, t=t, gate=gate: gate.piece_done(t))
        if self.forward is not None and t > 0:
            self.forward.pause()  # piece t-1's forward is issued: the other half's turn
        return None

    # ------------------------------------------------------------------ one step
    def run(self, micro: list, inv_count, n_micro: int, world: int):
        """All of a step's microbatches; returns (sum of the cross-entropy parts, terms)."""
        tr = self.trainer
        loss_sum = torch.zeros((), dtype=torch.float32, device=tr.device)
        terms: dict = {}
        n, r = len(micro), len(self.pieces)

        def account(parts) -> None:
            nonlocal loss_sum
            loss_sum = loss_sum + (parts.ce_sum * inv_count.squeeze()).detach()
            for name, v in parts.terms.items():
                terms[name] = terms.get(name, 0) + v.float().detach() / n_micro

        def forward(i: int, gate: "_BackwardGate"):
            """Microbatch i's forward and loss, marking its pieces' inputs for `gate`."""
            self.marking, self.forward_thread = gate, threading.get_ident()
            try:
                with self._stream(i):
                    return tr.forward_loss(micro[i], inv_count, n_micro, world)
            finally:
                self.marking = None

        def sync(last: bool):
            return tr.parallel.grad_sync(tr.model, last) if tr.parallel is not None else _null()

        self._fork()
        gate = _BackwardGate()
        loss, parts = forward(0, gate)                       # nothing to run beside it
        account(parts)
        for i in range(n - 1):
            nxt = _BackwardGate()
            back = Coroutine(lambda loss=loss, i=i: self._backward(loss, i), f"bux-backward-{i}")
            gate.coroutine = back
            self.forward = fwd = Coroutine(lambda i=i, nxt=nxt: forward(i + 1, nxt), f"bux-forward-{i + 1}")
            with sync(False):
                for _ in range(r):
                    a = fwd.resume()                         # piece t of i+1 ...
                    b = back.resume()                        # ... beside piece r-1-t of i
                    self.ticks += 1 if (a or b) else 0
                loss, parts = fwd.finish()                   # the loss of i+1
                back.finish()                                # what is left of i's backward (the first piece, the leaves)
            self.forward = None
            account(parts)
            gate = nxt
        gate.coroutine = None
        with sync(True):
            self._backward(loss, n - 1)                      # nothing left to run beside it
        self._join()
        return loss_sum, terms

    def _backward(self, loss, i: int) -> None:
        with self._stream(i):
            loss.backward()

    # ------------------------------------------------------------------ streams (GPU)
    def _stream(self, i: int):
        return torch.cuda.stream(self.streams[i % 2]) if self.streams is not None else _null()

    def _fork(self) -> None:
        if self.streams is not None:
            now = torch.cuda.current_stream(self.trainer.device)
            for s in self.streams:
                s.wait_stream(now)           # the batch, and the parameters the last update wrote

    def _join(self) -> None:
        if self.streams is not None:
            now = torch.cuda.current_stream(self.trainer.device)
            for s in self.streams:
                now.wait_stream(s)           # the optimizer reads gradients both streams wrote


class _BackwardGate:
    """Where one microbatch's backward pauses: after each piece, until its next tick."""

    def __init__(self):
        self.coroutine: Optional[Coroutine] = None

    def piece_done(self, t: int) -> None:
        if self.coroutine is not None and self.coroutine.alive:
            self.coroutine.pause()


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
