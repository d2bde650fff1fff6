"""The trainer: one step = forward/backward over the rank's microbatches, gradient
reduction, clipping, fused optimizer update; the loop launches step N+1 before it
reads step N's metrics, so the host never waits on the device between steps.

Reference: ``train/trainer.py:447-1649`` (`Trainer`, `train`, `directory`). There the
step is one traced XLA program; here it is explicit CUDA work on streams, and the
gradient paths (whole batch, microbatches reduced once, pipeline-scheduled) are
chosen from ``methods(...)`` by `bux_b200.parallel`.
"""

from __future__ import annotations

import json
import math
import re
import time
from pathlib import Path
from typing import Iterable, Optional

import numpy as np
import torch

from .. import runtime
from ..config import training as T
from ..lang import ir
from ..lang.printer import run_to_source
from ..models import Model, Precision, graph
from . import curriculum, data, objective, optim


def slug(name: str) -> str:
    return re.sub(r"[^A-Za-z0-9_.=+-]+", "_", name).strip("_")


def directory(run: ir.Run, out) -> Path:
    """``<out>/<slug(name)>-<id>/``: where a run writes."""
    return Path(out) / f"{slug(run.name)}-{run.id}"


def pick_device(spec: Optional[str] = None) -> torch.device:
    if spec:
        return torch.device(spec)
    if torch.cuda.is_available():
        return torch.device("cuda", runtime.local_rank())
    return torch.device("cpu")


class KernelWaitError(RuntimeError):
    """A kernel's bounded wait (on a peer's flag, a barrier) ran out during a step."""


class Timers:
    """Host timers of a step's parts, averaged over the steps between two logs."""

    def __init__(self):
        self.sums: dict = {}
        self.count = 0

    def add(self, name: str, seconds: float) -> None:
        self.sums[name] = self.sums.get(name, 0.0) + seconds

    def flush(self) -> dict:
        n = max(self.count, 1)
        out = {f"time/{k}_ms": v / n * 1000 for k, v in self.sums.items()}
        self.sums, self.count = {}, 0
        return out


class Trainer:
    def __init__(self, run: ir.Run, *, device=None, parallel=None, cache=".", seed=None,
                 fuse_optimizer: bool = False, moments: Optional[str] = None,
                 master: Optional[bool] = None):
        self.run, self.train = run, run.train
        t = run.train
        self.device = pick_device(device) if not isinstance(device, torch.device) else device
        self.parallel = parallel
        self.cache = cache
        cuda = self.device.type == "cuda"
        self.compute = torch.bfloat16 if (t.precision.compute == "bfloat16" and cuda) else torch.float32
        self.param_dtype = self.compute
        with parallel.placement(run.arch, self.param_dtype) if parallel is not None else _null():
            self.model = Model(run.arch, dtype=self.param_dtype, seed=t.seed if seed is None else seed,
                               device=self.device)
        if parallel is not None:
            parallel.prepare_model(self.model)
        from ..models.graph import count_outer_branches

        branches = count_outer_branches(self.model.graph)

        def edge(v) -> int:   # a number of branches, or a share of them (rounded up)
            return math.ceil(v * branches) if isinstance(v, float) else int(v)

        self.precision = Precision(compute=self.compute, matmuls=t.precision.matmuls,
                                   roles={k: v for k, v in t.precision.roles.model_dump().items()
                                          if k != "type" and v is not None},
                                   first=edge(t.precision.first), last=edge(t.precision.last),
                                   branches=branches, passes=tuple(t.precision.passes))
        experts_fmt = t.precision.experts()
        if experts_fmt:
            self.precision.roles["experts"] = experts_fmt
        self.model.set_remat(**self.remat_policy(t.methods.remat))
        use_master = (self.param_dtype != torch.float32) if master is None else master
        self.optimizer = optim.Optimizer(
            self.model.named_parameters(), t.optimizer, moments=moments or t.precision.moments,
            master=use_master, clip=t.clip,
            reduce=parallel.sum_scalar if parallel is not None else None,
            norm_weight=parallel.norm_weight if parallel is not None else None,
            shard_group=parallel.fsdp.group if parallel is not None and parallel.fsdp is not None else None,
            orthogonalize=t.methods.orthogonalize)
        self.lr_at = optim.lr_multiplier(t)
        self.step = 0
        self.tokens = 0
        self.stopping = False
        self.fuse_optimizer = fuse_optimizer
        self._pending_factor = None
        self._prev_norm_sq = None
        self._norm_acc = None
        self._hooks_installed = False
        self._status_host = None
        self.observing = None          # None, or {"histograms": bool}: what the next training forward observes
        self.pre_step: list = []       # callables of the number of the step that is about to run
        self.observed: dict = {}
        self.observed_histograms: dict = {}
        self.observed_gradients: dict = {}   # name -> (rms, histogram or None) of an observed step's gradients
        self._prefixes = None
        self._token_bytes = None
        self.stretches = curriculum.stretches(t)
        self._interleave = None        # the schedule of methods(interleave=true), made at the first step
        self.timers = Timers()

    # ------------------------------------------------------------------ setup
    # what the token mixers' names of ``remat(save=...)`` cover
    _MIXER_NAMES = {"attention", "attention.out", "recurrence", "recurrence.out"}

    def remat_policy(self, remat) -> dict:
        """``methods.remat`` → the arguments of `Model.set_remat`. Every pass of a repeat is
        checkpointed as a unit (only its input is kept, the pass is rerun in the backward);
        what a policy can keep on top of that here is the attention outputs:

        * ``none`` keeps everything; ``full`` (and ``dots`` / ``dots_no_batch``, whose finer
          grain — keeping every matmul's output — this framework does not have) keep only the
          passes' inputs; ``auto`` decides by a memory estimate (`bux_b200.train.fitting` by
          trial steps);
        * ``save_attention``, ``save_qkv_attention``, ``dots_attention`` also keep each
          attention's output and log-sum-exp, so the rerun skips the attention forward;
          ``offload_attention`` keeps them, and the passes' inputs, in pinned host memory;
        * ``remat(save=[...], offload=[...], first=N)``: ``attention`` (or ``attention.out``)
          in `save` keeps the attention outputs, in `offload` sends them (and the inputs) to
          the host; `first` checkpoints only the first N passes of each repeat.

        Reference: ``architecture/repeats/remat.py:128-145`` (`PRESETS`, `CANDIDATES`)."""
        if isinstance(remat, str):
            if remat in ("save_attention", "save_qkv_attention", "dots_attention"):
                return {"on": True, "keep_attention": True}
            if remat == "offload_attention":
                return {"on": True, "offload": self.device.type == "cuda", "keep_attention": True,
                        "kept_to_host": self.device.type == "cuda"}
            return {"on": self._remat_on(remat)}
        save = set(remat.save) & self._MIXER_NAMES
        off = set(remat.offload) & self._MIXER_NAMES
        cuda = self.device.type == "cuda"
        return {"on": True, "offload": bool(off) and cuda, "keep_attention": bool(save or off),
                "kept_to_host": bool(off) and cuda, "first": remat.first}

    def _remat_on(self, remat: str) -> bool:
        if remat == "none":
            return False
        if remat != "auto":
            return True
        if self.device.type != "cuda":
            return False
        t = self.train
        world = self.parallel.data_world if self.parallel is not None else 1
        rows = max(1, t.batch // world // t.methods.microbatches)
        layers = sum(1 for _ in self.run.arch.layers())
        est = rows * t.seq_len * self.run.arch.d_model * 2 * 12 * layers  # bytes kept without remat
        free, _ = torch.cuda.mem_get_info(self.device)
        return est > 0.5 * free

    def config_at(self, step: int) -> T.TrainConfig:
        for s in self.stretches:
            if s.start <= step < s.stop:
                return s.config
        return self.stretches[-1].config

    def batches(self, start: Optional[int] = None) -> Iterable:
        rank = self.parallel.data_rank if self.parallel is not None else 0
        world = self.parallel.data_world if self.parallel is not None else 1
        return data.batches(self.train, self.run.arch.vocab_size or 1, self.cache,
                            self.step if start is None else start, False, rank, world)

    # ------------------------------------------------------------------ a step
    def to_device(self, batch: data.Batch):
        def put(a, dtype):
            t = torch.from_numpy(np.ascontiguousarray(a))
            if self.device.type == "cuda":
                t = t.pin_memory().to(self.device, non_blocking=True)
            return t.to(dtype)

        ids, pos, mask = (put(batch.input_ids, torch.long), put(batch.position_ids, torch.long),
                          put(batch.loss_mask, torch.bool))
        # whether any row holds more than one document is read off the host copy (no device
        # sync); the segment ids themselves are formed on the device in `segments_of`
        host_pos = np.asarray(batch.position_ids)
        packed = bool(host_pos.shape[1] > 1 and (host_pos[:, 1:] <= host_pos[:, :-1]).any())
        return _DeviceBatch((ids, pos, mask), packed)

    def forward_loss(self, mb, inv_count, n_micro: int, world: int, training: bool = True):
        ids, pos, mask = mb
        segments = segments_of(pos) if getattr(mb, "packed", False) else None
        span = None
        if self.parallel is not None and self.parallel.context_group is not None:
            # this rank's positions; the loss still sees whole rows for its targets
            span = self.parallel.positions_span(ids.shape[1])
            ids, pos = ids[:, span[0]:span[1]], pos[:, span[0]:span[1]]
            if segments is not None:
                segments = segments[:, span[0]:span[1]]
        sw = self.train.precision.switch
        if sw is not None:   # from that share of the steps on, other GEMMs multiply in the format
            late = self.step >= round(sw.at * self.train.steps)
            self.precision.passes = tuple(sw.passes if late else self.train.precision.passes)
        ctx = self.model(ids, pos, segments, training=training, precision=self.precision,
                         methods=self.train.methods, parallel=self.parallel, step=self.step,
                         observe=self.observing if training else None)
        if ctx.observed or ctx.observed_histograms:   # an observed step: the hook reads them
            self.observed, self.observed_histograms = ctx.observed, ctx.observed_histograms
        parts = objective.compute(ctx, mb, self.train.loss, span=span, prefixes=self.prefix_table(),
                                  progress=self.step / max(1, self.train.steps))
        loss = parts.total_sum * inv_count + parts.per_batch / (n_micro * world)
        if span is not None:  # per-batch terms are reported by every rank of the row
            loss = parts.total_sum * inv_count + parts.per_batch / (n_micro * world * self.parallel.shape["context"])
        return loss, parts

    def train_step(self, batch: data.Batch) -> dict:
        """Run one optimizer step on this rank's rows of `batch`; returns device scalars."""
        t = self.train
        for before in self.pre_step:   # hooks that prepare the step about to run (its number is step + 1)
            before(self.step + 1)
        cfg = self.config_at(self.step)
        n_micro = max(1, min(t.methods.microbatches, batch.input_ids.shape[0]))
        world = self.parallel.data_world if self.parallel is not None else 1
        dev_batch = self.to_device(batch)
        rows = dev_batch[0].shape[0]
        micro = ([_DeviceBatch(tuple(x[i::n_micro] for x in dev_batch), dev_batch.packed) for i in range(n_micro)]
                 if n_micro > 1 else [dev_batch])
        # global number of targets: a device scalar, summed over ranks without a host sync
        count = torch.zeros(1, dtype=torch.float32, device=self.device)
        for mb in micro:
            _, m = objective.targets_and_mask(*mb)
            count += m.sum()
        if self.parallel is not None:
            count = self.parallel.sum_scalar(count, data_only=True)
        inv_count = 1.0 / count.clamp_min(1.0)
        lr_scale = self.lr_at(self.step)
        if self.fuse_optimizer:
            self._install_release_hooks()
            self._release = (lr_scale, self._delayed_clip_factor())
            self.optimizer.step_count += 1
        self.model.train()
        graph._OFFLOADED.clear()
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        terms: dict = {}
        pipe = getattr(self.parallel, "pipeline", None) if self.parallel is not None else None
        if pipe is not None:
            loss_sum, terms = pipe.run(self, micro, inv_count, n_micro, world)
            torch.distributed.all_reduce(loss_sum, group=pipe.group)  # the last stage holds it
        schedule = self._interleaved() if (pipe is None and len(micro) > 1 and t.methods.interleave) else None
        if schedule is not None:
            loss_sum, terms = schedule.run(micro, inv_count, n_micro, world)
        for k, mb in enumerate(micro if (pipe is None and schedule is None) else ()):
            last = k == len(micro) - 1
            sync = self.parallel.grad_sync(self.model, last) if self.parallel is not None else _null()
            with sync:
                loss, parts = self.forward_loss(mb, inv_count, n_micro, world)
                loss.backward()
            loss_sum += parts.ce_sum * inv_count.squeeze()
            for name, v in parts.terms.items():
                terms[name] = terms.get(name, 0) + v.float() / n_micro
        if self.parallel is not None:
            self.parallel.finish_grads(self.model)
        if self.observing is not None:   # an observed step: the gradients' statistics, before the update lets go of them
            from . import observe

            self.observed_gradients = observe.gradient_stats(self, bool(self.observing.get("histograms")))
        if self.fuse_optimizer:
            # parameters whose gradients had to be summed over ranks first are updated now,
            # with the same (delayed) clip factor as the ones updated during the backward
            lr_s, factor = self._release
            for name, p in self.model.named_parameters():
                g = self.optimizer.grad_of(p)
                if g is None or not p.requires_grad:
                    continue
                self._add_norm(g, p.device, self.parallel.norm_weight(name) if self.parallel else 1.0)
                self.optimizer.update_param(name, p, lr_s, 1.0, factor)
            if self._norm_acc is not None and self.parallel is not None:
                self._norm_acc = self.parallel.sum_scalar(self._norm_acc)
            norm = None if self._norm_acc is None else self._norm_acc.sqrt()
            self._prev_norm_sq = self._norm_acc
            self._norm_acc = None
        else:
            norm = self.optimizer.step(lr_scale)
        self.model.step_end_update()
        if self.parallel is not None:
            loss_sum = self.parallel.sum_scalar(loss_sum.view(1), data_only=True).view(())
            loss_sum = self.parallel.sum_positions(loss_sum)
        self.step += 1
        self.tokens += cfg.batch * cfg.seq_len
        self._snapshot_kernel_status()
        base_lr = t.optimizer.lr
        out = {"loss": loss_sum, "lr": base_lr * lr_scale, "tokens": self.tokens}
        if norm is not None:
            out["grad_norm"] = norm
        out.update(terms)
        return out

    def _interleaved(self):
        """The schedule of ``methods(interleave=true)``, or None (with a warning, once) where the
        step cannot be interleaved and its microbatches run one after another."""
        if self._interleave is None:
            from . import interleave

            why = interleave.unsupported(self)
            if why is None:
                try:
                    self._interleave = interleave.Interleaved(self)
                except TypeError as err:
                    why = str(err)
            if why is not None:
                import warnings

                warnings.warn(f"methods(interleave=true): {why}; the microbatches of a step run one after "
                              "another (the same gradients, nothing overlapped)")
                self._interleave = False
        return self._interleave or None

    def prefix_table(self):
        """Each id's prefix token for ``loss(prefix=...)`` (None without it): from the run's
        tokenizer; ids past the tokenizer's vocabulary, or every id without a tokenizer, have none."""
        if self.train.loss.prefix is None:
            return None
        if self._prefixes is None:
            vocab = self.run.arch.vocab_size or 1
            table = torch.full((vocab,), -1, dtype=torch.int64)
            if self.train.tokenizer is not None:
                from ..data import tokenizer as TK

                given = torch.from_numpy(TK.prefix_tokens(TK.load(self.train.tokenizer))).long()
                table[: min(vocab, given.numel())] = given[:vocab]
            self._prefixes = table.to(self.device)
        return self._prefixes

    # ---- the kernels' bounded waits
    def _snapshot_kernel_status(self) -> None:
        """Queue a copy of the device's status word (where a kernel's bounded wait records
        that it ran out) into pinned host memory behind the step's work: reading it later
        costs no synchronisation beyond the one the reader already made for that step."""
        if self.device.type != "cuda":
            return
        from ..ops import kernels as K

        if self._status_host is None:
            self._status_host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self._status_host.copy_(K.status_word(self.device), non_blocking=True)

    def check_kernels(self, what: str = "training step") -> None:
        """Raise on every rank if a bounded device wait ran out on any rank in a step whose
        results the host has already read (the log hook, before a checkpoint is written):
        such a kernel returned without writing its output, so the state is not to be kept."""
        if self._status_host is None:
            return
        code, count = (int(v) for v in self._status_host.tolist())
        bad = 1 if code else 0
        if self.parallel is not None and self.parallel.world > 1:
            bad = self.parallel.max_int(bad)
        if not bad:
            return
        from ..ops import kernels as K

        self.stopping = True
        K.status_word(self.device).zero_()
        self._status_host.zero_()
        where = (f"kernel {code >> 24}, site {(code >> 16) & 0xff}, block {code & 0xffff}; {count} waits in total"
                 if code else "on another rank")
        raise KernelWaitError(f"{what}: a bounded device wait ran out ({where}); the step's results are stale")

    # ---- optimizer fused into the backward (gradients released as they are produced)
    def _install_release_hooks(self) -> None:
        if self._hooks_installed:
            return
        self._hooks_installed = True
        names = {p: n for n, p in self.model.named_parameters()}
        later = {id(p) for p, _ in self.parallel.replicated} if self.parallel is not None else set()

        def hook(p):
            lr_scale, factor = self._release
            g = self.optimizer.grad_of(p)
            if g is not None:
                self._add_norm(g, p.device, 1.0)
            self.optimizer.update_param(names[p], p, lr_scale, 1.0, factor)

        for p in self.model.parameters():
            if p.requires_grad and id(p) not in later:
                p.register_post_accumulate_grad_hook(hook)

    def _add_norm(self, g, device, weight: float) -> None:
        if self.train.clip is None:
            return
        if self._norm_acc is None:
            self._norm_acc = torch.zeros(1, dtype=torch.float32, device=device)
        if weight == 1.0 and g.is_cuda and g.is_contiguous() and g.dtype in (torch.float32, torch.bfloat16):
            from ..ops import kernels as K

            K.sumsq(g, self._norm_acc)
        else:
            self._norm_acc += g.float().square().sum() * weight

    def _delayed_clip_factor(self):
        """With the update fused into the backward the step's own norm is not known
        until its end, so the clip factor comes from the previous step's norm."""
        if self.train.clip is None or self._prev_norm_sq is None:
            return None
        return self.optimizer.clip_factor(self._prev_norm_sq)

    # ------------------------------------------------------------------ eval
    @torch.no_grad()
    def evaluate(self, e: T.EvalConfig) -> dict:
        self.model.eval()
        self.precision.enabled = self.train.precision.eval != "compute"   # eval=compute: no low-precision matmuls
        rank = self.parallel.data_rank if self.parallel is not None else 0
        world = self.parallel.data_world if self.parallel is not None else 1
        nbytes = self.token_bytes()
        sums: dict = {}
        for b in data.eval_batches(self.train, e, self.run.arch.vocab_size or 1, self.cache, rank, world):
            mb = self.to_device(b)
            ctx = self.model(mb[0], mb[1], segments_of(mb[1]) if mb.packed else None, training=False,
                             precision=self.precision,
                             methods=self.train.methods, parallel=self.parallel, step=self.step)
            for name, (total, count) in objective.held_out(ctx, mb, nbytes, e.positions).items():
                acc = sums.setdefault(name, torch.zeros(2, dtype=torch.float32, device=self.device))
                acc[0] += total
                acc[1] += count
        self.model.train()
        self.precision.enabled = True
        out = {}
        for name in sorted(sums):   # every rank in the same order
            acc = sums[name]
            if self.parallel is not None:
                acc = self.parallel.sum_scalar(acc, data_only=True)
            total, count = acc.tolist()
            out[f"{e.name}_{name}"] = total / count if count > 0 else float("nan")
        return out

    def token_bytes(self):
        """The bytes of text each id stands for, for bits per byte (None without a tokenizer)."""
        if self.train.tokenizer is None:
            return None
        if self._token_bytes is None:
            from ..data import tokenizer as TK

            vocab = self.run.arch.vocab_size or 1
            table = torch.zeros(vocab, dtype=torch.int64)
            given = torch.from_numpy(TK.token_bytes(TK.load(self.train.tokenizer))).long()
            table[: min(vocab, given.numel())] = given[:vocab]
            self._token_bytes = table.to(self.device)
        return self._token_bytes

    # ------------------------------------------------------------------ state
    def state(self) -> dict:
        return {"model": self.model.state_dict(), "optimizer": self.optimizer.state_dict(),
                "step": self.step, "tokens": self.tokens}

    def load(self, state: dict) -> None:
        self.model.load_state_dict(state["model"])
        self.optimizer.load_state_dict(state["optimizer"])
        self.step, self.tokens = state["step"], state["tokens"]

    # ------------------------------------------------------------------ the loop
    def fit(self, hooks=(), sinks=()) -> None:
        t = self.train
        feed = data.prefetch(iter(self.batches()), 2)
        for h in hooks:
            h.start(self)
        pending = None  # (step, device scalars) of the step launched last
        while self.step < t.steps and not self.stopping:
            t0 = time.perf_counter()
            batch = next(feed)
            t1 = time.perf_counter()
            scalars = self.train_step(batch)
            t2 = time.perf_counter()
            self.timers.add("data", t1 - t0)
            self.timers.add("launch", t2 - t1)
            self.timers.count += 1
            if pending is not None:
                self._after_step(pending, hooks, sinks)
            pending = (self.step, scalars)
        if pending is not None:
            self._after_step(pending, hooks, sinks, last=True)
        for h in hooks:
            h.stop(self, sinks)
        for s in sinks:
            s.close()

    def _after_step(self, pending, hooks, sinks, last: bool = False) -> None:
        step, scalars = pending
        for h in hooks:
            if h.due(step, self, last=last or step >= self.train.steps):
                t0 = time.perf_counter()
                h(step, scalars, self, sinks)
                self.timers.add("hooks", time.perf_counter() - t0)


class _DeviceBatch(tuple):
    """(input_ids, position_ids, loss_mask) on the device, plus `packed`: whether some row
    holds more than one document (known from the host copy of the positions)."""

    def __new__(cls, parts, packed: bool = False):
        self = super().__new__(cls, parts)
        self.packed = packed
        return self


def segments_of(positions: torch.Tensor) -> torch.Tensor:
    """Document ids (from 1) of every position of packed rows: a document starts at a row's
    first position and wherever the position ids stop increasing (the reference's rule,
    ``architecture/common/segments.py:37`` there). Formed on the device, no host sync."""
    first = torch.ones_like(positions[:, :1], dtype=torch.bool)
    start = torch.cat([first, positions[:, 1:] <= positions[:, :-1]], dim=1)
    return start.long().cumsum(dim=1)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def count_params(arch: ir.Architecture) -> int:
    with torch.device("meta"):
        return Model(arch).num_params()


def train(run: ir.Run, out="runs", cache=".", hooks=None, sinks=None, device=None, parallel=None,
          resume: bool = True, quiet: bool = False) -> Trainer:
    """Train `run` into ``<out>/<name>-<id>/``: writes run.bux, run.json, metrics.jsonl,
    checkpoints; resumes from the latest checkpoint when there is one."""
    from . import hooks as H
    from . import sinks as S

    folder = directory(run, out)
    main = S.is_main_process()
    if main:
        folder.mkdir(parents=True, exist_ok=True)
        (folder / "run.bux").write_text(run_to_source(run))
        (folder / "run.json").write_text(run.model_dump_json(indent=1))
    trainer = Trainer(run, device=device, parallel=parallel, cache=cache)
    t = run.train
    resumed = None
    ckpt = H.Checkpoint(folder, t.checkpoint) if t.checkpoint is not None else None
    if ckpt is not None and resume:
        resumed = ckpt.restore(trainer)
    if sinks is None:
        sinks = [S.Console(run.name, t.steps), S.JSONL(folder, resume_step=resumed)] if not quiet \
            else [S.JSONL(folder, resume_step=resumed)]
    if not any(isinstance(s_, S.LatestMetrics) for s_ in sinks):
        sinks = [*sinks, S.LatestMetrics()]
    if main and not quiet:
        dev = f"{parallel.world if parallel is not None else 1} × {trainer.device.type}"
        n = trainer.model.num_params()
        S.echo(f"{run.name}: {folder}, on {dev}")
        from ..lang.printer import value_to_source

        S.echo(f"{run.name}: {curriculum.si(n)} parameters, {curriculum.summary(t)}, "
               f"{value_to_source(t.optimizer)}, {value_to_source(t.schedule)}")
        S.echo(f"{run.name}: log every {t.log.every}")
    if main and not quiet and t.log.trackers:
        from . import trackers

        sinks = [*sinks, *trackers.build(t.log.trackers, folder, run)]
    all_hooks = [H.Log(t.log, run, trainer)]
    if t.ema is not None:
        from .ema import Ship

        all_hooks.insert(0, Ship(t.ema, t.steps))   # before the eval and the checkpoint read the weights
    if t.observe is not None:
        from .observe import Observe

        all_hooks.append(Observe(t.observe, folder))
    for e in T.evals(t):
        all_hooks.append(H.Eval(e))
    if ckpt is not None:
        all_hooks.append(ckpt)
    if t.profile is not None:
        all_hooks.append(H.Profile(t.profile, folder))
    all_hooks += list(hooks or ())
    trainer.fit(all_hooks, sinks)
    return trainer
