"""Learning-rate schedules and optimizers (AdamW, Muon, NorMuon).

Schedules are plain host-side functions ``step -> multiplier`` (the step's learning
rate is a kernel argument, nothing is traced). The multiplier is the warmup ramp
``min((step+1)/warmup, 1)`` times the schedule's curve (reference:
``train/optim.py:86-245``).

`Optimizer` owns per-parameter state and updates with the fused sm_100a AdamW kernel
on CUDA (fp32 / bf16 / block-scaled 8-bit moments, fp32 master with a bf16 shadow
write) or a plain PyTorch statement on CPU. Gradient clipping uses one fused
sum-of-squares per tensor into a single device scalar, reduced across ranks once;
the clip factor reaches the update kernels as a device pointer (no host sync).
Muon orthogonalises 2-D hidden matrices by Newton–Schulz (`newton_schulz`).
"""

from __future__ import annotations

import math
from typing import Callable, Iterable, Optional

import torch

from ..config import training as T
from . import curriculum

# ------------------------------------------------------------------ schedules
_E1 = math.exp(-1)
SHAPES: dict = {
    "linear": lambda t: 1 - t,
    "sqrt": lambda t: 1 - math.sqrt(t),
    "cosine": lambda t: 0.5 * (1 + math.cos(math.pi * t)),
    "exp": lambda t: (math.exp(-t) - _E1) / (1 - _E1),
    "constant": lambda t: 0.0 if t > 0 else 1.0,
}


def _through(step: float, start: int, length: int) -> float:
    return min(max((step + 1 - start) / max(length, 1), 0.0), 1.0)


def _toward(start: float, end: float, shape: str, t: float) -> float:
    if shape == "geometric":
        return start * (end / start) ** t
    return end + (start - end) * SHAPES[shape](t)


def schedule_curve(c, train: T.TrainConfig) -> Callable:
    steps = train.steps
    if isinstance(c, T.ConstantSchedule):
        return lambda step: 1.0
    if isinstance(c, T.CosineSchedule):
        warm = T.warmup_steps(c, steps)
        length = round(c.horizon * steps) - warm
        return lambda step: _toward(1.0, c.final, "cosine", _through(step, warm, length))
    if isinstance(c, T.WSDSchedule):
        cool = c.cooldown(steps)
        return lambda step: _toward(1.0, c.final, c.shape, _through(step, steps - cool, cool))
    if isinstance(c, T.LinearDecaySchedule):
        warm = T.warmup_steps(c, steps)
        return lambda step: _toward(1.0, c.final, "linear", _through(step, warm, steps - warm))
    if isinstance(c, T.MultiStepSchedule):
        drops = [round(a * steps) for a in c.at]
        return lambda step: c.factor ** sum(step >= d for d in drops)
    if isinstance(c, T.PowerSchedule):
        cool = c.cooldown(steps)
        start, warm = steps - cool, T.warmup_steps(c, steps)
        parts = curriculum.stretches(train)
        each = [s.config.batch * s.config.seq_len for s in parts]
        before, total = [], 0
        for s, n in zip(parts, each):
            before.append(total)
            total += (s.stop - s.start) * n
        firsts = [s.start for s in parts]

        def power(step: float) -> float:
            step = min(max(step, warm - 1), start - 1)
            k = max(0, sum(f <= step for f in firsts) - 1)
            n = before[k] + (step - firsts[k] + 1) * each[k]
            return min(c.a * parts[k].config.batch * max(n, 1) ** c.b / train.optimizer.lr, 1.0)

        return lambda step: power(step) * _toward(1.0, c.final, c.shape, _through(step, start, cool))
    if isinstance(c, T.PiecewiseSchedule):
        ends = [round(p.until * steps) for p in c.pieces]
        starts = [T.warmup_steps(c, steps), *ends[:-1]]
        values = T.levels(c.pieces)

        def curve(step: float) -> float:
            found = None
            for k, (p, b, e) in enumerate(zip(c.pieces, starts, ends)):
                if found is None or step >= b:
                    found = _toward(values[k], values[k + 1], p.shape, _through(step, b, e - b))
            return found

        return curve
    raise ValueError(f"unknown schedule {c!r}")


def lr_multiplier(train: T.TrainConfig) -> Callable:
    curve = schedule_curve(train.schedule, train)
    warm = T.warmup_steps(train.schedule, train.steps)

    def multiplier(step: int) -> float:
        ramp = min((step + 1) / warm, 1.0) if warm else 1.0
        return ramp * curve(step)

    return multiplier


# ------------------------------------------------------------------ Newton–Schulz
NS_COEFFICIENTS = {
    "jordan": ((3.4445, -4.7750, 2.0315),),
    # Polar Express (Amsel et al. 2025): one triple per iteration, the last repeats
    "polar_express": (
        (8.28721201814563, -23.595886519098837, 17.300387312530933),
        (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
        (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
        (3.3184196573706015, -2.488488024314874, 0.51004894012372),
        (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
        (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
        (1.8750014808534479, -1.2500016453999487, 0.3750001645474248),
        (1.875, -1.25, 0.375),
    ),
}


def newton_schulz(g: torch.Tensor, steps: int = 5, coefficients: str = "jordan",
                  dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Approximate the orthogonal polar factor of each matrix of g [..., m, n] by the
    quintic iteration X ← aX + (bA + cA²)X with A = XXᵀ (Muon)."""
    table = NS_COEFFICIENTS[coefficients]
    x = g.to(dtype)
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(-1, -2)
    scale = 1.02 if coefficients == "polar_express" else 1.0
    x = x / (x.float().norm(dim=(-2, -1), keepdim=True) * scale + 1e-7).to(dtype)
    if x.is_cuda and dtype == torch.bfloat16 and _tensor_core_shapes(x):
        x = _newton_schulz_tcgen05(x.contiguous(), steps, table)
        return x.transpose(-1, -2) if transposed else x
    for i in range(steps):
        a, b, c = table[min(i, len(table) - 1)]
        gram = x @ x.transpose(-1, -2)
        x = a * x + (b * gram + c * (gram @ gram)) @ x
    return x.transpose(-1, -2) if transposed else x


def _tensor_core_shapes(x: torch.Tensor) -> bool:
    """The TMA descriptors of the GEMM want every row pitch a multiple of 16 bytes."""
    from ..ops import functional as ops
    return ops.kernels_on(x) and x.dim() in (2, 3) and x.shape[-1] % 8 == 0 and x.shape[-2] % 8 == 0


def _newton_schulz_tcgen05(x: torch.Tensor, steps: int, table) -> torch.Tensor:
    """The quintic iteration on this framework's own tcgen05 GEMM: three GEMMs per step
    (X·Xᵀ, A·A, and (bA + cA²)·X with X read as the MN-major operand, so nothing is
    transposed in memory), the polynomial and the `aX +` as two fused elementwise ops.
    A stack of matrices [e, m, n] runs matrix by matrix."""
    from ..ops import kernels as K
    if x.dim() == 3:
        return torch.stack([_newton_schulz_tcgen05(x[e].contiguous(), steps, table) for e in range(x.shape[0])])
    for i in range(steps):
        a, b, c = table[min(i, len(table) - 1)]
        gram = K.gemm_bf16(x, x)                    # [m, m] = X Xᵀ
        poly = K.gemm_bf16(gram, gram)              # A² (A is symmetric: A·Aᵀ)
        poly = torch.add(poly.mul_(c), gram, alpha=b)
        step = K.gemm_bf16(poly, x, b_mn=True)      # [m, n]: X stored [k=m, n]
        x = step.add_(x, alpha=a)
    return x


# ------------------------------------------------------------------ optimizer
def weight_decay_mask(name: str, p: torch.Tensor) -> bool:
    """Decoupled decay applies to matrices (ndim >= 2), not to gains, biases, sinks."""
    return p.ndim >= 2 and not getattr(p, "no_weight_decay", False)


def muon_eligible(name: str, p: torch.Tensor) -> bool:
    """Hidden 2-D (or stacked expert 3-D) matrices; embeddings and heads use AdamW, and so does
    what weight decay is told to skip (stacks of vectors, decay rates, tables: no linear maps)."""
    leaf = name.split(".")
    if p.ndim < 2 or getattr(p, "no_muon", False) or getattr(p, "no_weight_decay", False):
        return False
    return not ("embedding" in leaf or "proj" in leaf[-2:] and "head" in name or "tokens" in leaf
                or "router" in leaf or "positions" in leaf)


class Optimizer:
    """AdamW / Muon over named parameters with fused updates and device-side clipping.

    Args:
        named_params: (name, parameter) pairs. A parameter with a ``main_grad`` (fp32
            accumulator written by the weight-gradient GEMMs) is updated from it.
        config: ``adamw(...)``, ``muon(...)`` or ``normuon(...)`` settings.
        moments: "float32" | "bfloat16" | "fp8" (block-scaled e4m3, CUDA only).
        master: keep an fp32 master copy of low-precision parameters.
        clip: global-norm clip threshold or None.
        reduce: optional callable(tensor) that sums a device scalar across ranks.
    """

    def __init__(self, named_params: Iterable, config, *, moments: str = "float32",
                 master: bool = True, clip: Optional[float] = 1.0, reduce: Optional[Callable] = None,
                 norm_weight: Optional[Callable] = None, shard_group=None, orthogonalize: str = "gather"):
        self.c = config
        self.shard_group, self.orthogonalize = shard_group, orthogonalize
        self.named = [(n, p) for n, p in named_params if p.requires_grad]
        self.moments, self.clip, self.reduce = moments, clip, reduce
        self.norm_weight = norm_weight
        self.step_count = 0
        self.state: dict = {}
        self.is_muon = isinstance(config, T.MuonConfig)
        self.adam = config if not self.is_muon else (config.adam or T.AdamWConfig(lr=config.lr))
        for name, p in self.named:
            st: dict = {}
            use_muon = self.is_muon and muon_eligible(name, p)
            st["muon"] = use_muon
            low = p.dtype != torch.float32
            if master and low:
                st["master"] = p.detach().float().clone()
            if use_muon:
                st["momentum"] = torch.zeros_like(p, dtype=torch.float32)
                if isinstance(config, T.NorMuonConfig):
                    st["neuron_v"] = torch.zeros(*p.shape[:-1], 1, dtype=torch.float32, device=p.device)
            else:
                st.update(self._moment_buffers(p))
            self.state[name] = st

    def _moment_buffers(self, p) -> dict:
        n, dev = p.numel(), p.device
        if self.moments == "fp8" and p.is_cuda:
            blocks = (n + 31) // 32
            return {"m": torch.zeros(n, dtype=torch.uint8, device=dev),
                    "v": torch.zeros(n, dtype=torch.uint8, device=dev),
                    "m_sf": torch.ones(blocks, dtype=torch.uint8, device=dev),
                    "v_sf": torch.ones(blocks, dtype=torch.uint8, device=dev)}
        dt = torch.bfloat16 if self.moments == "bfloat16" else torch.float32
        return {"m": torch.zeros(n, dtype=dt, device=dev), "v": torch.zeros(n, dtype=dt, device=dev)}

    # ---- gradients
    @staticmethod
    def grad_of(p) -> Optional[torch.Tensor]:
        main = getattr(p, "main_grad", None)
        return main if main is not None else p.grad

    def grad_norm_sq(self) -> Optional[torch.Tensor]:
        """Device scalar: Σ g² over all parameters (weighted by `norm_weight(name)` for
        parameters that are replicated over some ranks), summed over ranks."""
        total = None
        for name, p in self.named:
            g = self.grad_of(p)
            if g is None:
                continue
            if total is None:
                total = torch.zeros(1, dtype=torch.float32, device=g.device)
            w = self.norm_weight(name) if self.norm_weight else 1.0
            if g.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous() and w == 1.0:
                from ..ops import kernels as K

                K.sumsq(g, total)
            else:
                total += g.float().square().sum() * w
        if total is not None and self.reduce is not None:
            total = self.reduce(total)
        return total

    def clip_factor(self, norm_sq: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if norm_sq is None or self.clip is None:
            return None
        norm = norm_sq.sqrt()
        return (self.clip / (norm + 1e-6)).clamp(max=1.0)

    # ---- updates
    def step(self, lr_scale: float = 1.0, grad_scale: float = 1.0) -> Optional[torch.Tensor]:
        """Apply one update; returns the global gradient norm (device scalar) or None."""
        self.step_count += 1
        norm_sq = self.grad_norm_sq() if self.clip is not None else None
        factor = self.clip_factor(norm_sq)
        for name, p in self.named:
            self.update_param(name, p, lr_scale, grad_scale, factor)
        return None if norm_sq is None else norm_sq.sqrt() * grad_scale

    def update_param(self, name: str, p, lr_scale: float, grad_scale: float = 1.0,
                     factor: Optional[torch.Tensor] = None, step: Optional[int] = None) -> None:
        """Update one parameter from its gradient and release the gradient."""
        g = self.grad_of(p)
        if g is None:
            return
        st = self.state[name]
        step = step if step is not None else max(self.step_count, 1)
        if st["muon"]:
            self._muon(name, p, g, st, lr_scale, grad_scale, factor)
        else:
            self._adamw(name, p, g, st, lr_scale, grad_scale, factor, step)
        if getattr(p, "main_grad", None) is not None:
            p.main_grad.zero_()
        p.grad = None

    def _adamw(self, name, p, g, st, lr_scale, grad_scale, factor, step) -> None:
        a = self.adam
        wd = a.weight_decay if weight_decay_mask(name, p) else 0.0
        lr = a.lr * lr_scale
        target = st.get("master", p.data)
        if p.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and not a.cautious_weight_decay:
            from ..ops import kernels as K

            K.adamw(target.view(-1), g.contiguous().view(-1), st["m"], st["v"], lr=lr, b1=a.b1, b2=a.b2,
                    eps=a.eps, wd=wd, step=step, m_sf=st.get("m_sf"), v_sf=st.get("v_sf"),
                    shadow=p.data.view(-1) if "master" in st and p.dtype == torch.bfloat16 else None,
                    grad_scale=factor, grad_scale_const=grad_scale)
            if "master" in st and p.dtype != torch.bfloat16:
                p.data.copy_(target)
            return
        gf = g.float().view(-1) * grad_scale
        if factor is not None:
            gf = gf * factor
        m, v = st["m"], st["v"]
        m.mul_(a.b1).add_(gf.to(m.dtype), alpha=1 - a.b1)
        v.mul_(a.b2).add_((gf * gf).to(v.dtype), alpha=1 - a.b2)
        mh = m.float() / (1 - a.b1 ** step)
        vh = v.float() / (1 - a.b2 ** step)
        upd = mh / (vh.sqrt() + a.eps)
        flat = target.view(-1)
        if wd:
            if a.cautious_weight_decay:
                upd = upd + wd * flat.float() * ((upd * flat.float()) > 0)
            else:
                upd = upd + wd * flat.float()
        flat.add_(upd.to(flat.dtype), alpha=-lr)
        if "master" in st:
            p.data.copy_(target)

    def _muon(self, name, p, g, st, lr_scale, grad_scale, factor) -> None:
        c = self.c
        gf = g.float() * grad_scale
        if factor is not None:
            gf = gf * factor
        buf = st["momentum"]
        buf.mul_(c.momentum).add_(gf, alpha=1 - c.momentum)
        upd = gf * (1 - c.momentum) + buf * c.momentum if c.nesterov else buf
        ns_dtype = torch.float32 if (c.ns_dtype == "float32" or not p.is_cuda) else torch.bfloat16
        whole_rows = getattr(p, "_bux_rows", None)
        if getattr(p, "_bux_sharded", False) and self.shard_group is not None and whole_rows is not None:
            o = self._orthogonalize_shards(name, upd, whole_rows, ns_dtype)
        else:
            o = newton_schulz(upd, c.ns_steps, c.ns_coefficients, ns_dtype).float()
        if "neuron_v" in st:  # NorMuon: per-neuron second moment of the orthogonal update
            v = st["neuron_v"]
            v.mul_(c.b2).add_(o.square().mean(-1, keepdim=True), alpha=1 - c.b2)
            scale_before = o.norm()
            o = o / (v.sqrt() + c.eps)
            o = o * (scale_before / (o.norm() + 1e-12))
        rows, cols = p.shape[-2], p.shape[-1]
        if whole_rows is not None and p.dim() == 2:
            rows = whole_rows  # the scale follows the whole matrix, not this rank's rows
        if c.consistent_rms is not None:
            o = o * (c.consistent_rms * math.sqrt(max(rows, cols)))
        else:
            o = o * math.sqrt(max(1.0, rows / cols))
        lr = c.lr * lr_scale
        target = st.get("master", p.data)
        wd = c.weight_decay if weight_decay_mask(name, p) else 0.0
        if wd:
            if c.cautious_weight_decay:
                target.add_(target * ((o * target.float()) > 0), alpha=-lr * wd)
            else:
                target.mul_(1 - lr * wd)
        target.add_(o.to(target.dtype), alpha=-lr)
        if "master" in st:
            p.data.copy_(target)

    def _orthogonalize_shards(self, name: str, upd: torch.Tensor, whole_rows: int, ns_dtype) -> torch.Tensor:
        """Newton–Schulz needs whole matrices; parameters sharded by rows over the fsdp
        group are put together first (reference: ``train/optim.py:829-1088`` there).
        ``gather`` (and ``gspmd``): every rank all-gathers the update, orthogonalises the
        whole matrix and keeps its rows. ``owner``: one rank per matrix (round robin by
        name) receives the rows, orthogonalises and sends each rank's rows back, so the
        Newton–Schulz FLOPs are spread over the ranks instead of repeated on all."""
        import torch.distributed as dist

        c, g = self.c, self.shard_group
        world, me = dist.get_world_size(g), dist.get_rank(g)
        upd = upd.contiguous()
        if self.orthogonalize != "owner":
            parts = [torch.empty_like(upd) for _ in range(world)]
            dist.all_gather(parts, upd, group=g)
            whole = newton_schulz(torch.cat(parts, dim=-2), c.ns_steps, c.ns_coefficients, ns_dtype).float()
            per = whole_rows // world
            return whole.narrow(-2, me * per, per).contiguous()
        owner = sum(name.encode()) % world
        src = dist.get_global_rank(g, owner)
        parts = [torch.empty_like(upd) for _ in range(world)] if me == owner else None
        dist.gather(upd, parts, dst=src, group=g)
        out = torch.empty_like(upd, dtype=torch.float32)
        pieces = None
        if me == owner:
            whole = newton_schulz(torch.cat(parts, dim=-2), c.ns_steps, c.ns_coefficients, ns_dtype).float()
            pieces = [x.contiguous() for x in whole.chunk(world, dim=-2)]
        dist.scatter(out, pieces, src=src, group=g)
        return out

    # ---- checkpointing
    MOMENT_KEYS = ("m", "v", "momentum", "neuron_v")

    def moments_for_checkpoint(self, name: str, shape) -> dict:
        """A parameter's optimizer tensors as a checkpoint holds them: in the parameter's
        shape (so that they shard and gather like the parameter), 8-bit block-scaled
        moments expanded to fp32 (their scale blocks follow this rank's flat layout, which
        another mesh does not share)."""
        st, out = self.state[name], {}
        for k in self.MOMENT_KEYS:
            t = st.get(k)
            if t is None:
                continue
            if k in ("m", "v") and f"{k}_sf" in st:
                t = _from_8bit(t, st[f"{k}_sf"], squared=k == "v")
            out[k] = t.view(shape) if t.numel() == math.prod(shape) else t
        return out

    def load_moment(self, name: str, key: str, value: torch.Tensor) -> None:
        """The inverse: take a checkpoint's tensor (parameter-shaped) into this rank's state."""
        st = self.state[name]
        dst = st[key]
        value = value.to(dst.device)
        if key in ("m", "v") and f"{key}_sf" in st:
            q, sf = _to_8bit(value.float().reshape(-1), squared=key == "v")
            dst.copy_(q)
            st[f"{key}_sf"].copy_(sf)
            return
        dst.copy_(value.to(dst.dtype).reshape(dst.shape))

    def state_dict(self) -> dict:
        return {"step": self.step_count, "state": self.state}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        for name, st in sd["state"].items():
            if name in self.state:
                for k, v in st.items():
                    if isinstance(v, torch.Tensor):
                        self.state[name][k].copy_(v)
                    else:
                        self.state[name][k] = v


def _from_8bit(q: torch.Tensor, sf: torch.Tensor, squared: bool) -> torch.Tensor:
    """fp32 values of block-scaled e4m3 moments (one E8M0 scale per 32 consecutive values;
    the second moment is held as its square root): what `adamw_kernel` reads."""
    n = q.numel()
    vals = q.view(torch.float8_e4m3fn).float()
    scale = torch.exp2(sf.clamp_min(1).float() - 127.0).repeat_interleave(32)[:n]
    out = vals * scale
    return out * out if squared else out


def _to_8bit(x: torch.Tensor, squared: bool) -> tuple:
    """(e4m3 bytes, E8M0 scale bytes) of fp32 moments, the layout `_from_8bit` reads."""
    n = x.numel()
    src = x.clamp_min(0).sqrt() if squared else x
    blocks = (n + 31) // 32
    padded = torch.zeros(blocks * 32, dtype=torch.float32, device=x.device)
    padded[:n] = src
    amax = padded.view(blocks, 32).abs().amax(1)
    exp = torch.ceil(torch.log2(amax.clamp_min(1e-38) / 448.0)).clamp(-126, 127)
    sf = (exp + 127).to(torch.uint8)
    q = (padded.view(blocks, 32) / torch.exp2(exp).unsqueeze(1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(-1)[:n], sf


def build_optimizer(model, train: T.TrainConfig, **kw) -> Optimizer:
    moments = kw.pop("moments", train.precision.moments)
    return Optimizer(model.named_parameters(), train.optimizer, moments=moments, clip=train.clip, **kw)
