"""Recurrent token mixers over a state S [dk, dv] per value head:

    S_t = diag(w_t) S_{t-1} + b_t (a_t^T S_{t-1}) + k_t v_t^T,      o_t = S_t^T q_t

``deltanet``, ``gdn``, ``kda``, ``gdn2``, ``gla``, ``lightning`` (reference:
``architecture/recurrent/linear_attention.py:686-971``), ``rwkv7`` (``rwkv7.py``),
``mamba`` and ``mamba2`` (``ssm.py:162-320``). The scans run by chunks of 64 positions in
fp32: everything inside a chunk is batched matmuls over all chunks at once, and only
the state is carried by a loop over the chunks (reference: ``chunkwise.py:40-441``).
A document start in a packed row resets the state: the decay there is e^-60 and the
rank-one read is dropped.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ...ops import reference as ref
from ..registry import BuildContext, Context, register
from .basic import Linear, Norm
from .conv import CausalDepthwise

CHUNK = 64
_RESET = -60.0


# ------------------------------------------------------------------ scans
def _chunks(x: torch.Tensor) -> torch.Tensor:
    """[b, t, h, e] → fp32 [b, h, n, CHUNK, e], the last chunk padded with zeros."""
    x = x.float().transpose(1, 2)
    pad = -x.shape[2] % CHUNK
    if pad:
        x = F.pad(x, (0, 0, 0, pad))
    return x.reshape(x.shape[0], x.shape[1], -1, CHUNK, x.shape[-1])


def _pair(x, y, gx, gy, strict: bool):
    """M[t, s] = sum_d x_t[d] y_s[d] exp(gx_t[d] - gy_s[d]) for s <= t (s < t if strict),
    else 0. One decay per head (last dim 1) goes through a plain matmul."""
    c = x.shape[-2]
    keep = torch.ones(c, c, dtype=torch.bool, device=x.device).tril(-1 if strict else 0)
    if gx.shape[-1] == 1:
        diff = (gx - gy.transpose(-1, -2)).masked_fill(~keep, float("-inf"))
        return (x @ y.transpose(-1, -2)) * diff.exp()
    out = []
    for i in range(x.shape[2]):  # a chunk at a time: the [t, s, d] decays are large
        diff = gx[:, :, i].unsqueeze(-2) - gy[:, :, i].unsqueeze(-3)
        diff = diff.masked_fill(~keep[..., None], float("-inf"))
        out.append(torch.einsum("bhtd,bhsd,bhtsd->bhts", x[:, :, i], y[:, :, i], diff.exp()))
    return torch.stack(out, 2)


_decoding = None   # (cache, layer) while a mixer runs with a `DecodeCache`: `scan` carries its state


class decoding:
    """While active, the layer's `scan` starts from the state the cache holds for it and leaves
    its last state there (incremental decoding, `bux_b200.models.cache`)."""

    def __init__(self, ctx, layer):
        self.slot = (ctx.cache, layer) if getattr(ctx, "cache", None) is not None else None

    def __enter__(self):
        global _decoding
        self.before, _decoding = _decoding, self.slot
        return self

    def __exit__(self, *exc):
        global _decoding
        _decoding = self.before
        return False


def scan(q, k, v, g, a=None, b=None, starts: Optional[torch.Tensor] = None, state=None, group=None):
    """`_scan`, continuing the state of a `DecodeCache` when a layer decodes with one."""
    slot = _decoding
    if slot is None:
        return _scan(q, k, v, g, a, b, starts, state, group)
    cache, layer = slot
    out, last = _scan(q, k, v, g, a, b, starts, cache.states.get(id(layer)) if state is None else state, group)
    cache.states[id(layer)] = last
    return out, last


def _scan(q, k, v, g, a=None, b=None, starts: Optional[torch.Tensor] = None, state=None, group=None):
    """The recurrence above from `state` (zero if None). q, k, a, b: [B, T, H, dk];
    v: [B, T, H, dv]; g = log w: [B, T, H, dk] or [B, T, H, 1] (<= 0); starts: bool [B, T],
    true where a document begins. With `group` the positions are split over its ranks
    (context parallelism) and the state is handed on between them. Returns (o [B, T, H, dv]
    in v's dtype, last state fp32)."""
    if group is not None:
        from ...parallel import recurrence

        return recurrence.pass_state(_scan, q, k, v, g, a, b, starts, group)
    if k.is_cuda and v.dtype == torch.bfloat16 and not torch.backends.cuda.matmul.allow_tf32:
        # bf16 activations: the chunk matrices end up as bf16 operands of the scan kernel, so
        # their fp32 matmuls may run on the tensor cores in TF32 (three more mantissa bits than bf16)
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            return _scan(q, k, v, g, a, b, starts, state, group)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = False
    bsz, t, h, dk = k.shape
    dv = v.shape[-1]
    if starts is not None:
        s_ = starts.view(bsz, t, 1, 1)
        g = torch.where(s_, torch.full_like(g, _RESET), g)
        if a is not None:
            a = a * (~s_).to(a.dtype)
    Q, K, V, Gs = _chunks(q), _chunks(k), _chunks(v), _chunks(g)
    G = Gs.cumsum(-2)                       # inclusive log decay inside the chunk
    Gp = G - Gs                             # exclusive: up to the position before
    end = G[..., -1:, :]
    n = Q.shape[2]
    S = torch.zeros(bsz, h, dk, dv, device=k.device) if state is None else state.float()
    Qd = Q * G.exp()
    Kd = K * (end - G).exp()
    Mqk = _pair(Q, K, G, G, False)
    rank1 = a is not None and b is not None
    if rank1:
        A, Bm = _chunks(a), _chunks(b)
        eye = torch.eye(CHUNK, device=k.device)
        T_ = torch.linalg.solve_triangular(eye - _pair(A, Bm, Gp, G, True), eye.expand(bsz, h, n, -1, -1),
                                           upper=False, unitriangular=True)
        P = T_ @ (A * Gp.exp())             # X = P S_0 + W V
        W = T_ @ _pair(A, K, Gp, G, True)
        Mqb = _pair(Q, Bm, G, G, False)
        Bd = Bm * (end - G).exp()
    from ...ops import functional as ops_f
    from ...ops import scan as scan_kernel

    if ops_f.kernels_on(v) and scan_kernel.supported(dk, dv, k.device):
        # the serial part on the tensor cores, the state in tensor memory across the chunks
        lam = end.exp().squeeze(-2).expand(bsz, h, n, dk)
        if rank1:
            o, last = scan_kernel.chunk_scan(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, state)
        else:
            o, last = scan_kernel.chunk_scan(None, Qd, None, Mqk, None, Kd, None, V, lam, state)
        out = o.reshape(bsz, h, n * CHUNK, dv)[:, :, :t].transpose(1, 2)
        return out.to(v.dtype), last
    local = Mqk @ V
    if rank1:
        U0 = W @ V
    outs = []
    decay_end = end.exp().transpose(-1, -2)  # [b, h, n, dk or 1, 1]
    for i in range(n):
        o = Qd[:, :, i] @ S + local[:, :, i]
        new = decay_end[:, :, i] * S + Kd[:, :, i].transpose(-1, -2) @ V[:, :, i]
        if rank1:
            X = P[:, :, i] @ S + U0[:, :, i]
            o = o + Mqb[:, :, i] @ X
            new = new + Bd[:, :, i].transpose(-1, -2) @ X
        S = new
        outs.append(o)
    out = torch.stack(outs, 2).reshape(bsz, h, n * CHUNK, dv)[:, :, :t].transpose(1, 2)
    return out.to(v.dtype), S


def scan_steps(q, k, v, g, a=None, b=None, starts=None, state=None):
    """The same recurrence one position at a time: the oracle of `scan`."""
    bsz, t, h, dk = k.shape
    S = torch.zeros(bsz, h, dk, v.shape[-1]) if state is None else state.float()
    outs = []
    for i in range(t):
        w = g[:, i].float().exp()
        ai = None if a is None else a[:, i].float()
        if starts is not None:
            st = starts[:, i].view(bsz, 1, 1)
            w = torch.where(st, torch.full_like(w, math.exp(_RESET)), w)
            if ai is not None:
                ai = ai * (~st).float()
        new = w.unsqueeze(-1) * S
        if ai is not None:
            read = torch.einsum("bhk,bhkv->bhv", ai, S)
            new = new + b[:, i].float().unsqueeze(-1) * read.unsqueeze(-2)
        S = new + k[:, i].float().unsqueeze(-1) * v[:, i].float().unsqueeze(-2)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, i].float(), S))
    return torch.stack(outs, 1).to(v.dtype), S


def delta_rule(q, k, v, g, beta, starts=None, state=None, group=None):
    """S_t = (I - beta k k^T) diag(w) S_{t-1} + beta k v^T, as the rank-one recurrence with
    a = -w k, b = beta k, written key beta k."""
    step = beta.float().unsqueeze(-1) * k.float()
    return scan(q, step, v, g, -g.float().exp() * k.float(), step, starts, state, group)


def l2norm(x, eps: float = 1e-6):
    y = x.float()
    return (y * torch.rsqrt(y.square().sum(-1, keepdim=True) + eps)).to(x.dtype)


def _starts(ctx: Context):
    if getattr(ctx, "segments", None) is None:
        return None
    s = ctx.positions == 0
    if _cp(ctx) is None:
        s[:, 0] = False  # the row's first position starts from the zero state anyway
    return s


def _cp(ctx: Context):
    """The process group the row's positions are split over, or None."""
    return getattr(ctx.parallel, "context_group", None) if getattr(ctx, "parallel", None) is not None else None


# ------------------------------------------------------------------ pieces
class LowRank(nn.Module):
    """act(x A) B + c through `rank` dims."""

    def __init__(self, n_in: int, rank: int, n_out: int, activation: Optional[str] = None,
                 bias: bool = False, std: float = 0.02):
        super().__init__()
        self.down = nn.Parameter(torch.randn(n_in, rank) * std)
        self.up = nn.Parameter(torch.randn(rank, n_out) * std)
        self.bias = nn.Parameter(torch.zeros(n_out)) if bias else None
        self.activation = activation

    def forward(self, x):
        h = x.float() @ self.down.float()
        if self.activation is not None:
            h = ref.activation(h, self.activation)
        y = h @ self.up.float()
        return y if self.bias is None else y + self.bias.float()


def time_step_bias(n: int, low: float = 1e-3, high: float = 0.1) -> torch.Tensor:
    """softplus^-1 of n time steps log-uniform in [low, high], floored at 1e-4."""
    dt = torch.exp(torch.empty(n).uniform_(math.log(low), math.log(high))).clamp_min(1e-4)
    return dt + torch.log(-torch.expm1(-dt))


def _log_uniform(n: int, low: float, high: float) -> torch.Tensor:
    return torch.log(torch.empty(n).uniform_(low, high))


class LinearAttention(nn.Module):
    """What the family shares: q, k, v projections, one short conv over the three side by
    side, SiLU, heads (each q/k head serves a group of adjacent value heads), and the
    output's norm, gate and projection."""

    def __init__(self, c, b: BuildContext, *, silu: bool = True, gate_rank: Optional[int] = None,
                 gate_bias: bool = False, norm_all_heads: bool = False):
        super().__init__()
        self.c = c
        width = b.width if isinstance(b.width, int) else b.d_model
        h, hv = c.num_heads, c.num_v_heads or c.num_heads
        dk, dv = c.head_dim, c.v_head_dim or c.head_dim
        self.h, self.hv, self.dk, self.dv, self.width = h, hv, dk, dv, width
        self.q = Linear(width, h * dk, False, b, role="q")
        self.k = Linear(width, h * dk, False, b, role="q")
        self.v = Linear(width, hv * dv, False, b, role="q")
        self.conv = CausalDepthwise(2 * h * dk + hv * dv, c.conv_size) if c.conv_size else None
        self.silu = silu
        if c.output_gate is not None:
            self.gate = (LowRank(width, gate_rank, hv * dv, bias=gate_bias) if gate_rank
                         else Linear(width, hv * dv, False, b, role="q"))
        self.norm_all_heads = norm_all_heads
        from ...config import layers as L

        self.norm = Norm(L.NormalizationConfig(type="rmsnorm", eps=c.norm_eps), hv * dv if norm_all_heads else dv)
        self.o = Linear(hv * dv, width, False, b, role="o", init_role="out")

    def qkv(self, x, ctx: Context):
        bsz, t, _ = x.shape
        q, k, v = self.q(x, ctx), self.k(x, ctx), self.v(x, ctx)
        if self.conv is not None:
            sizes = [q.shape[-1], k.shape[-1], v.shape[-1]]
            q, k, v = F.silu(self.conv(torch.cat([q, k, v], -1), ctx)).split(sizes, -1)
        elif self.silu:
            q, k, v = F.silu(q), F.silu(k), F.silu(v)
        group = self.hv // self.h
        q, k = (y.reshape(bsz, t, self.h, self.dk).repeat_interleave(group, 2) for y in (q, k))
        return q, k, v.reshape(bsz, t, self.hv, self.dv)

    def output(self, x, o, ctx: Context):
        bsz, t = o.shape[:2]
        o = self.norm(o.reshape(bsz, t, -1) if self.norm_all_heads else o, ctx).reshape(bsz, t, -1)
        if hasattr(self, "gate"):
            gate = self.gate(x, ctx) if isinstance(self.gate, Linear) else self.gate(x)
            o = (o.float() * ref.activation(gate.float(), self.c.output_gate)).to(o.dtype)
        return self.o(o, ctx)

    def forward(self, x, ctx: Context):
        with decoding(ctx, self):
            q, k, v = self.qkv(x, ctx)
            return self.output(x, self.mix(x, q, k, v, ctx), ctx)


class DeltaNet(LinearAttention):
    """Delta rule on L2-normalised q, k (q scaled by dk^-1/2), beta = sigmoid(W_b x), no decay."""

    def __init__(self, c, b, **kw):
        super().__init__(c, b, **kw)
        self.b = Linear(self.width, self.hv, False, b, role="router")

    def log_decay(self, x, ctx):
        return torch.zeros(*x.shape[:2], self.hv, 1, device=x.device)

    def mix(self, x, q, k, v, ctx):
        q, k = l2norm(q) * self.dk ** -0.5, l2norm(k)
        beta = torch.sigmoid(self.b(x, ctx).float())
        return delta_rule(q, k, v, self.log_decay(x, ctx), beta, _starts(ctx), group=_cp(ctx))[0]


class GatedDeltaNet(DeltaNet):
    """DeltaNet with a decay per value head: g = -exp(A_log) softplus(W_a x + dt_bias)."""

    def __init__(self, c, b):
        super().__init__(c, b)
        self.a = Linear(self.width, self.hv, False, b, role="router")
        self.A_log = nn.Parameter(_log_uniform(self.hv, 0.01, 16))
        self.dt_bias = nn.Parameter(time_step_bias(self.hv))

    def log_decay(self, x, ctx):
        rate = F.softplus(self.a(x, ctx).float() + self.dt_bias.float())
        return (-self.A_log.float().exp() * rate).unsqueeze(-1)


def channel_decay(f, A_log, lower_bound):
    rate = A_log.float().exp()[:, None]
    if lower_bound is not None:
        return lower_bound * torch.sigmoid(rate * f)
    return -rate * F.softplus(f)


def _channel_rates(heads: int, dk: int, lower_bound):
    A_log = _log_uniform(heads, 1, 16) if lower_bound is None else torch.zeros(heads)
    return nn.Parameter(A_log), nn.Parameter(time_step_bias(heads * dk))


class KDA(DeltaNet):
    """Gated DeltaNet with a decay per key channel from a low-rank f; low-rank output gate."""

    def __init__(self, c, b):
        super().__init__(c, b, gate_rank=c.output_gate_rank)
        self.f = LowRank(self.width, c.gate_rank or self.dk, self.hv * self.dk)
        self.A_log, self.dt_bias = _channel_rates(self.hv, self.dk, c.gate_lower_bound)

    def log_decay(self, x, ctx):
        bsz, t, _ = x.shape
        f = (self.f(x) + self.dt_bias.float()).reshape(bsz, t, self.hv, self.dk)
        return channel_decay(f, self.A_log, self.c.gate_lower_bound)


class GatedDeltaNet2(LinearAttention):
    """S_t = (I - k (b*k)^T) diag(e^g) S_{t-1} + k (w*v)^T with an erase gate b over the
    key channels and a write gate w over the value channels."""

    def __init__(self, c, b):
        dv = c.v_head_dim or c.head_dim
        super().__init__(c, b, gate_rank=c.output_gate_rank or dv, gate_bias=True)
        self.f = LowRank(self.width, c.gate_rank or dv, self.h * self.dk)
        self.erase = Linear(self.width, self.h * self.dk, False, b, role="q")
        self.write = Linear(self.width, self.hv * dv, False, b, role="q")
        self.A_log, self.dt_bias = _channel_rates(self.h, self.dk, c.gate_lower_bound)
        self.erase_scale = 2.0 if c.negative_eigenvalues else 1.0

    def mix(self, x, q, k, v, ctx):
        bsz, t, _ = x.shape
        group = self.hv // self.h
        q, k = l2norm(q) * self.dk ** -0.5, l2norm(k)
        f = (self.f(x) + self.dt_bias.float()).reshape(bsz, t, self.h, self.dk)
        g = channel_decay(f, self.A_log, self.c.gate_lower_bound).repeat_interleave(group, 2)
        erase = self.erase_scale * torch.sigmoid(self.erase(x, ctx).float()).reshape(bsz, t, self.h, self.dk)
        erase = erase.repeat_interleave(group, 2)
        write = torch.sigmoid(self.write(x, ctx).float()).reshape(bsz, t, self.hv, -1)
        a = -g.exp() * erase * k.float()
        return scan(q, k, write * v.float(), g, a, k.float(), _starts(ctx), group=_cp(ctx))[0].to(v.dtype)


class GLA(LinearAttention):
    """Linear attention with a decay per key channel, log w = log sigmoid(f) / 16."""

    def __init__(self, c, b):
        super().__init__(c, b, silu=False)
        self.f = LowRank(self.width, c.gate_rank, self.hv * self.dk, bias=True)

    def mix(self, x, q, k, v, ctx):
        g = F.logsigmoid(self.f(x).reshape(*k.shape)) / 16
        return scan(q * self.dk ** -0.5, k, v, g, starts=_starts(ctx), group=_cp(ctx))[0]


def slopes(heads: int, layer: int, layers: int) -> torch.Tensor:
    """MiniMax's decay rates 2^(-8 i / heads), scaled down with depth."""
    factor = 1 - layer / (layers - 1 + 1e-5) + 1e-5
    return 2 ** (-8 / heads * torch.arange(1, heads + 1, dtype=torch.float32)) * factor


class Lightning(LinearAttention):
    """Linear attention on SiLU'd q, k, v with a fixed decay per head by depth."""

    def __init__(self, c, b):
        super().__init__(c, b, norm_all_heads=True)
        self.register_buffer("slopes", slopes(self.hv, b.layer_index, max(b.num_layers, 1)), persistent=False)

    def mix(self, x, q, k, v, ctx):
        g = (-self.slopes.float()[:, None]).expand(*q.shape[:3], 1)
        return scan(q, k, v, g, starts=_starts(ctx), group=_cp(ctx))[0]


class RWKV7(nn.Module):
    """Token shift, r/k/v, low-rank decay w and in-context learning rate a, the
    generalised delta rule S_t = (diag(w) - (a kk) kk^T) S_{t-1} + k v^T, a per-head
    layernorm plus the bonus (r k r_k) v, gate, projection. Port ``v``: value residual."""
    no_weight_decay = ("shift", "r_k")


    def __init__(self, c, b: BuildContext):
        super().__init__()
        if c.conv_size is not None:
            raise NotImplementedError("rwkv7 with a short conv (it shifts tokens)")
        self.c = c
        width = b.width if isinstance(b.width, int) else b.d_model
        h, hv = c.num_heads, c.num_v_heads or c.num_heads
        dk, dv = c.head_dim, c.v_head_dim or c.head_dim
        self.h, self.hv, self.dk, self.dv = h, hv, dk, dv
        nk, nv = h * dk, hv * dv
        self.shift = nn.Parameter(torch.zeros(6, width))
        self.r = Linear(width, nk, False, b, role="q")
        self.k = Linear(width, nk, False, b, role="q")
        self.v = Linear(width, nv, False, b, role="q")
        self.w = LowRank(width, c.decay_rank, nk, "tanh", bias=True)
        self.a = LowRank(width, c.a_rank, nk, bias=True)
        self.ports = b.ports or ()
        if any(p.name == "v" and p.mode != "write" for p in self.ports):
            self.v_mix = LowRank(width, c.v_rank, nv, bias=True)
        if c.output_gate is not None:
            self.g = LowRank(width, c.gate_rank, nv, c.output_gate)
        self.k_k = nn.Parameter(torch.full((nk,), 0.85))
        self.k_a = nn.Parameter(torch.ones(nk))
        self.r_k = nn.Parameter(torch.zeros(hv, dk))
        self.norm_scale = nn.Parameter(torch.ones(hv, dv))
        self.norm_bias = nn.Parameter(torch.zeros(hv, dv))
        self.eps = dv * c.norm_eps
        self.o = Linear(nv, width, False, b, role="o", init_role="out")

    def forward(self, x, ctx: Context):
        bsz, t, _ = x.shape
        h, hv, dk, dv = self.h, self.hv, self.dk, self.dv
        prev = F.pad(x[:, :-1], (0, 0, 1, 0))
        cache = getattr(ctx, "cache", None)
        if cache is not None:     # incremental decoding: the token before this call's first one
            last = cache.tails.get(("shift", id(self)))
            if last is not None:
                prev = torch.cat([last, x[:, :-1]], dim=1)
            cache.tails[("shift", id(self))] = x[:, -1:]
        if _cp(ctx) is not None:  # the token before this rank's first one lives on the rank before
            from ...parallel import recurrence

            prev = torch.cat([recurrence.halo(x, 1, _cp(ctx)), x[:, :-1]], dim=1)
        st = _starts(ctx)
        if st is not None:
            prev = prev * (~st).unsqueeze(-1).to(x.dtype)
        shifted = x.unsqueeze(0) + (prev - x).unsqueeze(0) * self.shift.to(x.dtype)[:, None, None]
        xr, xw, xk, xv, xa, xg = shifted
        r, k = self.r(xr, ctx).float(), self.k(xk, ctx).float()
        v = self.v(xv, ctx).reshape(bsz, t, hv, dv)
        for p in self.ports:
            if p.name == "v" and p.mode != "write":
                mix = torch.sigmoid(self.v_mix(xv)).reshape(v.shape)
                v = (v.float() + (ctx.read(p.tap, p.mode == "pop").float() - v.float()) * mix).to(v.dtype)
        for p in self.ports:
            if p.name == "v" and p.mode == "write":
                ctx.push(p.tap, v)
        log_w = -math.exp(-0.5) * torch.sigmoid(self.w(xw))
        a = torch.sigmoid(self.a(xa))
        kk = k * self.k_k.float()
        k = k * (1 + (a - 1) * self.k_a.float())

        def split(y):
            return y.reshape(bsz, t, h, dk).repeat_interleave(hv // h, 2)

        r, k, log_w, a, kk = map(split, (r, k, log_w, a, kk))
        kk = l2norm(kk, eps=1e-12)
        with decoding(ctx, self):
            o, _ = scan(r, k, v, log_w, -kk, kk * a, st, group=_cp(ctx))
        o = F.layer_norm(o.float(), (dv,), eps=self.eps) * self.norm_scale.float() + self.norm_bias.float()
        o = o + (r * k * self.r_k.float()).sum(-1, keepdim=True) * v.float()
        o = o.reshape(bsz, t, -1)
        if hasattr(self, "g"):
            o = o * self.g(xg)
        return self.o(o.to(x.dtype), ctx)


# ------------------------------------------------------------------ state space models
def mamba_scan(x, dt, A, B, C, starts=None, state=None, last: Optional[list] = None):
    """Every channel's state S = exp(dt A) S + (dt x) B, read as y = S·C, one position at a
    time in fp32. x, dt: [b, t, d]; A: [d, n]; B, C: [b, t, n]. From `state` (zero if None);
    the state after the last position is appended to `last` when a list is given."""
    xs, dt, A, B, C = x.float(), dt.float(), A.float(), B.float(), C.float()
    bsz, t, d = xs.shape
    s = xs.new_zeros(bsz, d, A.shape[-1]) if state is None else state.float()
    ys = []
    for i in range(t):
        if starts is not None:
            s = s * (~starts[:, i]).view(bsz, 1, 1).float()
        s = (dt[:, i, :, None] * A).exp() * s + (dt[:, i] * xs[:, i]).unsqueeze(-1) * B[:, i, None]
        ys.append((s * C[:, i, None]).sum(-1))
    if last is not None:
        last.append(s)
    return torch.stack(ys, 1).to(x.dtype)


class Mamba(nn.Module):
    no_weight_decay = ("A_log",)

    def __init__(self, c, b: BuildContext):
        super().__init__()
        from ...config import layers as L

        width = b.width if isinstance(b.width, int) else b.d_model
        d_inner, n = c.expand * width, c.state_size
        r = c.dt_rank or math.ceil(width / 16)
        self.rank, self.n = r, n
        self.in_proj = Linear(width, 2 * d_inner, False, b)
        self.conv = CausalDepthwise(d_inner, c.conv_size, bias=True)
        self.x_proj = Linear(d_inner, r + 2 * n, False, b)
        self.dt_proj = nn.Parameter(torch.randn(r, d_inner) * r ** -0.5)
        self.dt_bias = nn.Parameter(time_step_bias(d_inner, c.dt_min, c.dt_max))
        rms = L.NormalizationConfig(type="rmsnorm")
        self.dt_norm, self.b_norm, self.c_norm = Norm(rms, r), Norm(rms, n), Norm(rms, n)
        self.A_log = nn.Parameter(torch.log(torch.arange(1, n + 1, dtype=torch.float32)).repeat(d_inner, 1))
        self.D = nn.Parameter(torch.ones(d_inner))
        self.out_proj = Linear(d_inner, width, False, b, init_role="out")

    def forward(self, x, ctx: Context):
        u, z = self.in_proj(x, ctx).chunk(2, -1)
        u = F.silu(self.conv(u, ctx))
        dt, B, C = self.x_proj(u, ctx).split([self.rank, self.n, self.n], -1)
        dt = F.softplus(self.dt_norm(dt, ctx).float() @ self.dt_proj.float() + self.dt_bias.float())
        if _cp(ctx) is not None:
            raise NotImplementedError("mamba: a state per channel and position is not handed on between ranks; "
                                      "use mamba2 (or another mixer of the family) under mesh(context=...)")
        cache = getattr(ctx, "cache", None)
        kept: Optional[list] = [] if cache is not None else None
        y = mamba_scan(u, dt, -self.A_log.float().exp(), self.b_norm(B, ctx), self.c_norm(C, ctx), _starts(ctx),
                       state=cache.states.get(id(self)) if cache is not None else None, last=kept)
        if cache is not None:
            cache.states[id(self)] = kept[0]
        y = (y.float() + u.float() * self.D.float()) * F.silu(z.float())
        return self.out_proj(y.to(x.dtype), ctx)


class Mamba2(nn.Module):
    no_weight_decay = ("A_log",)

    def __init__(self, c, b: BuildContext):
        super().__init__()
        from ...config import layers as L

        width = b.width if isinstance(b.width, int) else b.d_model
        d_inner, n, g = c.expand * width, c.state_size, c.num_groups
        if c.num_heads is not None:
            d_inner = c.num_heads * c.head_dim
        h = d_inner // c.head_dim
        self.inner, self.heads, self.head_dim, self.groups, self.n = d_inner, h, c.head_dim, g, n
        self.in_proj = Linear(width, 2 * d_inner + 2 * g * n + h, False, b)
        self.conv = CausalDepthwise(d_inner + 2 * g * n, c.conv_size, bias=True)
        self.dt_bias = nn.Parameter(time_step_bias(h, c.dt_min, c.dt_max))
        self.A_log = nn.Parameter(_log_uniform(h, 1, 16))
        self.D = nn.Parameter(torch.ones(h))
        self.norm = Norm(L.NormalizationConfig(type="rmsnorm", eps=1e-5), d_inner // g)
        self.out_proj = Linear(d_inner, width, False, b, init_role="out")

    def forward(self, x, ctx: Context):
        bsz, t, _ = x.shape
        d, g, n, h = self.inner, self.groups, self.n, self.heads
        z, ubc, dt = self.in_proj(x, ctx).split([d, d + 2 * g * n, h], -1)
        u, B, C = F.silu(self.conv(ubc, ctx)).split([d, g * n, g * n], -1)
        u = u.reshape(bsz, t, h, self.head_dim)
        B, C = (y.reshape(bsz, t, g, n).repeat_interleave(h // g, 2) for y in (B, C))
        dt = F.softplus(dt.float() + self.dt_bias.float())
        A = -self.A_log.float().exp()
        with decoding(ctx, self):
            y, _ = scan(C, B, dt.unsqueeze(-1) * u.float(), (dt * A).unsqueeze(-1), starts=_starts(ctx), group=_cp(ctx))
        y = (y.float() + u.float() * self.D.float()[:, None]).reshape(bsz, t, d) * F.silu(z.float())
        y = self.norm(y.reshape(bsz, t, g, -1).to(x.dtype), ctx).reshape(bsz, t, d)
        return self.out_proj(y, ctx)


for _name, _cls in (("deltanet", DeltaNet), ("gdn", GatedDeltaNet), ("kda", KDA), ("gdn2", GatedDeltaNet2),
                    ("gla", GLA), ("lightning", Lightning), ("rwkv7", RWKV7), ("mamba", Mamba),
                    ("mamba2", Mamba2)):
    register(_name)(lambda c, b, _cls=_cls: _cls(c, b))
