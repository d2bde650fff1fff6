"""Residual algebras: what a top-level residual branch ``[f]`` does instead of
``x + f(x)``, and ``merge``, which reads a widened stream back into one.

``residual = hc() | mhc() | gr() | attnres() | msar() | vpgate()`` at the top of an
architecture picks one (reference: ``architecture/residual.py:150-691``):

* hc / mhc / gr widen the stream to n copies, ``[b, t, n, d]``;
* attnres keeps the embedding and every branch output so far, ``[b, t, 1+L, d]``;
* msar keeps raw outputs, finished blocks' conv expansions and the head's read;
* vpgate keeps one stream and mixes ``a·x + b·f(x)`` per channel.

Every algebra is called as ``algebra(x, body, ctx)`` with the stream as it holds it;
what a branch reads follows from the state alone, so a shared block can run at several
depths. Coefficient math runs in fp32 and is cast to the stream's dtype.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from ..config import layers as L
from .layers.conv import CausalDepthwise
from .registry import BuildContext, Context, register

_EPS = 1e-6


def widening(residual) -> Optional[int]:
    """Copies of the stream the widened stream starts as; None when it is not widened."""
    if isinstance(residual, (L.HyperConnectionsConfig, L.GatedResidualConfig)):
        return residual.expansion
    if isinstance(residual, (L.AttentionResidualConfig, L.MultiStreamAttentionResidualConfig)):
        return 1
    return None


def widen(x: torch.Tensor, n: int) -> torch.Tensor:
    return x.unsqueeze(2).expand(-1, -1, n, -1).contiguous()


def weighted(w: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """sum_j w[b,t,j] x[b,t,j,:]"""
    return torch.einsum("btn,btnd->btd", w.to(x.dtype), x)


def mixed(m: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """stream k = sum_j m[b,t,j,k] x[b,t,j,:]"""
    return torch.einsum("btjk,btjd->btkd", m.to(x.dtype), x)


def sinkhorn(logits: torch.Tensor, iters: int) -> torch.Tensor:
    """Doubly stochastic matrix of exp(logits): softmax over rows, columns divided by
    their sums, then iters-1 more rounds of rows and columns (columns last)."""
    m = torch.softmax(logits.float(), -1) + _EPS
    m = m / (m.sum(-2, keepdim=True) + _EPS)
    for _ in range(iters - 1):
        m = m / (m.sum(-1, keepdim=True) + _EPS)
        m = m / (m.sum(-2, keepdim=True) + _EPS)
    return m


def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    y = x.float()
    return (y * torch.rsqrt(y.square().mean(-1, keepdim=True) + eps)).to(x.dtype)


def _pending(ctx: Context, x: torch.Tensor) -> torch.Tensor:
    """Coefficients of a single-pass read: the last branch's, or stream 0 alone."""
    if getattr(ctx, "pending_read", None) is not None:
        return ctx.pending_read
    first = torch.zeros(x.shape[2], dtype=x.dtype, device=x.device)
    first[0] = 1
    return first.expand(*x.shape[:3])


def _single_pass(computed: torch.Tensor, x: torch.Tensor, ctx: Context) -> torch.Tensor:
    read = _pending(ctx, x)
    ctx.pending_read = computed
    return read


class _Dynamic(nn.Module):
    """s·tanh(layernorm(H) W) at every stream of H; W from 0, s from 0.01."""

    def __init__(self, d: int, columns: int, eps: float):
        super().__init__()
        self.proj = nn.Parameter(torch.zeros(d, columns))
        self.scale = nn.Parameter(torch.tensor(0.01))
        self.eps = eps

    def forward(self, x):
        y = nn.functional.layer_norm(x.float(), x.shape[-1:], eps=self.eps)
        return self.scale * torch.tanh(y @ self.proj)


class HyperConnections(nn.Module):
    """h = A_m^T H;  H' = A_r^T H + B^T f(h). Branch k starts as a pre-norm residual on
    stream k mod n (A_m = e_k, A_r = I, B = 1); without f it is the read alone, which
    starts as the sum of the streams."""

    no_weight_decay = ("static_alpha", "static_beta")

    def __init__(self, c: L.HyperConnectionsConfig, d: int, index: int, write: bool = True):
        super().__init__()
        n = c.expansion
        self.single_pass, self.write = c.single_pass, write
        a_m = torch.zeros(n)
        if write:
            a_m[index % n] = 1
        else:
            a_m.fill_(1)
        a = torch.cat([a_m[:, None], torch.eye(n)], 1)
        self.static_alpha = nn.Parameter(a if write else a[:, :1].clone())
        if write:
            self.static_beta = nn.Parameter(torch.ones(n))
        columns = a.shape[1] if write else 1
        if c.dynamic:
            self.dynamic_alpha = _Dynamic(d, columns, c.norm_eps)
            if write:
                self.dynamic_beta = _Dynamic(d, 1, c.norm_eps)

    def _alpha(self, x):
        a = self.static_alpha.float().expand(*x.shape[:3], -1)
        return a + self.dynamic_alpha(x) if hasattr(self, "dynamic_alpha") else a

    def read(self, x, ctx=None):
        return weighted(self._alpha(x)[..., 0], x)

    def forward(self, x, body, ctx: Context):
        alpha = self._alpha(x)
        read = alpha[..., 0]
        if self.single_pass:
            read = _single_pass(read, x, ctx)
        y = body(weighted(read, x), ctx)
        beta = self.static_beta.float().expand(*x.shape[:3])
        if hasattr(self, "dynamic_beta"):
            beta = beta + self.dynamic_beta(x)[..., 0]
        return mixed(alpha[..., 1:], x) + beta.to(y.dtype).unsqueeze(-1) * y.unsqueeze(2)


class ManifoldHyperConnections(nn.Module):
    """pre = sigmoid(a_pre r W_pre + b_pre), post = 2 sigmoid(...), res = sinkhorn(...),
    with r the n streams flattened and RMS-normalised: f reads sum_j pre_j x_j and
    stream k becomes sum_j res_jk x_j + post_k f(h)."""

    def __init__(self, c: L.HyperConnectionsConfig, d: int, index: int, write: bool = True):
        super().__init__()
        n = c.expansion
        self.n, self.write, self.single_pass = n, write, c.single_pass
        self.iters, self.eps = c.sinkhorn_iters, c.norm_eps
        if write:
            fav = torch.zeros(n)
            fav[index % n] = 1
            pre, post = (b * (2 * fav - 1) for b in (c.pre_bias, c.post_bias))
            res = c.res_bias * (1 - torch.eye(n))
            bias = torch.cat([pre, post, res.reshape(-1)])
        else:
            bias = torch.full((n,), -math.log(n - 1))
        self.bias = nn.Parameter(bias.float())
        if c.dynamic:
            self.proj = nn.Parameter(torch.zeros(n * d, bias.shape[0]))
            self.scale = nn.Parameter(torch.full((3 if write else 1,), 0.01))

    def _logits(self, x):
        b, t, n, d = x.shape
        if not hasattr(self, "proj"):
            return self.bias.expand(b, t, -1)
        flat = x.reshape(b, t, n * d).float()
        rms = torch.rsqrt(flat.square().mean(-1, keepdim=True) + self.eps)
        widths = (n, n, n * n)[: self.scale.shape[0]]
        a = torch.cat([s.expand(w) for s, w in zip(self.scale, widths)])
        return (flat @ self.proj.float()) * rms * a + self.bias

    def read(self, x, ctx=None):
        return weighted(torch.sigmoid(self._logits(x)[..., : self.n]) + _EPS, x)

    def forward(self, x, body, ctx: Context):
        b, t, n, _ = x.shape
        logits = self._logits(x)
        read = torch.sigmoid(logits[..., :n]) + _EPS
        if self.single_pass:
            read = _single_pass(read, x, ctx)
        post = 2 * torch.sigmoid(logits[..., n: 2 * n])
        res = sinkhorn(logits[..., 2 * n:].reshape(b, t, n, n), self.iters)
        y = body(weighted(read, x), ctx)
        return mixed(res, x) + post.to(y.dtype).unsqueeze(-1) * y.unsqueeze(2)


class GatedResidual(nn.Module):
    """Streams RMS-normalised with their own gains; f reads mean_j g_j r_j with
    g = sigmoid(W_u silu(W_d r / n)); f is added to stream j by 2 sigmoid(W_w r / n)_j."""

    def __init__(self, c: L.GatedResidualConfig, d: int, write: bool = True, std: float = 0.02):
        super().__init__()
        n = c.expansion
        self.n, self.eps = n, c.norm_eps
        self.gain = nn.Parameter(torch.ones(n, d))
        self.down = nn.Parameter(torch.randn(c.rank, n * d) * std)
        self.up = nn.Parameter(torch.randn(n * d, c.rank) * std)
        if write:
            self.write_proj = nn.Parameter(torch.randn(n, n * d) * std)

    def _norm(self, x):
        return (_rms(x, self.eps).float() * self.gain).to(x.dtype)

    def _read(self, r):
        b, t, n, d = r.shape
        flat = r.reshape(b, t, n * d).float()
        gate = nn.functional.silu(flat @ self.down.float().t() / n) @ self.up.float().t()
        return (torch.sigmoid(gate).view(b, t, n, d) * r.float()).mean(2).to(r.dtype)

    def read(self, x, ctx=None):
        return self._read(self._norm(x))

    def forward(self, x, body, ctx: Context):
        b, t, n, d = x.shape
        r = self._norm(x)
        y = body(self._read(r), ctx)
        weight = 2 * torch.sigmoid(r.reshape(b, t, n * d).float() @ self.write_proj.float().t() / n)
        return x + weight.to(y.dtype).unsqueeze(-1) * y.unsqueeze(2)


def sources(state: torch.Tensor, block_size: Optional[int]) -> torch.Tensor:
    """What attnres reads from: the embedding, then every output (or sums of blocks of
    `block_size` outputs, the block under way included once it has one)."""
    if block_size is None:
        return state
    b, t, s, d = state.shape
    outputs = state[:, :, 1:]
    full = (s - 1) // block_size
    parts = [state[:, :, :1], outputs[:, :, : full * block_size].reshape(b, t, full, block_size, d).sum(3)]
    if full * block_size < s - 1:
        parts.append(outputs[:, :, full * block_size:].sum(2, keepdim=True))
    return torch.cat(parts, 2)


class AttentionResidual(nn.Module):
    """f reads the softmax over the sources v of dot(w, rmsnorm(v)); w starts at 0 (their
    average). f's output joins the state."""

    def __init__(self, c: L.AttentionResidualConfig, d: int, write: bool = True):
        super().__init__()
        self.query = nn.Parameter(torch.zeros(d))
        self.key_gain = nn.Parameter(torch.ones(d))
        self.block_size, self.eps = c.block_size, c.norm_eps

    def read(self, x, ctx=None):
        v = sources(x, self.block_size)
        keys = _rms(v, self.eps).float() * self.key_gain
        scores = torch.einsum("btmd,d->btm", keys, self.query.float())
        return weighted(torch.softmax(scores, -1), v)

    def forward(self, x, body, ctx: Context):
        y = body(self.read(x), ctx)
        return torch.cat([x, y.unsqueeze(2)], 2)


def _msar_layout(s: int, block: int, expansions: int):
    """(finished blocks, outputs of the block under way) of an msar state of s entries;
    None for a fresh one (the embedding alone)."""
    if s == 1:
        return None
    rest = s - 1 - (1 + expansions)
    width = block + expansions
    k = (rest - 1) % width + 1
    if rest < 1 or k > block:
        raise ValueError(f"msar: a state of {s} entries is none of blocks of {block}")
    return (rest - k) // width, k


class MultiStreamAttentionResidual(nn.Module):
    """Block MSAR: each source (embedding, finished block sums, the block under way)
    expands into m streams (itself and causal depthwise convs of it); per stream a
    softmax over depth, then a sigmoid mix over the streams."""

    no_weight_decay = ("scale", "bias")

    def __init__(self, c: L.MultiStreamAttentionResidualConfig, d: int, write: bool = True):
        super().__init__()
        self.eps = c.norm_eps
        self.block = c.block_size or 1
        self.expansions = len(c.kernel_sizes)
        if not write:
            return
        m = 1 + self.expansions
        self.convs = nn.ModuleList(CausalDepthwise(d, k, zero=True) for k in c.kernel_sizes)
        self.query = nn.Parameter(torch.zeros(m, d))
        self.proj = nn.Parameter(torch.zeros(m * d, m))
        self.scale = nn.Parameter(torch.tensor(0.01))
        self.bias = nn.Parameter(torch.full((m,), -math.log(max(m - 1, 1))))

    def read(self, x, ctx=None):
        return x[:, :, 0] if x.shape[2] == 1 else x[:, :, -1]

    def _sources(self, x, at):
        b, t, _, d = x.shape
        m = self.expansions + 1
        if at is None:
            return x.new_zeros(b, t, 0, m, d), x[:, :, 0], True
        blocks, under_way = at
        width = self.block + m - 1
        streams = [x[:, :, :m]]
        for j in range(blocks):
            first = m + j * width
            total = x[:, :, first: first + self.block].sum(2, keepdim=True)
            streams.append(torch.cat([total, x[:, :, first + self.block: first + width]], 2))
        newest = m + blocks * width
        return torch.stack(streams, 2), x[:, :, newest: newest + under_way].sum(2), under_way == self.block

    def _mix(self, src):
        b, t, _, m, d = src.shape
        scores = torch.einsum("btnmd,md->btnm", _rms(src, self.eps).float(), self.query.float())
        z = torch.einsum("btnm,btnmd->btmd", torch.softmax(scores, 2).to(src.dtype), src)
        flat = z.reshape(b, t, m * d).float()
        rms = torch.rsqrt(flat.square().mean(-1, keepdim=True) + self.eps)
        logits = (flat @ self.proj.float()) * rms * self.scale + self.bias
        return weighted(torch.sigmoid(logits), z)

    def forward(self, x, body, ctx: Context):
        at = _msar_layout(x.shape[2], self.block, self.expansions)
        done, newest, finished = self._sources(x, at)
        expanded = torch.stack([newest, *(conv(newest, ctx) for conv in self.convs)], 2)
        h = self._mix(torch.cat([done, expanded.unsqueeze(2)], 2))
        y = body(h, ctx)
        kept = x if at is None else x[:, :, :-1]
        new = [kept, expanded[:, :, 1:]] if finished else [kept]
        new += [y.unsqueeze(2), (h + y).unsqueeze(2)]
        return torch.cat(new, 2)


class ResidualGate(nn.Module):
    """x' = a·x + b·f(x) per channel, b = sigmoid(g / T), a = sqrt(max(1 - b², eps));
    branch k starts at b = 1/sqrt(k+2)."""

    def __init__(self, c: L.ResidualGateConfig, d: int, index: int):
        super().__init__()
        b = 1 / math.sqrt(index + 2)
        self.gate = nn.Parameter(torch.full((d,), c.temperature * math.log(b / (1 - b))))
        self.temperature, self.eps = c.temperature, c.eps

    def weights(self):
        w = self.gate.float() / self.temperature
        b = torch.sigmoid(w)
        return torch.sqrt(torch.clamp(torch.sigmoid(-w) * (1 + b), min=self.eps)), b

    def forward(self, x, body, ctx: Context):
        a, b = self.weights()
        return a.to(x.dtype) * x + b.to(x.dtype) * body(x, ctx)


def build(residual, d: int, index: int = 0, write: bool = True) -> nn.Module:
    if isinstance(residual, L.HyperConnectionsConfig):
        cls = HyperConnections if residual.type == "hc" else ManifoldHyperConnections
        return cls(residual, d, index, write)
    if isinstance(residual, L.GatedResidualConfig):
        return GatedResidual(residual, d, write)
    if isinstance(residual, L.AttentionResidualConfig):
        return AttentionResidual(residual, d, write)
    if isinstance(residual, L.MultiStreamAttentionResidualConfig):
        return MultiStreamAttentionResidual(residual, d, write)
    if isinstance(residual, L.ResidualGateConfig):
        return ResidualGate(residual, d, index)
    raise ValueError("merge reads a widened residual stream, but there is none")


class Merge(nn.Module):
    """The read of a widened stream back into one. Single-pass hc / mhc read with the
    coefficients the last branch computed."""

    def __init__(self, reader: Optional[nn.Module]):
        super().__init__()
        if reader is not None:
            self.reader = reader

    def forward(self, x, ctx: Context):
        reader = getattr(self, "reader", None)
        if reader is None:
            return weighted(_pending(ctx, x), x)
        return reader.read(x, ctx)


@register("merge")
def _merge(c, b: BuildContext):
    r = b.residual
    if isinstance(r, L.HyperConnectionsConfig) and r.single_pass:
        return Merge(None)
    return Merge(build(r, b.d_model, write=False))
