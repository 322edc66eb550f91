"""Differentiable front ends of the native kernels (torch.autograd Functions).

Each op has two implementations with the same contract:
  * CUDA tensors: the hand-written sm_100a kernels through ``momijo_b200._C`` (no fallback);
  * CPU tensors: plain torch in fp32 (so the framework and its tests run without a GPU).

Weight gradients can be written straight into a flat gradient buffer: when a parameter carries
a ``main_grad`` view (set by the sharded/data-parallel wrappers) the backward GEMM stores or
accumulates into it and autograd receives ``None`` for that parameter.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as tF

from .. import _C
from .gemm import gemm, _gelu_tanh, _gelu_tanh_grad

bf16 = torch.bfloat16


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
def _wgrad_target(p):
    """(buffer, accumulate) when ``p`` owns a slice of a flat gradient buffer, else (None, False)."""
    mg = getattr(p, "main_grad", None)
    if mg is None:
        return None, False
    acc = not getattr(p, "_mg_fresh", False)
    p._mg_fresh = False
    return mg, acc


def _colsum(x2d, out=None, accumulate=False):
    """Column sums of a bf16 matrix -> bf16 vector (bias gradient)."""
    M, N = x2d.shape
    if out is None:
        out = torch.empty(N, dtype=bf16, device=x2d.device)
        accumulate = False
    if not x2d.is_cuda:
        s = x2d.float().sum(0)
        if accumulate:
            s = s + out.float()
        out.copy_(s.to(out.dtype))
        return out
    S = _C.lib().mmj_colsum_splits(M)
    scratch = torch.empty(S * N, dtype=torch.float32, device=x2d.device)
    f32 = out.dtype == torch.float32   # fp32 gradient buffers take the sums unrounded
    _C.call("mmj_colsum_bf16", _C.ptr(x2d), x2d.stride(0), None if f32 else _C.ptr(out), _C.ptr(out) if f32 else None,
            _C.ptr(scratch), M, N, int(accumulate), _C.current_stream())
    return out


def _bias_grad(b, dy2d):
    if b is None:
        return None
    buf, acc = _wgrad_target(b)
    if buf is not None:
        _colsum(dy2d, out=buf, accumulate=acc)
        return None
    return _colsum(dy2d)


def _weight_grad(w, dy2d, x2d):
    """dW[N, K] = dy^T x, into main_grad when present."""
    buf, acc = _wgrad_target(w)
    if buf is not None:
        gemm(dy2d, x2d, a_mn=True, b_mn=True, out=buf, accumulate=acc)
        return None
    return gemm(dy2d, x2d, a_mn=True, b_mn=True)


# --------------------------------------------------------------------------------------------
# linear / MLP
# --------------------------------------------------------------------------------------------
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual):
        x2 = x.reshape(-1, x.shape[-1])
        res2 = residual.reshape(-1, w.shape[0]) if residual is not None else None
        zg = getattr(w, "_zero_gather", None)
        if zg is not None and zg.pending:
            # sharded data parallel: the other ranks' pieces of this weight have not been gathered
            # yet; this GEMM pulls them over NVLink while it computes (and leaves w complete)
            y = zg.gemm(x2, w, bias=b, add_aux=res2)
        else:
            y = gemm(x2, w, bias=b, add_aux=res2)
        ctx.save_for_backward(x2, w)
        ctx.b = b
        ctx.w_ref = w
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = gemm(dy2, w, b_mn=True).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(ctx.w_ref, dy2, x2) if ctx.needs_input_grad[1] else None
        db = _bias_grad(ctx.b, dy2) if (ctx.b is not None and ctx.needs_input_grad[2]) else None
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


def linear(x, w, b=None, residual=None):
    """y = x @ w.T + b (+ residual). x: [..., K] bf16, w: [N, K] bf16."""
    if x.dtype != bf16 or not x.is_cuda:
        y = tF.linear(x, w.to(x.dtype), None if b is None else b.to(x.dtype))
        return y if residual is None else y + residual
    return _Linear.apply(x, w, b, residual)


class _MlpGelu(torch.autograd.Function):
    """fc1 -> GELU(tanh) -> fc2 (+ residual) with the activation fused into both GEMM epilogues."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        x2 = x.reshape(-1, x.shape[-1])
        act, pre = gemm(x2, w1, bias=b1, gelu=True)
        res2 = residual.reshape(-1, w2.shape[0]) if residual is not None else None
        y = gemm(act, w2, bias=b2, add_aux=res2)
        ctx.save_for_backward(x2, w1, w2, pre, act)
        ctx.refs = (w1, b1, w2, b2)
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, pre, act = ctx.saved_tensors
        rw1, rb1, rw2, rb2 = ctx.refs
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dw2 = _weight_grad(rw2, dy2, act)
        db2 = _bias_grad(rb2, dy2)
        dpre = gemm(dy2, w2, b_mn=True, dgelu_aux=pre)  # (dy @ W2) * gelu'(pre)
        dw1 = _weight_grad(rw1, dpre, x2)
        db1 = _bias_grad(rb1, dpre)
        dx = gemm(dpre, w1, b_mn=True).view(ctx.xshape)
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None)


def mlp_gelu(x, w1, b1, w2, b2, residual=None):
    if x.dtype != bf16 or not x.is_cuda:
        h = _gelu_tanh(tF.linear(x, w1.to(x.dtype), None if b1 is None else b1.to(x.dtype)))
        y = tF.linear(h, w2.to(x.dtype), None if b2 is None else b2.to(x.dtype))
        return y if residual is None else y + residual
    return _MlpGelu.apply(x, w1, b1, w2, b2, residual)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * F)
        y = torch.empty((g2.shape[0], F), dtype=bf16, device=gu.device)
        _C.call("mmj_swiglu_fwd", _C.ptr(g2), _C.ptr(y), g2.shape[0], F, _C.current_stream())
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return y.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        F = g2.shape[1] // 2
        dy2 = dy.reshape(-1, F).contiguous()
        dgu = torch.empty_like(g2)
        _C.call("mmj_swiglu_bwd", _C.ptr(g2), _C.ptr(dy2), _C.ptr(dgu), g2.shape[0], F,
                _C.current_stream())
        return dgu.view(ctx.shape)


def swiglu(gu):
    """silu(gate) * up where gate/up are the two halves of the last dimension."""
    if gu.dtype != bf16 or not gu.is_cuda or (gu.shape[-1] // 2) % 8:
        g, u = gu.chunk(2, dim=-1)
        return tF.silu(g) * u
    return _SwiGLU.apply(gu.contiguous())


_ACT_IDS = {"gelu": 0, "silu": 1, "relu": 2, "leaky_relu": 3, "sigmoid": 4, "tanh": 5}


class _Act(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, alpha):
        x = x.contiguous()
        y = torch.empty_like(x)
        _C.call("mmj_act_fwd", _C.ptr(x), _C.ptr(y), x.numel(), op, alpha, _C.current_stream())
        ctx.save_for_backward(x)
        ctx.op, ctx.alpha = op, alpha
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        _C.call("mmj_act_bwd", _C.ptr(x), _C.ptr(dy), _C.ptr(dx), x.numel(), ctx.op, ctx.alpha,
                _C.current_stream())
        return dx, None, None


def activation(x, kind: str, alpha: float = 0.01):
    if x.dtype != bf16 or not x.is_cuda or x.numel() % 8:
        if kind == "gelu":
            return _gelu_tanh(x)
        if kind == "silu":
            return tF.silu(x)
        if kind == "relu":
            return torch.relu(x)
        if kind == "leaky_relu":
            return tF.leaky_relu(x, alpha)
        if kind == "sigmoid":
            return torch.sigmoid(x)
        return torch.tanh(x)
    return _Act.apply(x, _ACT_IDS[kind], float(alpha))


# --------------------------------------------------------------------------------------------
# normalisation
# --------------------------------------------------------------------------------------------
class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, residual, eps, mode):
        C = x.shape[-1]
        x2 = x.reshape(-1, C)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if mode == 0 else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        res2 = residual.reshape(-1, C) if residual is not None else None
        res_out = torch.empty_like(x2) if residual is not None else None
        _C.call("mmj_norm_fwd", _C.ptr(x2), _C.ptr(res2), _C.ptr(res_out), _C.ptr(gamma),
                _C.ptr(beta), _C.ptr(y), _C.ptr(mean), _C.ptr(rstd), rows, C, eps, mode,
                _C.ptr(_C.status_tensor(x.device)), _C.current_stream())
        xin = res_out if residual is not None else x2
        ctx.save_for_backward(xin, gamma, mean if mean is not None else rstd, rstd)
        ctx.refs = (gamma, beta)
        ctx.mode = mode
        ctx.shape = x.shape
        ctx.has_res = residual is not None
        if residual is not None:
            return y.view(x.shape), res_out.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dres_out):
        xin, gamma, mean, rstd = ctx.saved_tensors
        rgamma, rbeta = ctx.refs
        C = xin.shape[1]
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, C)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres2 = None
        if dres_out is not None:
            dres2 = dres_out.reshape(-1, C)
            if not dres2.is_contiguous():
                dres2 = dres2.contiguous()
        dx = torch.empty_like(xin)
        nparts = _C.lib().mmj_norm_bwd_parts(rows)
        scratch = torch.empty(2 * nparts * C, dtype=torch.float32, device=xin.device)
        gbuf, gacc = _wgrad_target(rgamma)
        bbuf, bacc = _wgrad_target(rbeta) if rbeta is not None else (None, False)
        direct = gbuf is not None and gbuf.dtype == bf16 and (rbeta is None or bbuf is not None) and (
            rbeta is None or gacc == bacc)
        if direct:
            dg, db, acc = gbuf, bbuf, gacc
        else:
            dg = torch.empty(C, dtype=bf16, device=xin.device)
            db = torch.empty(C, dtype=bf16, device=xin.device) if rbeta is not None else None
            acc = False
        _C.call("mmj_norm_bwd", _C.ptr(dy2), _C.ptr(xin), _C.ptr(gamma),
                _C.ptr(mean) if ctx.mode == 0 else None, _C.ptr(rstd), _C.ptr(dres2), _C.ptr(dx),
                _C.ptr(dg), _C.ptr(db), _C.ptr(scratch), rows, C, ctx.mode, int(acc),
                _C.ptr(_C.status_tensor(xin.device)), _C.current_stream())
        if direct:
            dg_ret, db_ret = None, None
        else:
            dg_ret, db_ret = dg, db
            if gbuf is not None:  # mixed case: fold manually
                gbuf.copy_(gbuf + dg if gacc else dg)
                dg_ret = None
            if bbuf is not None:
                bbuf.copy_(bbuf + db if bacc else db)
                db_ret = None
        dxv = dx.view(ctx.shape)
        # with a fused residual the same gradient flows to both x and residual
        return dxv, dg_ret, db_ret, (dxv if ctx.has_res else None), None, None


def _norm_ref(x, gamma, beta, residual, eps, mode):
    if residual is not None:
        x = x + residual
    xf = x.float()
    if mode == 0:
        y = tF.layer_norm(xf, (x.shape[-1],), gamma.float(), None if beta is None else beta.float(), eps)
    else:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    y = y.to(x.dtype)
    return (y, x) if residual is not None else (y, None)


def layer_norm(x, gamma, beta, eps=1e-5, residual=None):
    """LayerNorm over the last dim. With ``residual`` returns (norm(x + residual), x + residual)."""
    if x.dtype != bf16 or not x.is_cuda or x.shape[-1] % 8 or x.shape[-1] > 8192:
        y, r = _norm_ref(x, gamma, beta, residual, eps, 0)
    else:
        y, r = _Norm.apply(x.contiguous(), gamma, beta,
                           None if residual is None else residual.contiguous(), eps, 0)
    return (y, r) if residual is not None else y


def rms_norm(x, gamma, eps=1e-5, residual=None):
    if x.dtype != bf16 or not x.is_cuda or x.shape[-1] % 8 or x.shape[-1] > 8192:
        y, r = _norm_ref(x, gamma, None, residual, eps, 1)
    else:
        y, r = _Norm.apply(x.contiguous(), gamma, None,
                           None if residual is None else residual.contiguous(), eps, 1)
    return (y, r) if residual is not None else y


# --------------------------------------------------------------------------------------------
# rotary embedding
# --------------------------------------------------------------------------------------------
_ROPE_CACHE = {}


def rope_table(T: int, D: int, theta: float, device):
    """[T, D/2, 2] fp32 table of (cos, sin) for the half-split rotary embedding."""
    key = (T, D, float(theta), str(device))
    t = _ROPE_CACHE.get(key)
    if t is None:
        inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
        t = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()
        _ROPE_CACHE[key] = t
    return t


def rope_inplace(x2d, table, head_off, n_heads, D, T, sign=1.0):
    """Rotate ``n_heads`` heads that start at column ``head_off`` of a [rows, ld] bf16 matrix."""
    if not x2d.is_cuda:
        rows = x2d.shape[0]
        half = D // 2
        pos = torch.arange(rows, device=x2d.device) % T
        cs = table[pos]  # [rows, half, 2]
        c, s = cs[..., 0][:, None, :], sign * cs[..., 1][:, None, :]
        v = x2d[:, head_off:head_off + n_heads * D].reshape(rows, n_heads, D).float()
        a, b = v[..., :half], v[..., half:]
        out = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
        x2d[:, head_off:head_off + n_heads * D] = out.reshape(rows, n_heads * D).to(x2d.dtype)
        return x2d
    _C.call("mmj_rope", _C.ptr(x2d), _C.ptr(table), x2d.shape[0], x2d.stride(0), head_off, n_heads,
            D, T, float(sign), _C.current_stream())
    return x2d


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def _attn_ref(q, k, v, causal, scale):
    """q: [B, Hq, T, D], k/v: [B, Hkv, T, D] -> [B, Hq, T, D], fp32 softmax."""
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    if Hkv != Hq:
        k = k.repeat_interleave(Hq // Hkv, dim=1)
        v = v.repeat_interleave(Hq // Hkv, dim=1)
    s = (q.float() @ k.float().transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ v.float()).to(q.dtype)


class _AttnPacked(torch.autograd.Function):
    """Causal/full attention on a packed [B*T, (Hq + 2*Hkv)*D] projection (Q | K | V)."""

    @staticmethod
    def forward(ctx, qkv, B, T, Hq, Hkv, D, causal, scale, rope):
        qkv = qkv.contiguous()
        ld = qkv.shape[1]
        qc, kc, vc = 0, Hq * D, (Hq + Hkv) * D
        if rope is not None:
            qkv = qkv.clone()
            rope_inplace(qkv, rope, qc, Hq, D, T, 1.0)
            rope_inplace(qkv, rope, kc, Hkv, D, T, 1.0)
        out = torch.empty((B * T, Hq * D), dtype=bf16, device=qkv.device)
        lse = torch.empty((B, Hq, T), dtype=torch.float32, device=qkv.device)
        st = _C.status_tensor(qkv.device)
        _C.call("mmj_attn_fwd", _C.ptr(qkv), ld, qc, _C.ptr(qkv), ld, kc, _C.ptr(qkv), ld, vc,
                _C.ptr(out), out.stride(0), 0, _C.ptr(lse), B, T, Hq, Hkv, D, scale, int(causal),
                _C.ptr(st), _C.current_stream())
        ctx.save_for_backward(qkv, out, lse)
        ctx.cfg = (B, T, Hq, Hkv, D, causal, scale)
        ctx.rope = rope
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        B, T, Hq, Hkv, D, causal, scale = ctx.cfg
        ld = qkv.shape[1]
        qc, kc, vc = 0, Hq * D, (Hq + Hkv) * D
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        dq_acc = torch.empty((B * T, Hq * D), dtype=torch.float32, device=qkv.device)   # cleared by the kernel
        delta = torch.empty((B, Hq, T), dtype=torch.float32, device=qkv.device)
        st = _C.status_tensor(qkv.device)
        _C.call("mmj_attn_bwd", _C.ptr(qkv), ld, qc, _C.ptr(qkv), ld, kc, _C.ptr(qkv), ld, vc,
                _C.ptr(out), out.stride(0), 0, _C.ptr(dout), dout.stride(0), 0, _C.ptr(lse),
                _C.ptr(delta), _C.ptr(dq_acc), dq_acc.stride(0), 0, _C.ptr(dqkv), ld, kc,
                _C.ptr(dqkv), ld, vc, B, T, Hq, Hkv, D, scale, int(causal), _C.ptr(st),
                _C.current_stream())
        _C.call("mmj_cast_f32_to_bf16_2d", _C.ptr(dq_acc), dq_acc.stride(0), _C.ptr(dqkv), ld,
                B * T, Hq * D, _C.current_stream())
        if ctx.rope is not None:
            rope_inplace(dqkv, ctx.rope, qc, Hq, D, T, -1.0)
            rope_inplace(dqkv, ctx.rope, kc, Hkv, D, T, -1.0)
        return dqkv, None, None, None, None, None, None, None, None


def attention_packed(qkv, B, T, Hq, Hkv, D, causal=True, scale=None, rope=None):
    """qkv: [B*T, (Hq+2Hkv)*D] -> [B*T, Hq*D]. ``rope``: table from ``rope_table`` or None."""
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if qkv.dtype == bf16 and qkv.is_cuda and D in (64, 128):
        return _AttnPacked.apply(qkv, B, T, Hq, Hkv, D, bool(causal), float(scale), rope)
    x = qkv
    if rope is not None:
        x = x.clone()
        # differentiable rotation for the reference path
        rows = x.shape[0]
        half = D // 2
        pos = torch.arange(rows, device=x.device) % T
        cs = rope[pos]
        c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]

        def rot(v, n):
            v = v.reshape(rows, n, D).float()
            a, b = v[..., :half], v[..., half:]
            return torch.cat([a * c - b * s, b * c + a * s], dim=-1).reshape(rows, n * D).to(qkv.dtype)

        q2 = rot(qkv[:, :Hq * D], Hq)
        k2 = rot(qkv[:, Hq * D:(Hq + Hkv) * D], Hkv)
        x = torch.cat([q2, k2, qkv[:, (Hq + Hkv) * D:]], dim=1)
    q = x[:, :Hq * D].reshape(B, T, Hq, D).transpose(1, 2)
    k = x[:, Hq * D:(Hq + Hkv) * D].reshape(B, T, Hkv, D).transpose(1, 2)
    v = x[:, (Hq + Hkv) * D:].reshape(B, T, Hkv, D).transpose(1, 2)
    o = _attn_ref(q, k, v, causal, scale)
    return o.transpose(1, 2).reshape(B * T, Hq * D)


# --------------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tok, wte, wpe, T):
        tok1 = tok.reshape(-1).contiguous()
        rows, C = tok1.numel(), wte.shape[1]
        out = torch.empty((rows, C), dtype=bf16, device=wte.device)
        _C.call("mmj_embedding_fwd", _C.ptr(tok1), _C.ptr(wte), _C.ptr(wpe), _C.ptr(out), rows, C,
                T, wte.shape[0], _C.current_stream())
        ctx.save_for_backward(tok1)
        ctx.refs = (wte, wpe)
        ctx.T = T
        return out.view(*tok.shape, C)

    @staticmethod
    def backward(ctx, dout):
        (tok1,) = ctx.saved_tensors
        wte, wpe = ctx.refs
        C = wte.shape[1]
        d2 = dout.reshape(-1, C).contiguous()
        rows = d2.shape[0]
        ebuf, eacc = _wgrad_target(wte)
        fold_wte = ebuf is not None and ebuf.dtype != bf16   # fp32 gradient buffer: scatter in bf16, then fold
        if ebuf is None or fold_wte:
            dwte = torch.zeros_like(wte)
        else:
            dwte = ebuf
            if not eacc:
                dwte.zero_()
        dwpe, pacc, fold_wpe = None, False, False
        if wpe is not None:
            pbuf, pacc = _wgrad_target(wpe)
            fold_wpe = pbuf is not None and pbuf.dtype != bf16
            pacc_buf = pacc
            dwpe = pbuf if (pbuf is not None and not fold_wpe) else torch.empty_like(wpe)
            if pbuf is None or fold_wpe:
                pacc = False
            if wpe.shape[0] > ctx.T and not pacc:
                dwpe.zero_()
        _C.call("mmj_embedding_bwd", _C.ptr(tok1), _C.ptr(d2), _C.ptr(dwte), _C.ptr(dwpe), rows, C,
                ctx.T, wte.shape[0], int(pacc), _C.current_stream())
        if fold_wte:
            if eacc:
                ebuf.add_(dwte)
            else:
                ebuf.copy_(dwte)
        if wpe is not None and fold_wpe:
            if pacc_buf:
                pbuf.add_(dwpe)
            else:
                pbuf.copy_(dwpe)
        return (None, None if ebuf is not None else dwte,
                None if (wpe is None or getattr(wpe, "main_grad", None) is not None) else dwpe, None)


def embedding(tok, wte, wpe=None, T=None):
    """wte[tok] (+ wpe[position]); tok: int64 [B, T]."""
    if T is None:
        T = tok.shape[-1]
    if not wte.is_cuda or wte.dtype != bf16:
        y = tF.embedding(tok, wte)
        if wpe is not None:
            y = y + wpe[:T]
        return y
    return _Embedding.apply(tok, wte, wpe, T)


# --------------------------------------------------------------------------------------------
# LM head + cross entropy
# --------------------------------------------------------------------------------------------
def pad_vocab(V: int, mult: int = 128) -> int:
    return (V + mult - 1) // mult * mult


def _inv_valid(t1, ignore_index):
    """Device scalar 1 / max(1, #targets != ignore_index): the factor of a mean over counted rows."""
    inv = torch.empty(1, dtype=torch.float32, device=t1.device)
    _C.call("mmj_ce_count_valid", _C.ptr(t1), t1.numel(), ignore_index, _C.ptr(inv), _C.current_stream())
    return inv


def softmax_cross_entropy(logits, targets, ignore_index=-100, reduction="mean"):
    """Fused softmax cross-entropy returning (loss, dlogits) like the reference's
    ``softmax_cross_entropy`` (legacy/src/momijo/learn/losses/losses.mojo:72-85);
    ``dlogits`` is the gradient of the reduced loss with respect to the logits. The mean runs over
    the rows whose target is not ``ignore_index`` (on both the CUDA and the CPU path)."""
    V = logits.shape[-1]
    l2 = logits.reshape(-1, V)
    t1 = targets.reshape(-1).contiguous()
    n = l2.shape[0]
    if l2.is_cuda and l2.dtype == bf16:
        work_buf = torch.empty((n, (V + 7) // 8 * 8), dtype=bf16, device=l2.device)
        work = work_buf[:, :V]
        work.copy_(l2)
        loss_row = torch.empty(n, dtype=torch.float32, device=l2.device)
        inv = _inv_valid(t1, ignore_index) if reduction == "mean" else None
        _C.call("mmj_ce_fwd_bwd", _C.ptr(work), work.stride(0), V, _C.ptr(t1), _C.ptr(loss_row), n,
                1.0, _C.ptr(inv), ignore_index, 1, _C.current_stream())
        loss = torch.empty(1, dtype=torch.float32, device=l2.device)
        _C.call("mmj_reduce_mean", _C.ptr(loss_row), _C.ptr(loss), n, 1.0, _C.ptr(inv),
                _C.current_stream())
        return loss[0], work.reshape(logits.shape)
    lf = l2.float()
    logp = torch.log_softmax(lf, dim=-1)
    valid = t1 != ignore_index
    tt = t1.clamp(min=0)
    loss_row = -(logp.gather(1, tt[:, None])[:, 0]) * valid
    d = (torch.softmax(lf, -1) - tF.one_hot(tt, V).float()) * valid[:, None]
    if reduction == "mean":
        nv = valid.sum().clamp(min=1)
        return loss_row.sum() / nv, (d / nv).to(logits.dtype).view(logits.shape)
    return loss_row.sum(), d.to(logits.dtype).view(logits.shape)


class _LMHeadCE(torch.autograd.Function):
    """logits = x @ wte.T, cross-entropy averaged over the counted rows, with dlogits produced in the
    forward pass (in place over the logits) so the backward is two GEMMs. The incoming loss gradient is
    a device scalar: a kernel that leaves at once when it equals 1 scales dlogits by it otherwise, so
    that both gradient products (the weight gradient written straight into a flat ``main_grad`` buffer
    included) carry the factor, without a host synchronisation."""

    @staticmethod
    def forward(ctx, x, wte, targets, V, ignore_index):
        x2 = x.reshape(-1, x.shape[-1])
        M = x2.shape[0]
        Vp = pad_vocab(V)
        logits = torch.empty((M, Vp), dtype=bf16, device=x.device)
        gemm(x2, wte, out=logits[:, :wte.shape[0]] if wte.shape[0] != Vp else logits)
        t1 = targets.reshape(-1).contiguous()
        loss_row = torch.empty(M, dtype=torch.float32, device=x.device)
        inv = _inv_valid(t1, ignore_index)
        _C.call("mmj_ce_fwd_bwd", _C.ptr(logits), logits.stride(0), V, _C.ptr(t1), _C.ptr(loss_row),
                M, 1.0, _C.ptr(inv), ignore_index, 1, _C.current_stream())
        loss = torch.empty(1, dtype=torch.float32, device=x.device)
        _C.call("mmj_reduce_mean", _C.ptr(loss_row), _C.ptr(loss), M, 1.0, _C.ptr(inv), _C.current_stream())
        ctx.save_for_backward(x2, wte, logits)
        ctx.w_ref = wte
        ctx.xshape = x.shape
        ctx.consumed = False
        return loss[0]

    @staticmethod
    def backward(ctx, dloss):
        x2, wte, dlogits = ctx.saved_tensors
        if ctx.consumed:
            raise RuntimeError("lm_head_cross_entropy keeps its logit gradient in place: backward runs once")
        ctx.consumed = True
        nrow = wte.shape[0]
        dl = dlogits[:, :nrow]
        ds = dloss.detach().reshape(1).to(torch.float32)
        _C.call("mmj_scale_bf16_dev", _C.ptr(dlogits), dlogits.stride(0), dlogits.shape[0],
                dlogits.shape[1], _C.ptr(ds), _C.current_stream())
        dx = gemm(dl, wte, b_mn=True)
        dw = _weight_grad(ctx.w_ref, dl, x2)
        return dx.view(ctx.xshape), dw, None, None, None


def lm_head_cross_entropy(x, wte, targets, vocab_size, ignore_index=-100):
    """Mean next-token loss of ``x @ wte.T`` against ``targets`` (tied or untied head)."""
    if not x.is_cuda or x.dtype != bf16:
        logits = tF.linear(x.reshape(-1, x.shape[-1]), wte.to(x.dtype))[:, :vocab_size]
        return tF.cross_entropy(logits.float(), targets.reshape(-1), ignore_index=ignore_index)
    return _LMHeadCE.apply(x, wte, targets, vocab_size, ignore_index)
