"""Autograd functions over the trainer kernels (csrc/kernels/train_kernels.cu,
gemm_kernels.cu). CUDA tensors always run the sm_100a kernels; CPU tensors run a
plain PyTorch restatement of the same math, which is what the multi-process
`gloo` tests of the parallel layers use (there is no GPU fallback path).

Weight gradients follow the Megatron convention: when a parameter carries a
`.main_grad` fp32 buffer, backward accumulates into it (wgrad GEMM with fp32
accumulate epilogue) and returns None for that parameter.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _lib
from . import gemm as G

_scratch: dict[tuple, torch.Tensor] = {}


def scratch(device, nfloats: int, tag: str = "") -> torch.Tensor:
    """Per-device, per-tag fp32 scratch buffer that only ever grows (stream-ordered reuse)."""
    key = (device.index, tag)
    t = _scratch.get(key)
    if t is None or t.numel() < nfloats:
        t = torch.empty(max(nfloats, 1 << 16), dtype=torch.float32, device=device)
        _scratch[key] = t
    return t


def _accum_param_grad(p: torch.Tensor, g_fp32_or_none, compute):
    """compute(out_fp32, accumulate) writes the gradient; returns what autograd should see."""
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        compute(mg, True)
        return None
    out = torch.empty(p.shape, dtype=torch.float32, device=p.device)
    compute(out, False)
    return out.to(p.dtype)


# --------------------------------------------------------------------------- LayerNorm (+ residual add)
class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, gamma, beta, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        M = x2.shape[0]
        has_res = res is not None
        if x.is_cuda:
            x2 = x2.contiguous()
            r2 = res.reshape(-1, H).contiguous() if has_res else None
            y = torch.empty_like(x2)
            xo = torch.empty_like(x2) if has_res else None
            mean = torch.empty(M, dtype=torch.float32, device=x.device)
            rstd = torch.empty(M, dtype=torch.float32, device=x.device)
            rc = _lib.lib().cocclkLayerNormFwd(x2.data_ptr(), _lib.ptr(r2), gamma.data_ptr(), beta.data_ptr(),
                                               y.data_ptr(), _lib.ptr(xo), mean.data_ptr(), rstd.data_ptr(), M, H,
                                               eps, _lib.cur_stream())
            _lib.check(rc, "cocclkLayerNormFwd")
            xs = xo if has_res else x2
        else:
            xs = (x2.float() + res.reshape(-1, H).float()).to(x.dtype) if has_res else x2
            xf = xs.float()
            mean = xf.mean(-1)
            rstd = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
            y = (((xf - mean[:, None]) * rstd[:, None]) * gamma.float() + beta.float()).to(x.dtype)
        ctx.save_for_backward(xs, mean, rstd, gamma, beta)
        ctx.has_res = has_res
        ctx.shape = x.shape
        if has_res:
            return y.reshape(x.shape), xs.reshape(x.shape)
        return y.reshape(x.shape), None

    @staticmethod
    def backward(ctx, dy, dxs):
        xs, mean, rstd, gamma, beta = ctx.saved_tensors
        H = xs.shape[-1]
        M = xs.shape[0]
        dy2 = dy.reshape(-1, H)
        dres = dxs.reshape(-1, H) if dxs is not None else None
        if xs.is_cuda:
            dy2 = dy2.contiguous()
            dres = dres.contiguous() if dres is not None else None
            dx = torch.empty_like(xs)
            grid = _lib.lib().cocclkLayerNormBwdGrid(M)
            sc = scratch(xs.device, grid * 2 * H, "ln")

            def run(dg, db, acc):
                rc = _lib.lib().cocclkLayerNormBwd(dy2.data_ptr(), xs.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                                   gamma.data_ptr(), _lib.ptr(dres), dx.data_ptr(), dg.data_ptr(),
                                                   db.data_ptr(), int(acc), sc.data_ptr(), M, H, _lib.cur_stream())
                _lib.check(rc, "cocclkLayerNormBwd")

            mg, mb = getattr(gamma, "main_grad", None), getattr(beta, "main_grad", None)
            if mg is not None and mb is not None:
                run(mg, mb, True)
                dgamma = dbeta = None
            else:
                dg = torch.empty(H, dtype=torch.float32, device=xs.device)
                db = torch.empty(H, dtype=torch.float32, device=xs.device)
                run(dg, db, False)
                dgamma, dbeta = dg.to(gamma.dtype), db.to(beta.dtype)
        else:
            xh = (xs.float() - mean[:, None]) * rstd[:, None]
            d = dy2.float()
            dyg = d * gamma.float()
            c1 = dyg.mean(-1, keepdim=True)
            c2 = (dyg * xh).mean(-1, keepdim=True)
            dxf = rstd[:, None] * (dyg - c1 - xh * c2)
            if dres is not None:
                dxf = dxf + dres.float()
            dx = dxf.to(xs.dtype)
            dg, db = (d * xh).sum(0), d.sum(0)
            dgamma = _cpu_param_grad(gamma, dg)
            dbeta = _cpu_param_grad(beta, db)
        dx = dx.reshape(ctx.shape)
        return dx, (dx if ctx.has_res else None), dgamma, dbeta, None


def _cpu_param_grad(p, g32):
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        mg.add_(g32.reshape(mg.shape))
        return None
    return g32.to(p.dtype)


def layer_norm(x, gamma, beta, eps: float = 1e-5, residual=None):
    """y = LN(x + residual); returns (y, x + residual) when a residual is given, else y."""
    y, xs = _LayerNorm.apply(x, residual, gamma, beta, eps)
    return (y, xs) if residual is not None else y


# --------------------------------------------------------------------------- Linear (+bias, +GELU)
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, gelu):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        N = w.shape[0]
        z = None
        if x.is_cuda:
            if gelu:
                y, z = G.gemm(x2, w, bias=bias, gelu=True, save_preact=True)
            else:
                y = G.gemm(x2, w, bias=bias)
        else:
            yf = x2.float() @ w.float().t()
            if bias is not None:
                yf = yf + bias.float()
            if gelu:
                z = yf.to(x.dtype)
                yf = F.gelu(z.float(), approximate="tanh")
            y = yf.to(x.dtype)
        ctx.save_for_backward(x2, w, bias if bias is not None else None, z)
        ctx.gelu = gelu
        ctx.has_bias = bias is not None
        ctx.in_shape = x.shape
        return y.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w, bias, z = ctx.saved_tensors
        N, K = w.shape
        dy2 = dy.reshape(-1, N)
        M = dy2.shape[0]
        if dy2.is_cuda:
            dy2 = dy2.contiguous()
            if ctx.gelu:
                dz = torch.empty_like(dy2)
                rc = _lib.lib().cocclkGeluBwd(dy2.data_ptr(), z.data_ptr(), dz.data_ptr(), dz.numel(), _lib.cur_stream())
                _lib.check(rc, "cocclkGeluBwd")
                dy2 = dz
            dx = G.gemm(dy2, w.t()) if ctx.needs_input_grad[0] else None
            dw = _accum_param_grad(w, None, lambda out, acc: G.gemm(dy2.t(), x2.t(), out=out, accumulate=acc))
            db = None
            if ctx.has_bias:
                def colsum(out, acc):
                    sc = scratch(dy2.device, _lib.lib().cocclkColSumBlocks(M) * N, "colsum")
                    rc = _lib.lib().cocclkColSum(dy2.data_ptr(), out.data_ptr(), int(acc), sc.data_ptr(), M, N,
                                                 _lib.cur_stream())
                    _lib.check(rc, "cocclkColSum")
                db = _accum_param_grad(bias, None, colsum)
        else:
            d = dy2.float()
            if ctx.gelu:
                zf = z.float().requires_grad_(True)
                with torch.enable_grad():
                    a = F.gelu(zf, approximate="tanh")
                d = torch.autograd.grad(a, zf, d)[0].to(dy.dtype).float()
            dx = (d @ w.float()).to(dy.dtype) if ctx.needs_input_grad[0] else None
            dw = _cpu_param_grad(w, d.t() @ x2.float())
            db = _cpu_param_grad(bias, d.sum(0)) if ctx.has_bias else None
        if dx is not None:
            dx = dx.reshape(ctx.in_shape)
        return dx, dw, db, None


def linear(x, w, bias=None, gelu: bool = False):
    """y = act(x @ w.T + bias); w is [out, in]; GELU (tanh form) fused into the GEMM epilogue."""
    return _Linear.apply(x, w, bias, gelu)


# --------------------------------------------------------------------------- cross-entropy
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, scale, unit_grad):
        V = logits.shape[-1]
        lg = logits.reshape(-1, V)
        tg = targets.reshape(-1)
        M = lg.shape[0]
        if lg.is_cuda:
            assert lg.stride(1) == 1
            loss = torch.empty(M, dtype=torch.float32, device=lg.device)
            rc = _lib.lib().cocclkCrossEntropy(lg.data_ptr(), tg.data_ptr(), loss.data_ptr(), M, V, lg.stride(0),
                                               float(scale), _lib.cur_stream())
            _lib.check(rc, "cocclkCrossEntropy")
            grad = lg  # overwritten in place with (softmax - onehot) * scale
        else:
            lf = lg.float()
            lse = torch.logsumexp(lf, -1)
            valid = tg >= 0
            tcl = tg.clamp(min=0)
            loss = torch.where(valid, lse - lf.gather(1, tcl[:, None])[:, 0], torch.zeros_like(lse))
            p = torch.softmax(lf, -1)
            p[torch.arange(M), tcl] -= 1.0
            p = p * valid[:, None]
            grad = (p * scale).to(lg.dtype)
        ctx.save_for_backward(grad)
        ctx.shape = logits.shape
        ctx.unit_grad = unit_grad
        return loss.sum() * scale

    @staticmethod
    def backward(ctx, dloss):
        (grad,) = ctx.saved_tensors
        if not ctx.unit_grad:
            grad = grad * dloss.to(grad.dtype)
        return grad.reshape(ctx.shape), None, None, None


def cross_entropy(logits, targets, scale: float, unit_grad: bool = True):
    """sum_i CE(logits_i, targets_i) * scale. On CUDA the logits buffer is consumed (turned into its gradient).

    unit_grad=True (the trainer's case) assumes the result is the root of backward(), i.e. the incoming
    gradient is 1, and skips one pass over the [tokens, vocab] gradient."""
    return _CrossEntropy.apply(logits, targets, scale, unit_grad)


# --------------------------------------------------------------------------- optimizer kernels
def adam_step(master, m, v, grad, param_bf16, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=None):
    n = master.numel()
    if master.is_cuda:
        rc = _lib.lib().cocclkAdam(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
                                   int(grad.dtype == torch.bfloat16), _lib.ptr(param_bf16), n, lr, beta1, beta2, eps,
                                   weight_decay, step, _lib.ptr(grad_scale), _lib.cur_stream())
        _lib.check(rc, "cocclkAdam")
        return
    g = grad.float() * (grad_scale.item() if grad_scale is not None else 1.0)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * master
    master.add_(upd, alpha=-lr)
    if param_bf16 is not None:
        param_bf16.copy_(master)


def sum_squares(x, out, accumulate=False):
    """out[0] (+)= sum(x^2) without a host sync."""
    if x.is_cuda:
        sc = scratch(x.device, _lib.lib().cocclkSumSqBlocks(x.numel()), "sumsq")
        rc = _lib.lib().cocclkSumSq(x.data_ptr(), int(x.dtype == torch.bfloat16), x.numel(), out.data_ptr(),
                                    int(accumulate), sc.data_ptr(), _lib.cur_stream())
        _lib.check(rc, "cocclkSumSq")
    else:
        s = x.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s


def clip_coef(sumsq, max_norm: float, grad_scale_in: float, coef, norm_out=None):
    if sumsq.is_cuda:
        rc = _lib.lib().cocclkClipCoef(sumsq.data_ptr(), max_norm, grad_scale_in, coef.data_ptr(), _lib.ptr(norm_out),
                                       _lib.cur_stream())
        _lib.check(rc, "cocclkClipCoef")
    else:
        norm = sumsq[0].sqrt() * grad_scale_in
        if norm_out is not None:
            norm_out[0] = norm
        c = 1.0
        if max_norm > 0 and norm > max_norm:
            c = max_norm / (norm + 1e-6)
        coef[0] = c * grad_scale_in
