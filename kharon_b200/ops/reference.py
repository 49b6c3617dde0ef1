"""PyTorch evaluation of every operator, in fp32 math, writing into the caller's buffers.

Used (a) on CPU tensors, where it is the execution path of the CPU test tier and of the
fp32 oracle model, and (b) by the GPU tests as the plain-PyTorch reference each CUDA kernel
is compared against.  Storage dtype follows the tensors passed in (fp32 or bf16).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESID, EPI_DGELU, EPI_RESID = range(6)

_K = 0.79788456
_C = 0.044715


def gelu(x):
    return 0.5 * x * (1.0 + torch.tanh(_K * (x + _C * x * x * x)))


def gelu_grad(x):
    u = _K * (x + _C * x * x * x)
    t = torch.tanh(u)
    return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * _K * (1.0 + 3.0 * _C * x * x)


#: fp32 matrix product used by ``gemm``; the operator layer installs the native CUDA-core kernel
#: for GPU tensors (see ``ops._matmul_f32``), CPU tensors use torch.
matmul_f32 = None


def _mm(A, B):
    if matmul_f32 is not None and A.is_cuda:
        return matmul_f32(A, B)
    return A @ B


def gemm(a, b, out, a_mn, b_mn, accumulate, epi, bias, aux, alpha):
    A = a.float().t() if a_mn else a.float()
    Bm = b.float() if b_mn else b.float().t()
    acc = _mm(A, Bm) * alpha
    if epi in (EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESID):
        acc = acc + bias.float()
    if epi == EPI_BIAS_GELU:
        aux.copy_(acc)
        acc = gelu(aux.float())
    elif epi in (EPI_BIAS_RESID, EPI_RESID):
        acc = acc + aux.float()
    elif epi == EPI_DGELU:
        acc = acc * gelu_grad(aux.float())
    if accumulate:
        out.add_(acc.to(out.dtype))
    else:
        out.copy_(acc)
    return out


def embed_fwd(tok, pos, wte, wpe, out, T):
    rows = out.shape[0]
    p = pos.long() if pos is not None else (torch.arange(rows, device=out.device) % T)
    out.copy_(wte.float()[tok.long()] + wpe.float()[p])
    return out


def embed_bwd(tok, dx, dwte, dwpe, B, T):
    d = dx.shape[1]
    if dwte is not None:
        dwte.index_add_(0, tok.long().reshape(-1), dx.float())
    if dwpe is not None:
        dwpe[:T].add_(dx.float().reshape(B, T, d).sum(0))


def colsum(x, out, accumulate):
    s = x.float().sum(0)
    if accumulate:
        out.add_(s)
    else:
        out.copy_(s)


def layernorm_fwd(x, w, b, y, mean, rstd):
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = ((xf - mu) ** 2).mean(-1, keepdim=True)
    rs = torch.rsqrt(var + 1e-5)
    y.copy_((xf - mu) * rs * w.float() + b.float())
    if mean is not None:
        mean.copy_(mu.squeeze(-1))
    if rstd is not None:
        rstd.copy_(rs.squeeze(-1))
    return y


def layernorm_bwd(dy, x, w, mean, rstd, dres, dx, dw, db):
    g = dy.float()
    xh = (x.float() - mean.float()[:, None]) * rstd.float()[:, None]
    gw = g * w.float()
    s1 = gw.mean(-1, keepdim=True)
    s2 = (gw * xh).mean(-1, keepdim=True)
    o = rstd.float()[:, None] * (gw - s1 - xh * s2)
    if dres is not None:
        o = o + dres.float()
    dw.add_((g * xh).sum(0))
    db.add_(g.sum(0))
    dx.copy_(o)


def xent(logits, V, target, coef, uniform, rowloss, prob, write_grad):
    R = logits.shape[0]
    lg = logits[:, :V].float()
    lse = torch.logsumexp(lg, -1)
    t = target.long()
    valid = (t >= 0) & (t < V)
    ts = t.clamp(0, V - 1)
    xt = lg.gather(1, ts[:, None]).squeeze(1)
    if rowloss is not None:
        rowloss.copy_(torch.where(valid, lse - xt, torch.zeros_like(xt)))
    if prob is not None:
        prob.copy_(torch.where(valid, torch.exp(xt - lse), torch.zeros_like(xt)))
    if write_grad:
        sc = coef.float() if coef is not None else torch.full((R,), float(uniform), device=logits.device)
        sc = torch.where(valid, sc, torch.zeros_like(sc))
        p = torch.exp(lg - lse[:, None])
        onehot = F.one_hot(ts, V).float()
        logits.zero_()
        logits[:, :V] = ((p - onehot) * sc[:, None]).to(logits.dtype)


def xent_stats(logits, V, target, v0, stats):
    lg = logits[:, :V].float()
    m = lg.max(-1).values
    s = torch.exp(lg - m[:, None]).sum(-1)
    t = target.long() - v0
    inside = (t >= 0) & (t < V)
    xt = lg.gather(1, t.clamp(0, V - 1)[:, None]).squeeze(1)
    stats[:, 0] = m
    stats[:, 1] = s
    stats[:, 2] = torch.where(inside, xt, torch.full_like(xt, float("-inf")))


def xent_grad(logits, V, target, v0, gmax, gsum, coef, uniform):
    R = logits.shape[0]
    lg = logits[:, :V].float()
    tg = target.long()
    sc = coef.float() if coef is not None else torch.full((R,), float(uniform), device=logits.device)
    sc = torch.where(tg >= 0, sc, torch.zeros_like(sc))
    p = torch.exp(lg - gmax.float()[:, None]) / gsum.float()[:, None]
    t = tg - v0
    inside = (t >= 0) & (t < V)
    onehot = F.one_hot(t.clamp(0, V - 1), V).float() * inside[:, None].float()
    logits.zero_()
    logits[:, :V] = ((p - onehot) * sc[:, None]).to(logits.dtype)


def adamw(p, g, m, v, pb, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, zero_grad):
    gk = g * grad_scale
    m.mul_(b1).add_(gk, alpha=1.0 - b1)
    v.mul_(b2).addcmul_(gk, gk, value=1.0 - b2)
    p.mul_(1.0 - lr * wd).sub_(lr * (m / bc1) / (torch.sqrt(v / bc2) + eps))
    if pb is not None:
        pb.copy_(p)
    if zero_grad:
        g.zero_()


def _heads(qkv, B, T, H, hd):
    d = H * hd
    x = qkv[:, : 3 * d].float().reshape(B, T, 3, H, hd)
    q, k, v = x[:, :, 0], x[:, :, 1], x[:, :, 2]
    return q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)   # [B,H,T,hd]


def flash_fwd(qkv, out, lse, B, T, H, hd):
    q, k, v = _heads(qkv, B, T, H, hd)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    l = torch.logsumexp(s, -1)
    p = torch.exp(s - l[..., None])
    o = p @ v
    out.copy_(o.transpose(1, 2).reshape(B * T, H * hd))
    if lse is not None:
        lse.copy_(l)


def flash_bwd(qkv, out, dout, lse, dqkv, B, T, H, hd):
    q, k, v = _heads(qkv, B, T, H, hd)
    d = H * hd
    do = dout.float().reshape(B, T, H, hd).transpose(1, 2)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    ds = p * (dp - (dp * p).sum(-1, keepdim=True)) / math.sqrt(hd)
    dq = ds @ k
    dk = ds.transpose(-1, -2) @ q
    res = torch.stack([dq, dk, dv], 0).permute(1, 3, 0, 2, 4).reshape(B * T, 3 * d)
    dqkv[:, : 3 * d] = res.to(dqkv.dtype)


def append_kv(qkv, kc, vc, pos, slot, btab, bs, H, hd, ntok):
    d = H * hd
    p = pos[:ntok].long()
    blk = btab[slot[:ntok].long(), p // bs].long()
    kc[blk, p % bs] = qkv[:ntok, d:2 * d].reshape(ntok, H, hd).to(kc.dtype)
    vc[blk, p % bs] = qkv[:ntok, 2 * d:3 * d].reshape(ntok, H, hd).to(vc.dtype)


def paged_attn(qkv, kc, vc, out, pos, slot, btab, bs, H, hd, ntok):
    d = H * hd
    p = pos[:ntok].long()
    ctx = int(p.max()) + 1
    j = torch.arange(ctx, device=qkv.device)
    blk = btab[slot[:ntok].long()][:, j // bs].long().clamp_(min=0)          # [ntok, ctx]
    K = kc[blk, (j % bs)[None, :]].float()                                   # [ntok, ctx, H, hd]
    Vv = vc[blk, (j % bs)[None, :]].float()
    q = qkv[:ntok, :d].float().reshape(ntok, H, hd)
    s = torch.einsum("the,tjhe->thj", q, K) / math.sqrt(hd)
    s = s.masked_fill((j[None, :] > p[:, None])[:, None, :], float("-inf"))
    out[:ntok] = torch.einsum("thj,tjhe->the", torch.softmax(s, -1), Vv).reshape(ntok, d).to(out.dtype)


def sample(logits, V, temperature, seed, step, rep, out, nseq):
    lg = logits[:nseq, :V].float()
    if temperature <= 0:
        idx = lg.argmax(-1)
        out[:nseq * rep].copy_(idx.repeat_interleave(rep).to(out.dtype))
        return
    g = torch.Generator().manual_seed((int(seed) * 1000003 + int(step)) & 0x7FFFFFFF)
    p = torch.softmax(lg / temperature, -1).cpu()
    idx = torch.multinomial(p, rep, replacement=True, generator=g).to(out.device)
    out[:nseq * rep].copy_(idx.reshape(-1).to(out.dtype))
