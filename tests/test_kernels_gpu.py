"""Numerics of each CUDA kernel against the plain-PyTorch fp32 evaluation of the same op."""
import pytest
import torch

from kharon_b200 import ops
from kharon_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def relerr(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 64, 0), (256, 512, 256, 256), (384, 320, 192, 128), (200, 136, 72, 64),
                                      (1024, 1024, 1024, 0), (8, 1024, 512, 0)])
def test_gemm_majors(a_mn, b_mn, M, N, K, bn):
    torch.manual_seed(0)
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("pitch not 16-byte aligned for this major")
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, b, out, a_mn=a_mn, b_mn=b_mn, block_n=bn)
    want = torch.empty(M, N, device=DEV)
    ref.gemm(a, b, want, a_mn, b_mn, False, 0, None, None, 1.0)
    torch.cuda.synchronize()
    assert ops.error_word() == 0
    assert relerr(out, want) < 6e-3, relerr(out, want)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (384, 328, 192), (1000, 1024, 1024), (4096, 2048, 512)])
def test_gemm_cta_pairs(a_mn, b_mn, M, N, K):
    """256 x 256 tiles on CTA pairs (cta_group::2) against the PyTorch product, ragged edges included."""
    torch.manual_seed(10)
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    bias, resid = _rand(N), _rand(M, N)
    out = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, b, out, a_mn=a_mn, b_mn=b_mn, block_n=512, epi=ops.EPI_BIAS_RESID, bias=bias, aux=resid)
    want = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ref.gemm(a, b, want, a_mn, b_mn, False, ops.EPI_BIAS_RESID, bias, resid, 1.0)
    torch.cuda.synchronize()
    assert ops.error_word() == 0
    assert relerr(out, want) < 6e-3, relerr(out, want)
    acc = torch.ones(M, N, device=DEV)
    ops.gemm(a, b, acc, a_mn=a_mn, b_mn=b_mn, block_n=512, accumulate=True)
    wf = torch.empty(M, N, device=DEV)
    ref.gemm(a, b, wf, a_mn, b_mn, False, 0, None, None, 1.0)
    assert relerr(acc, 1 + wf) < 1e-4


def test_gemm_fp32_accumulate_and_alpha():
    torch.manual_seed(1)
    M, N, K = 256, 384, 320
    a, b = _rand(K, M), _rand(K, N)
    out = torch.randn(M, N, device=DEV)
    base = out.clone()
    ops.gemm(a, b, out, a_mn=True, b_mn=True, accumulate=True, alpha=0.5)
    want = base + 0.5 * (a.float().t() @ b.float())
    assert relerr(out, want) < 1e-5
    ops.gemm(a, b, out, a_mn=True, b_mn=True, accumulate=False)
    assert relerr(out, a.float().t() @ b.float()) < 1e-5


@pytest.mark.parametrize("M,N,K,bn", [(256, 256, 64, 0), (384, 328, 200, 256), (2048, 512, 4096, 512), (1000, 1024, 1032, 0),
                                      (136, 64, 72, 64), (3072, 2048, 2048, 0), (512, 1536, 640, 128)])
def test_gemm_weight_gradient_with_bias_gradient(M, N, K, bn):
    """dW += dY^T X with db += column sums of dY taken from the operand tiles in shared memory
    (single tiles, CTA pairs, ragged M / N / K, several tiles per CTA) against PyTorch."""
    torch.manual_seed(12)
    dy, x = _rand(K, M), _rand(K, N)
    dw = torch.randn(M, N, device=DEV)
    db = torch.randn(M, device=DEV)
    want_w = dw + dy.float().t() @ x.float()
    want_b = db + dy.float().sum(0)
    ops.gemm(dy, x, dw, a_mn=True, b_mn=True, accumulate=True, block_n=bn, colsum=db)
    torch.cuda.synchronize()
    assert ops.error_word() == 0
    assert relerr(dw, want_w) < 1e-4, relerr(dw, want_w)
    assert relerr(db, want_b) < 1e-5, relerr(db, want_b)
    # overwrite form, and run-to-run identical bits
    db2, db3 = torch.full((M,), 3.0, device=DEV), torch.full((M,), -1.0, device=DEV)
    ops.gemm(dy, x, dw, a_mn=True, b_mn=True, block_n=bn, colsum=db2)
    ops.gemm(dy, x, dw, a_mn=True, b_mn=True, block_n=bn, colsum=db3)
    assert torch.equal(db2, db3) and relerr(db2, dy.float().sum(0)) < 1e-5


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_f32_oracle_kernel(ta, tb):
    torch.manual_seed(13)
    M, N, K = 150, 77, 203
    A = torch.randn(K, M, device=DEV).t() if ta else torch.randn(M, K, device=DEV)
    B = torch.randn(N, K, device=DEV).t() if tb else torch.randn(K, N, device=DEV)
    got = ops._matmul_f32(A, B)
    want = (A.double() @ B.double()).float()
    assert relerr(got, want) < 2e-6


@pytest.mark.parametrize("epi", [ops.EPI_BIAS, ops.EPI_BIAS_GELU, ops.EPI_BIAS_RESID, ops.EPI_DGELU, ops.EPI_RESID])
@pytest.mark.parametrize("N", [512, 328])
def test_gemm_epilogues(epi, N):
    torch.manual_seed(2)
    M, K = 320, 256
    a, b = _rand(M, K, scale=0.5), _rand(N, K, scale=0.1)
    bias = _rand(N)
    aux = _rand(M, N)
    aux_ref = aux.clone()
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    want = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(a, b, out, epi=epi, bias=bias, aux=aux)
    ref.gemm(a, b, want, False, False, False, epi, bias, aux_ref, 1.0)
    assert relerr(out, want) < 8e-3
    if epi == ops.EPI_BIAS_GELU:
        assert relerr(aux, aux_ref) < 8e-3


def test_gemm_vocab_shapes():
    """Head shapes: N = 50257 (ragged), and the M-major weight-gradient with M = 50304 padded."""
    torch.manual_seed(3)
    R, d, V, Vp = 256, 128, 50257, 50304
    x, wte = _rand(R, d), _rand(V, d, scale=0.05)
    logits = torch.zeros(R, Vp, device=DEV, dtype=torch.bfloat16)
    ops.gemm(x, wte, logits[:, :V])
    want = x.float() @ wte.float().t()
    assert relerr(logits[:, :V], want) < 6e-3
    assert logits[:, V:].abs().max().item() == 0
    dl = _rand(R, Vp, scale=0.01)
    dl[:, V:] = 0
    dx = torch.empty(R, d, device=DEV, dtype=torch.bfloat16)
    ops.gemm(dl[:, :V], wte, dx, b_mn=True)
    assert relerr(dx, dl[:, :V].float() @ wte.float()) < 6e-3
    dw = torch.zeros(V, d, device=DEV)
    ops.gemm(dl[:, :V], x, dw, a_mn=True, b_mn=True, accumulate=True)
    assert relerr(dw, dl[:, :V].float().t() @ x.float()) < 1e-4


def test_layernorm_fwd_bwd():
    torch.manual_seed(4)
    for rows, d in [(64, 128), (1000, 512), (4096, 2048)]:
        x, w, b = _rand(rows, d), _rand(d), _rand(d)
        dy, dres = _rand(rows, d), _rand(rows, d)
        y = torch.empty_like(x); mean = torch.empty(rows, device=DEV); rstd = torch.empty(rows, device=DEV)
        ops.layernorm_fwd(x, w, b, y, mean, rstd)
        y2 = torch.empty_like(x); m2 = torch.empty_like(mean); r2 = torch.empty_like(rstd)
        ref.layernorm_fwd(x, w, b, y2, m2, r2)
        assert relerr(y, y2) < 4e-3 and relerr(mean, m2) < 1e-4 and relerr(rstd, r2) < 1e-4
        dx = torch.empty_like(x); dw = torch.ones(d, device=DEV); db = torch.ones(d, device=DEV)
        part = torch.zeros(ops.layernorm_bwd_scratch_elems(rows, d), device=DEV)
        ops.layernorm_bwd(dy, x, w, mean, rstd, dres, dx, dw, db, part)
        dx2 = torch.empty_like(x); dw2 = torch.ones(d, device=DEV); db2 = torch.ones(d, device=DEV)
        ref.layernorm_bwd(dy, x, w, m2, r2, dres, dx2, dw2, db2)
        assert relerr(dx, dx2) < 5e-3 and relerr(dw, dw2) < 1e-3 and relerr(db, db2) < 1e-3


def test_xent_vocab_slices_combine_to_full_softmax():
    """Per-slice statistics + combined gradient equal the full-row cross-entropy."""
    torch.manual_seed(6)
    R, V, parts = 96, 1003, 2
    vs = (V + parts - 1) // parts
    ld = (vs + 63) // 64 * 64
    full = _rand(R, V, scale=2.0)
    tgt = torch.randint(0, V, (R,), device=DEV, dtype=torch.int32)
    tgt[5] = -1
    stats, bufs = [], []
    for r in range(parts):
        v0, v1 = r * vs, min(V, (r + 1) * vs)
        lg = torch.full((R, ld), 77.0, device=DEV, dtype=torch.bfloat16)
        lg[:, :v1 - v0] = full[:, v0:v1]
        st = torch.empty(R, 3, device=DEV); st2 = torch.empty(R, 3, device=DEV)
        ops.xent_stats(lg, v1 - v0, tgt, v0, st)
        ref.xent_stats(lg, v1 - v0, tgt, v0, st2)
        assert torch.equal(torch.isinf(st[:, 2]), torch.isinf(st2[:, 2]))
        fin = ~torch.isinf(st2[:, 2])
        assert relerr(st[:, :2], st2[:, :2]) < 1e-3 and relerr(st[fin, 2], st2[fin, 2]) < 1e-6
        stats.append(st); bufs.append((lg, v0, v1))
    sa = torch.stack(stats)
    gm = sa[..., 0].max(0).values
    gs = (sa[..., 1] * torch.exp(sa[..., 0] - gm)).sum(0)
    loss = torch.where(tgt >= 0, torch.log(gs) + gm - sa[..., 2].max(0).values, torch.zeros_like(gm))
    want = full.clone().float()
    lp = torch.log_softmax(want, -1)
    want_loss = torch.where(tgt >= 0, -lp.gather(1, tgt.clamp(min=0).long()[:, None]).squeeze(1), torch.zeros(R, device=DEV))
    assert relerr(loss, want_loss) < 1e-3
    grad = torch.softmax(want, -1)
    grad[torch.arange(R, device=DEV), tgt.clamp(min=0).long()] -= 1.0
    grad[tgt < 0] = 0
    grad *= 0.25
    for lg, v0, v1 in bufs:
        ops.xent_grad(lg, v1 - v0, tgt, v0, gm, gs, uniform=0.25)
        assert relerr(lg[:, :v1 - v0], grad[:, v0:v1]) < 1e-2
        pad8 = (v1 - v0 + 7) // 8 * 8
        assert lg[:, v1 - v0:pad8].abs().max().item() == 0 if pad8 > v1 - v0 else True


def test_xent():
    torch.manual_seed(5)
    for R, V, ld in [(64, 256, 256), (130, 50257, 50304), (32, 1000, 1008)]:
        logits = torch.zeros(R, ld, device=DEV, dtype=torch.bfloat16)
        logits[:, :V] = _rand(R, V, scale=2.0)
        logits[:, V:] = 99.0   # padding must be ignored
        tgt = torch.randint(0, V, (R,), device=DEV, dtype=torch.int32)
        tgt[3] = -1
        coef = torch.randn(R, device=DEV)
        l2 = logits.clone()
        rl = torch.empty(R, device=DEV); pr = torch.empty(R, device=DEV)
        rl2 = torch.empty(R, device=DEV); pr2 = torch.empty(R, device=DEV)
        ops.xent(logits, V, tgt, coef=coef, rowloss=rl, prob=pr)
        ref.xent(l2, V, tgt, coef, 1.0, rl2, pr2, True)
        assert relerr(rl, rl2) < 1e-3 and relerr(pr, pr2) < 2e-3
        assert relerr(logits, l2) < 1e-2
        if ld > V:
            assert logits[:, V:].abs().max().item() == 0
        assert logits[3].abs().max().item() == 0


def test_adamw_matches_torch_and_emits_bf16():
    torch.manual_seed(6)
    n = 100003
    p = torch.randn(n + 1, device=DEV)[:n]
    p = torch.randn(n, device=DEV); g = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV); v = torch.zeros(n, device=DEV)
    pb = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    pt = torch.nn.Parameter(p.clone()); pt.grad = g.clone()
    opt = torch.optim.AdamW([pt], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        gg = g.clone()
        ops.adamw(p, gg, m, v, pb, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=step)
        assert gg.abs().max().item() == 0
        opt.step()
        assert torch.allclose(p, pt.data, rtol=1e-5, atol=1e-6)
        assert torch.equal(pb, p.to(torch.bfloat16))


def test_embed_and_colsum():
    torch.manual_seed(7)
    B, T, d, V = 4, 64, 128, 300
    tok = torch.randint(0, V, (B * T,), device=DEV, dtype=torch.int32)
    tok[5] = tok[17] = tok[200] = 11
    wte, wpe = _rand(V, d), _rand(T, d)
    out = torch.empty(B * T, d, device=DEV, dtype=torch.bfloat16)
    ops.embed_fwd(tok, None, wte, wpe, out, T)
    want = torch.empty_like(out); ref.embed_fwd(tok, None, wte, wpe, want, T)
    assert relerr(out, want) < 4e-3
    dx = _rand(B * T, d)
    dwte = torch.ones(V, d, device=DEV); dwpe = torch.ones(T, d, device=DEV)
    ops.embed_bwd(tok, dx, dwte, dwpe, B, T)
    dwte2 = torch.ones(V, d, device=DEV); dwpe2 = torch.ones(T, d, device=DEV)
    ref.embed_bwd(tok, dx, dwte2, dwpe2, B, T)
    assert relerr(dwte, dwte2) < 1e-5 and relerr(dwpe, dwpe2) < 1e-5
    for rows, N in [(777, 322), (4096, 2048), (100, 64)]:
        x = _rand(rows, (N + 7) // 8 * 8)[:, :N]
        cs = torch.ones(N, device=DEV)
        ops.colsum(x, cs, accumulate=True)
        assert relerr(cs, 1 + x.float().sum(0)) < 1e-5


@pytest.mark.parametrize("B,T,H,hd", [(2, 256, 4, 64), (1, 512, 2, 128), (3, 64, 2, 64), (2, 200, 2, 128), (1, 1024, 1, 64),
                                      (2, 384, 3, 128), (1, 130, 2, 64), (40, 512, 8, 128), (5, 72, 1, 128)])
def test_flash_fwd_bwd(B, T, H, hd):
    torch.manual_seed(8)
    d = H * hd
    qkv = _rand(B * T, 3 * d, scale=1.0)
    out = torch.zeros(B * T, d, device=DEV, dtype=torch.bfloat16)
    lse = torch.zeros(B, H, T, device=DEV)
    ops.flash_fwd(qkv, out, lse, B, T, H, hd)
    out2 = torch.empty_like(out); lse2 = torch.empty_like(lse)
    ref.flash_fwd(qkv, out2, lse2, B, T, H, hd)
    torch.cuda.synchronize()
    assert ops.error_word() == 0
    assert relerr(out, out2) < 1e-2, relerr(out, out2)
    assert relerr(lse, lse2) < 1e-3
    dout = _rand(B * T, d)
    dqkv = torch.zeros_like(qkv); delta = torch.empty(B, H, T, device=DEV)
    ops.flash_bwd(qkv, out, dout, lse, dqkv, delta, B, T, H, hd)
    dqkv2 = torch.zeros_like(qkv)
    ref.flash_bwd(qkv, out2, dout, lse2, dqkv2, B, T, H, hd)
    torch.cuda.synchronize()
    assert ops.error_word() == 0
    for i, name in enumerate("qkv"):
        e = relerr(dqkv[:, i * d:(i + 1) * d], dqkv2[:, i * d:(i + 1) * d])
        assert e < 2e-2, (name, e)
    # every output element has one writer and a fixed summation order: identical bits on a second run
    out3, lse3, dqkv3 = torch.zeros_like(out), torch.zeros_like(lse), torch.zeros_like(dqkv)
    ops.flash_fwd(qkv, out3, lse3, B, T, H, hd)
    ops.flash_bwd(qkv, out, dout, lse, dqkv3, delta, B, T, H, hd)
    assert torch.equal(out, out3) and torch.equal(lse, lse3) and torch.equal(dqkv, dqkv3)


def test_flash_large_scores_rescale():
    """Scores that keep growing along the keys force the in-place rescaling of the output accumulator."""
    torch.manual_seed(21)
    B, T, H, hd = 1, 512, 2, 128
    d = H * hd
    qkv = _rand(B * T, 3 * d, scale=1.0)
    ramp = torch.linspace(0.2, 6.0, T, device=DEV)[:, None]
    qkv[:, d:2 * d] = (qkv[:, d:2 * d].float() * ramp).bfloat16()      # later keys have larger norms
    out = torch.zeros(B * T, d, device=DEV, dtype=torch.bfloat16)
    lse = torch.zeros(B, H, T, device=DEV)
    ops.flash_fwd(qkv, out, lse, B, T, H, hd)
    out2 = torch.empty_like(out); lse2 = torch.empty_like(lse)
    ref.flash_fwd(qkv, out2, lse2, B, T, H, hd)
    torch.cuda.synchronize()
    assert ops.error_word() == 0
    assert relerr(out, out2) < 1e-2, relerr(out, out2)
    assert relerr(lse, lse2) < 1e-3


@pytest.mark.parametrize("M", [1, 8, 17, 32, 64])
@pytest.mark.parametrize("N,K", [(3072, 1024), (1024, 4096), (50257, 1024), (200, 192)])
def test_gemm_skinny(M, N, K):
    torch.manual_seed(9)
    x = _rand(M, K, scale=0.5)
    w = _rand(N, K, scale=0.1)
    bias = _rand(N)
    ld = (N + 63) // 64 * 64
    scratch = torch.zeros(ops.gemm_skinny_scratch_elems(M, N, K), device=DEV)
    for epi in (ops.EPI_NONE, ops.EPI_BIAS, ops.EPI_BIAS_GELU, ops.EPI_BIAS_RESID):
        aux = _rand(M, ld)[:, :N]
        aux_ref = aux.clone()
        out = torch.zeros(M, ld, device=DEV, dtype=torch.bfloat16)[:, :N]
        want = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        ops.gemm_skinny(x, w, out, scratch, epi=epi, bias=bias, aux=aux)
        ref.gemm(x, w, want, False, False, False, epi, bias, aux_ref, 1.0)
        assert relerr(out, want) < 8e-3, (epi, relerr(out, want))
        out2 = torch.zeros_like(out)
        ops.gemm_skinny(x, w, out2, scratch, epi=epi, bias=bias, aux=aux_ref.clone())
        assert torch.equal(out, out2)               # split-K partials are added in a fixed order
    torch.cuda.synchronize()
    assert ops.error_word() == 0


@pytest.mark.parametrize("M", [1, 5, 16])
@pytest.mark.parametrize("N,K", [(3072, 1024), (4096, 1024), (50257, 1024), (200, 192)])
def test_gemm_skinny_with_layernorm_prologue(M, N, K):
    """LayerNorm folded into the weight-streaming GEMM equals LayerNorm followed by the GEMM."""
    torch.manual_seed(10)
    x = _rand(M, K, scale=2.0) + 0.5
    w = _rand(N, K, scale=0.1)
    bias = _rand(N)
    lw, lb = (1.0 + 0.1 * torch.randn(K, device=DEV)).bfloat16(), (0.1 * torch.randn(K, device=DEV)).bfloat16()
    ld = (N + 63) // 64 * 64
    scratch = torch.zeros(ops.gemm_skinny_scratch_elems(M, N, K), device=DEV)
    y = torch.empty_like(x)
    ref.layernorm_fwd(x, lw, lb, y, None, None)
    for epi in (ops.EPI_NONE, ops.EPI_BIAS, ops.EPI_BIAS_GELU):
        aux = torch.zeros(M, ld, device=DEV, dtype=torch.bfloat16)[:, :N]
        aux_ref = aux.clone()
        out = torch.zeros(M, ld, device=DEV, dtype=torch.bfloat16)[:, :N]
        want = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        ops.gemm_skinny(x, w, out, scratch, epi=epi, bias=bias, aux=aux, ln_w=lw, ln_b=lb)
        ref.gemm(y, w, want, False, False, False, epi, bias, aux_ref, 1.0)
        assert relerr(out, want) < 1e-2, (epi, relerr(out, want))
    torch.cuda.synchronize()
    assert ops.error_word() == 0


def test_tensor_map_cache_overflow_keeps_descriptors_valid():
    """The descriptor cache drops its index when full; descriptors handed out before (the A map of
    the very launch whose B map caused the overflow) must stay valid, so results stay right."""
    from kharon_b200 import _native
    lib = _native.cuda()
    old = lib.kh_tmap_cache_limit(7)
    try:
        torch.manual_seed(11)
        big_a = _rand(128 + 400, 192, scale=0.5)
        big_b = _rand(256 + 400, 192, scale=0.2)
        out = torch.empty(128, 256, device=DEV, dtype=torch.bfloat16)
        want = torch.empty_like(out)
        for i in range(0, 400, 3):          # every launch sees operands at new addresses
            a, b = big_a[i:i + 128], big_b[i + 1:i + 257]
            ops.gemm(a, b, out)
            ref.gemm(a, b, want, False, False, False, ops.EPI_NONE, None, None, 1.0)
            assert relerr(out, want) < 8e-3, i
    finally:
        lib.kh_tmap_cache_limit(old)
    torch.cuda.synchronize()
    assert ops.error_word() == 0


def test_bounded_wait_status_word_is_clean():
    assert ops.error_word() == 0


def test_bounded_wait_runs_out_and_reports_status():
    """A wait on a flag that nothing sets gives up after its limit, reports code 5 through the status
    word, and leaves the context usable; once the flag is set the same wait succeeds."""
    flag = torch.zeros(1, device=DEV, dtype=torch.int32)
    status = torch.full((1,), -1, device=DEV, dtype=torch.int32)
    ops.wait_probe(flag, 1, 30, status)
    torch.cuda.synchronize()
    assert status.item() == 5 and ops.error_word() == 5      # read-and-clear
    assert ops.error_word() == 0
    flag.fill_(1)
    ops.wait_probe(flag, 1, 30, status)
    torch.cuda.synchronize()
    assert status.item() == 0 and ops.error_word() == 0
    assert torch.ones(4, device=DEV).sum().item() == 4.0     # the context still works


def test_mailbox_put_then_wait_and_wait_that_runs_out():
    """The pipeline mailbox primitives on one device (the slot is local memory here): a put delivers
    the bytes and raises the slot counter, the wait queued behind it passes and advances its expected
    count; a wait for a message nobody sends gives up after its limit with code 7."""
    src = _rand(300, 64)
    dst = torch.zeros_like(src)
    flag = torch.zeros(1, device=DEV, dtype=torch.int32)
    state = torch.zeros(2, device=DEV, dtype=torch.int32)
    expected = torch.zeros(1, device=DEV, dtype=torch.int32)
    for k in range(1, 4):
        src.add_(1.0)
        ops.p2p_put(src, dst.data_ptr(), flag.data_ptr(), state)
        ops.p2p_wait(flag.data_ptr(), expected, 500)
        torch.cuda.synchronize()
        assert torch.equal(dst, src) and flag.item() == k and expected.item() == k
        assert state.tolist() == [k, 0] and ops.error_word() == 0
    ops.p2p_wait(flag.data_ptr(), expected, 50)          # message 4 never comes
    torch.cuda.synchronize()
    assert ops.error_word() == 7 and expected.item() == 3
    assert ops.error_word() == 0


def test_guard_bands_stay_intact_through_training_steps():
    from kharon_b200.engine import TrainEngine
    from kharon_b200.models import gpt
    from kharon_b200.utils.guards import GuardedAlloc
    from kharon_b200.utils.rng import Rng
    ga = GuardedAlloc()
    gpt.set_allocator(ga)
    try:
        e = TrainEngine(layers=2, d_model=128, heads=2, vocab=1000, seq=96, mbatch=3, n_micro=2, device="cuda")
    finally:
        gpt.set_allocator(None)
    idx, tgt = Rng(4).batch(e.tokens_per_step, 1000)
    for _ in range(3):
        e.train_step(idx, tgt)
    torch.cuda.synchronize()
    assert len(ga.bufs) > 20 and ga.check() == []
    ga.bufs[0][1][3] = 0          # a damaged band is reported
    assert ga.check() == [ga.bufs[0][0]]


def test_merge_attention_equals_attention_over_all_keys():
    torch.manual_seed(11)
    H, T, hd = 2, 64, 64
    q, k, v = (torch.randn(H, T, hd, device=DEV) for _ in range(3))
    def attn(kk, vv):
        s = (q @ kk.transpose(-1, -2)) / hd ** 0.5
        return torch.softmax(s, -1) @ vv, torch.logsumexp(s, -1)
    o_all, l_all = attn(k, v)
    o1, l1 = attn(k[:, :40], v[:, :40])
    o2, l2 = attn(k[:, 40:], v[:, 40:])
    o, l = ops.merge_attention(o1, l1, o2, l2)
    assert torch.allclose(o, o_all, atol=1e-5) and torch.allclose(l, l_all, atol=1e-5)


def test_grpo_device_advantages_and_coefficients_match_host():
    """Device versions of the group-relative advantages and the per-token GRPO coefficients against the
    runtime library's host functions (reference src/core/grpo.c:7-20, src/grpo_train.c:164-174)."""
    torch.manual_seed(30)
    NP, G, T = 6, 8, 18
    rows = NP * G
    rew = torch.rand(rows)
    rew[8:16] = 0.5                                   # a group with zero variance
    p_cur, p_ref = torch.rand(rows * T) * 0.9 + 1e-3, torch.rand(rows * T) * 0.9 + 1e-3
    adv_h, coef_h = torch.empty(rows), torch.empty(rows * T)
    ops.grpo_advantages(rew, NP, G, 1e-4, adv_h)
    ops.grpo_coef(adv_h, p_cur, p_ref, rows, T, 8, T - 2, 0.04, coef_h)
    adv_d, coef_d = torch.empty(rows, device=DEV), torch.empty(rows * T, device=DEV)
    ops.grpo_advantages(rew.to(DEV), NP, G, 1e-4, adv_d)
    ops.grpo_coef(adv_d, p_cur.to(DEV), p_ref.to(DEV), rows, T, 8, T - 2, 0.04, coef_d)
    assert torch.allclose(adv_d.cpu(), adv_h, rtol=1e-5, atol=1e-6)
    assert torch.allclose(coef_d.cpu(), coef_h, rtol=1e-4, atol=1e-7)
