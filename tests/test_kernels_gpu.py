"""Each sm_100a kernel against a plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from oslo_b200 import ops
    from oslo_b200.ops import cuda_ops
    assert ops.load_ext(required=True) is not None
    return ops, cuda_ops


def _close(a, b, atol, rtol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert torch.allclose(a, b, atol=atol, rtol=rtol), f"max abs err {err}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 200), (1024, 128, 4096), (77 * 8, 1024, 1024), (8, 16384, 4096),
                                   (2560, 2048, 320), (2504, 2320, 520), (4096, 4352, 1024)])
def test_gemm_layouts(dtype, a_mn, b_mn, M, N, K):
    ops, co = _ops()
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=dtype)
    B = torch.randn(N, K, device="cuda", dtype=dtype)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
        pytest.skip("row stride must be a multiple of 16 bytes")
    out = co.gemm(a, b, a_mn, b_mn)
    ref = A.float() @ B.float().t()
    _close(out, ref, atol=0.02 * math.sqrt(K), rtol=2e-2)
    assert co.device_error_code(out) == 0


@pytest.mark.parametrize("M,N,K", [(384, 768, 512), (2500, 2096, 256)])  # single-CTA tiles; 256 x 256 tiles on CTA pairs
def test_gemm_epilogues(M, N, K):
    ops, co = _ops()
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * 0.5
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    z_ref = x.float() @ w.float().t() + bias.float()
    z = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    y = co.gemm(x, w, bias=bias, aux_out=z, flags=co.FLAG_BIAS | co.FLAG_GELU | co.FLAG_SAVE_PREACT)
    _close(z, z_ref, atol=0.03)
    _close(y, ops.reference.gelu_tanh(z_ref), atol=0.03)
    y2 = co.gemm(x, w, bias=bias, aux=res, flags=co.FLAG_BIAS | co.FLAG_RESIDUAL)
    _close(y2, z_ref + res.float(), atol=0.05)
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    co.gemm(x, w, out=acc, flags=co.FLAG_OUT_FP32 | co.FLAG_ACCUMULATE, alpha=0.5)
    _close(acc, 1.0 + 0.5 * (x.float() @ w.float().t()), atol=0.03)
    g = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * 0.5
    dz = co.gemm(g, w, aux=z, flags=co.FLAG_DGELU)
    zz = z.float().requires_grad_(True)
    ops.reference.gelu_tanh(zz).backward(torch.ones_like(zz))
    _close(dz, (g.float() @ w.float().t()) * zz.grad, atol=0.05)


@pytest.mark.parametrize("reversed_", [False, True])
@pytest.mark.parametrize("act", [None, "gelu_new"])
def test_linear_autograd(reversed_, act):
    ops, co = _ops()
    torch.manual_seed(2)
    x = (torch.randn(4, 96, 256, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(256, 512, device="cuda") * 0.05).to(torch.bfloat16)
    w = (w if reversed_ else w.t().contiguous()).requires_grad_(True)
    b = torch.randn(512, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = ops.linear(x, w, b, reversed_, act)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = ops.reference.linear(xf, wf, bf, reversed_, act)
    yr.backward(g.float())
    _close(y, yr, atol=0.05)
    _close(x.grad, xf.grad, atol=0.05)
    _close(w.grad, wf.grad, atol=0.3, rtol=3e-2)
    _close(b.grad, bf.grad, atol=0.3, rtol=3e-2)


@pytest.mark.parametrize("dtype,cols", [(torch.bfloat16, 4096), (torch.bfloat16, 768), (torch.float32, 2048), (torch.float16, 48)])
def test_layernorm(dtype, cols):
    ops, _ = _ops()
    torch.manual_seed(3)
    x = torch.randn(37, 5, cols, device="cuda").to(dtype).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(dtype).requires_grad_(True)
    b = (0.1 * torch.randn(cols, device="cuda")).to(dtype).requires_grad_(True)
    y = ops.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = ops.reference.layer_norm(xf, wf, bf, 1e-5)
    yr.backward(g.float())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    _close(y, yr, atol=tol)
    _close(x.grad, xf.grad, atol=tol)
    _close(w.grad, wf.grad, atol=tol * 20, rtol=3e-2)
    _close(b.grad, bf.grad, atol=tol * 20, rtol=3e-2)


def test_bias_gelu_and_dropout():
    ops, _ = _ops()
    torch.manual_seed(4)
    x = torch.randn(64, 33, 1024, device="cuda").to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(1024, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = ops.bias_gelu(x, b)
    g = torch.randn_like(y)
    y.backward(g)
    xf, bf = x.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    yr = ops.reference.bias_gelu(xf, bf)
    yr.backward(g.float())
    _close(y, yr, atol=2e-2)
    _close(x.grad, xf.grad, atol=2e-2)
    _close(b.grad, bf.grad, atol=1.0, rtol=3e-2)
    r = torch.randn_like(x)
    out = ops.bias_dropout_residual(x.detach(), b.detach(), r, 0.0, True)
    _close(out, x.detach().float() + b.detach().float() + r.float(), atol=3e-2)
    xd = x.detach().clone().requires_grad_(True)
    out = ops.bias_dropout_residual(xd, None, None, 0.25, True)
    kept = (out != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.01
    out.backward(torch.ones_like(out))
    assert torch.equal((xd.grad != 0), (out != 0) | ((xd.detach() == 0) & (xd.grad != 0)))
    _close(xd.grad[out != 0], torch.full_like(xd.grad[out != 0], 1 / 0.75), atol=1e-2)


def test_rotary():
    ops, _ = _ops()
    torch.manual_seed(5)
    x = torch.randn(2, 33, 4, 256, device="cuda").to(torch.bfloat16).requires_grad_(True)
    pos = torch.arange(7, 40, device="cuda").unsqueeze(0).expand(2, -1).contiguous()
    y = ops.rotary_interleaved(x, pos, 64)
    g = torch.randn_like(y)
    y.backward(g)
    xf = x.detach().float().requires_grad_(True)
    yr = ops.reference.rotary_interleaved(xf, pos, 64)
    yr.backward(g.float())
    _close(y, yr, atol=2e-2)
    _close(x.grad, xf.grad, atol=2e-2)
    # a non-leaf input takes the in-place kernel (first rotary_dim dims only); its backward overwrites the incoming
    # gradient, so hand it a copy
    x2 = x.detach().clone().requires_grad_(True)
    y2 = ops.rotary_interleaved(x2 * 1.0, pos, 64)
    y2.backward(g.clone())
    _close(y2, yr, atol=2e-2)
    _close(x2.grad, xf.grad, atol=2e-2)


def test_softmax_kernels():
    ops, _ = _ops()
    torch.manual_seed(6)
    x = torch.randn(6, 40, 40, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = ops.scaled_upper_triang_masked_softmax(x, 0.3)
    g = torch.randn_like(y)
    y.backward(g)
    xf = x.detach().float()
    yr = ops.reference.scaled_upper_triang_masked_softmax(xf, 0.3)
    _close(y, yr, atol=1e-2)
    assert (y.triu(1) == 0).all()
    _close(x.grad, ops.reference.softmax_backward(yr, g.float(), 0.3), atol=1e-2)
    x4 = torch.randn(2, 3, 17, 50, device="cuda").to(torch.float16)
    mask = (torch.rand(2, 1, 17, 50, device="cuda") < 0.3).to(torch.uint8)
    _close(ops.scaled_masked_softmax(x4, mask, 2.0), ops.reference.scaled_masked_softmax(x4.float(), mask, 2.0), atol=2e-3)


@pytest.mark.parametrize("vocab", [50400, 1000, 50257])
def test_cross_entropy(vocab):
    ops, _ = _ops()
    torch.manual_seed(7)
    lg = (torch.randn(65, vocab, device="cuda") * 2).to(torch.bfloat16).requires_grad_(True)
    lab = torch.randint(0, vocab, (65,), device="cuda")
    lab[3] = -100
    loss = ops.cross_entropy(lg, lab)
    loss.backward()
    lf = lg.detach().float().requires_grad_(True)
    lr = ops.reference.cross_entropy(lf, lab)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-3
    _close(lg.grad, lf.grad, atol=2e-4, rtol=5e-2)


def test_linear_cross_entropy_fused():
    ops, _ = _ops()
    torch.manual_seed(8)
    h = (torch.randn(300, 256, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(1024, 256, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn(1024, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    lab = torch.randint(0, 1024, (300,), device="cuda")
    lab[:5] = -100
    loss = ops.linear_cross_entropy(h, w, b, lab, chunk_rows=128)
    loss.backward()
    hf, wf, bf = (t.detach().float().requires_grad_(True) for t in (h, w, b))
    lr = ops.reference.cross_entropy(ops.reference.linear(hf, wf, bf), lab)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 5e-3
    _close(h.grad, hf.grad, atol=2e-4, rtol=5e-2)
    _close(w.grad, wf.grad, atol=2e-4, rtol=5e-2)
    _close(b.grad, bf.grad, atol=2e-4, rtol=5e-2)


@pytest.mark.parametrize("M,N,K,lo,with_bias", [(300, 1000, 256, 0, True), (128, 264, 64, 500, False),
                                                (2560, 50400, 512, 0, True), (1024, 25200, 1024, 25200, True)])
def test_lm_head_gemm_with_cross_entropy_epilogue(M, N, K, lo, with_bias):
    """Row statistics and (softmax - onehot) * scale straight out of the GEMM accumulators against fp32 statements on
    the 16-bit-rounded logits; labels outside this shard's columns and ignored labels included."""
    ops, co = _ops()
    ext = ops.load_ext()
    torch.manual_seed(11)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.1).to(torch.bfloat16)
    b = (torch.randn(N, device="cuda") * 0.2).to(torch.bfloat16) if with_bias else None
    full = lo + N + 300
    lab = torch.randint(0, full, (M,), device="cuda")           # some labels belong to other shards
    lab[1] = lo
    lab[2] = lo + N - 1
    lab[3] = -100
    logits = x.float() @ w.float().t()
    if b is not None:
        logits = logits + b.float()
    logits = logits.to(torch.bfloat16).float()
    mx, se, tg = ext.gemm_ce_stats(x, w, 0, b, lab, lo)
    want_mx = logits.max(-1).values
    want_se = torch.exp(logits - want_mx[:, None]).sum(-1)
    local = lab - lo
    inside = (local >= 0) & (local < N)
    want_tg = torch.where(inside, logits.gather(1, local.clamp(0, N - 1)[:, None]).squeeze(1), torch.zeros_like(want_mx))
    # sums of K products in another order than the library's: bf16 rounding may differ by one step for a few logits
    _close(mx, want_mx, atol=0.05, rtol=1e-2)
    lse, want_lse = torch.log(se) + mx, torch.log(want_se) + want_mx
    _close(lse, want_lse, atol=0.02, rtol=1e-3)
    _close(tg, want_tg, atol=0.05, rtol=1e-2)
    scale = torch.rand(M, device="cuda") * (lab != -100)
    d = ext.gemm_ce_grad(x, w, 0, b, lab, lo, want_lse.contiguous(), scale.contiguous())
    p = torch.exp(logits - want_lse[:, None])
    rows = torch.nonzero(inside, as_tuple=True)[0]
    p[rows, local[rows]] -= 1.0
    p *= scale[:, None]
    _close(d, p, atol=3e-3, rtol=5e-2)
    assert d[3].abs().max() == 0
    assert co.device_error_code(x) == 0


def test_linear_cross_entropy_epilogue_and_separate_kernels_agree():
    """Whole loss + gradients: the GEMM-epilogue route and the logits-chunk route give the same numbers."""
    ops, _ = _ops()
    from oslo_b200.config import set_config
    res = {}
    for flag in (True, False):
        set_config(ce_in_gemm_epilogue=flag)
        torch.manual_seed(8)
        h = (torch.randn(700, 256, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
        w = (torch.randn(2048, 256, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
        b = (torch.randn(2048, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
        lab = torch.randint(0, 2048, (700,), device="cuda")
        lab[:5] = -100
        loss = ops.linear_cross_entropy(h, w, b, lab, chunk_rows=256)
        loss.backward()
        res[flag] = (loss.item(), h.grad.clone(), w.grad.clone(), b.grad.clone())
    set_config(ce_in_gemm_epilogue=True)
    assert abs(res[True][0] - res[False][0]) < 2e-3
    for a, c in zip(res[True][1:], res[False][1:]):
        _close(a, c, atol=3e-4, rtol=5e-2)


def test_adam_and_ngram():
    ops, co = _ops()
    ext = ops.load_ext()
    torch.manual_seed(9)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    plp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    for step in (1, 2, 3):
        ext.adam_step(p, g, m, v, plp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0, None)
        ops.reference.adam_step(pr, g, mr, vr, step, 1e-2, 0.9, 0.95, 1e-8, 0.1)
    _close(p, pr, atol=1e-5, rtol=1e-4)
    _close(plp, pr, atol=2e-2)
    assert abs(ext.sumsq(g).item() - g.float().pow(2).sum().item()) / n < 1e-3
    toks = torch.tensor([[1, 2, 3, 1, 2], [5, 5, 5, 5, 5], [1, 2, 3, 4, 5]], device="cuda")
    lp = torch.zeros(3, 10, device="cuda")
    out = ops.ban_repeated_ngrams(toks, lp.clone(), 3)
    want = ops.reference.ban_repeated_ngrams(toks.cpu(), lp.cpu().clone(), 3)
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("Sq,Sk,window,use_kpm", [(128, 128, None, False), (200, 200, 48, False), (77, 333, None, True), (256, 256, 256, False)])
def test_flash_attention(D, Sq, Sk, window, use_kpm):
    ops, _ = _ops()
    torch.manual_seed(10)
    B, H = 2, 3
    mk = lambda s: (torch.randn(B, s, H, D, device="cuda") * 0.7).to(torch.bfloat16).permute(0, 2, 1, 3).requires_grad_(True)
    q, k, v = mk(Sq), mk(Sk), mk(Sk)
    kpm = None
    if use_kpm:
        kpm = torch.ones(B, Sk, device="cuda", dtype=torch.long)
        kpm[0, :9] = 0
    scale = 1.0 / math.sqrt(D)
    o = ops.attention(q, k, v, True, window, scale, kpm)
    g = torch.randn(B, H, Sq, D, device="cuda").to(torch.bfloat16)
    o.backward(g)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf = ops.reference.attention(qf, kf, vf, True, window, scale, kpm)
    orf.backward(g.float())
    _close(o, orf, atol=2e-2)
    _close(q.grad, qf.grad, atol=3e-2, rtol=5e-2)
    _close(k.grad, kf.grad, atol=3e-2, rtol=5e-2)
    _close(v.grad, vf.grad, atol=3e-2, rtol=5e-2)


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Sq,Sk,causal,window,use_kpm", [
    (640, 640, True, None, False), (300, 300, False, None, False), (128, 517, True, None, True),
    (1, 130, True, None, False), (513, 513, True, 100, False), (384, 384, False, None, True)])
def test_flash_forward_tcgen05(D, dtype, Sq, Sk, causal, window, use_kpm):
    """tcgen05/TMEM forward kernel against the fp32 statement (output and log-sum-exp), many key blocks,
    ragged tails, prefix offset (Sk > Sq), window, padding, and a second call on the same inputs."""
    ops, _ = _ops()
    ext = ops.load_ext(required=True)
    torch.manual_seed(11)
    B, H = 2, 3
    mk = lambda s: (torch.randn(B, s, H, D, device="cuda") * 0.8).to(dtype).permute(0, 2, 1, 3)
    q, k, v = mk(Sq), mk(Sk), mk(Sk)
    kpm = kpm8 = None
    if use_kpm:
        kpm = torch.ones(B, Sk, device="cuda", dtype=torch.long)
        kpm[0, :9] = 0
        kpm[1, 100:140] = 0
        kpm8 = kpm.to(torch.uint8)
    scale = 1.0 / math.sqrt(D)
    o, lse = ext.flash_fwd(q, k, v, scale, causal, int(window or 0), kpm8, 1)
    o2, lse2 = ext.flash_fwd(q, k, v, scale, causal, int(window or 0), kpm8, 1)
    want = ops.reference.attention(q.float(), k.float(), v.float(), causal, window, scale, kpm)
    assert int(ext.error_word(q).item()) == 0
    _close(o, want, atol=2e-2)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    o_old, lse_old = ext.flash_fwd(q, k, v, scale, causal, int(window or 0), kpm8, 0)
    _close(lse, lse_old, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("D,window", [(256, None), (128, 37), (64, None)])
def test_decode_attention(D, window):
    ops, _ = _ops()
    torch.manual_seed(11)
    B, H, T = 3, 4, 300
    q = torch.randn(B, H, D, device="cuda").to(torch.bfloat16)
    kc = torch.randn(B, H, T, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(B, H, T, D, device="cuda").to(torch.bfloat16)
    lengths = torch.tensor([300, 1, 129], device="cuda", dtype=torch.int32)
    out = ops.decode_attention(q, kc, vc, lengths, 1 / math.sqrt(D), window)
    want = ops.functional.decode_attention(q.cpu().float(), kc.cpu().float(), vc.cpu().float(), lengths.cpu(),
                                           1 / math.sqrt(D), window)
    _close(out.cpu(), want, atol=2e-2)


@pytest.mark.parametrize("kind", ["gptj", "gpt2", "gpt_neo"])
def test_fused_model_matches_eager_model(kind):
    """Whole-model check: loss and every parameter gradient of the fused (kernel) model against the eager one."""
    import oslo_b200 as ob
    torch.manual_seed(0)
    if kind == "gptj":
        cfg = ob.GPTJConfig(vocab_size=512, n_positions=128, n_embd=256, n_layer=2, n_head=4, rotary_dim=16)
        cls = ob.GPTJForCausalLM
    elif kind == "gpt2":
        cfg = ob.GPT2Config(vocab_size=512, n_positions=128, n_embd=256, n_layer=2, n_head=4, resid_pdrop=0.0,
                            embd_pdrop=0.0, attn_pdrop=0.0)
        cls = ob.GPT2LMHeadModel
    else:
        cfg = ob.GPTNeoConfig(vocab_size=512, max_position_embeddings=128, hidden_size=256, num_layers=2, num_heads=4,
                              window_size=32)
        cls = ob.GPTNeoForCausalLM
    eager = cls(cfg).to(torch.bfloat16).cuda().train()
    fused = cls(cfg).to(torch.bfloat16).cuda().train()
    fused.load_state_dict(eager.state_dict())
    fused.fuse()
    ids = torch.randint(0, 512, (3, 128), device="cuda")
    le = eager(input_ids=ids, labels=ids).loss
    lf = fused(input_ids=ids, labels=ids, output_logits=False).loss
    le.backward()
    lf.backward()
    assert abs(le.item() - lf.item()) < 0.03, (le.item(), lf.item())
    ge = dict(eager.named_parameters())
    worst = 0.0
    for n, p in fused.named_parameters():
        a, b = p.grad.float(), ge[n].grad.float()
        rel = (a - b).norm() / (b.norm() + 1e-6)
        worst = max(worst, rel.item())
        assert rel < 0.08, (n, rel.item())


def test_graphed_greedy_decoder_gpu():
    """CUDA-graph replayed greedy decoding produces exactly the tokens of the same step run eagerly, and the fused
    decode step (device-positioned cache) agrees with the general cached forward on the next-token logits."""
    import oslo_b200 as ob
    from oslo_b200.generation import GraphedGreedyDecoder
    from oslo_b200.models.common import StaticKVCache
    torch.manual_seed(0)
    cfg = ob.GPTJConfig(vocab_size=1024, n_positions=256, n_embd=256, n_layer=2, n_head=4, rotary_dim=16)
    model = ob.GPTJForCausalLM(cfg).to(torch.bfloat16).cuda().fuse().eval()
    ids = torch.randint(0, 1024, (3, 33), device="cuda")
    graphed = GraphedGreedyDecoder(model, max_len=128, use_graph=True)
    eager = GraphedGreedyDecoder(model, max_len=128, use_graph=False)
    for prompt, n_new in ((33, 40), (20, 30)):
        got = graphed.generate(ids[:, :prompt], n_new)
        want = eager.generate(ids[:, :prompt], n_new)
        assert torch.equal(got, want)
    assert graphed.replays > 0 and eager.replays == 0
    nxt = torch.randint(0, 1024, (3, 1), device="cuda")
    logits = []
    with torch.no_grad():
        for device_positions in (True, False):
            cache = StaticKVCache(64)
            model(input_ids=ids, past_key_values=cache, use_cache=True)
            pos = None
            if device_positions:
                cache.use_device_positions(True)
                pos = cache.lengths_dev.to(torch.long).unsqueeze(1)
            out = model(input_ids=nxt, past_key_values=cache, position_ids=pos, use_cache=True)
            logits.append(out.logits[:, -1].float())
    assert getattr(model.transformer.h[0], "_packed2_w", None) is not None   # the fused step really ran
    _close(logits[0], logits[1], atol=3e-2)


@pytest.mark.parametrize("M,K1,K2,N", [(1, 512, 2048, 4096), (3, 256, 0, 1024), (4, 4096, 0, 28672), (2, 264, 520, 260)])
def test_gemv_rows(M, K1, K2, N):
    ops, co = _ops()
    ext = ops.load_ext(required=True)
    torch.manual_seed(5)
    x1 = torch.randn(M, K1, device="cuda", dtype=torch.bfloat16) * 0.5
    x2 = torch.randn(M, K2, device="cuda", dtype=torch.bfloat16) * 0.5 if K2 else None
    w = torch.randn(N, K1 + K2, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    y = ext.gemv_rows(x1, x2, w, b, N // 2)
    xin = x1.float() if x2 is None else torch.cat([x1.float(), x2.float()], dim=1)
    ref = xin @ w.float().t() + b.float()
    ref[:, N // 2:] = ops.reference.gelu_tanh(ref[:, N // 2:])
    _close(y, ref, atol=0.03)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    z = ext.gemv_rows(x1, x2, w, None, -1, res)
    _close(z, xin @ w.float().t() + res.float(), atol=0.04)


@pytest.mark.parametrize("M,N,K,rev", [(1, 4096, 4096, False), (8, 512, 4096, False), (32, 16384, 4096, True),
                                        (5, 4096, 16384, False), (64, 264, 520, True), (3, 50400, 1024, False)])
def test_small_m_linear(M, N, K, rev):
    """Decode-sized linear layers (split-K path) against fp32, and bit-identical when repeated."""
    ops, co = _ops()
    torch.manual_seed(3)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * 0.5
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    wt = w.t().contiguous() if rev else w
    with torch.no_grad():
        y = co.linear(x, wt, b, rev, "gelu_new")
        y2 = co.linear(x, wt, b, rev, "gelu_new")
        z = co.linear(x, wt, None, rev, None)
    ref = x.float() @ w.float().t()
    _close(z, ref, atol=0.03)
    _close(y, ops.reference.gelu_tanh(ref + b.float()), atol=0.03)
    assert torch.equal(y, y2)
    assert co.device_error_code(y) == 0


def test_packed_decode_projection_matches_per_layer_path():
    """GPT-J decode step: the packed q/k/v/fc_in GEMM gives the logits of the per-layer path."""
    import oslo_b200 as ob
    from oslo_b200.config import set_config
    torch.manual_seed(0)
    cfg = ob.GPTJConfig(vocab_size=1024, n_positions=256, n_embd=256, n_layer=2, n_head=4, rotary_dim=16)
    model = ob.GPTJForCausalLM(cfg).to(torch.bfloat16).cuda().fuse().eval()
    ids = torch.randint(0, 1024, (3, 1), device="cuda")
    outs = []
    try:
        for flag in (True, False):
            set_config(packed_decode=flag)
            with torch.no_grad():
                outs.append(model(input_ids=ids, use_cache=False).logits.float())
    finally:
        set_config(packed_decode=True)
    assert getattr(model.transformer.h[0], "_packed_w", None) is not None
    _close(outs[0], outs[1], atol=2e-2)


def test_weight_gradients_accumulate_into_flat_buffer():
    """Weight-gradient GEMMs that add straight into the optimizer's flat gradient buffer give the gradients of the
    ordinary autograd accumulation over two micro-batches."""
    import oslo_b200 as ob
    from oslo_b200.optim import FusedAdamW
    torch.manual_seed(0)
    cfg = ob.GPTJConfig(vocab_size=1024, n_positions=128, n_embd=256, n_layer=2, n_head=4, rotary_dim=16)
    model = ob.GPTJForCausalLM(cfg).to(torch.bfloat16).cuda().fuse().train()
    opt = FusedAdamW(model.parameters(), lr=1e-3)
    ids = torch.randint(0, 1024, (4, 64), device="cuda")
    flagged = [p for p in opt.buf.params if getattr(p, "_oslo_accum_grad", False)]
    assert flagged
    grads = []
    for fused in (True, False):
        for p in flagged:
            p._oslo_accum_grad = fused
        opt.zero_grad()
        for mb in (ids[:2], ids[2:]):
            (model(input_ids=mb, labels=mb, output_logits=False).loss / 2).backward()
        grads.append(opt.buf.flat_g.float().clone())
    for p in flagged:
        p._oslo_accum_grad = True
    assert grads[0].abs().max() > 0
    _close(grads[0], grads[1], atol=2e-3, rtol=5e-2)


def test_fused_mlp_autograd():
    """fc_in -> GeLU -> fc_out as one autograd node (dGeLU inside the dgrad GEMM epilogue) against fp32 autograd."""
    ops, co = _ops()
    torch.manual_seed(8)
    rows, E, F = 200, 256, 1024
    x = (torch.randn(2, rows // 2, E, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w_in = (torch.randn(F, E, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    b_in = (torch.randn(F, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    w_out = (torch.randn(E, F, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    b_out = (torch.randn(E, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    assert co.fused_mlp_ok(x, w_in, w_out)
    y = co.fused_mlp(x, w_in, b_in, w_out, b_out)
    g = torch.randn_like(y)
    y.backward(g)
    ref_in = [t.detach().float().requires_grad_(True) for t in (x, w_in, b_in, w_out, b_out)]
    xf, wi, bi, wo, bo = ref_in
    yr = ops.reference.gelu_tanh(xf @ wi.t() + bi) @ wo.t() + bo
    yr.backward(g.float())
    _close(y, yr, atol=3e-2)
    for got, want in zip((x, w_in, b_in, w_out, b_out), ref_in):
        _close(got.grad, want.grad, atol=5e-2, rtol=5e-2)
