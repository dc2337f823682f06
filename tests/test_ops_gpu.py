"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture(scope="module")
def dev():
    from elf_b200.ops import _ext

    assert _ext.available(), "the native extension must be built for GPU tests"
    return torch.device("cuda", 0)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (200, 264, 72), (1000, 520, 328), (4096, 1024, 2048), (96, 8, 8)])
def test_gemm_family(dev, m, n, k):
    from elf_b200.ops import gemm as G

    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05
    dy = torch.randn(m, n, device=dev, dtype=torch.bfloat16)
    bias = torch.randn(n, device=dev, dtype=torch.bfloat16)
    assert rel_err(G.linear_forward(x, w, bias), x.float() @ w.float().t() + bias.float()) < 5e-3
    assert rel_err(G.linear_forward(x, w), x.float() @ w.float().t()) < 5e-3
    assert rel_err(G.linear_input_grad(dy, w), dy.float() @ w.float()) < 5e-3
    ref_dw = dy.float().t() @ x.float()
    assert rel_err(G.linear_weight_grad(dy, x), ref_dw) < 5e-3
    acc32 = torch.full((n, k), 0.5, device=dev, dtype=torch.float32)
    G.linear_weight_grad(dy, x, out=acc32)
    assert rel_err(acc32, ref_dw + 0.5) < 1e-4
    acc16 = torch.ones(n, k, device=dev, dtype=torch.bfloat16)
    G.linear_weight_grad(dy, x, out=acc16)
    assert rel_err(acc16, ref_dw + 1) < 5e-3
    G.check_status()


@pytest.mark.parametrize("m,n,k", [(4096, 5120, 1024), (4000, 5064, 1000), (3900, 4872, 520)])
def test_gemm_k_split_tail(dev, m, n, k):
    """Shapes with more tiles than CTA pairs and a small last wave: the pair kernel splits that wave
    along K and adds the partial sums in L2.  Ragged rows / columns / K, bias, accumulation and an
    output with a row pitch larger than its width (the pre-clearing then runs as a 2-D memset)."""
    from elf_b200.ops import _ext
    from elf_b200.ops import gemm as G

    torch.manual_seed(m + n + k)
    x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(n, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(m, n, device=dev, dtype=torch.bfloat16)
    ref = x.float() @ w.float().t()
    for split in (True, False):
        G.set_variant(1, split)
        try:
            assert rel_err(G.linear_forward(x, w), ref) < 5e-3
            assert rel_err(G.linear_forward(x, w, bias), ref + bias.float()) < 5e-3
            assert rel_err(G.linear_input_grad(dy, w), dy.float() @ w.float()) < 5e-3
            acc = torch.full((n, k), 0.25, device=dev, dtype=torch.float32)
            G.linear_weight_grad(dy, x, out=acc)
            assert rel_err(acc, dy.float().t() @ x.float() + 0.25) < 1e-4
            # strided output: a [m, n] window of a wider buffer whose other columns must stay untouched
            wide = torch.full((m, n + 64), 7.0, device=dev, dtype=torch.bfloat16)
            _ext.get().gemm(x, w, wide[:, :n], None, False, False, False, 1.0, G.status(dev), 1, split)
            assert rel_err(wide[:, :n], ref) < 5e-3
            assert bool((wide[:, n:] == 7.0).all())
        finally:
            G.set_variant(1, True)
    G.check_status(dev)


def test_gemm_fp16_and_strided(dev):
    from elf_b200.ops import gemm as G

    x = torch.randn(300, 512, device=dev, dtype=torch.float16)[:, :256]  # row pitch 512
    w = torch.randn(128, 256, device=dev, dtype=torch.float16) * 0.05
    assert rel_err(G.linear_forward(x, w), x.float() @ w.float().t()) < 2e-3
    G.check_status()


def test_linear_dw_layer_matches_autograd(dev):
    from elf_b200.zb_utils import LinearDW

    torch.manual_seed(0)
    lin = torch.nn.Linear(256, 512, bias=True, device=dev, dtype=torch.bfloat16)
    ref = torch.nn.Linear(256, 512, bias=True, device=dev, dtype=torch.float32)
    ref.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})
    dw = LinearDW(lin)
    x = torch.randn(4, 96, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    xr = x.detach().float().requires_grad_()
    y = dw(x)
    g = torch.randn_like(y)
    y.backward(g)
    ref(xr).backward(g.float())
    assert dw.weight.grad is None  # B pass leaves parameters alone
    dw.move_last_computed("input", 0)
    dw.move_last_computed("grad_output", 0)
    dw.backward(0)
    assert rel_err(y, ref(xr)) < 5e-3
    assert rel_err(x.grad, xr.grad) < 5e-3
    assert rel_err(dw.weight.grad, ref.weight.grad) < 5e-3
    assert rel_err(dw.bias.grad, ref.bias.grad) < 5e-3


@pytest.mark.parametrize("rows,dim", [(64, 256), (300, 4096), (17, 8192)])
def test_rmsnorm(dev, rows, dim):
    from elf_b200.ops import fused as Fu

    torch.manual_seed(1)
    x = torch.randn(rows, dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(dim, device=dev)).to(torch.bfloat16).requires_grad_()
    y = Fu.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = F.rms_norm(xf, (dim,), wf, 1e-5)
    yr.backward(g.float())
    assert rel_err(y, yr) < 5e-3 and rel_err(x.grad, xf.grad) < 1e-2 and rel_err(w.grad, wf.grad) < 1e-2
    # fused residual add + norm
    x.grad = None
    w.grad = None
    y2, h = Fu.add_rms_norm(x, r, w, 1e-5)
    gy, gh = torch.randn_like(y2), torch.randn_like(h)
    torch.autograd.backward([y2, h], [gy, gh])
    xf, rf, wf = x.detach().float().requires_grad_(), r.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    hr = (xf + rf).to(torch.bfloat16).float().detach() + (xf + rf - (xf + rf).detach())  # h rounded to bf16 as the kernel stores it
    yr = F.rms_norm(hr, (dim,), wf, 1e-5)
    torch.autograd.backward([yr, hr], [gy.float(), gh.float()])
    assert rel_err(h, hr) < 5e-3 and rel_err(y2, yr) < 5e-3
    assert rel_err(x.grad, xf.grad) < 1e-2 and rel_err(r.grad, rf.grad) < 1e-2 and rel_err(w.grad, wf.grad) < 1e-2


def test_rope(dev):
    from elf_b200.ops import fused as Fu

    b, s, hq, hkv, d = 2, 128, 4, 2, 128
    cos, sin = Fu.rope_tables(s, d, 500000.0, dev)
    x = torch.randn(b * s, (hq + 2 * hkv) * d, device=dev, dtype=torch.bfloat16)
    ref = Fu._rope_ref(x.float(), cos, sin, hq + hkv, d, s, 1.0)
    leaf = x.clone().requires_grad_()
    out = Fu.rope_(leaf * 1, cos, sin, hq + hkv, d, s)
    assert rel_err(out, ref) < 5e-3
    g = torch.randn_like(out)
    gref = Fu._rope_ref(g.float(), cos, sin, hq + hkv, d, s, -1.0)
    out.backward(g)
    assert rel_err(leaf.grad, gref) < 5e-3


def test_swiglu(dev):
    from elf_b200.ops import fused as Fu

    gu = torch.randn(300, 2 * 1408, device=dev, dtype=torch.bfloat16, requires_grad=True)
    out = Fu.swiglu(gu)
    g = torch.randn_like(out)
    out.backward(g)
    guf = gu.detach().float().requires_grad_()
    a, b = guf.chunk(2, -1)
    ref = F.silu(a) * b
    ref.backward(g.float())
    assert rel_err(out, ref) < 5e-3 and rel_err(gu.grad, guf.grad) < 1e-2


@pytest.mark.parametrize("rows,vocab", [(64, 1024), (33, 32000), (16, 128256)])
def test_cross_entropy(dev, rows, vocab):
    from elf_b200.ops import fused as Fu

    torch.manual_seed(2)
    logits = (torch.randn(rows, vocab, device=dev) * 2).to(torch.bfloat16)
    tgt = torch.randint(0, vocab, (rows,), device=dev)
    lf = logits.float().requires_grad_()
    ref = F.cross_entropy(lf, tgt, reduction="sum")
    (ref / 7).backward()
    leaf = logits.clone().requires_grad_()
    loss = Fu.cross_entropy(leaf, tgt, reduction="sum")
    (loss / 7).backward()
    assert abs(loss.item() - ref.item()) / abs(ref.item()) < 1e-3
    assert rel_err(leaf.grad, lf.grad) < 1e-2


def test_embedding(dev):
    from elf_b200.ops import fused as Fu

    table = torch.randn(1000, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (4, 77), device=dev)
    out = Fu.embedding(table, ids)
    assert torch.equal(out, F.embedding(ids, table))
    g = torch.randn_like(out)
    out.backward(g)
    tf = table.detach().float().requires_grad_()
    F.embedding(ids, tf).backward(g.float())
    assert rel_err(table.grad, tf.grad) < 1e-2


def test_embedding_backward_into_the_gradient_buffer(dev):
    """Many repeated tokens, two micro-batches accumulating into one bf16 and one fp32 gradient
    buffer, against an fp32 index_add; the result must also be bit-identical from run to run."""
    from elf_b200.ops import fused as Fu

    torch.manual_seed(5)
    vocab, dim = 500, 512
    for grad_dtype in (torch.bfloat16, torch.float32):
        table = torch.nn.Parameter(torch.randn(vocab, dim, device=dev, dtype=torch.bfloat16))
        ref = torch.zeros(vocab, dim, device=dev, dtype=torch.float32)
        runs = []
        for attempt in range(2):
            buf = torch.zeros(vocab, dim, device=dev, dtype=grad_dtype)
            if grad_dtype == torch.bfloat16:
                table.grad = buf
            else:
                table.grad, table.main_grad = None, buf
            gen = torch.Generator(device=dev).manual_seed(11)
            for mb in range(2):
                ids = torch.randint(0, 40 if mb == 0 else vocab, (2, 300), device=dev, generator=gen)  # heavy repetition in the first
                g = torch.randn(2, 300, dim, device=dev, dtype=torch.bfloat16, generator=gen)
                Fu.embedding(table, ids, into_grad=True).backward(g)
                if attempt == 0:
                    ref.index_add_(0, ids.reshape(-1), g.reshape(-1, dim).float())
            runs.append(buf.clone())
        assert torch.equal(runs[0], runs[1]), "embedding backward is not deterministic"
        assert rel_err(runs[0], ref) < (1e-2 if grad_dtype == torch.bfloat16 else 1e-6)
        if hasattr(table, "main_grad"):
            del table.main_grad


def test_fused_adamw(dev):
    from elf_b200.optim import FusedAdamW

    torch.manual_seed(3)
    ps = [torch.nn.Parameter(torch.randn(257, 33, device=dev).to(torch.bfloat16)), torch.nn.Parameter(torch.randn(1001, device=dev).to(torch.bfloat16))]
    ref = [torch.nn.Parameter(p.detach().float().clone()) for p in ps]
    opt = FusedAdamW(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-5, weight_decay=0.1)
    ropt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.95), eps=1e-5, weight_decay=0.1)
    for _ in range(4):
        for p, q in zip(ps, ref):
            g = torch.randn_like(p)
            p.grad.copy_(g)
            q.grad = g.float()
        opt.step()
        ropt.step()
        opt.zero_grad()
    for (w, q) in zip([opt.master[0]], [torch.cat([r.detach().reshape(-1) for r in ref])]):
        got = torch.cat([w[o : o + p.numel()] for o, p in zip(opt.groups[0].offsets, ps)])
        assert rel_err(got, q) < 1e-5
    for p, q in zip(ps, ref):
        assert rel_err(p, q) < 5e-3


def _attention_reference(qkv, hq, hkv):
    import math

    q = qkv[:, :, :hq].transpose(1, 2)
    k = qkv[:, :, hq : hq + hkv].transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    v = qkv[:, :, hq + hkv :].transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    n = s.shape[-1]
    s = s.masked_fill(torch.triu(torch.ones(n, n, device=s.device, dtype=torch.bool), 1), float("-inf"))
    return (torch.softmax(s, -1) @ v).transpose(1, 2), torch.logsumexp(s, -1)


@pytest.mark.parametrize(
    "batch,seq,hq,hkv,mult",
    [(1, 128, 1, 1, 1.0), (1, 384, 2, 2, 1.0), (1, 512, 3, 1, 1.0), (2, 384, 4, 2, 1.0), (1, 1024, 8, 2, 3.0), (1, 2048, 4, 1, 1.0)],
)
def test_attention_forward_kernel(dev, batch, seq, hq, hkv, mult):
    """tcgen05 flash attention forward against fp32 softmax(QK^T)V; `mult` widens the score
    range so that the lazy re-scaling of the running maximum is exercised.  Even group sizes
    pair two heads per work item, odd ones (and multi-head attention) pair two query tiles,
    with a lone first tile when the tile count is odd."""
    from elf_b200.ops import attention_native as A
    from elf_b200.ops import gemm as G

    torch.manual_seed(seq + hq)
    qkv = (torch.randn(batch, seq, hq + 2 * hkv, 128, device=dev) * mult).bfloat16()
    out, lse = A.forward_packed(qkv, hq, hkv)
    G.check_status(dev)
    ref_out, ref_lse = _attention_reference(qkv.float(), hq, hkv)
    assert rel_err(out, ref_out) < 1e-2
    assert (lse - ref_lse).abs().max().item() < 2e-2


@pytest.mark.parametrize("backward", ["native", "library"])
@pytest.mark.parametrize("batch,seq,hq,hkv", [(2, 256, 4, 2), (1, 512, 2, 2), (1, 384, 3, 1)])
def test_attention_native_backward(dev, backward, batch, seq, hq, hkv):
    """Gradient of the native attention op against fp32 autograd of the plain formula: own
    backward kernels (dK / dV in tensor memory, dQ through the fp32 accumulator) and the
    variant that feeds the library's fused backward with our output and log-sum-exp."""
    from elf_b200.ops import attention_native as A
    from elf_b200.ops import gemm as G

    torch.manual_seed(7)
    qkv = torch.randn(batch, seq, hq + 2 * hkv, 128, device=dev).bfloat16()
    g = torch.randn(batch, seq, hq, 128, device=dev).bfloat16()
    x = qkv.clone().requires_grad_()
    old = A._BACKWARD
    A._BACKWARD = backward
    try:
        for _ in range(2):  # the second pass re-uses the cached (re-zeroed) dQ accumulator
            x.grad = None
            A.native_attention_packed(x, hq, hkv).backward(g)
    finally:
        A._BACKWARD = old
    G.check_status(dev)
    x32 = qkv.float().requires_grad_()
    _attention_reference(x32, hq, hkv)[0].backward(g.float())
    assert rel_err(x.grad[:, :, :hq], x32.grad[:, :, :hq]) < 1e-2
    assert rel_err(x.grad[:, :, hq : hq + hkv], x32.grad[:, :, hq : hq + hkv]) < 1e-2
    assert rel_err(x.grad[:, :, hq + hkv :], x32.grad[:, :, hq + hkv :]) < 1e-2


def test_llama_layer_with_native_attention(dev):
    """The Llama decoder layer gives the same output and input gradient whether attention runs on
    the library or on the hand-written kernels."""
    from elf_b200.models.llama import LlamaConfig, LlamaDecoderLayer, init_llama_
    from elf_b200.ops import attention_native as A

    torch.manual_seed(3)
    cfg = LlamaConfig(n_layers=1, d_model=512, n_heads=4, n_kv_heads=2, ffn=1024, vocab=1024, seq_len=256)
    layer = init_llama_(LlamaDecoderLayer(cfg).to(dev).to(torch.bfloat16), 0.05, seed=1)
    x = torch.randn(2, 256, 512, device=dev, dtype=torch.bfloat16)
    results = []
    default_mode = A._MODE
    for mode in ("library", "native"):
        A.set_mode(mode)
        try:
            xi = x.clone().requires_grad_()
            y = layer(xi)
            y.float().square().mean().backward()
            results.append((y.detach(), xi.grad.detach()))
        finally:
            A.set_mode(default_mode)
    assert rel_err(results[1][0], results[0][0]) < 1e-2
    assert rel_err(results[1][1], results[0][1]) < 2e-2


def test_llama_layer_matches_fp32_reference(dev):
    """A decoder layer on the kernels vs. the same module in fp32 on torch ops."""
    from elf_b200.models.llama import LlamaConfig, LlamaDecoderLayer, init_llama_
    from elf_b200.ops import gemm
    from elf_b200.zb_utils import LayerDW, replace_layer_with_layer_dw

    cfg = LlamaConfig(n_layers=1, d_model=512, n_heads=4, n_kv_heads=2, ffn=1024, vocab=1024, seq_len=256)
    torch.manual_seed(0)
    layer = init_llama_(LlamaDecoderLayer(cfg).to(dev).to(torch.bfloat16), 0.05, seed=1)
    ref = LlamaDecoderLayer(cfg).to(dev).float()
    ref.load_state_dict({k: v.float() for k, v in layer.state_dict().items()})
    replace_layer_with_layer_dw(layer)
    x = torch.randn(2, 256, 512, device=dev, dtype=torch.bfloat16, requires_grad=True)
    xr = x.detach().float().requires_grad_()
    y = layer(x)
    g = torch.randn_like(y)
    y.backward(g)
    for m in layer.modules():
        if isinstance(m, LayerDW):
            m.move_last_computed("input", 0)
            m.move_last_computed("grad_output", 0)
            m.backward(0)
    gemm.set_enabled(False)
    try:
        yr = ref(xr)
        yr.backward(g.float())
    finally:
        gemm.set_enabled(True)
    assert rel_err(y, yr) < 2e-2
    assert rel_err(x.grad, xr.grad) < 3e-2
    for (n, p), (_, q) in zip(layer.named_parameters(), ref.named_parameters()):
        assert rel_err(p.grad, q.grad) < 3e-2, n
    gemm.check_status()


def test_smoke_entry(dev):
    import __graft_entry__

    __graft_entry__.smoke()


def test_attention_at_the_benchmark_shape(dev):
    """B=1, S=4096, 32 query / 8 KV heads (the Llama-3-8B layer): all 148 CTAs persistent, 32 key
    tiles per head.  The fp32 formula is evaluated on a sample of heads only (the full score
    matrix would be 2 GB per head group); forward output, log-sum-exp and all three gradients."""
    from elf_b200.ops import attention_native as A
    from elf_b200.ops import gemm as G

    torch.manual_seed(11)
    seq, hq, hkv = 4096, 32, 8
    qkv = torch.randn(1, seq, hq + 2 * hkv, 128, device=dev).bfloat16()
    g = torch.randn(1, seq, hq, 128, device=dev).bfloat16()
    out, lse = A.forward_packed(qkv, hq, hkv)
    dqkv = A.backward_packed(g, qkv, out, lse, hq, hkv)
    G.check_status(dev)
    group = hq // hkv
    for kv in (0, 5, 7):  # first, a middle and the last KV head, with the 4 query heads that share it
        heads = list(range(kv * group, (kv + 1) * group))
        sub = torch.cat([qkv[:, :, heads], qkv[:, :, hq + kv : hq + kv + 1], qkv[:, :, hq + hkv + kv : hq + hkv + kv + 1]], dim=2).float().requires_grad_()
        ref_out, ref_lse = _attention_reference(sub, group, 1)
        assert rel_err(out[:, :, heads], ref_out) < 1e-2
        assert (lse[:, heads] - ref_lse).abs().max().item() < 2e-2
        ref_out.backward(g[:, :, heads].float())
        want = sub.grad
        assert rel_err(dqkv[:, :, heads], want[:, :, :group]) < 2e-2  # dQ
        assert rel_err(dqkv[:, :, hq + kv], want[:, :, group]) < 2e-2  # dK, summed over the group
        assert rel_err(dqkv[:, :, hq + hkv + kv], want[:, :, group + 1]) < 2e-2  # dV


def test_residual_add_and_norm_gain_gradient_into_bf16(dev):
    from elf_b200.ops import _ext

    ext = _ext.get()
    torch.manual_seed(2)
    a = torch.randn(300, 4096, device=dev, dtype=torch.bfloat16)
    b = torch.randn_like(a)
    want = (a.float() + b.float()).bfloat16()
    got = ext.residual_add(a, b)
    assert got.data_ptr() == a.data_ptr() and torch.equal(got, want)
    # RMSNorm backward adding the gain's gradient to a bf16 buffer that already holds something
    x = torch.randn(300, 4096, device=dev).bfloat16()
    dy = torch.randn_like(x)
    w = (1 + 0.1 * torch.randn(4096, device=dev)).bfloat16()
    _, rstd, _ = ext.rmsnorm_fwd(x, w, 1e-5, None)
    dw32 = torch.empty(4096, device=dev, dtype=torch.float32)
    dx_ref = ext.rmsnorm_bwd(dy, x, w, rstd, dw32, False, None, None)
    buf = torch.full((4096,), 0.5, device=dev, dtype=torch.bfloat16)
    dx = ext.rmsnorm_bwd(dy, x, w, rstd, buf, True, None, None)
    assert torch.equal(dx, dx_ref)
    assert rel_err(buf, dw32 + 0.5) < 5e-3
    with pytest.raises(RuntimeError, match="only be accumulated"):
        ext.rmsnorm_bwd(dy, x, w, rstd, buf, False, None, None)


@pytest.mark.parametrize("block", ["layer", "attention", "mlp"])
def test_single_node_layer_matches_the_composed_layer(dev, block):
    """The hand-written backward (one autograd node per layer or half layer) against the same
    module run as a chain of small autograd functions: output, input gradient, the W-pass
    operands it files and every parameter gradient after the W pass."""
    from elf_b200.models import llama as L
    from elf_b200.zb_utils import LayerDW, replace_layer_with_layer_dw

    cfg = L.LlamaConfig(n_layers=1, d_model=512, n_heads=4, n_kv_heads=2, ffn=1536, vocab=1024, seq_len=256, rope_theta=500000.0)
    cls = {"layer": L.LlamaDecoderLayer, "attention": L.LlamaAttentionBlock, "mlp": L.LlamaMLPBlock}[block]
    results = {}
    for fused in (False, True):
        torch.manual_seed(0)
        with torch.device(dev):
            m = cls(cfg).to(torch.bfloat16)
        L.init_llama_(m, 0.02, 3)
        replace_layer_with_layer_dw(m)
        m.fused = fused
        x = torch.randn(2, cfg.seq_len, cfg.d_model, device=dev, generator=torch.Generator(device=dev).manual_seed(1)).bfloat16().requires_grad_()
        g = torch.randn(2, cfg.seq_len, cfg.d_model, device=dev, generator=torch.Generator(device=dev).manual_seed(2)).bfloat16()
        layers = [mod for mod in m.modules() if isinstance(mod, LayerDW)]
        for mb in range(2):  # two micro-batches: gradients accumulate
            y = m(x)
            for layer in layers:
                layer.move_last_computed("input", mb)
            y.backward(g)
            for layer in layers:
                layer.move_last_computed("grad_output", mb)
        for mb in range(2):
            for layer in layers:
                layer.backward(mb)
        results[fused] = (y.detach(), x.grad.clone(), {n: p.grad.clone() for n, p in m.named_parameters()})
    (y0, dx0, g0), (y1, dx1, g1) = results[False], results[True]
    assert rel_err(y1, y0) < 2e-3
    assert rel_err(dx1, dx0) < 1e-2
    assert set(g0) == set(g1)
    for name in g0:
        assert rel_err(g1[name], g0[name]) < 1e-2, name


def test_embedding_skips_and_records_an_id_outside_the_table(dev):
    """An out-of-range token id must not become an out-of-range read: its row comes back zero, its
    gradient is dropped, and the status word says which row and id."""
    from elf_b200.ops import fused as Fu
    from elf_b200.ops import gemm

    torch.cuda.synchronize()
    gemm.check_status()
    table = torch.nn.Parameter(torch.randn(64, 32, device=dev).bfloat16())
    ids = torch.tensor([[3, 64, 5, -2]], device=dev)
    out = Fu.embedding(table, ids, into_grad=True)
    assert torch.equal(out[0, 0], table[3]) and torch.equal(out[0, 2], table[5])
    assert out[0, 1].abs().sum() == 0 and out[0, 3].abs().sum() == 0
    out.float().sum().backward()
    assert table.grad[3].float().sum() == 32 and table.grad.float().sum() == 64  # rows 3 and 5 only
    rec = gemm.status(dev).tolist()
    assert rec[0] == 4 and rec[1] == 1 and (rec[2], rec[3]) in ((1, 64), (3, -2))
    with pytest.raises(RuntimeError, match="index outside its table"):
        gemm.check_status()
    gemm.check_status()  # the record is cleared by the check that raised


def test_partial_replay_through_a_single_node_layer(dev):
    """B -> W recompute on the fused layer: the replay refills the output-gradient stashes of
    the layer's linears with the values of the first backward and adds nothing to the norm
    gains' gradients a second time."""
    from elf_b200.models import llama as L
    from elf_b200.zb_utils import LayerDW, partial_dx_recomputation, replace_layer_with_layer_dw

    cfg = L.LlamaConfig(n_layers=1, d_model=512, n_heads=4, n_kv_heads=2, ffn=1536, vocab=1024, seq_len=256, rope_theta=500000.0)
    torch.manual_seed(0)
    with torch.device(dev):
        m = L.LlamaDecoderLayer(cfg).to(torch.bfloat16)
    L.init_llama_(m, 0.02, 3)
    replace_layer_with_layer_dw(m)
    m.fused = True
    layers = [mod for mod in m.modules() if isinstance(mod, LayerDW)]
    x = torch.randn(2, cfg.seq_len, cfg.d_model, device=dev).bfloat16().requires_grad_()
    g = torch.randn(2, cfg.seq_len, cfg.d_model, device=dev).bfloat16()
    y = m(x)
    for layer in layers:
        layer.move_last_computed("input", 0)
    y.backward(g, retain_graph=True)
    first = [layer.last_grad_output.clone() for layer in layers]
    gains = {n: p.grad.clone() for n, p in m.named_parameters() if "norm" in n}
    assert gains and all(t is not None for t in first)
    for layer in layers:
        layer.last_grad_output = None
    partial_dx_recomputation(y, g)
    for layer, ref in zip(layers, first):
        assert layer.last_grad_output is not None and rel_err(layer.last_grad_output, ref) < 1e-3
    for n, p in m.named_parameters():
        if "norm" in n:
            assert torch.equal(p.grad, gains[n]), n


def test_chunked_head_loss_matches_the_plain_head(dev):
    """LM head + cross entropy with the vocabulary in chunks (ragged last chunk, an ignored row)
    against fp32 logits: loss, hidden-state gradient, weight gradient added to what is there."""
    from elf_b200.ops.head_loss import chunked_head_loss

    torch.manual_seed(4)
    rows, d, vocab = 300, 512, 5000 * 8 // 8 + 8  # 5008: not a multiple of the chunk
    h = (torch.randn(rows, d, device=dev) * 0.5).bfloat16().requires_grad_()
    w = torch.nn.Parameter((torch.randn(vocab, d, device=dev) * 0.05).bfloat16())
    w.grad = torch.full_like(w, 0.25)
    t = torch.randint(0, vocab, (rows,), device=dev)
    t[7] = -100
    loss = chunked_head_loss(h, w, t, reduction="sum", chunk=1024)
    loss.backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = F.cross_entropy(hf @ wf.t(), t, reduction="sum", ignore_index=-100)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    assert rel_err(h.grad, hf.grad) < 2e-2
    assert rel_err(w.grad.float() - 0.25, wf.grad) < 2e-2
