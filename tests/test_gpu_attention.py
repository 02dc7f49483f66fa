"""tcgen05 variable-length attention (forward + backward) against the fp32 padded reference."""
import pytest
import torch

from nmtgminor_b200 import ops
from nmtgminor_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[0, 1, 2], ids=["auto", "general", "general_no_ws"])
def variant(request):
    """0 = automatic choice (persistent single-tile kernels up to 128 tokens, warp-specialised multi-tile kernels for long
    sequences), 1 = multi-tile kernels only, warp-specialised wherever they apply, 2 = multi-tile kernels without warp
    specialisation."""
    ops.ext().set_attention_variant(request.param)
    yield request.param
    ops.ext().set_attention_variant(0)


def _cu(lengths):
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    return cu.to(DEV)


def _poison():
    """Leave NaNs in the allocator's free blocks: the kernels must not rely on fresh memory being zero."""
    x = torch.full((32 << 20,), float("nan"), device=DEV, dtype=torch.bfloat16)
    del x


def _err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-6)).item()


@pytest.mark.parametrize("lengths", [[5], [128], [20, 100, 37, 64, 1], [16, 17, 31, 32, 33, 63, 64, 65, 96, 97, 127, 2, 3],
                                     [129, 200, 77], [300, 17], [0, 12, 0, 40]])
@pytest.mark.parametrize("causal", [False, True])
def test_self_attention_fwd_bwd(lengths, causal, variant):
    torch.manual_seed(0)
    heads, W = 4, 256
    n = sum(lengths)
    cap = (n + 127) // 128 * 128
    qkv = torch.randn(cap, 3 * W, device=DEV).bfloat16().requires_grad_(True)
    cu = _cu(lengths)
    _poison()
    out = ops.self_attention(qkv, cu, heads, max(lengths), causal=causal, dropout_p=0.0, training=True)
    assert ops.check_status() == 0
    dout = torch.randn(cap, W, device=DEV).bfloat16()
    dout[n:] = 0
    _poison()
    out.backward(dout)
    assert ops.check_status() == 0
    q32 = qkv.detach().float().requires_grad_(True)
    o_ref = ref.attention(q32[:, :W], q32[:, W:2 * W], q32[:, 2 * W:], cu, cu, heads, causal, 0.0)
    o_ref.backward(dout.float())
    assert _err(out[:n], o_ref[:n]) < 2e-2
    assert out[n:].abs().max().item() == 0 if cap > n else True
    g, gr = qkv.grad, q32.grad
    assert _err(g[:n, :W], gr[:n, :W]) < 3e-2, "dq"
    assert _err(g[:n, W:2 * W], gr[:n, W:2 * W]) < 3e-2, "dk"
    assert _err(g[:n, 2 * W:], gr[:n, 2 * W:]) < 3e-2, "dv"
    if cap > n:
        assert g[n:].abs().max().item() == 0


@pytest.mark.parametrize("lq,lk", [([7, 30], [50, 3]), ([100, 64, 12, 33], [128, 17, 99, 1]), ([100, 64, 12], [128, 129, 260]),
                                   ([140], [20])])
def test_cross_attention_fwd_bwd(lq, lk, variant):
    torch.manual_seed(1)
    heads, W = 2, 128
    nq, nk = sum(lq), sum(lk)
    cq, ck = nq + 24, nk + 40                      # spare rows past the last sequence, as in fixed-capacity batches
    q = torch.randn(cq, W, device=DEV).bfloat16().requires_grad_(True)
    kv = torch.randn(ck, 2 * W, device=DEV).bfloat16().requires_grad_(True)
    cu_q, cu_k = _cu(lq), _cu(lk)
    _poison()
    out = ops.cross_attention(q, kv, cu_q, cu_k, heads, max(lq), max(lk), 0.0, True)
    dout = torch.randn(cq, W, device=DEV).bfloat16()
    dout[nq:] = 0
    _poison()
    out.backward(dout)
    assert ops.check_status() == 0
    q32 = q.detach().float().requires_grad_(True)
    kv32 = kv.detach().float().requires_grad_(True)
    o_ref = ref.attention(q32, kv32[:, :W], kv32[:, W:], cu_q, cu_k, heads, False, 0.0)
    o_ref.backward(dout.float())
    assert _err(out[:nq], o_ref[:nq]) < 2e-2
    assert _err(q.grad[:nq], q32.grad[:nq]) < 3e-2
    assert _err(kv.grad[:nk], kv32.grad[:nk]) < 3e-2
    assert out[nq:].abs().max().item() == 0 and q.grad[nq:].abs().max().item() == 0 and kv.grad[nk:].abs().max().item() == 0


def test_many_items_per_cta_pipeline():
    """More (sequence, head) items than SMs so every persistent CTA walks several items."""
    torch.manual_seed(5)
    import numpy as np
    rng = np.random.RandomState(0)
    lengths = [int(v) for v in rng.randint(1, 101, size=200)]
    heads, W = 8, 512
    n = sum(lengths)
    cu = _cu(lengths)
    qkv = torch.randn(n, 3 * W, device=DEV).bfloat16().requires_grad_(True)
    out = ops.self_attention(qkv, cu, heads, 100, causal=True, dropout_p=0.0, training=True)
    dout = torch.randn(n, W, device=DEV).bfloat16()
    out.backward(dout)
    assert ops.check_status() == 0
    q32 = qkv.detach().float().requires_grad_(True)
    o_ref = ref.attention(q32[:, :W], q32[:, W:2 * W], q32[:, 2 * W:], cu, cu, heads, True, 0.0)
    o_ref.backward(dout.float())
    assert _err(out, o_ref) < 2e-2
    assert _err(qkv.grad, q32.grad) < 3e-2


def test_attention_dropout_is_replayed_in_backward(variant):
    """With dropout the op must stay a deterministic function of (seed, stream): finite differences of the
    forward agree with the analytic backward only if backward regenerates the forward mask."""
    torch.manual_seed(2)
    heads, W = 1, 64
    lengths = [40, 70]
    n = sum(lengths)
    cu = _cu(lengths)
    qkv = (torch.randn(n, 3 * W, device=DEV) * 0.5).bfloat16()
    ops.manual_seed(7)
    ops.reset_stream_counter()
    a = ops.self_attention(qkv, cu, heads, 70, dropout_p=0.2, training=True)
    ops.reset_stream_counter()
    b = ops.self_attention(qkv, cu, heads, 70, dropout_p=0.2, training=True)
    assert torch.equal(a, b)
    c = ops.self_attention(qkv, cu, heads, 70, dropout_p=0.0, training=True)
    assert not torch.equal(a, c)
    # linearity in V: out(v1 + v2) = out(v1) + out(v2) for a fixed mask; backward wrt V must equal P_drop^T dO
    x = qkv.clone().requires_grad_(True)
    ops.reset_stream_counter()
    o = ops.self_attention(x, cu, heads, 70, dropout_p=0.2, training=True)
    do = torch.randn_like(o)
    o.backward(do)
    dv = x.grad[:, 2 * W:].float()
    # probe: directional derivative along a random V direction
    dirv = torch.randn(n, W, device=DEV).bfloat16()
    x2 = qkv.clone()
    x2[:, 2 * W:] = dirv
    ops.reset_stream_counter()
    o_dir = ops.self_attention(x2, cu, heads, 70, dropout_p=0.2, training=True)   # = P_drop @ dirv
    lhs = (o_dir.float() * do.float()).sum().item()
    rhs = (dv * dirv.float()).sum().item()
    assert abs(lhs - rhs) <= 3e-2 * max(1.0, abs(lhs)), (lhs, rhs)


@pytest.mark.parametrize("lengths", [[5], [100, 37, 64], [129, 200, 77], [300, 17]])
@pytest.mark.parametrize("causal", [False, True])
def test_self_attention_with_additive_bias(lengths, causal):
    """An fp32 bias [batch, heads, T, T] on the scaled scores (relative-position terms): output, input gradients and the
    gradient of the bias itself against the fp32 padded statement.  The bias tensor is a padded view (row stride larger
    than the longest sequence), as models hand it over."""
    torch.manual_seed(3)
    heads, W = 4, 256
    n = sum(lengths)
    T = max(lengths)
    cap = (n + 127) // 128 * 128
    qkv = torch.randn(cap, 3 * W, device=DEV).bfloat16().requires_grad_(True)
    cu = _cu(lengths)
    store = torch.randn(len(lengths), heads, T + 3, T + 8, device=DEV)
    bias = store[:, :, :T, :T].detach().requires_grad_(True)
    _poison()
    out = ops.self_attention(qkv, cu, heads, T, causal=causal, dropout_p=0.0, training=True, bias=bias)
    assert ops.check_status() == 0
    dout = torch.randn(cap, W, device=DEV).bfloat16()
    dout[n:] = 0
    out.backward(dout)
    assert ops.check_status() == 0
    q32 = qkv.detach().float().requires_grad_(True)
    b32 = bias.detach().clone().requires_grad_(True)
    o_ref = ref.attention(q32[:, :W], q32[:, W:2 * W], q32[:, 2 * W:], cu, cu, heads, causal, 0.0, bias=b32)
    o_ref.backward(dout.float())
    assert _err(out[:n], o_ref[:n]) < 2e-2
    g, gr = qkv.grad, q32.grad
    assert _err(g[:n, :W], gr[:n, :W]) < 3e-2, "dq"
    assert _err(g[:n, W:2 * W], gr[:n, W:2 * W]) < 3e-2, "dk"
    assert _err(g[:n, 2 * W:], gr[:n, 2 * W:]) < 3e-2, "dv"
    assert _err(bias.grad, b32.grad) < 3e-2, "dbias"
    # pairs outside the sequences get no gradient
    for i, L in enumerate(lengths):
        assert bias.grad[i, :, L:, :].abs().max().item() == 0 if L < T else True
        assert bias.grad[i, :, :, L:].abs().max().item() == 0 if L < T else True


def test_wavlm_and_shaw_attention_run_on_the_fused_path():
    """The two relative-position attention modules of the speech encoders agree between the kernel path (bias operand)
    and the PyTorch statement of the same module on the CPU."""
    from nmtgminor_b200.models.layers import PackedSeqs
    from nmtgminor_b200.models.speech_encoders import GatedRelPosSelfAttention
    from nmtgminor_b200.models.w2vbert import ShawRelPosSelfAttention
    from nmtgminor_b200.parallel.flat import FlatParameterStore
    lengths = [150, 40]
    n = sum(lengths)
    cu = torch.zeros(3, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    for cls in (GatedRelPosSelfAttention, ShawRelPosSelfAttention):
        torch.manual_seed(1)
        mod = cls(128, 2, 0.0).eval()
        x = torch.randn(n, 128)
        seqs = PackedSeqs(torch.zeros(n, dtype=torch.long), torch.zeros(n, dtype=torch.long), cu, max(lengths))
        with torch.no_grad():
            want = mod(x, seqs)
        launches = ops.LAUNCHES[0]
        gpu = cls(128, 2, 0.0).eval()
        gpu.load_state_dict(mod.state_dict())
        gpu = gpu.to(DEV)
        FlatParameterStore(gpu, torch.device(DEV))
        with torch.no_grad():
            got = gpu(x.to(DEV).bfloat16(), seqs.to(DEV))
        assert ops.LAUNCHES[0] > launches and ops.check_status() == 0
        assert _err(got.float().cpu(), want) < 4e-2, cls.__name__


@pytest.mark.parametrize("causal", [False, True])
def test_relative_self_attention_long_sequences_use_the_bias_operand(causal):
    """Transformer-XL style attention over sequences longer than one tile: the position term and the content bias enter the
    tcgen05 kernels as an additive operand; output and gradients against the fp32 padded statement on CPU."""
    import copy
    from nmtgminor_b200.models.layers import PackedSeqs
    from nmtgminor_b200.models.relative_transformer import RelativeSelfAttention
    torch.manual_seed(11)
    H, h = 128, 2
    m32 = RelativeSelfAttention(H, h, 0.0, causal).eval()
    with torch.no_grad():
        m32.r_w_bias.normal_(0, 0.2)
        m32.r_r_bias.normal_(0, 0.2)
    lengths = [200, 150, 37]
    n = sum(lengths)
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    x32 = (torch.randn(n, H) * 0.5).requires_grad_()
    seqs_cpu = PackedSeqs(torch.zeros(n, dtype=torch.long), torch.zeros(n, dtype=torch.long), cu, max(lengths))
    want = m32(x32, seqs_cpu)
    gw = torch.autograd.grad(want.square().sum(), [x32, m32.r_w_bias, m32.r_r_bias])
    from nmtgminor_b200.parallel.flat import FlatParameterStore
    m = copy.deepcopy(m32).to(DEV)
    FlatParameterStore(m, torch.device(DEV))
    calls = ops.LAUNCHES[0]
    x = x32.detach().to(DEV).to(torch.bfloat16).requires_grad_()
    seqs = PackedSeqs(torch.zeros(n, dtype=torch.long, device=DEV), torch.zeros(n, dtype=torch.long, device=DEV), cu.to(DEV), max(lengths))
    got = m(x, seqs)
    gg = torch.autograd.grad(got.float().square().sum(), [x, m.r_w_bias, m.r_r_bias])
    assert ops.LAUNCHES[0] > calls and ops.check_status() == 0
    assert (got.float().cpu() - want).abs().max() < 0.06 * max(1.0, float(want.abs().max()))
    for a, b in zip(gg, gw):
        scale = max(1.0, float(b.abs().max()))
        assert (a.float().cpu() - b).abs().max() < 0.08 * scale


@pytest.mark.parametrize("hd", [32, 16, 48])
@pytest.mark.parametrize("cross", [False, True])
def test_heads_narrower_than_64_run_on_the_kernels(hd, cross):
    """Head sizes below 64 are zero-padded to the kernels' 64 columns; output and gradients against the fp32 statement."""
    torch.manual_seed(2)
    heads = 4
    W = heads * hd
    lq, lk = [70, 150, 9], [33, 140, 128]
    cu_q, cu_k = _cu(lq), _cu(lq if not cross else lk)
    nq, nk = sum(lq), sum(lq if not cross else lk)
    launches = ops.LAUNCHES[0]
    if cross:
        q = torch.randn(nq, W, device=DEV).bfloat16().requires_grad_(True)
        kv = torch.randn(nk, 2 * W, device=DEV).bfloat16().requires_grad_(True)
        out = ops.cross_attention(q, kv, cu_q, cu_k, heads, max(lq), max(lk), 0.0, True)
        leaves = [q, kv]
    else:
        qkv = torch.randn(nq, 3 * W, device=DEV).bfloat16().requires_grad_(True)
        out = ops.self_attention(qkv, cu_q, heads, max(lq), causal=True, dropout_p=0.0, training=True)
        leaves = [qkv]
    assert ops.LAUNCHES[0] > launches and ops.check_status() == 0
    dout = torch.randn(nq, W, device=DEV).bfloat16()
    grads = torch.autograd.grad(out, leaves, dout)
    l32 = [t.detach().float().requires_grad_(True) for t in leaves]
    if cross:
        o_ref = ref.attention(l32[0], l32[1][:, :W], l32[1][:, W:], cu_q, cu_k, heads, False, 0.0)
    else:
        o_ref = ref.attention(l32[0][:, :W], l32[0][:, W:2 * W], l32[0][:, 2 * W:], cu_q, cu_q, heads, True, 0.0)
    g_ref = torch.autograd.grad(o_ref, l32, dout.float())
    assert _err(out, o_ref) < 2e-2
    for g, gr in zip(grads, g_ref):
        assert _err(g, gr) < 3e-2


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("ws", [1, 2], ids=["ws", "no_ws"])
def test_long_sequences_walk_many_tiles(causal, ws):
    """Sequences of up to six 128-token tiles: every double buffer of the pipelined backward is reused several times."""
    torch.manual_seed(13)
    ops.ext().set_attention_variant(ws)
    try:
        heads, W = 2, 128
        lengths = [700, 333, 129, 5]
        n = sum(lengths)
        cu = _cu(lengths)
        qkv = (torch.randn(n, 3 * W, device=DEV) * 0.7).bfloat16().requires_grad_(True)
        out = ops.self_attention(qkv, cu, heads, max(lengths), causal=causal, dropout_p=0.0, training=True)
        dout = torch.randn(n, W, device=DEV).bfloat16()
        out.backward(dout)
        assert ops.check_status() == 0
        q32 = qkv.detach().float().requires_grad_(True)
        o_ref = ref.attention(q32[:, :W], q32[:, W:2 * W], q32[:, 2 * W:], cu, cu, heads, causal, 0.0)
        o_ref.backward(dout.float())
        assert _err(out, o_ref) < 2e-2
        g, gr = qkv.grad, q32.grad
        assert _err(g[:, :W], gr[:, :W]) < 3e-2, "dq"
        assert _err(g[:, W:2 * W], gr[:, W:2 * W]) < 3e-2, "dk"
        assert _err(g[:, 2 * W:], gr[:, 2 * W:]) < 3e-2, "dv"
        # encoder-decoder shape: 300 queries over 650 keys, and the dropout mask of the forward pass replayed
        lq, lk = [300, 40], [650, 200]
        cq, ck = _cu(lq), _cu(lk)
        q = (torch.randn(sum(lq), W, device=DEV) * 0.7).bfloat16().requires_grad_(True)
        kv = (torch.randn(sum(lk), 2 * W, device=DEV) * 0.7).bfloat16().requires_grad_(True)
        o = ops.cross_attention(q, kv, cq, ck, heads, max(lq), max(lk), 0.0, True)
        do = torch.randn_like(o)
        o.backward(do)
        assert ops.check_status() == 0
        q3, kv3 = q.detach().float().requires_grad_(True), kv.detach().float().requires_grad_(True)
        o3 = ref.attention(q3, kv3[:, :W], kv3[:, W:], cq, ck, heads, False, 0.0)
        o3.backward(do.float())
        assert _err(o, o3) < 2e-2 and _err(q.grad, q3.grad) < 3e-2 and _err(kv.grad, kv3.grad) < 3e-2
    finally:
        ops.ext().set_attention_variant(0)


def test_pipelined_backward_replays_the_dropout_mask_on_long_sequences():
    """dV = P_drop^T dO checked through the linearity of the forward pass in V, on four key tiles."""
    torch.manual_seed(3)
    heads, W = 1, 64
    lengths = [500, 260]
    n = sum(lengths)
    cu = _cu(lengths)
    qkv = (torch.randn(n, 3 * W, device=DEV) * 0.5).bfloat16()
    ops.manual_seed(11)
    x = qkv.clone().requires_grad_(True)
    ops.reset_stream_counter()
    o = ops.self_attention(x, cu, heads, 500, dropout_p=0.2, training=True)
    do = torch.randn_like(o)
    o.backward(do)
    assert ops.check_status() == 0
    dv = x.grad[:, 2 * W:].float()
    dirv = torch.randn(n, W, device=DEV).bfloat16()
    x2 = qkv.clone()
    x2[:, 2 * W:] = dirv
    ops.reset_stream_counter()
    o_dir = ops.self_attention(x2, cu, heads, 500, dropout_p=0.2, training=True)
    lhs = (o_dir.float() * do.float()).sum().item()
    rhs = (dv * dirv.float()).sum().item()
    assert abs(lhs - rhs) <= 3e-2 * max(1.0, abs(lhs)), (lhs, rhs)
