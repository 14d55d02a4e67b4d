"""The fp32 row ops of the ternary15m block stack (rmsnorm, swiglu, softmax cross-entropy, batched
grouped-query attention, their backward kernels, the sgd step) through the C ABI, against float64
restatements of MotifCL's shader arithmetic (kernels/vulkan/rmsnorm_f32.comp, rmsnorm_bwd_x_f32.comp,
rmsnorm_bwd_w_f32.comp, swiglu_f32.comp, swiglu_bwd_f32.comp, ce_fwd_rows_f32.comp, ce_bwd_f32.comp,
gqa_fwd_general_f32.comp, gqa_bwd_probs_f32.comp, gqa_bwd_dkv_f32.comp).  These are floating-point
kernels whose reduction order differs from the shaders', so the bar is a tolerance, stated per test:
relative L2 error <= 2e-6 against the float64 result (fp32 rounding of sums of a few hundred terms).
"""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-6


def rel_l2(a, ref):
    a = a.detach().double().cpu()
    ref = ref.detach().double().cpu()
    return float((a - ref).norm() / max(float(ref.norm()), 1e-30))


def dev(a):
    return a.to("cuda", torch.float32).contiguous()


@pytest.mark.parametrize("rows,cols", [(7, 288), (256, 288), (33, 100), (4, 4096)])
def test_rmsnorm_forward_and_backward(ctx, rows, cols):
    g = torch.Generator().manual_seed(rows * 1000 + cols)
    x = torch.randn(rows, cols, generator=g, dtype=torch.float64)
    w = torch.rand(cols, generator=g, dtype=torch.float64) + 0.5
    dy = torch.randn(rows, cols, generator=g, dtype=torch.float64)
    eps = 1e-5
    inv = 1.0 / torch.sqrt((x * x).mean(dim=1, keepdim=True) + eps)
    ref_y = x * inv * w
    dot = (dy * w * x).sum(dim=1, keepdim=True)
    ref_dx = dy * w * inv - x * inv ** 3 * dot / cols
    ref_dw = (dy * x * inv).sum(dim=0)

    xd, wd, dyd = dev(x), dev(w), dev(dy)
    y = torch.empty_like(xd)
    ctx.rmsnorm(xd, wd, y, rows, cols, eps)
    dx = torch.empty_like(xd)
    ctx.rmsnorm_backward_x(xd, wd, dyd, dx, rows, cols, eps)
    row_inv = torch.empty(rows, device="cuda")
    dw = torch.full((cols,), 123.0, device="cuda")          # must be overwritten, not accumulated into
    ctx.rmsnorm_backward_weight(xd, dyd, row_inv, dw, rows, cols, eps)
    torch.cuda.synchronize()
    assert rel_l2(y, ref_y) <= TOL
    assert rel_l2(dx, ref_dx) <= TOL
    assert rel_l2(row_inv, inv.squeeze(1)) <= TOL
    assert rel_l2(dw, ref_dw) <= TOL


@pytest.mark.parametrize("rows,hidden", [(5, 768), (300, 64), (1, 1)])
def test_swiglu_forward_and_backward(ctx, rows, hidden):
    g = torch.Generator().manual_seed(rows + hidden)
    packed = torch.randn(rows, 2 * hidden, generator=g, dtype=torch.float64) * 2
    dy = torch.randn(rows, hidden, generator=g, dtype=torch.float64)
    gate, up = packed[:, :hidden], packed[:, hidden:]
    sig = torch.sigmoid(gate)
    ref = gate * sig * up
    ref_d = torch.cat([dy * up * (sig + gate * sig * (1 - sig)), dy * gate * sig], dim=1)
    pd, dyd = dev(packed), dev(dy)
    out = torch.empty(rows, hidden, device="cuda")
    ctx.swiglu(pd, out, rows, hidden)
    dp = torch.empty_like(pd)
    ctx.swiglu_backward(pd, dyd, dp, rows, hidden)
    torch.cuda.synchronize()
    assert rel_l2(out, ref) <= TOL
    assert rel_l2(dp, ref_d) <= TOL


@pytest.mark.parametrize("rows,cols", [(9, 32000), (64, 257), (1, 2)])
def test_softmax_cross_entropy_forward_and_backward(ctx, rows, cols):
    g = torch.Generator().manual_seed(rows * 7 + cols)
    logits = torch.randn(rows, cols, generator=g, dtype=torch.float64) * 3
    targets = torch.randint(0, cols, (rows,), generator=g, dtype=torch.int32)
    if rows > 2:
        targets[1] = -1            # outside [0, cols): contributes a zero loss, like the reference's shader
    valid = (targets >= 0) & (targets < cols)
    lse = torch.logsumexp(logits, dim=1)
    picked = logits[torch.arange(rows), targets.clamp(0, cols - 1).long()]
    ref_rows = torch.where(valid, lse - picked, torch.zeros_like(lse))
    ref_loss = ref_rows.sum() / rows
    go = 0.75
    onehot = torch.zeros_like(logits)
    onehot[torch.arange(rows)[valid], targets[valid].long()] = 1.0
    ref_grad = go / rows * (torch.softmax(logits, dim=1) - onehot)

    ld, td = dev(logits), targets.to("cuda")
    partial = torch.empty(rows, device="cuda")
    out = torch.empty(1, device="cuda")
    ctx.softmax_cross_entropy(ld, td, partial, out, rows, cols)
    grad = torch.empty_like(ld)
    ctx.softmax_cross_entropy_backward(ld, td, torch.tensor([go], device="cuda"), grad, rows, cols)
    torch.cuda.synchronize()
    assert rel_l2(partial, ref_rows) <= TOL
    assert abs(float(out[0]) - float(ref_loss)) <= TOL * max(1.0, abs(float(ref_loss)))
    assert rel_l2(grad, ref_grad) <= TOL


def _attention_reference(q, k, v, B, Tq, Tk, H, G, hd, vhd, causal, q_off, window, scale):
    """float64 attention with the reference's masking rules; returns out and the probabilities."""
    qh = q.view(B, Tq, H, hd).permute(0, 2, 1, 3)
    kh = k.view(B, Tk, G, hd).permute(0, 2, 1, 3).repeat_interleave(H // G, dim=1)
    vh = v.view(B, Tk, G, vhd).permute(0, 2, 1, 3).repeat_interleave(H // G, dim=1)
    s = qh @ kh.transpose(-1, -2) * scale
    tq = torch.arange(Tq).view(Tq, 1) + q_off
    tk = torch.arange(Tk).view(1, Tk)
    allowed = torch.ones(Tq, Tk, dtype=torch.bool)
    if causal:
        allowed &= tk <= tq
    if window:
        allowed &= tk >= (tq + 1 - window).clamp(min=0)
    s = s.masked_fill(~allowed, float("-inf"))
    p = torch.softmax(s, dim=-1)
    out = (p @ vh).permute(0, 2, 1, 3).reshape(B * Tq, H * vhd)
    return out, p


@pytest.mark.parametrize("B,Tq,Tk,H,G,hd,causal,q_off,window", [
    (2, 64, 64, 6, 6, 48, False, 0, 0),        # the block stack's call: batched, unmasked
    (2, 64, 64, 6, 6, 48, True, 0, 0),         # the trainer's call: causal
    (1, 5, 37, 4, 2, 16, True, 32, 0),         # grouped heads, decode-style offset
    (1, 40, 40, 2, 1, 8, True, 0, 7),          # sliding window
    (1, 3, 300, 2, 2, 130, False, 0, 0),       # head_dim above one block's thread count
])
def test_gqa_forward_and_backward(ctx, B, Tq, Tk, H, G, hd, causal, q_off, window):
    g = torch.Generator().manual_seed(B * 100 + Tq + Tk + hd)
    q = torch.randn(B * Tq, H * hd, generator=g, dtype=torch.float64, requires_grad=True)
    k = torch.randn(B * Tk, G * hd, generator=g, dtype=torch.float64, requires_grad=True)
    v = torch.randn(B * Tk, G * hd, generator=g, dtype=torch.float64, requires_grad=True)
    dout = torch.randn(B * Tq, H * hd, generator=g, dtype=torch.float64)
    scale = 1.0 / math.sqrt(hd)
    ref, p = _attention_reference(q, k, v, B, Tq, Tk, H, G, hd, hd, causal, q_off, window, scale)

    qd, kd, vd = dev(q), dev(k), dev(v)
    out = torch.empty(B * Tq, H * hd, device="cuda")
    ctx.gqa_forward(qd, kd, vd, out, B, Tq, Tk, Tk, H, G, hd, hd, causal, q_off, window, scale)
    torch.cuda.synchronize()
    assert rel_l2(out, ref) <= TOL

    if window:
        return                                  # the reference's backward has no sliding window either
    ref.backward(dout)
    probs = torch.empty(B * H * Tq * Tk, device="cuda")
    ds = torch.empty_like(probs)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    ctx.gqa_backward(qd, kd, vd, dev(dout), probs, ds, dq, dk, dv, B, Tq, Tk, H, G, hd, causal, q_off, scale)
    torch.cuda.synchronize()
    assert rel_l2(probs.view(B, H, Tq, Tk), p) <= TOL
    assert rel_l2(dq, q.grad) <= 2 * TOL
    assert rel_l2(dk, k.grad) <= 2 * TOL
    assert rel_l2(dv, v.grad) <= 2 * TOL


def test_gqa_padded_key_stride(ctx):
    """Keys stored with a stride larger than key_tokens (a KV cache with room to grow)."""
    B, Tq, Tk, stride, H, G, hd = 2, 3, 10, 16, 4, 2, 32
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B * Tq, H * hd, generator=g, dtype=torch.float64)
    kfull = torch.randn(B, stride, G * hd, generator=g, dtype=torch.float64)
    vfull = torch.randn(B, stride, G * hd, generator=g, dtype=torch.float64)
    scale = 0.2
    ref, _ = _attention_reference(q, kfull[:, :Tk].reshape(B * Tk, -1), vfull[:, :Tk].reshape(B * Tk, -1),
                                  B, Tq, Tk, H, G, hd, hd, True, Tk - Tq, 0, scale)
    out = torch.empty(B * Tq, H * hd, device="cuda")
    ctx.gqa_forward(dev(q), dev(kfull.reshape(B * stride, -1)), dev(vfull.reshape(B * stride, -1)), out,
                    B, Tq, Tk, stride, H, G, hd, hd, True, Tk - Tq, 0, scale)
    torch.cuda.synchronize()
    assert rel_l2(out, ref) <= TOL


def test_sgd_step_and_argument_checks(ctx):
    n = 1000
    p = torch.randn(n, device="cuda")
    gr = torch.randn(n, device="cuda")
    out = torch.empty_like(p)
    ctx.eltwise(6, p, gr, out, n, 0.01)
    torch.cuda.synchronize()
    assert rel_l2(out, p.double() - 0.01 * gr.double()) <= TOL
    x = torch.zeros(4, 4, device="cuda")
    with pytest.raises(RuntimeError, match="non-zero"):
        ctx.rmsnorm(x, x, x, 0, 4, 1e-5)
    with pytest.raises(RuntimeError, match="n_head % n_kv_head"):
        ctx.gqa_forward(x, x, x, x, 1, 1, 1, 1, 3, 2, 1, 1, False, 0, 0, 1.0)
    with pytest.raises(RuntimeError, match="key_stride"):
        ctx.gqa_forward(x, x, x, x, 1, 1, 4, 2, 1, 1, 1, 1, False, 0, 0, 1.0)


def test_embedding_forward_and_backward(ctx):
    B, T, V, D = 3, 10, 50, 24
    g = torch.Generator().manual_seed(11)
    tw = torch.randn(V, D, generator=g, dtype=torch.float64)
    pw = torch.randn(T + 4, D, generator=g, dtype=torch.float64)       # a position table longer than the sequence
    ids = torch.randint(0, V, (B * T,), generator=g, dtype=torch.int32)
    ids[3] = -1                                                        # outside the table: token part is zero
    ids[4] = V
    ok = (ids >= 0) & (ids < V)
    tok = torch.where(ok.view(-1, 1), tw[ids.clamp(0, V - 1).long()], torch.zeros(1, D, dtype=torch.float64))
    ref = tok + pw[torch.arange(B * T) % T]
    out = torch.empty(B * T, D, device="cuda")
    ctx.token_position_embedding(dev(tw), dev(pw), ids.cuda(), out, B * T, V, T, D)
    gather = torch.empty(B * T, D, device="cuda")
    ctx.token_position_embedding(dev(tw), None, ids.cuda(), gather, B * T, V, 1, D)
    torch.cuda.synchronize()
    assert rel_l2(out, ref) <= TOL
    assert rel_l2(gather, tok) <= TOL

    go = torch.randn(B * T, D, generator=g, dtype=torch.float64)
    ref_gw = torch.zeros(V, D, dtype=torch.float64)
    ref_gw.index_add_(0, ids[ok].long(), go[ok])
    gw = torch.full((V, D), 9.0, device="cuda")
    ctx.embedding_weight_backward(ids.cuda(), dev(go), gw, V, D, B * T, zero_first=True)
    acc = torch.ones(V, D, device="cuda")
    ctx.embedding_weight_backward(ids.cuda(), dev(go), acc, V, D, B * T, zero_first=False)
    gp = torch.empty(T, D, device="cuda")
    ctx.position_embedding_backward(dev(go), gp, B, T, D)
    torch.cuda.synchronize()
    assert rel_l2(gw, ref_gw) <= TOL
    assert rel_l2(acc, ref_gw + 1.0) <= TOL
    assert rel_l2(gp, go.view(B, T, D).sum(0)) <= TOL


def _rope_reference(x, B, T, H, hd, rd, off, theta, inverse, split_half):
    x = x.view(B, T, -1).clone()
    out = x.clone()
    rd = hd if rd <= 0 else min(rd, hd)
    rd -= rd & 1
    half = hd // 2
    pos = (torch.arange(T, dtype=torch.float64) + off).view(1, T)
    for h in range(H):
        for pair in range(rd // 2):
            lo, hi = (pair, half + pair) if split_half else (2 * pair, 2 * pair + 1)
            ang = pos / theta ** (2 * pair / hd)
            if inverse:
                ang = -ang
            a, b = x[:, :, h * hd + lo], x[:, :, h * hd + hi]
            out[:, :, h * hd + lo] = a * torch.cos(ang) - b * torch.sin(ang)
            out[:, :, h * hd + hi] = a * torch.sin(ang) + b * torch.cos(ang)
    return out.view(B * T, -1)


@pytest.mark.parametrize("split_half", [False, True])
@pytest.mark.parametrize("rd,off", [(0, 0), (8, 5)])
def test_rope_forward_and_inverse(ctx, split_half, rd, off):
    B, T, H, hd = 2, 9, 3, 16
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B * T, H * hd, generator=g, dtype=torch.float64)
    ref = _rope_reference(x, B, T, H, hd, rd, off, 10000.0, False, split_half)
    xd = dev(x)
    y = torch.empty_like(xd)
    ctx.rope(xd, y, B, T, H * hd, H, hd, rd, off, 10000.0, False, split_half)
    back = torch.empty_like(xd)
    ctx.rope(y, back, B, T, H * hd, H, hd, rd, off, 10000.0, True, split_half)
    torch.cuda.synchronize()
    # angles reach ~13 rad and are formed in fp32 (position / theta^e), as in the shader
    assert rel_l2(y, ref) <= 5e-6
    assert rel_l2(back, x) <= 5e-6


def test_adam_update(ctx):
    n = 5000
    g = torch.Generator().manual_seed(1)
    p = torch.randn(n, generator=g, dtype=torch.float64)
    gr = torch.randn(n, generator=g, dtype=torch.float64)
    m = torch.randn(n, generator=g, dtype=torch.float64) * 0.1
    v = torch.rand(n, generator=g, dtype=torch.float64) * 0.01
    lr, b1, b2, eps, wd, step = 6e-3, 0.9, 0.95, 1e-8, 0.1, 3
    c1, c2 = 1 / (1 - b1 ** step), 1 / (1 - b2 ** step)
    mn = b1 * m + (1 - b1) * gr
    vn = b2 * v + (1 - b2) * gr * gr
    ref = p - lr * (mn * c1 / (torch.sqrt(vn * c2) + eps) + wd * p)
    pd, md, vd = dev(p), dev(m), dev(v)
    ctx.adam_update(pd, dev(gr), md, vd, n, lr, b1, b2, eps, wd, c1, c2)
    torch.cuda.synchronize()
    assert rel_l2(pd, ref) <= TOL and rel_l2(md, mn) <= TOL and rel_l2(vd, vn) <= TOL


def test_reference_known_answer_inputs_for_rmsnorm_swiglu_add(ctx):
    """The fixed inputs and tolerances MotifCL's own backend test uses for these ops
    (tests/test_vulkan_backend.cpp:159-220): RMSNorm of two rows of four with eps 1e-6 (1e-5 abs), SwiGLU of two packed
    rows [gate | up] (1e-5 abs), add (1e-6 abs); expectations are the test's own float formulas."""
    dev = "cuda:0"
    t = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    rms_x = [1.0, 2.0, 3.0, 4.0, -2.0, 0.0, 2.0, 4.0]
    rms_w = [1.0, 0.5, 1.5, 2.0]
    out = torch.empty(8, dtype=torch.float32, device=dev)
    ctx.rmsnorm(t(rms_x), t(rms_w), out, 2, 4, 1.0e-6)
    ctx.finish()
    got = out.cpu().numpy()
    for r in range(2):
        ss = np.float32(0.0)
        for c in range(4):
            ss = np.float32(ss + np.float32(rms_x[r * 4 + c]) * np.float32(rms_x[r * 4 + c]))
        inv = np.float32(1.0) / np.sqrt(np.float32(ss / np.float32(4.0) + np.float32(1.0e-6)))
        for c in range(4):
            assert abs(got[r * 4 + c] - np.float32(rms_x[r * 4 + c]) * inv * np.float32(rms_w[c])) <= 1e-5
    sw = [1.0, -2.0, 0.5, 4.0, -1.5, 3.0, -2.0, 0.25]
    out = torch.empty(4, dtype=torch.float32, device=dev)
    ctx.swiglu(t(sw), out, 2, 2)
    ctx.finish()
    got = out.cpu().numpy()
    for r in range(2):
        for c in range(2):
            gate, up = np.float32(sw[r * 4 + c]), np.float32(sw[r * 4 + 2 + c])
            assert abs(got[r * 2 + c] - gate / (np.float32(1.0) + np.exp(-gate)) * up) <= 1e-5
    a, b = [1.0, -2.0, 3.5, 4.0], [4.0, 5.0, -0.5, -1.0]
    out = torch.empty(4, dtype=torch.float32, device=dev)
    ctx.eltwise(0, t(a), t(b), out, 4)
    ctx.finish()
    assert np.abs(out.cpu().numpy() - (np.float32(a) + np.float32(b))).max() <= 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 255, 256, 4096, 70001])
def test_mse_loss_and_backward_follow_the_opencl_kernels_order(ctx, n):
    """MotifCL kernels/loss.cl:1-43: chunk sums of 256 elements left to right, 256 strided lanes over the chunk sums, a
    128..1 tree, one division: restated here in float32 with numpy, and the result must be the same float."""
    rng = np.random.default_rng(n)
    pred = rng.standard_normal(n).astype(np.float32)
    target = rng.standard_normal(n).astype(np.float32)
    chunks = (n + 255) // 256
    partial = np.zeros(chunks, np.float32)
    for g in range(chunks):
        acc = np.float32(0.0)
        for i in range(g * 256, min(n, g * 256 + 256)):
            d = np.float32(pred[i] - target[i])
            acc = np.float32(acc + np.float32(d * d))
        partial[g] = acc
    scratch = np.zeros(256, np.float32)
    for lid in range(256):
        acc = np.float32(0.0)
        for i in range(lid, chunks, 256):
            acc = np.float32(acc + partial[i])
        scratch[lid] = acc
    stride = 128
    while stride > 0:
        scratch[:stride] = (scratch[:stride] + scratch[stride:2 * stride]).astype(np.float32)
        stride >>= 1
    want = np.float32(scratch[0] / np.float32(n))
    dev = torch.device("cuda:0")
    p_d, t_d = torch.from_numpy(pred).to(dev), torch.from_numpy(target).to(dev)
    part_d = torch.zeros(chunks, dtype=torch.float32, device=dev)
    out_d = torch.zeros(1, dtype=torch.float32, device=dev)
    ctx.mse_loss(p_d, t_d, part_d, out_d, n)
    assert np.array_equal(part_d.cpu().numpy().view(np.uint32), partial.view(np.uint32))
    assert out_d.cpu().numpy().view(np.uint32)[0] == want.view(np.uint32)
    g_out = torch.tensor([0.75], dtype=torch.float32, device=dev)
    g_d = torch.empty(n, dtype=torch.float32, device=dev)
    ctx.mse_backward(p_d, t_d, g_out, g_d, n)
    want_g = ((np.float32(0.75) * np.float32(2.0)) * (pred - target).astype(np.float32)).astype(np.float32) / np.float32(n)
    assert np.array_equal(g_d.cpu().numpy().view(np.uint32), want_g.astype(np.float32).view(np.uint32))

