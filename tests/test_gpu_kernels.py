"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from zenyx_b200.ops import _ext

    return _ext.C()


def _status_ok():
    from zenyx_b200.ops import _ext

    _ext.check_status()


def _rel_err(a, b):
    a = a.float()
    b = b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _close(a, ref, rel=2e-2, max_abs=3e-2):
    """Frobenius-relative error below `rel` AND no single element off by more than `max_abs` of the
    reference's largest magnitude (a wrong row or tile hides easily inside a norm)."""
    a, ref = a.float(), ref.float()
    worst = ((a - ref).abs().max() / (ref.abs().max() + 1e-12)).item()
    return _rel_err(a, ref) < rel and worst < max_abs


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 264, 136), (1000, 768, 520)])
def test_gemm_layouts(C, a_t, b_t, M, N, K):
    torch.manual_seed(0)
    dev = "cuda"
    if a_t and M % 8:
        pytest.skip("transposed A needs M % 8 == 0")
    a = torch.randn(M, K, device=dev).bfloat16()
    b = torch.randn(N, K, device=dev).bfloat16()
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_t else a
    b_in = b.t().contiguous() if b_t else b
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    C.gemm(a_in, b_in, out, a_t, b_t, None)
    _status_ok()
    assert _rel_err(out, ref) < 1e-2
    # fp32 output with an fp32 addend aliasing the output (gradient accumulation)
    acc = torch.randn(M, N, device=dev, dtype=torch.float32)
    ref2 = acc + ref
    C.gemm(a_in, b_in, acc, a_t, b_t, acc)
    _status_ok()
    assert _rel_err(acc, ref2) < 1e-3
    # bf16 output with a bf16 addend (residual connection)
    res = torch.randn(M, N, device=dev).bfloat16()
    out3 = torch.empty_like(res)
    C.gemm(a_in, b_in, out3, a_t, b_t, res)
    _status_ok()
    assert _rel_err(out3, ref + res.float()) < 1e-2


@pytest.mark.parametrize("with_addend", [False, True])
@pytest.mark.parametrize("M,N,K", [(1000, 264, 136), (130, 72, 64), (257, 512, 320)])
def test_gemm_output_view_leaves_its_surroundings_alone(C, M, N, K, with_addend):
    """bf16 output (and addend) as a window of a larger matrix: the epilogue's TMA stores clip at the window's
    edge, and the addend's TMA loads read zeros beyond it instead of the neighbouring values."""
    torch.manual_seed(3)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    big = torch.full((M + 3, N + 24), 7.0, device="cuda", dtype=torch.bfloat16)
    out = big[1:M + 1, 8:N + 8]
    res_big = torch.full((M + 2, N + 16), 1000.0, device="cuda", dtype=torch.bfloat16)
    res = res_big[2:, 8:N + 8]
    res.copy_(torch.randn(M, N, device="cuda"))
    C.gemm(a, b, out, False, False, res if with_addend else None)
    _status_ok()
    ref = a.float() @ b.float().t() + (res.float() if with_addend else 0)
    assert _close(out, ref)
    mask = torch.ones_like(big, dtype=torch.bool)
    mask[1:M + 1, 8:N + 8] = False
    assert (big[mask] == 7.0).all()


def test_gemm_large_persistent(C):
    torch.manual_seed(1)
    M, N, K = 4096, 4096, 1024
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    C.gemm(a, b, out, False, False, None)
    _status_ok()
    ref = a.float() @ b.float().t()
    assert _rel_err(out, ref) < 1e-2


def _attn_ref(q, k, v, scale, qpos, kpos, causal, window_blocks=0, global_every=0):
    """q [B,Sq,Hq,D], k/v [B,Skv,Hkv,D]; qpos/kpos global token positions. fp32 math."""
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * scale
    mask = torch.ones(Sq, k.shape[1], dtype=torch.bool, device=q.device)
    if causal:
        mask &= kpos[None, :] <= qpos[:, None]
    if window_blocks > 0:
        qb = (qpos // 128)[:, None]
        kb = (kpos // 128)[None, :]
        keep = (qb - kb).abs() < window_blocks
        if global_every > 0:
            keep |= (kb % global_every) == 0
        mask &= keep
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum("bhqk,bhkd->bhqd", p, vf).permute(0, 2, 1, 3)
    return o, lse


def _positions(chunk_pos, S):
    n = len(chunk_pos)
    L = S // n
    return torch.cat([torch.arange(p, p + L) for p in chunk_pos]).cuda()


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 256, 4, 1), (2, 512, 8, 2), (1, 384, 4, 4)])
def test_attn_fwd_basic(C, causal, B, S, Hq, Hkv):
    torch.manual_seed(2)
    D = 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    C.attn_fwd(q, k, v, o, lse, scale, causal, 0, 0, [0], [0], False, 0, 0, 0)
    _status_ok()
    pos = torch.arange(S, device="cuda")
    o_ref, lse_ref = _attn_ref(q, k, v, scale, pos, pos, causal)
    assert _close(o, o_ref)
    assert (lse - lse_ref).abs().max().item() < 2e-2


def test_attn_fwd_strided_qkv_and_long(C):
    """Q/K/V as column blocks of one fused projection buffer; enough KV tiles to cycle the ring."""
    torch.manual_seed(3)
    B, S, Hq, Hkv, D = 1, 2048, 4, 2, 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    q = qkv[:, : Hq * D].view(B, S, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].view(B, S, Hkv, D)
    o = torch.empty(B, S, Hq, D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    C.attn_fwd(q, k, v, o, lse, scale, True, 0, 0, [0], [0], False, 0, 0, 0)
    _status_ok()
    pos = torch.arange(S, device="cuda")
    o_ref, lse_ref = _attn_ref(q, k, v, scale, pos, pos, True)
    assert _close(o, o_ref)
    assert (lse - lse_ref).abs().max().item() < 2e-2


def test_attn_fwd_zigzag_ring_merge(C):
    """Emulates a 2-rank zigzag ring on one GPU: rank 0 holds chunks (0, 3), rank 1 holds (1, 2).
    Two calls (own KV, then the peer's KV with merge_prev) must equal full causal attention."""
    torch.manual_seed(4)
    B, S, Hq, Hkv, D = 1, 1024, 4, 2, 128
    L = S // 4
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(D)
    pos = torch.arange(S, device="cuda")
    o_ref, lse_ref = _attn_ref(q, k, v, scale, pos, pos, True)
    chunks = {0: [0, 3], 1: [1, 2]}

    def shard(t, r):
        return torch.cat([t[:, c * L : (c + 1) * L] for c in chunks[r]], dim=1).contiguous()

    for r in (0, 1):
        qr = shard(q, r)
        o = torch.empty_like(qr)
        lse = torch.empty(B, Hq, 2 * L, device="cuda", dtype=torch.float32)
        qpos = [c * L for c in chunks[r]]
        for step, owner in enumerate([r, 1 - r]):
            C.attn_fwd(qr, shard(k, owner), shard(v, owner), o, lse, scale, True, 0, 0, qpos,
                       [c * L for c in chunks[owner]], step > 0, 0, 0, 0)
        _status_ok()
        o_exp = shard(o_ref, r)
        lse_exp = torch.cat([lse_ref[:, :, c * L : (c + 1) * L] for c in chunks[r]], dim=2)
        assert _close(o, o_exp)
        assert (lse - lse_exp).abs().max().item() < 2e-2


def test_attn_fwd_block_sparse(C):
    torch.manual_seed(5)
    B, S, Hq, Hkv, D = 1, 2048, 2, 1, 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    C.attn_fwd(q, k, v, o, lse, scale, True, 3, 4, [0], [0], False, 0, 0, 0)
    _status_ok()
    pos = torch.arange(S, device="cuda")
    o_ref, lse_ref = _attn_ref(q, k, v, scale, pos, pos, True, 3, 4)
    assert _close(o, o_ref)
    assert (lse - lse_ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("rows,H", [(777, 4096), (130, 2048), (33, 1024), (50, 6144), (9, 8192 + 512)])
def test_rmsnorm(C, rows, H):
    # 4096 / 2048: row-in-registers forward; H <= 4096: one vector per thread backward, <= 8192: two, above: fallback
    torch.manual_seed(6)
    x = torch.randn(rows, H, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device="cuda")
    C.rmsnorm_fwd(x, w, y, rstd, 1e-5)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    assert _rel_err(y, ref) < 1e-2
    assert _rel_err(rstd, torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)) < 1e-4
    dy = torch.randn_like(x)
    ref.backward(dy.float())
    dx = torch.empty_like(x)
    dw = torch.zeros(H, device="cuda")
    C.rmsnorm_bwd(dy, x, w, rstd, dx, dw, None)
    assert _rel_err(dx, xf.grad) < 1e-2
    assert _rel_err(dw, wf.grad) < 1e-2
    # with the gradient of the residual branch added in, and dw accumulating on top of the first call
    dres = torch.randn_like(x)
    dx2 = torch.empty_like(x)
    C.rmsnorm_bwd(dy, x, w, rstd, dx2, dw, dres)
    assert _rel_err(dx2, xf.grad + dres.float()) < 1e-2
    assert _rel_err(dw, 2 * wf.grad) < 1e-2
    _status_ok()


def test_swiglu(C):
    torch.manual_seed(7)
    T, F = 300, 1024
    gu = torch.randn(T, 2 * F, device="cuda").bfloat16()
    h = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
    C.swiglu_fwd(gu, h)
    guf = gu.float().requires_grad_(True)
    ref = torch.nn.functional.silu(guf[:, :F]) * guf[:, F:]
    assert _rel_err(h, ref) < 1e-2
    dh = torch.randn_like(h)
    ref.backward(dh.float())
    dgu = torch.empty_like(gu)
    C.swiglu_bwd(gu, dh, dgu)
    assert _rel_err(dgu, guf.grad) < 1e-2


def test_rope(C):
    torch.manual_seed(8)
    T, Hq, Hkv, D = 256, 4, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    pos = torch.arange(T, device="cuda").float() * 3 + 5
    inv = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = pos[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()

    def rot(x):  # x [T, H, D]
        x1, x2 = x[..., : D // 2], x[..., D // 2 :]
        return torch.cat([x1 * cos[:, None] - x2 * sin[:, None], x2 * cos[:, None] + x1 * sin[:, None]], -1)

    qf = qkv[:, : Hq * D].float().view(T, Hq, D)
    kf = qkv[:, Hq * D : (Hq + Hkv) * D].float().view(T, Hkv, D)
    vf = qkv[:, (Hq + Hkv) * D :].float().view(T, Hkv, D).clone()
    work = qkv.clone()
    k_out = torch.empty(T, Hkv, D, device="cuda", dtype=torch.bfloat16)
    v_out = torch.empty(T, Hkv, D, device="cuda", dtype=torch.bfloat16)
    C.rope_qkv(work, cos, sin, k_out, v_out, Hq, Hkv, D, T, False)
    assert _rel_err(work[:, : Hq * D].view(T, Hq, D), rot(qf)) < 1e-2
    assert _rel_err(k_out, rot(kf)) < 1e-2
    assert torch.equal(v_out.float(), vf)
    # in place + inverse restores the input up to bf16 rounding
    work2 = qkv.clone()
    C.rope_qkv(work2, cos, sin, None, None, Hq, Hkv, D, T, False)
    C.rope_qkv(work2, cos, sin, None, None, Hq, Hkv, D, T, True)
    assert _rel_err(work2, qkv) < 1e-2


def test_embedding_and_ce(C):
    torch.manual_seed(9)
    V, H, T = 1024, 256, 500
    table = torch.randn(V, H, device="cuda").bfloat16()
    ids = torch.randint(0, V, (T,), device="cuda")
    out = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    C.embedding_fwd(ids, table, out)
    assert torch.equal(out, table[ids])
    dout = torch.randn(T, H, device="cuda").bfloat16()
    dtab = torch.zeros(V, H, device="cuda")
    C.embedding_bwd(ids, dout, dtab)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, ids, dout.float())
    assert _rel_err(dtab, ref) < 1e-5

    logits = (3 * torch.randn(T, V, device="cuda")).bfloat16()
    tgt = torch.randint(0, V, (T,), device="cuda")
    lf = logits.float().requires_grad_(True)
    loss_ref = torch.nn.functional.cross_entropy(lf, tgt, reduction="none")
    loss_ref.sum().backward()
    work = logits.clone()
    loss = torch.empty(T, device="cuda")
    C.ce_fwd_bwd(work, tgt, loss, 0.5, -100)
    assert (loss - loss_ref).abs().max().item() < 2e-2
    assert _close(work, 0.5 * lf.grad)


def test_kv_quant(C):
    torch.manual_seed(10)
    T, Hkv, D = 512, 2, 128
    x = (torch.randn(T, Hkv, D, device="cuda") * torch.rand(1, Hkv, 1, device="cuda") * 4).bfloat16()
    q = torch.empty(T, Hkv, D, device="cuda", dtype=torch.uint8)
    scales = torch.empty(T // 128, Hkv, device="cuda")
    C.kv_quant_e4m3(x, q, scales, None, 128)
    amax = x.float().view(T // 128, 128, Hkv, D).abs().amax(dim=(1, 3))
    assert torch.allclose(scales, amax / 448.0, rtol=1e-6)
    ref_q = (x.float().view(T // 128, 128, Hkv, D) / scales[:, None, :, None]).view(T, Hkv, D).to(torch.float8_e4m3fn)
    mismatch = (q.view(torch.float8_e4m3fn).float() != ref_q.float()).float().mean().item()
    assert mismatch < 1e-3
    back = torch.empty_like(x)
    C.kv_dequant_e4m3(q, scales, back, 128)
    assert _rel_err(back, x) < 0.05


def test_adamw_split_master(C):
    torch.manual_seed(11)
    n = 4096 * 3
    w0 = torch.randn(n, device="cuda")
    p = torch.nn.Parameter(w0.clone())
    opt = torch.optim.AdamW([p], lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    bits = w0.view(torch.int32)
    hi = ((bits + 0x8000) >> 16).to(torch.int16)
    lo = (bits - (hi.to(torch.int32) << 16)).to(torch.int16)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        p.grad = g.clone()
        opt.step()
        C.adamw(hi, lo, m, v, g, 3e-4, 0.9, 0.95, 1e-8, 0.1, step, 1.0, None)
    master = ((hi.to(torch.int32) << 16) + lo.to(torch.int32)).view(torch.float32)
    assert (master - p.data).abs().max().item() < 1e-6
    # the bf16 half is the nearest-bf16 of the master (ties up)
    assert _rel_err(hi.view(torch.bfloat16), master) < 4e-3
    ss = torch.zeros(1, device="cuda")
    C.sumsq(g, ss)
    assert abs(ss.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-4


@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_zero_step_kernel_matches_the_host_path(C, state_dtype):
    """The fused optimizer kernel (norm pass, clip, AdamW on the split master, parameter refresh) against the same
    optimizer on CPU tensors, for fp32 and for bf16 moments."""
    from zenyx_b200.models.llama import FlatBuffers
    from zenyx_b200.parallel.zero import ZeroAdamW

    specs = [("w", (256, 384), True), ("n", (256,), False)]
    torch.manual_seed(21)
    gpu = FlatBuffers(specs, "cuda")
    cpu = FlatBuffers(specs, "cpu")
    init = (torch.randn(gpu.total) * 0.1).bfloat16()
    gpu.params.copy_(init)
    cpu.params.copy_(init)
    kw = dict(lr=1e-2, weight_decay=0.1, max_grad_norm=1.0, single_process=True, state_dtype=state_dtype)
    og, oc = ZeroAdamW(gpu, **kw), ZeroAdamW(cpu, **kw)
    assert og.fused_peer and og.m.dtype == state_dtype
    for _ in range(6):
        g = torch.randn(gpu.total) * 0.5
        gpu.grads.copy_(g)
        cpu.grads.copy_(g)
        og.step()
        oc.step()
    _status_ok()
    assert float(gpu.grads.abs().sum()) == 0.0                      # consumed and cleared
    assert _rel_err(gpu.params.float().cpu(), cpu.params.float()) < 4e-3
    assert _rel_err(og.m.float().cpu(), oc.m.float()) < (1e-5 if state_dtype == torch.float32 else 6e-3)
    assert _rel_err(og.v.float().cpu(), oc.v.float()) < (1e-5 if state_dtype == torch.float32 else 6e-3)
    assert abs(og.grad_norm.item() - oc.grad_norm.item()) / oc.grad_norm.item() < 1e-4


def _attn_bwd_ref(q, k, v, do, scale, qpos, kpos, causal, wb=0, ge=0):
    qf = q.float().requires_grad_(True)
    kf = k.float().requires_grad_(True)
    vf = v.float().requires_grad_(True)
    o, _ = _attn_ref(qf, kf, vf, scale, qpos, kpos, causal, wb, ge)
    o.backward(do.float())
    return qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 256, 4, 1), (2, 512, 4, 2), (1, 1024, 2, 2)])
def test_attn_bwd_basic(C, causal, B, S, Hq, Hkv):
    torch.manual_seed(12)
    D = 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    C.attn_fwd(q, k, v, o, lse, scale, causal, 0, 0, [0], [0], False, 0, 0, 0)
    delta = torch.empty_like(lse)
    dq = torch.empty(B, S, Hq, D, device="cuda")
    dk = torch.zeros(B, S, Hkv, D, device="cuda")
    dv = torch.zeros(B, S, Hkv, D, device="cuda")
    C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, causal, 0, 0, [0], [0], True, False, 0, 0, 0)
    _status_ok()
    pos = torch.arange(S, device="cuda")
    dq_r, dk_r, dv_r = _attn_bwd_ref(q, k, v, do, scale, pos, pos, causal)
    assert _close(dv, dv_r)
    assert _close(dk, dk_r)
    assert _close(dq, dq_r)


def test_attn_bwd_zigzag_ring(C):
    """Two emulated zigzag ranks: each rank's backward runs one call per KV owner, accumulating dQ
    locally and adding dK/dV into the owner's buffers, exactly like the ring does over peer memory."""
    torch.manual_seed(13)
    B, S, Hq, Hkv, D = 1, 1024, 4, 2, 128
    L = S // 4
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(D)
    pos = torch.arange(S, device="cuda")
    dq_r, dk_r, dv_r = _attn_bwd_ref(q, k, v, do, scale, pos, pos, True)
    chunks = {0: [0, 3], 1: [1, 2]}

    def shard(t, r):
        return torch.cat([t[:, c * L : (c + 1) * L] for c in chunks[r]], dim=1).contiguous()

    dk_own = {r: torch.zeros(B, 2 * L, Hkv, D, device="cuda") for r in (0, 1)}
    dv_own = {r: torch.zeros(B, 2 * L, Hkv, D, device="cuda") for r in (0, 1)}
    for r in (0, 1):
        qr, dor = shard(q, r), shard(do, r)
        o = torch.empty_like(qr)
        lse = torch.empty(B, Hq, 2 * L, device="cuda", dtype=torch.float32)
        qpos = [c * L for c in chunks[r]]
        order = [r, 1 - r]
        for step, owner in enumerate(order):
            C.attn_fwd(qr, shard(k, owner), shard(v, owner), o, lse, scale, True, 0, 0, qpos,
                       [c * L for c in chunks[owner]], step > 0, 0, 0, 0)
        delta = torch.empty_like(lse)
        dq = torch.empty(B, 2 * L, Hq, D, device="cuda")
        for step, owner in enumerate(order):
            C.attn_bwd(qr, shard(k, owner), shard(v, owner), o, dor, lse, delta, dq, dk_own[owner], dv_own[owner],
                       scale, True, 0, 0, qpos, [c * L for c in chunks[owner]], step == 0, step > 0, 0, 0, 0)
        _status_ok()
        assert _close(dq, shard(dq_r, r))
    for r in (0, 1):
        assert _close(dk_own[r], shard(dk_r, r))
        assert _close(dv_own[r], shard(dv_r, r))


def test_attn_bwd_block_sparse(C):
    torch.manual_seed(14)
    B, S, Hq, Hkv, D = 1, 1536, 2, 1, 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    C.attn_fwd(q, k, v, o, lse, scale, True, 2, 4, [0], [0], False, 0, 0, 0)
    delta = torch.empty_like(lse)
    dq = torch.empty(B, S, Hq, D, device="cuda")
    dk = torch.zeros(B, S, Hkv, D, device="cuda")
    dv = torch.zeros(B, S, Hkv, D, device="cuda")
    C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, True, 2, 4, [0], [0], True, False, 0, 0, 0)
    _status_ok()
    pos = torch.arange(S, device="cuda")
    dq_r, dk_r, dv_r = _attn_bwd_ref(q, k, v, do, scale, pos, pos, True, 2, 4)
    assert _close(dv, dv_r)
    assert _close(dk, dk_r)
    assert _close(dq, dq_r)


def test_peer_barrier_wait_is_bounded(C):
    """A flag that nothing sets: the barrier kernel must give up within its limit, report the
    timeout through the status word, and leave the context usable."""
    import time

    from zenyx_b200.ops import _ext

    flags = C.peer_alloc(256)
    try:
        t0 = time.perf_counter()
        # pretend to be rank 0 of 2 with both flag arrays in our own memory: slot 1 is never written
        C.peer_barrier([flags, flags + 128], 0, 1, 200.0)
        with pytest.raises(_ext.KernelError) as ei:
            _ext.check_status()
        assert "timed out" in str(ei.value) and "peer barrier" in str(ei.value)
        assert time.perf_counter() - t0 < 5.0
        _ext.check_status()                      # the word was cleared; the context still works
        x = torch.ones(8, device="cuda")
        assert x.sum().item() == 8.0
    finally:
        torch.cuda.synchronize()
        C.peer_free(flags)


# ------------------------------------------------------------------------------------------------
# Out-of-bounds and race detection without a sanitizer: guard bands and repeatability
# ------------------------------------------------------------------------------------------------
def _guarded(shape, dtype, fill, guard_elems=4096):
    """A tensor of `shape` carved out of a larger buffer whose head and tail hold a known pattern."""
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * guard_elems,), fill, device="cuda", dtype=dtype)
    return buf, buf[guard_elems: guard_elems + n].view(*shape), guard_elems


def _guards_intact(buf, guard, fill):
    head, tail = buf[:guard], buf[-guard:]
    ref = torch.full_like(head, fill)
    return torch.equal(head.view(torch.int16 if buf.element_size() == 2 else torch.int32),
                       ref.view(torch.int16 if buf.element_size() == 2 else torch.int32)) and \
        torch.equal(tail.view(torch.int16 if buf.element_size() == 2 else torch.int32),
                    ref.view(torch.int16 if buf.element_size() == 2 else torch.int32))


def test_kernels_write_only_inside_their_outputs(C):
    """Every output of the GEMM (ragged M and N), of the attention forward and of the attention backward
    sits between guard bands filled with a pattern; the bands must come back untouched."""
    torch.manual_seed(21)
    M, N, K = 1000, 264, 520                       # ragged against the 128 x 256 x 64 tiles
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    gbuf, out, g = _guarded((M, N), torch.bfloat16, 77.0)
    C.gemm(a, b, out, False, False, None)
    _status_ok()
    assert _guards_intact(gbuf, g, 77.0)
    assert _rel_err(out, a.float() @ b.float().t()) < 1e-2
    fbuf, outf, g = _guarded((M, N), torch.float32, 77.0)
    outf.zero_()
    C.gemm(a, b, outf, False, False, outf)          # fp32 accumulate-into-self (weight-gradient epilogue)
    _status_ok()
    assert _guards_intact(fbuf, g, 77.0)
    B, S, Hq, Hkv, D = 1, 384, 4, 2, 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    obuf, o, g = _guarded((B, S, Hq, D), torch.bfloat16, 77.0)
    lbuf, lse, _ = _guarded((B, Hq, S), torch.float32, 77.0)
    scale = 1.0 / math.sqrt(D)
    C.attn_fwd(q, k, v, o, lse, scale, True, 0, 0, [0], [0], False, 0, 0, 0)
    _status_ok()
    assert _guards_intact(obuf, g, 77.0) and _guards_intact(lbuf, g, 77.0)
    dbuf, delta, _ = _guarded((B, Hq, S), torch.float32, 77.0)
    qbuf, dq, _ = _guarded((B, S, Hq, D), torch.float32, 77.0)
    kbuf, dk, _ = _guarded((B, S, Hkv, D), torch.float32, 77.0)
    vbuf, dv, _ = _guarded((B, S, Hkv, D), torch.float32, 77.0)
    dk.zero_()
    dv.zero_()
    C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, True, 0, 0, [0], [0], True, False, 0, 0, 0)
    _status_ok()
    for buf in (dbuf, qbuf, kbuf, vbuf):
        assert _guards_intact(buf, g, 77.0)
    pos = torch.arange(S, device="cuda")
    dq_r, dk_r, dv_r = _attn_bwd_ref(q, k, v, do, scale, pos, pos, True)
    assert _close(dq, dq_r) and _close(dk, dk_r) and _close(dv, dv_r)


def test_kernels_are_repeatable(C):
    """The same launch twice: GEMM, attention forward and dQ are deterministic and must match bit for
    bit; dK/dV are accumulated with fp32 atomics across query heads and tiles, so they may differ in
    the last bits only. A data race inside a kernel shows up here as a mismatch."""
    torch.manual_seed(22)
    a = torch.randn(1536, 1024, device="cuda").bfloat16()
    b = torch.randn(2048, 1024, device="cuda").bfloat16()
    outs = []
    for _ in range(2):
        o = torch.empty(1536, 2048, device="cuda", dtype=torch.bfloat16)
        C.gemm(a, b, o, False, False, None)
        outs.append(o)
    assert torch.equal(outs[0], outs[1])
    B, S, Hq, Hkv, D = 1, 2048, 8, 2, 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(D)
    res = []
    for _ in range(2):
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
        C.attn_fwd(q, k, v, o, lse, scale, True, 0, 0, [0], [0], False, 0, 0, 0)
        delta = torch.empty_like(lse)
        dq = torch.empty(B, S, Hq, D, device="cuda")
        dk = torch.zeros(B, S, Hkv, D, device="cuda")
        dv = torch.zeros(B, S, Hkv, D, device="cuda")
        C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, True, 0, 0, [0], [0], True, False, 0, 0, 0)
        res.append((o, lse, dq, dk, dv))
    _status_ok()
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    assert torch.equal(res[0][2], res[1][2])
    assert _rel_err(res[0][3], res[1][3]) < 1e-5 and _rel_err(res[0][4], res[1][4]) < 1e-5


@pytest.mark.parametrize("causal,wb,ge,chunks", [
    (True, 2, 0, [0]),                 # causal window, no global blocks
    (False, 2, 4, [0]),                # two-sided window plus global blocks
    (False, 3, 0, [0]),                # two-sided window only
    (True, 3, 4, [1024, 0]),           # two position chunks stored out of order (zigzag-style layout)
    (True, 1, 8, [512, 1536, 0, 1024]),  # four chunks, window of one block
])
def test_attn_sparse_tile_iteration_matches_reference(C, causal, wb, ge, chunks):
    """The windowed kernels jump over runs of excluded tiles; forward and backward must still agree with
    a reference that applies the mask element by element, for every combination of causal / two-sided
    windows, with and without global blocks, and for piecewise-contiguous position layouts."""
    torch.manual_seed(31)
    B, S, Hq, Hkv, D = 1, 2048, 2, 1, 128
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
    do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device="cuda", dtype=torch.float32)
    scale = 1.0 / math.sqrt(D)
    n = len(chunks)
    clen = S // n
    pos = torch.cat([torch.arange(c, c + clen, device="cuda") for c in chunks])
    C.attn_fwd(q, k, v, o, lse, scale, causal, wb, ge, chunks, chunks, False, 0, 0, 0)
    _status_ok()
    o_ref, lse_ref = _attn_ref(q, k, v, scale, pos, pos, causal, wb, ge)
    assert _close(o, o_ref)
    assert (lse - lse_ref).abs().max().item() < 2e-2
    delta = torch.empty_like(lse)
    dq = torch.empty(B, S, Hq, D, device="cuda")
    dk = torch.zeros(B, S, Hkv, D, device="cuda")
    dv = torch.zeros(B, S, Hkv, D, device="cuda")
    C.attn_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scale, causal, wb, ge, chunks, chunks, True, False, 0, 0, 0)
    _status_ok()
    dq_r, dk_r, dv_r = _attn_bwd_ref(q, k, v, do, scale, pos, pos, causal, wb, ge)
    assert _close(dv, dv_r)
    assert _close(dk, dk_r)
    assert _close(dq, dq_r)


# ------------------------------------------------------------------------------------------------
# Checked build (-DZX_CHECKED): same kernels with in-kernel index checks
# ------------------------------------------------------------------------------------------------
_CHECKED_SCRIPT = r"""
import math, torch
from zenyx_b200.ops import _ext
C = _ext.C()
torch.manual_seed(0)
B, S, Hq, Hkv, D = 2, 384, 4, 2, 128
q = torch.randn(B, S, Hq, D, device="cuda").bfloat16(); k = torch.randn(B, S, Hkv, D, device="cuda").bfloat16()
v = torch.randn(B, S, Hkv, D, device="cuda").bfloat16(); do = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
o = torch.empty_like(q); lse = torch.empty(B, Hq, S, device="cuda"); sc = 1 / math.sqrt(D)
C.attn_fwd(q, k, v, o, lse, sc, True, 0, 0, [0], [0], False, 0, 0, 0)
dq = torch.empty(B, S, Hq, D, device="cuda"); dk = torch.zeros(B, S, Hkv, D, device="cuda"); dv = torch.zeros_like(dk)
C.attn_bwd(q, k, v, o, do, lse, torch.empty_like(lse), dq, dk, dv, sc, True, 0, 0, [0], [0], True, False, 0, 0, 0)
a = torch.randn(200, 264, device="cuda").bfloat16(); b = torch.randn(136, 264, device="cuda").bfloat16()
out = torch.empty(200, 136, device="cuda", dtype=torch.bfloat16)
C.gemm(a, b, out, False, False, None)
_ext.check_status()      # raises if any index check fired
qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
ref = torch.nn.functional.scaled_dot_product_attention(qf, kf.repeat_interleave(2, 1), vf.repeat_interleave(2, 1), is_causal=True).permute(0, 2, 1, 3)
assert ((o.float() - ref).norm() / ref.norm()).item() < 2e-2
assert ((out.float() - a.float() @ b.float().t()).norm() / (a.float() @ b.float().t()).norm()).item() < 1e-2
assert torch.isfinite(dq).all() and torch.isfinite(dk).all() and torch.isfinite(dv).all()
print("checked ok")
"""


def test_checked_build_runs_clean():
    """The -DZX_CHECKED build of the kernels (``python -m zenyx_b200._build --checked``) runs attention forward
    and backward and a ragged GEMM with every epilogue row index tested in the kernel; no check fires and the
    results agree with fp32 math."""
    import os
    import subprocess
    import sys

    import zenyx_b200

    d = os.path.join(os.path.dirname(zenyx_b200.__file__), "_checked")
    if not os.path.exists(os.path.join(d, "_C.so")):
        pytest.skip("checked build not present: python -m zenyx_b200._build --checked")
    env = dict(os.environ, ZENYX_B200_EXT_DIR=d, PYTHONPATH=os.path.dirname(os.path.dirname(zenyx_b200.__file__)))
    res = subprocess.run([sys.executable, "-c", _CHECKED_SCRIPT], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "checked ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
