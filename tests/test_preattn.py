"""RMSNorm + rotary embedding of Q and K in one pass (the ops a video-DiT layer runs before the operator).
CPU: the oracle against the reference's complex-multiplication formula.  GPU: the fused kernel against the
oracle, and the operator on the strided (B,S,H,D) results against contiguous (B,H,S,D) copies."""
import math

import pytest
import torch

from oracle import vecattn_oracle as O


def _tables(s, d, seed):
    g = torch.Generator().manual_seed(seed)
    ang = torch.rand(s, d // 2, generator=g) * 6.283
    return torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous()


def test_oracle_rope_equals_complex_multiplication():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 3, 40, 128, generator=g).to(torch.bfloat16)
    cos, sin = _tables(40, 128, 2)
    freqs = torch.complex(cos.double(), sin.double())
    want = torch.view_as_real(torch.view_as_complex(x.double().unflatten(3, (-1, 2))) * freqs).flatten(3, 4)
    got = O.rope_interleaved(x, cos, sin)
    # equal to the double-precision product rounded once; torch's own cast rounds twice (through float32) and may
    # differ on isolated ties
    assert (got.double() - want).abs().max() <= (want.abs() * 2.0 ** -8).max()
    assert (got != want.to(x.dtype)).float().mean() <= 1e-4
    x64 = torch.tensor([1.00390625 + 2.0 ** -30, 1.00390625 - 2.0 ** -30, -1.00390625 - 2.0 ** -30], dtype=torch.float64)
    assert O._round_from_double(x64, torch.bfloat16).tolist() == [1.0078125, 1.0, -1.0078125]   # ties broken by the tail
    skipped = O.rope_interleaved(x, cos[:30], sin[:30], skip=10)
    assert torch.equal(skipped[:, :, :10], x[:, :, :10]) and not torch.equal(skipped[:, :, 10:], x[:, :, 10:])
    w = torch.rand(128, generator=g).to(torch.bfloat16)
    y = O.rms_norm(x, w, 1e-6)
    ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float())
    assert (y.float() - ref).abs().max() <= 2.0 ** -7 * ref.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads,kv_heads,s,skip", [(40, 40, 333, 0), (24, 24, 1000, 17), (28, 4, 512, 0), (3, 1, 64, 0)])
def test_fused_norm_rope_matches_oracle(built_library, dtype, heads, kv_heads, s, skip):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from vecattention_b200.preattn import qk_norm_rope
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, s, heads * 128, generator=g).to(dtype)
    k = torch.randn(2, s, kv_heads * 128, generator=g).to(dtype)
    wq = (1 + 0.1 * torch.randn(heads * 128, generator=g)).to(dtype)
    wk = (1 + 0.1 * torch.randn(kv_heads * 128, generator=g)).to(dtype)
    cos, sin = _tables(s - skip, 128, 4)
    qg, kg = qk_norm_rope(q.cuda(), k.cuda(), wq.cuda(), wk.cuda(), 1e-6, cos.cuda(), sin.cuda(), skip, heads=heads,
                          kv_heads=kv_heads)
    assert tuple(qg.shape) == (2, heads, s, 128) and tuple(kg.shape) == (2, kv_heads, s, 128)
    for got, x, w, h in ((qg, q, wq, heads), (kg, k, wk, kv_heads)):
        ref = O.rope_interleaved(O.rms_norm(x, w, 1e-6).view(2, s, h, 128).transpose(1, 2), cos, sin, skip)
        diff = (got.cpu() != ref)
        # the association of the sum of squares may move rstd by one fp32 step: isolated results land on the
        # neighbouring 16-bit value
        assert diff.float().mean() <= 2e-3, diff.float().mean().item()
        # one 16-bit step of a normalised element moves a rotated result by up to that step of the PAIR's magnitude
        rf = ref.float()
        mag = (rf[..., 0::2] ** 2 + rf[..., 1::2] ** 2).sqrt().repeat_interleave(2, dim=-1).clamp_min(1e-3)
        step = mag * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)
        assert bool(((got.cpu().float() - rf).abs() <= 2.01 * step).all())
    # norm only, rotation only, in place
    qn, _ = qk_norm_rope(q.cuda(), k.cuda(), wq.cuda(), wk.cuda(), 1e-6, heads=heads, kv_heads=kv_heads)
    assert (qn.cpu().float() - O.rms_norm(q, wq, 1e-6).view(2, s, heads, 128).transpose(1, 2).float()).abs().max() <= 0.07
    qr, _ = qk_norm_rope(q.cuda(), k.cuda(), None, None, 0.0, cos.cuda(), sin.cuda(), skip, heads=heads, kv_heads=kv_heads)
    assert torch.equal(qr.cpu(), O.rope_interleaved(q.view(2, s, heads, 128).transpose(1, 2), cos, sin, skip))
    qd = q.cuda()
    qi, _ = qk_norm_rope(qd, k.cuda(), wq.cuda(), wk.cuda(), 1e-6, cos.cuda(), sin.cuda(), skip, heads=heads,
                         kv_heads=kv_heads, inplace=True)
    assert qi.data_ptr() == qd.data_ptr() and torch.equal(qi, qg)


@pytest.mark.gpu
def test_operator_reads_the_prepared_layout_in_place(built_library):
    """The (B,H,S,D) views of (B,S,H*D) storage go straight into the operator: same bits as contiguous copies."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import vecattention_b200 as va
    from vecattention_b200.preattn import as_heads, qk_norm_rope
    g = torch.Generator().manual_seed(5)
    b, s, h = 1, 2000, 6
    q, k, v = (torch.randn(b, s, h * 128, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    w = torch.ones(h * 128, dtype=torch.bfloat16, device="cuda")
    cos, sin = (t.cuda() for t in _tables(s, 128, 6))
    qh, kh = qk_norm_rope(q, k, w, w, 1e-6, cos, sin, heads=h)
    vh = as_heads(v, h)
    assert not qh.is_contiguous()
    out = va.VecAttention_prefill(qh, kh, vh, 0.6, 64, 16, 8192, False, 32768)
    ref = va.VecAttention_prefill(qh.contiguous(), kh.contiguous(), vh.contiguous(), 0.6, 64, 16, 8192, False, 32768)
    assert torch.equal(out, ref)


def test_oracle_txtlast_rope_is_the_rotation_when_pairs_share_an_angle():
    """Per-element tables whose two entries of a pair carry the same angle (how the reference's callers fill
    them) turn the text-last formula into the plain rotation of the pair; the text tokens stay as they are."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, 2, 50, 128, generator=g).to(torch.bfloat16)
    c64, s64 = _tables(40, 128, 6)
    cos, sin = c64.repeat_interleave(2, dim=1).contiguous(), s64.repeat_interleave(2, dim=1).contiguous()
    got = O.rope_interleaved_txtlast(x, cos, sin, txt_len=10)
    want = O.rope_interleaved(x[:, :, :40], c64, s64)
    assert torch.equal(got[:, :, 40:], x[:, :, 40:])
    step = want.float().abs().clamp_min(2.0 ** -6) * 2.0 ** -7
    assert bool(((got[:, :, :40].float() - want.float()).abs() <= step).all())   # float32 against double arithmetic


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,heads,kv_heads,l,txt", [(1, 24, 24, 1000, 256), (2, 6, 2, 333, 0), (1, 3, 3, 17, 17), (1, 2, 1, 64, 5)])
def test_head_norm_and_txtlast_rope_match_oracle(built_library, dtype, b, heads, kv_heads, l, txt):
    """The per-head preparation (RMSNorm over 128 elements, rotary embedding on all but the last text tokens) against
    the oracle; parity unpinned: the reference's CUDA extension for these two ops is not built here."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from vecattention_b200.preattn import qk_head_norm_rope
    g = torch.Generator().manual_seed(7)
    q = torch.randn(b, heads, l, 128, generator=g).to(dtype)
    k = torch.randn(b, kv_heads, l, 128, generator=g).to(dtype)
    wq = (1 + 0.1 * torch.randn(128, generator=g)).to(dtype)
    wk = (1 + 0.1 * torch.randn(128, generator=g)).to(dtype)
    ang = torch.rand(max(l - txt, 1), 128, generator=g) * 6.283
    cos, sin = torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous()
    qg, kg = qk_head_norm_rope(q.cuda(), k.cuda(), wq.cuda(), wk.cuda(), 1e-6, cos.cuda(), sin.cuda(), txt)
    tiny = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    for got, x, w in ((qg, q, wq), (kg, k, wk)):
        ref = O.rope_interleaved_txtlast(O.rms_norm(x, w, 1e-6), cos[: l - txt], sin[: l - txt], txt)
        diff = got.cpu() != ref
        # the approximate reciprocal square root and the order of the sum may move a normalised element to the
        # neighbouring 16-bit value, and with it the two rotated results of its pair
        assert diff.float().mean() <= 2e-2, diff.float().mean().item()
        rf = ref.float()
        mag = (rf[..., 0::2] ** 2 + rf[..., 1::2] ** 2).sqrt().repeat_interleave(2, dim=-1).clamp_min(1e-3)
        assert bool(((got.cpu().float() - rf).abs() <= 3.01 * mag * tiny).all())
    # the text tokens are normalised but not rotated; rotation only is exact; in place
    if txt:
        assert torch.equal(qg[:, :, l - txt:].cpu(), qk_head_norm_rope(q.cuda(), k.cuda(), wq.cuda(), wk.cuda(), 1e-6)[0][:, :, l - txt:].cpu())
    qr, kr = qk_head_norm_rope(q.cuda(), k.cuda(), None, None, 0.0, cos.cuda(), sin.cuda(), txt)
    assert torch.equal(qr.cpu(), O.rope_interleaved_txtlast(q, cos[: l - txt], sin[: l - txt], txt))
    assert torch.equal(kr.cpu(), O.rope_interleaved_txtlast(k, cos[: l - txt], sin[: l - txt], txt))
    qd, kd = q.cuda(), k.cuda()
    qi, ki = qk_head_norm_rope(qd, kd, wq.cuda(), wk.cuda(), 1e-6, cos.cuda(), sin.cuda(), txt, inplace=True)
    assert qi.data_ptr() == qd.data_ptr() and torch.equal(qi, qg) and torch.equal(ki, kg)
    # strided input (a slice of a longer sequence, as the two-stream blocks pass it)
    big = torch.randn(b, heads, l + 8, 128, generator=g).to(dtype).cuda()
    qs, _ = qk_head_norm_rope(big[:, :, 3: 3 + l], k.cuda(), wq.cuda(), wk.cuda(), 1e-6, cos.cuda(), sin.cuda(), txt)
    qc, _ = qk_head_norm_rope(big[:, :, 3: 3 + l].contiguous(), k.cuda(), wq.cuda(), wk.cuda(), 1e-6, cos.cuda(), sin.cuda(), txt)
    assert torch.equal(qs, qc)
