"""e4m3 LM-head weights with per-row scales (FMMS_FLAG_W_FP8) against the CPU oracle.

The oracle dequantises both operands (per-row e4m3 weights as stored, hidden states quantised per row the
way the kernels do it) and multiplies in fp32; e4m3 x e4m3 products are exact in fp32, so the kernels'
sums differ from it only by summation order.  Tolerances: logits atol = rtol = 1e-4 of the logit scale
(as for bf16), sampled ids equal on every draw whose top-2 gap exceeds 1e-3 relative, chi-square p > 0.01
against the softmax of the QUANTISED logits.
"""

import numpy as np
import pytest
import torch

from oracle import fmms_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fs():
    import flashsampling_b200 as fs
    from flashsampling_b200 import build

    build.build_library()
    return fs


def _dev():
    return torch.device("cuda", 0)


def _head(V, D, B, seed, w_std=None):
    from flashsampling_b200.quant import quantize_rows_e4m3
    from flashsampling_b200.testing import gaussian_head

    w, h = gaussian_head(V, D, B, w_std or 1.5 / np.sqrt(D), seed)
    w_q, w_s = quantize_rows_e4m3(w)
    return w_q, w_s, h


def test_package_quantiser_equals_the_oracles():
    from flashsampling_b200.quant import dequantize_rows, quantize_rows_e4m3

    x = torch.randn(300, 200, generator=torch.Generator().manual_seed(0)) * 0.02
    q, s = quantize_rows_e4m3(x)
    q2, s2 = O.quantize_rows_e4m3(x)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
    assert float((dequantize_rows(q, s) - x).abs().max() / x.abs().max()) < 0.07  # 3 mantissa bits


@pytest.mark.parametrize("V,D,B", [(100, 16, 1), (1000, 256, 3), (4097, 528, 17), (20000, 512, 64), (9000, 256, 130)])
def test_fp8_logits_match_dequantised_matmul(fs, V, D, B):
    w_q, w_s, h = _head(V, D, B, seed=V + B)
    ids, logits = fs.fused_mm_sample(w_q.to(_dev()), h.to(_dev()), 1, torch.empty((), device=_dev()), seed=0,
                                     greedy_sampling=True, return_logits=True, weight_scale=w_s.to(_dev()))
    fs.check_status()
    assert fs.last_path() == "mma"
    ref = O.quantized_logits(w_q, w_s, h)
    torch.testing.assert_close(logits.cpu(), ref, atol=1e-4 * float(ref.abs().max()), rtol=1e-4)
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 1e-3 * top2[:, 0].abs()
    assert torch.equal(ids.cpu()[clear, 0], ref.argmax(-1)[clear])


@pytest.mark.parametrize("V,D,B,S", [(20000, 512, 3, 2), (20000, 512, 48, 1), (30000, 256, 64, 2), (9000, 1024, 130, 1),
                                     (5000, 128, 300, 1), (40000, 256, 200, 1), (33000, 512, 256, 2)])
def test_fp8_external_noise_parity(fs, V, D, B, S):
    w_q, w_s, h = _head(V, D, B, seed=V + B + S)
    g = torch.Generator().manual_seed(S)
    noise = O.gumbel_from_uniform(torch.rand(S, B, V, generator=g).clamp_min(1e-30))
    temp = torch.rand(B, generator=g) * 1.2 + 0.4
    ids, vals = fs.fused_mm_sample(w_q.to(_dev()), h.to(_dev()), S, temp.to(_dev()), seed=0, noise=noise.to(_dev()),
                                   weight_scale=w_s.to(_dev()), return_values=True)
    fs.check_status()
    want, decisive, ymax = O.gumbel_argmax(O.quantized_logits(w_q, w_s, h), temp, noise, rel_gap=1e-3)
    bad = (ids.cpu() != want) & decisive
    assert not bad.any(), f"{int(bad.sum())} decisive draws differ"
    assert decisive.float().mean() > 0.75
    torch.testing.assert_close(vals.cpu()[decisive], ymax[decisive], atol=2e-3, rtol=2e-4)


def test_fp8_qwen_head_full_size(fs):
    """V=151936, d=4096, B=64: the benchmark shape with e4m3 weights (0.62 GB streamed instead of 1.24)."""
    from flashsampling_b200.quant import quantize_rows_e4m3

    V, D, B = 151936, 4096, 64
    g = torch.Generator(device=_dev()).manual_seed(3)
    w = torch.empty((V, D), dtype=torch.bfloat16, device=_dev())
    for r0 in range(0, V, 16384):
        r1 = min(V, r0 + 16384)
        w[r0:r1] = (torch.randn((r1 - r0, D), generator=g, device=_dev()) * 0.02).bfloat16()
    h = torch.randn((B, D), generator=g, device=_dev()).bfloat16()
    w_q, w_s = quantize_rows_e4m3(w)
    noise = O.gumbel_from_uniform(torch.rand(1, B, V, generator=torch.Generator().manual_seed(1)).clamp_min(1e-30))
    t = torch.tensor(0.7, device=_dev())
    ids = fs.fused_mm_sample(w_q, h, 1, t, seed=0, noise=noise.to(_dev()), weight_scale=w_s)
    fs.check_status()
    want, decisive, _ = O.gumbel_argmax(O.quantized_logits(w_q.cpu(), w_s.cpu(), h.cpu()), 0.7, noise, rel_gap=1e-3)
    assert not ((ids.cpu() != want) & decisive).any() and decisive.float().mean() > 0.75
    # how far the quantised head's distribution is from the bf16 head's, for the record: total variation per row
    p8 = torch.softmax(O.quantized_logits(w_q.cpu(), w_s.cpu(), h.cpu()[:4]) / 0.7, -1)
    p16 = torch.softmax((h.cpu()[:4].float() @ w.cpu().float().T) / 0.7, -1)
    print("total variation fp8 vs bf16 head, 4 rows:", [round(float(x), 4) for x in 0.5 * (p8 - p16).abs().sum(-1)])


def test_fp8_distribution_chi_square(fs):
    from flashsampling_b200.testing import chi_square_row

    V, D, B, S, T = 4096, 256, 64, 64, 0.8
    w_q, w_s, h1 = _head(V, D, 1, seed=77, w_std=2.0 / np.sqrt(D))
    hd = h1.expand(B, D).contiguous().to(_dev())
    wd, sd = w_q.to(_dev()), w_s.to(_dev())
    t = torch.tensor(T, device=_dev())
    counts = torch.zeros(V, dtype=torch.int64, device=_dev())
    calls = 64
    for c in range(calls):
        ids = fs.fused_mm_sample(wd, hd, S, t, seed=c * S, weight_scale=sd)
        counts += torch.bincount(ids.flatten(), minlength=V)
    fs.check_status()
    n = calls * B * S
    probs = O.softmax_probs(O.quantized_logits(w_q, w_s, h1)[0], T)
    pval, stat, dof, mass = chi_square_row(counts.cpu().numpy(), probs, n)
    print(f"fp8: draws={n} dof={dof} mass={mass:.4f} p={pval:.4f}")
    assert mass > 0.9 and pval > 0.01


def test_fp8_with_log_probabilities_and_top_k(fs):
    V, D, B, S = 12000, 256, 40, 2
    w_q, w_s, h = _head(V, D, B, seed=5)
    wd, sd, hd = w_q.to(_dev()), w_s.to(_dev()), h.to(_dev())
    t = torch.tensor(0.9, device=_dev())
    ids, lp = fs.fused_mm_sample(wd, hd, S, t, seed=9, weight_scale=sd, return_logprobs=True)
    plain = fs.fused_mm_sample(wd, hd, S, t, seed=9, weight_scale=sd)
    assert torch.equal(ids, plain)
    logits = O.quantized_logits(w_q, w_s, h)
    want_lp, _ = O.log_probs(logits, 0.9, ids.cpu())
    assert float((lp.cpu().double() - want_lp).abs().max()) < 1e-3
    top = fs.fused_mm_sample(wd, hd, S, t, seed=9, weight_scale=sd, top_k=20)
    for b in range(B):
        kth = logits[b].topk(20).values[-1]
        assert bool((logits[b][top[b].cpu()] >= kth - 1e-4 * kth.abs()).all())
    fs.check_status()


def test_fp8_argument_errors(fs):
    w = torch.zeros(64, 32, dtype=torch.float8_e4m3fn, device=_dev())
    h = torch.zeros(2, 32, dtype=torch.bfloat16, device=_dev())
    t = torch.tensor(1.0, device=_dev())
    with pytest.raises(TypeError):
        fs.fused_mm_sample(w, h, 1, t, seed=0)  # fp8 weights without scales
    with pytest.raises(ValueError):
        fs.fused_mm_sample(w, h, 1, t, seed=0, weight_scale=torch.ones(63, device=_dev()))
    with pytest.raises(ValueError):
        fs.fused_mm_sample(w, h, 1, t, seed=0, weight_scale=torch.ones(64, device=_dev()), kernel="gemv")
