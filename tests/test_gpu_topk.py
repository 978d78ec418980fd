"""Top-k / top-p sampling on the GPU against the CPU oracle.

The oracle (``oracle.topk_topp_probs``) restates the reference's second stage
(src/fused_mm_sampling/tl_fused_mm_topk.py:76-107) and is pinned to outputs of the reference's own
function (tests/golden/reference_topk_golden.npz).  Checked here:

* the reference's own test (tests/test_core.py:102-140): 5000 draws on ramps of known logits hit
  exactly the allowed tokens;
* with externally supplied Gumbel noise the sampled id is the argmax of (logit / T + noise) over the
  oracle's allowed set, draw for draw, wherever the decision is not within fp32 accumulation noise
  (top-2 gap above 1e-3 relative and the k-th / (k+1)-th logits apart by more than 1e-4 relative);
* a restricted draw equals the unrestricted draw of the same seed whenever that one is allowed;
* chi-square of 2^17 draws against the oracle's probabilities, p > 0.01;
* log-probabilities under the truncated distribution within 1e-3;
* rows whose candidate list overflows (ascending logits over the full vocabulary) are redone exactly
  by the second pass, and are reported (-1, status word) when the caller gave no scratch for it.
"""

import ctypes

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


def _allowed(logits_row, temp, k, p):
    """(allowed ids in descending order of probability, their probabilities, boundary gap)."""
    ids, probs = O.topk_topp_probs(logits_row[None], float(temp), k, p)
    keep = probs[0] > 0
    z = logits_row.float() / float(temp)
    top = z.topk(min(k + 1, z.numel())).values
    gap = float((top[k - 1] - top[k]).abs() / top[k - 1].abs().clamp_min(1e-30)) if top.numel() > k else 1.0
    return ids[0][keep], probs[0][keep], gap


@pytest.mark.parametrize("nh", [1, 2])
@pytest.mark.parametrize("V", [100, 200, 256])
def test_top_k_top_p_restricts_to_allowed_tokens(fs, V, nh):
    """tests/test_core.py:102-140 of the reference, through the provider registry."""
    from flashsampling_b200.testing import make_synthetic_inputs

    inp = make_synthetic_inputs(vocab_size=V, n_hidden_states=nh, device=_dev())
    t = torch.tensor(1.0, device=_dev())
    sampler = fs.get_sampler("fused-topk", weights=inp.weights).prepare()
    samples = sampler.sample(weights=inp.weights, hidden_states=inp.hidden_states, num_samples=5000, temperature=t,
                             top_k=10, top_p=0.9)
    fs.check_status()
    assert samples.shape == (nh, 5000)
    logits = O.logits_fp32(inp.weights.cpu(), inp.hidden_states.cpu())
    for r in range(nh):
        ids, _, _ = _allowed(logits[r], 1.0, 10, 0.9)
        assert set(samples[r].cpu().tolist()) == set(ids.tolist()), r


@pytest.mark.parametrize("B,k,p", [(3, 1, None), (3, 10, 0.8), (24, 20, 0.9), (70, 50, None), (70, 64, 0.95), (200, 20, 0.5), (300, 8, None)])
def test_external_noise_parity_top_k(fs, B, k, p):
    from flashsampling_b200.testing import gaussian_head

    V, D, S = 20000, 256, 3
    w, h = gaussian_head(V, D, B, 1.5 / np.sqrt(D), seed=B + k)
    g = torch.Generator().manual_seed(k)
    noise = O.gumbel_from_uniform(torch.rand(S, B, V, generator=g).clamp_min(1e-30))
    temp = torch.rand(B, generator=g) * 1.2 + 0.4
    out = fs.fused_mm_sample(w.to(_dev()), h.to(_dev()), S, temp.to(_dev()), seed=0, noise=noise.to(_dev()),
                             top_k=k, top_p=p, return_values=True, return_logprobs=True)
    ids, vals, lps = (x.cpu() for x in out)
    fs.check_status()
    logits = O.logits_fp32(w, h)
    checked = 0
    for b in range(B):
        allowed, probs, gap = _allowed(logits[b], temp[b], k, p)
        if gap < 1e-4:
            continue  # the k-th and (k+1)-th logits are within accumulation noise of each other
        z = logits[b][allowed] / temp[b]
        for s in range(S):
            y = z + noise[s, b][allowed]
            top2 = y.topk(min(2, y.numel())).values
            assert int(ids[b, s]) in set(allowed.tolist()), (b, s)
            if y.numel() > 1 and float((top2[0] - top2[1]) / top2[0].abs().clamp_min(1e-30)) <= 1e-3:
                continue
            want = int(allowed[y.argmax()])
            assert int(ids[b, s]) == want, (b, s, int(ids[b, s]), want)
            assert abs(float(vals[b, s]) - float(top2[0])) < 2e-3 + 2e-4 * abs(float(top2[0]))
            want_lp = float(torch.log(probs[allowed == want].double())[0])
            if p is None or probs.numel() > 1:  # a nucleus of borderline size would shift the normaliser
                assert abs(float(lps[b, s]) - want_lp) < 2e-3, (b, s, float(lps[b, s]), want_lp)
            checked += 1
    assert checked >= 0.7 * B * S


def test_restricted_draw_equals_unrestricted_draw_when_allowed(fs):
    from flashsampling_b200.testing import gaussian_head

    V, D, B, S, k = 30000, 128, 64, 4, 64
    w, h = gaussian_head(V, D, B, 2.0 / np.sqrt(D), seed=5)
    wd, hd = w.to(_dev()), h.to(_dev())
    t = torch.tensor(0.6, device=_dev())
    free = fs.fused_mm_sample(wd, hd, S, t, seed=77, kernel="mma").cpu()
    topk = fs.fused_mm_sample(wd, hd, S, t, seed=77, top_k=k).cpu()
    fs.check_status()
    logits = O.logits_fp32(w, h)
    inside = same = 0
    for b in range(B):
        allowed = set(_allowed(logits[b], 0.6, k, None)[0].tolist())
        for s in range(S):
            assert int(topk[b, s]) in allowed
            if int(free[b, s]) in allowed:
                inside += 1
                same += int(free[b, s]) == int(topk[b, s])
    assert inside > 0.3 * B * S and same >= inside - 2  # (z*invT + g) is rounded once there, twice here


@pytest.mark.parametrize("k,p", [(16, None), (50, 0.9)])
def test_top_k_distribution_chi_square(fs, k, p):
    from flashsampling_b200.testing import chi_square_row, gaussian_head

    V, D, B, S, T = 8192, 128, 64, 256, 0.9
    w, h1 = gaussian_head(V, D, 1, 2.0 / np.sqrt(D), seed=31)
    hd = h1.expand(B, D).contiguous().to(_dev())
    wd = w.to(_dev())
    t = torch.tensor(T, device=_dev())
    counts = torch.zeros(V, dtype=torch.int64, device=_dev())
    calls = 8
    for c in range(calls):
        ids = fs.fused_mm_sample(wd, hd, S, t, seed=c * S, top_k=k, top_p=p)
        counts += torch.bincount(ids.flatten(), minlength=V)
    fs.check_status()
    n = calls * B * S
    allowed, probs, _ = _allowed(O.logits_fp32(w, h1)[0], T, k, p)
    full = np.zeros(V)
    full[allowed.numpy()] = probs.double().numpy()
    assert int(counts.cpu()[full == 0].sum()) == 0
    pval, stat, dof, mass = chi_square_row(counts.cpu().numpy(), full, n)
    print(f"top_k={k} top_p={p}: draws={n} dof={dof} mass={mass:.4f} p={pval:.4f}")
    assert pval > 0.01


def test_overflowing_rows_take_the_exact_pass(fs):
    """Logits that rise (or fall) steadily over the whole vocabulary concentrate the largest entries in a
    few CTAs and defeat the running bound, which needs large entries in 64 different classes: the rows'
    candidate lists overflow and the rows are redone from their materialised logits."""
    from flashsampling_b200 import _lib
    from flashsampling_b200.testing import make_synthetic_inputs

    V = 151936
    inp = make_synthetic_inputs(vocab_size=V, hidden_size=15, n_hidden_states=2, device=_dev())
    t = torch.tensor(1.0, device=_dev())
    S, k = 2000, 10
    samples = fs.fused_mm_sample(inp.weights, inp.hidden_states, S, t, seed=3, top_k=k)
    fs.check_status()
    # bf16 rounding of the weights turns the ramps into noisy ramps (logits ~1e5, neighbours a few units
    # apart), so membership is checked by value: every sampled id has a logit at or above the k-th largest,
    # up to fp32 accumulation noise at this magnitude
    logits = O.logits_fp32(inp.weights.cpu(), inp.hidden_states.cpu())
    for r in range(2):
        kth = logits[r].topk(k).values[-1]
        picked = logits[r][samples[r].cpu()]
        assert bool((picked >= kth - 1e-6 * kth.abs() - 0.05).all()), r
        assert int(samples[r].min()) >= 0 and int(samples[r].max()) < V
    # the same call with a scratch too small for the exact pass: the overflowing rows are reported, not guessed
    lib = _lib.load()
    full, small = _lib.query_topk_workspace(V, 2)
    assert small < full
    tws = torch.zeros(small, dtype=torch.uint8, device=_dev())
    ws = torch.zeros(_lib.query_workspace(V, inp.weights.shape[1], 2, S), dtype=torch.uint8, device=_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out = torch.zeros((2, S), dtype=torch.int64, device=_dev())
    c = _lib.FmmsCall()
    c.struct_bytes = ctypes.sizeof(_lib.FmmsCall)
    c.W_bf16, c.H_bf16, c.temperature = inp.weights.data_ptr(), inp.hidden_states.data_ptr(), t.data_ptr()
    c.V_local, c.D, c.B, c.S, c.seed = V, inp.weights.shape[1], 2, S, 3
    c.out_idx, c.workspace, c.workspace_bytes = out.data_ptr(), ws.data_ptr(), ws.numel()
    c.status_dev, c.stream = status.data_ptr(), torch.cuda.current_stream().cuda_stream
    c.top_k, c.top_p, c.topk_workspace, c.topk_workspace_bytes = k, 0.0, tws.data_ptr(), tws.numel()
    assert lib.fmms_run(ctypes.byref(c)) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.ERR_TOPK_OVERFLOW
    assert (out == -1).all()
    status.zero_()
    # and the scratch is left clean: the next call with room for the exact pass gives the first answer
    tws2 = torch.zeros(full, dtype=torch.uint8, device=_dev())
    c.topk_workspace, c.topk_workspace_bytes = tws2.data_ptr(), tws2.numel()
    for _ in range(2):
        out.zero_()
        assert lib.fmms_run(ctypes.byref(c)) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and torch.equal(out, samples)


@pytest.mark.parametrize("seed,B", [(2, 256), (3, 200)])
def test_gaussian_rows_stay_out_of_the_exact_pass_with_two_m_tiles(fs, seed, B):
    """Full-size Gaussian heads at more than 128 rows: a thread of the two-M-tile layout scans four times the
    columns of the one-M-tile layout, and with a single 16-entry segment per thread one or two rows per call
    used to overflow (seeds below) and send the whole call through the exact pass (~1 ms instead of ~0.35).
    Run with a scratch too small for the exact pass, an overflow would be reported in the status word."""
    from flashsampling_b200 import _lib

    lib = _lib.load()
    V, D, S, k = 151936, 4096, 1, 50
    torch.manual_seed(seed)
    w = (torch.randn(V, D, device=_dev()) * 0.02).bfloat16()
    h = torch.randn(B, D, device=_dev()).bfloat16()
    t = torch.tensor(0.7, device=_dev())
    _, small = _lib.query_topk_workspace(V, B)
    tws = torch.zeros(small, dtype=torch.uint8, device=_dev())
    ws = torch.zeros(_lib.query_workspace(V, D, B, S), dtype=torch.uint8, device=_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out = torch.zeros((B, S), dtype=torch.int64, device=_dev())
    c = _lib.FmmsCall()
    c.struct_bytes = ctypes.sizeof(_lib.FmmsCall)
    c.W_bf16, c.H_bf16, c.temperature = w.data_ptr(), h.data_ptr(), t.data_ptr()
    c.V_local, c.D, c.B, c.S, c.seed = V, D, B, S, 3
    c.out_idx, c.workspace, c.workspace_bytes = out.data_ptr(), ws.data_ptr(), ws.numel()
    c.status_dev, c.stream = status.data_ptr(), torch.cuda.current_stream().cuda_stream
    c.top_k, c.top_p, c.topk_workspace, c.topk_workspace_bytes = k, 0.9, tws.data_ptr(), tws.numel()
    assert lib.fmms_run(ctypes.byref(c)) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(out.min()) >= 0
    # and the ids are those of the allowed set
    logits = (h[:4].float() @ w.float().T).cpu()
    for r in range(4):
        allowed = set(_allowed(logits[r], 0.7, k, 0.9)[0].tolist())
        assert int(out[r, 0]) in allowed


def test_clustered_large_logits_use_the_spill_list(fs):
    """A head whose first 2000 vocabulary rows carry three times the weight scale (frequent tokens at the low ids
    of a vocabulary): a couple of hundred of their logits pass the pivot, all inside two CTAs' vocabulary
    ranges, i.e. eight threads' segments per row.  What does not fit goes to the row's spill list, not to the
    exact pass: with a scratch too small for that pass no row may be reported, and every id is an allowed one."""
    from flashsampling_b200 import _lib

    lib = _lib.load()
    V, D, B, S, k = 151936, 1024, 40, 2, 50
    torch.manual_seed(11)
    w = torch.randn(V, D, device=_dev()) * 0.03
    w[:2000] *= 3.0
    w = w.bfloat16()
    h = torch.randn(B, D, device=_dev()).bfloat16()
    t = torch.tensor(0.8, device=_dev())
    _, small = _lib.query_topk_workspace(V, B)
    tws = torch.zeros(small, dtype=torch.uint8, device=_dev())
    ws = torch.zeros(_lib.query_workspace(V, D, B, S), dtype=torch.uint8, device=_dev())
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    out = torch.zeros((B, S), dtype=torch.int64, device=_dev())
    c = _lib.FmmsCall()
    c.struct_bytes = ctypes.sizeof(_lib.FmmsCall)
    c.W_bf16, c.H_bf16, c.temperature = w.data_ptr(), h.data_ptr(), t.data_ptr()
    c.V_local, c.D, c.B, c.S, c.seed = V, D, B, S, 5
    c.out_idx, c.workspace, c.workspace_bytes = out.data_ptr(), ws.data_ptr(), ws.numel()
    c.status_dev, c.stream = status.data_ptr(), torch.cuda.current_stream().cuda_stream
    c.top_k, c.top_p, c.topk_workspace, c.topk_workspace_bytes = k, 0.0, tws.data_ptr(), tws.numel()
    for _ in range(2):  # the second call finds the spill counters reset
        assert lib.fmms_run(ctypes.byref(c)) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and int(out.min()) >= 0
        logits = (h.float() @ w.float().T).cpu()
        inside_cluster = 0
        for r in range(B):
            allowed = set(_allowed(logits[r], 0.8, k, None)[0].tolist())
            assert all(int(x) in allowed for x in out[r].tolist()), r
            inside_cluster += sum(1 for x in allowed if x < 2000)
        assert inside_cluster > 0.9 * B * k  # the allowed sets do sit in the clustered range


def test_top_k_argument_errors(fs):
    w = torch.zeros(256, 16, dtype=torch.bfloat16, device=_dev())
    h = torch.zeros(2, 16, dtype=torch.bfloat16, device=_dev())
    t = torch.tensor(1.0, device=_dev())
    with pytest.raises(ValueError):
        fs.fused_mm_sample(w, h, 1, t, seed=0, top_k=65)
    with pytest.raises(ValueError):
        fs.fused_mm_sample(w, h, 1, t, seed=0, top_p=0.9)
    with pytest.raises(ValueError):
        fs.fused_mm_sample(w, h, 1, t, seed=0, top_k=5, return_logits=True)
