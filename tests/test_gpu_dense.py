"""GPU parity of flash_attn_varlen_func forward + backward
(grid modelled on tests/test_fmha_sm100.py:187-197, scaled down so the fp32 CPU oracle runs in seconds)."""
import pytest
import torch

from golden_io import load
from oracle import dense, gen
from oracle.check import check_is_allclose

pytestmark = pytest.mark.gpu

# tests/test_fmha_sm100.py:126-133
TOL = dict(abs_tol=1e-3, rel_tol=8.01 / 128, cos_diff_tol=7e-6)
LSE_TOL = dict(abs_tol=1e-6, rel_tol=2.01 / 65536)


def _run(c, causal, bwd):
    import flashmla_windows_linux_sm120_b200 as fm
    q, k, v = (c[n].cuda().requires_grad_(bwd) for n in ("q", "k", "v"))
    out, lse = fm.flash_attn_varlen_func(q, k, v, c["cu_q"].cuda(), c["cu_k"].cuda(), c["max_q"], c["max_k"],
                                         softmax_scale=c["scale"], causal=causal)
    grads = None
    if bwd:
        out.backward(c["d_out"].cuda())
        grads = (q.grad.cpu(), k.grad.cpu(), v.grad.cpu())
    torch.cuda.synchronize()
    return out.detach().cpu(), lse.detach().cpu(), grads


@pytest.mark.parametrize("d,dv", [(192, 128), (128, 128)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("varlen", [False, True])
def test_dense_fwd_bwd(d, dv, causal, varlen):
    c = gen.make_dense_case(gen.DenseCase(b=3, mean_sq=200, mean_sk=200, varlen=varlen, h=4, h_k=4, d=d, dv=dv,
                                          causal=causal))
    out, lse, (dq, dk, dvv) = _run(c, causal, True)
    r_out, r_lse, r_dq, r_dk, r_dv = dense.dense_fwd_bwd_ref(c["q"], c["k"], c["v"], c["d_out"], c["cu_q"], c["cu_k"],
                                                             causal, c["scale"])
    assert check_is_allclose("out", out, r_out, **TOL)
    assert check_is_allclose("lse", lse, r_lse, **LSE_TOL)
    assert check_is_allclose("dq", dq, r_dq, **TOL)
    assert check_is_allclose("dk", dk, r_dk, **TOL)
    assert check_is_allclose("dv", dvv, r_dv, **TOL)


@pytest.mark.parametrize("d", [192, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_dense_fwd_bwd_long(d, causal):
    """Sequences of several 128-row tiles and key blocks (the rings wrap and every barrier changes phase),
    with more keys than queries so that the causal mask is bottom-right aligned."""
    c = gen.make_dense_case(gen.DenseCase(b=2, mean_sq=520, mean_sk=760, varlen=True, h=2, h_k=2, d=d, dv=128, causal=causal))
    out, lse, (dq, dk, dvv) = _run(c, causal, True)
    r_out, r_lse, r_dq, r_dk, r_dv = dense.dense_fwd_bwd_ref(c["q"], c["k"], c["v"], c["d_out"], c["cu_q"], c["cu_k"],
                                                             causal, c["scale"])
    assert check_is_allclose("out", out, r_out, **TOL)
    assert check_is_allclose("lse", lse, r_lse, **LSE_TOL)
    assert check_is_allclose("dq", dq, r_dq, **TOL)
    assert check_is_allclose("dk", dk, r_dk, **TOL)
    assert check_is_allclose("dv", dvv, r_dv, **TOL)


@pytest.mark.parametrize("seed", range(8))
def test_dense_fwd_bwd_random_lengths(seed):
    """Seeded random sequence lengths including single tokens, key counts below and above a block, and (non-causal)
    more queries than keys."""
    import random
    rng = random.Random(2000 + seed)
    causal = rng.random() < 0.6
    b = rng.randint(1, 5)
    sq = [rng.choice([1, 7, 64, 127, 128, 129, 255, 300, 513]) for _ in range(b)]
    sk = [max(q if causal else 1, rng.choice([1, 5, 63, 64, 65, 128, 200, 257, 640])) for q in sq]
    d = rng.choice([192, 128])
    cu_q = torch.tensor([0] + sq, dtype=torch.int32).cumsum(0).to(torch.int32)
    cu_k = torch.tensor([0] + sk, dtype=torch.int32).cumsum(0).to(torch.int32)
    g = torch.Generator().manual_seed(seed)
    mk = lambda *shape: (torch.randn(*shape, generator=g) / 10).to(torch.bfloat16)
    h = 2
    c = dict(q=mk(sum(sq), h, d), k=mk(sum(sk), h, d), v=mk(sum(sk), h, 128), d_out=mk(sum(sq), h, 128), cu_q=cu_q, cu_k=cu_k,
             max_q=max(sq), max_k=max(sk), scale=(d + 100) ** -0.5)
    out, lse, (dq, dk, dvv) = _run(c, causal, True)
    r_out, r_lse, r_dq, r_dk, r_dv = dense.dense_fwd_bwd_ref(c["q"], c["k"], c["v"], c["d_out"], c["cu_q"], c["cu_k"],
                                                             causal, c["scale"])
    assert check_is_allclose("out", out, r_out, **TOL)
    assert check_is_allclose("lse", lse, r_lse, **LSE_TOL)
    assert check_is_allclose("dq", dq, r_dq, **TOL)
    assert check_is_allclose("dk", dk, r_dk, **TOL)
    assert check_is_allclose("dv", dvv, r_dv, **TOL)


@pytest.mark.parametrize("causal", [False, True])
def test_dense_neighbour_sequence_does_not_leak(causal):
    """A tile that overhangs the end of its sequence reads rows of the next one.  Non-finite values there
    must not reach this sequence's outputs: the result equals the one computed for the sequence alone."""
    c = gen.make_dense_case(gen.DenseCase(b=2, mean_sq=200, mean_sk=200, varlen=True, h=2, h_k=2, d=192, dv=128, causal=causal))
    cu_q, cu_k = c["cu_q"], c["cu_k"]
    lq0, lk0 = int(cu_q[1]), int(cu_k[1])
    assert lq0 % 64 and lk0 % 64, "the case must leave partial tiles"
    both = {n: c[n].clone() for n in ("q", "k", "v", "d_out")}
    both["q"][lq0:] = float("nan")
    both["d_out"][lq0:] = float("inf")
    both["k"][lk0:] = float("nan")
    both["v"][lk0:] = float("inf")
    poisoned = dict(c, **both)
    out, lse, (dq, dk, dvv) = _run(poisoned, causal, True)
    alone = dict(c, q=c["q"][:lq0], k=c["k"][:lk0], v=c["v"][:lk0], d_out=c["d_out"][:lq0], cu_q=cu_q[:2], cu_k=cu_k[:2],
                 max_q=lq0, max_k=lk0)
    a_out, a_lse, (a_dq, a_dk, a_dv) = _run(alone, causal, True)
    assert torch.equal(out[:lq0], a_out) and torch.equal(lse[:lq0], a_lse)
    assert torch.equal(dq[:lq0], a_dq) and torch.equal(dk[:lk0], a_dk) and torch.equal(dvv[:lk0], a_dv)


def test_dense_packed_inputs_are_read_in_place():
    """flash_attn_varlen_qkvpacked_func / kvpacked_func hand strided views of one packed tensor to the kernels
    (no copy): results and gradients equal those of the same values passed as separate tensors, bit for bit."""
    import flashmla_windows_linux_sm120_b200 as fm
    c = gen.make_dense_case(gen.DenseCase(b=2, mean_sq=180, mean_sk=180, varlen=False, h=4, h_k=4, d=192, dv=128, causal=True))
    cu, mx = c["cu_q"].cuda(), c["max_q"]
    q, k, v, d_out = (c[n].cuda() for n in ("q", "k", "v", "d_out"))
    qs, ks, vs = (t.clone().requires_grad_() for t in (q, k, v))
    out, lse = fm.flash_attn_varlen_func(qs, ks, vs, cu, cu, mx, mx, softmax_scale=c["scale"], causal=True)
    out.backward(d_out)

    qkv = torch.cat([q, k, v], dim=-1).requires_grad_()
    out_p, lse_p = fm.flash_attn_varlen_qkvpacked_func(qkv, cu, mx, 192, softmax_scale=c["scale"], causal=True)
    out_p.backward(d_out)
    assert torch.equal(out_p, out) and torch.equal(lse_p, lse)
    assert torch.equal(qkv.grad[..., :192], qs.grad) and torch.equal(qkv.grad[..., 192:384], ks.grad)
    assert torch.equal(qkv.grad[..., 384:], vs.grad)

    qk, kv = q.clone().requires_grad_(), torch.cat([k, v], dim=-1).requires_grad_()
    out_k, lse_k = fm.flash_attn_varlen_kvpacked_func(qk, kv, cu, cu, mx, mx, 192, softmax_scale=c["scale"], causal=True)
    out_k.backward(d_out)
    assert torch.equal(out_k, out) and torch.equal(lse_k, lse)
    assert torch.equal(qk.grad, qs.grad) and torch.equal(kv.grad[..., :192], ks.grad) and torch.equal(kv.grad[..., 192:], vs.grad)


def test_dense_fwd_causal_more_queries_than_keys():
    """Bottom-right aligned causal mask with s_q > s_k: the first s_q - s_k queries see no key: O = 0, lse = -inf."""
    torch.manual_seed(3)
    sq, sk, h, d = 300, 130, 2, 192
    mk = lambda *shape: (torch.randn(*shape) / 10).to(torch.bfloat16)
    c = dict(q=mk(sq, h, d), k=mk(sk, h, d), v=mk(sk, h, 128), d_out=mk(sq, h, 128), cu_q=torch.tensor([0, sq], dtype=torch.int32),
             cu_k=torch.tensor([0, sk], dtype=torch.int32), max_q=sq, max_k=sk, scale=0.06)
    out, lse, _ = _run(c, True, False)
    r_out, r_lse = dense.dense_fwd_ref(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], True, c["scale"])
    assert torch.all(out[:sq - sk] == 0) and torch.all(lse[:sq - sk] == float("-inf"))
    assert check_is_allclose("out", out, r_out, **TOL)
    assert check_is_allclose("lse", lse[sq - sk:], r_lse[sq - sk:], **LSE_TOL)


def test_dense_fwd_gqa_32_over_4():
    """the reference grid's GQA shape (tests/test_fmha_sm100.py:189): 32 query heads over 4 kv heads"""
    c = gen.make_dense_case(gen.DenseCase(b=2, mean_sq=200, mean_sk=330, varlen=True, h=32, h_k=4, d=192, dv=128, causal=True))
    out, lse, _ = _run(c, True, False)
    r_out, r_lse = dense.dense_fwd_ref(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], True, c["scale"])
    assert check_is_allclose("out", out, r_out, **TOL)
    assert check_is_allclose("lse", lse, r_lse, **LSE_TOL)


@pytest.mark.parametrize("d", [192, 128])
def test_dense_fwd_gqa(d):
    c = gen.make_dense_case(gen.DenseCase(b=2, mean_sq=150, mean_sk=260, varlen=True, h=8, h_k=2, d=d, dv=128, causal=True))
    out, lse, _ = _run(c, True, False)
    r_out, r_lse = dense.dense_fwd_ref(c["q"], c["k"], c["v"], c["cu_q"], c["cu_k"], True, c["scale"])
    assert check_is_allclose("out", out, r_out, **TOL)
    assert check_is_allclose("lse", lse, r_lse, **LSE_TOL)


def test_dense_bitwise_determinism():
    c = gen.make_dense_case(gen.DenseCase(b=2, mean_sq=300, mean_sk=300, varlen=True, h=4, h_k=4, d=192, dv=128, causal=True))
    first = _run(c, True, True)
    for _ in range(3):
        again = _run(c, True, True)
        assert torch.equal(first[0], again[0]) and torch.equal(first[1], again[1])
        for a, b in zip(first[2], again[2]):     # dq too: every output has a single, ordered producer
            assert torch.equal(a, b)


def test_dense_deterministic_flag_is_accepted():
    import flashmla_windows_linux_sm120_b200 as fm
    c = gen.make_dense_case(gen.DenseCase(b=1, mean_sq=130, mean_sk=130, varlen=False, h=2, h_k=2, d=128, dv=128, causal=True))
    cu = c["cu_q"].cuda()
    res = []
    for det in (False, True):
        q, k, v = (c[n].cuda().requires_grad_() for n in ("q", "k", "v"))
        out, _ = fm.flash_attn_varlen_func(q, k, v, cu, cu, c["max_q"], c["max_k"], softmax_scale=c["scale"], causal=True,
                                           deterministic=det)
        out.backward(c["d_out"].cuda())
        res.append((out.detach(), q.grad, k.grad, v.grad))
    assert all(torch.equal(a, b) for a, b in zip(*res))


def test_dense_bwd_rejects_gqa():
    c = gen.make_dense_case(gen.DenseCase(b=1, mean_sq=64, mean_sk=64, varlen=False, h=4, h_k=2, d=128, dv=128, causal=False))
    with pytest.raises(ValueError):
        _run(c, False, True)


def test_dense_rejects_unsupported_head_dim():
    import flashmla_windows_linux_sm120_b200 as fm
    q = torch.zeros(64, 2, 64, dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        fm.flash_attn_varlen_func(q, q, q, cu, cu, 64, 64)


@pytest.mark.parametrize("name", ["dense_mla192_causal", "dense_128_plain_gqa"])
def test_dense_golden(name):
    import flashmla_windows_linux_sm120_b200 as fm
    g = load(name)
    causal = bool(g["causal"])
    bwd = "dq" in g
    q, k, v = (g[n].cuda().requires_grad_(bwd) for n in ("q", "k", "v"))
    cu_q, cu_k = g["cu_q"], g["cu_k"]
    mq = int((cu_q[1:] - cu_q[:-1]).max())
    mk = int((cu_k[1:] - cu_k[:-1]).max())
    out, lse = fm.flash_attn_varlen_func(q, k, v, cu_q.cuda(), cu_k.cuda(), mq, mk, softmax_scale=g["scale"], causal=causal)
    assert check_is_allclose("out", out.detach(), g["out"], **TOL)
    assert check_is_allclose("lse", lse.detach(), g["lse"], **LSE_TOL)
    if bwd:
        out.backward(g["d_out"].cuda())
        assert check_is_allclose("dq", q.grad, g["dq"], **TOL)
        assert check_is_allclose("dk", k.grad, g["dk"], **TOL)
        assert check_is_allclose("dv", v.grad, g["dv"], **TOL)
