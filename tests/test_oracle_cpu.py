"""The CPU oracle against the golden vectors and against itself (no GPU).

Mirrors the reference's CPU-side tests: common/src/lib.rs:84-113 (metrics, generator)
and the finite-difference self-check of 02-flash-attention/src/main.rs:339-390,504-508.
"""
import numpy as np
import pytest

import oracle
from mx230_b200 import common

RTOL, ATOL = 1e-3, 1e-4  # 02-flash-attention/src/main.rs:17-18


def test_pseudo_rand_matches_golden_and_host(golden):
    assert np.array_equal(oracle.pseudo_rand(16, 1), golden["rand_seed1_first16"])
    assert np.array_equal(oracle.pseudo_rand(16, 42), golden["rand_seed42_first16"])
    assert np.array_equal(common.pseudo_rand(257, 5), oracle.pseudo_rand(257, 5))


def test_library_generators_equal_the_oracle_generators():
    """The library's host-side generators (what the benchmark draws its inputs from) against the oracle's,
    bit for bit: the uniform stream of common/src/lib.rs:67-78 and the N(0,1) stream built on it."""
    for seed in (0, 1, 42, 1234):
        assert np.array_equal(common.pseudo_rand(1000, seed + 1), oracle.pseudo_rand(1000, seed + 1))
        for idx in (0, 3):
            assert np.array_equal(common.normal((7, 143), seed, idx), oracle.normal((7, 143), seed, idx))
    z = common.normal((200000,), 0, 0)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01


def test_pseudo_rand_is_deterministic_and_bounded():
    a, b = oracle.pseudo_rand(1000, 42), oracle.pseudo_rand(1000, 42)
    assert np.array_equal(a, b)
    assert ((a >= -1.0) & (a < 1.0)).all()
    assert not np.array_equal(oracle.pseudo_rand(1000, 43), a)


def test_max_rel_err_basics():
    a = np.array([1.0, 2.0, 3.0], np.float32)
    assert oracle.max_rel_err(a, a) == 0.0
    got = np.array([1.0, 2.2, 3.0], np.float32)
    assert abs(oracle.max_rel_err(got, a) - 0.1) < 1e-6
    assert abs(common.max_rel_err(got, a) - 0.1) < 1e-6


def test_allclose_err_threshold():
    want = np.array([0.0, 100.0], np.float32)
    got = np.array([0.05, 101.0], np.float32)
    assert oracle.allclose_err(got, want, 1e-2, 5e-2) <= 1.0 + 1e-6
    bad = np.array([0.10, 102.0], np.float32)
    assert oracle.allclose_err(bad, want, 1e-2, 5e-2) > 1.0
    assert abs(common.allclose_err(bad, want, 1e-2, 5e-2) - oracle.allclose_err(bad, want, 1e-2, 5e-2)) < 1e-5


def test_normal_generator_moments():
    x = oracle.normal((200000,), 0, 0)
    assert abs(float(x.mean())) < 1e-2 and abs(float(x.std()) - 1.0) < 1e-2
    assert not np.array_equal(oracle.normal((64,), 0, 0), oracle.normal((64,), 0, 1))
    assert np.array_equal(oracle.normal((64,), 3, 2), oracle.normal((64,), 3, 2))


@pytest.mark.parametrize("causal", [0, 1])
def test_forward_matches_golden(golden, causal):
    n = 64
    q, k, v = (oracle.pseudo_rand(n * 64, s).reshape(n, 64) for s in (1, 2, 3))
    o, lse = oracle.attn_fwd(q, k, v, bool(causal))
    assert oracle.allclose_err(o, golden[f"fwd_o_c{causal}"], RTOL, ATOL) < 1.0
    assert np.abs(lse - golden[f"fwd_lse_c{causal}"]).max() < 1e-5


@pytest.mark.parametrize("causal", [0, 1])
def test_backward_matches_golden(golden, causal):
    n = 64
    q, k, v, do = (oracle.pseudo_rand(n * 64, s).reshape(n, 64) for s in (11, 12, 13, 14))
    dq, dk, dv = oracle.attn_bwd(q, k, v, do, bool(causal))
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert oracle.allclose_err(got, golden[f"bwd_{name}_c{causal}"], RTOL, ATOL) < 1.0, name


@pytest.mark.parametrize("causal", [False, True])
def test_backward_matches_finite_difference(causal):
    """fd_check, 02-flash-attention/src/main.rs:339-390: N=128, seeds 21-24, eps 1e-3,
    six sampled indices, relative error abs(fd-g)/(1e-3+abs(g)) under 5e-2."""
    n, d = 128, 64
    q, k, v, do = (oracle.pseudo_rand(n * d, s).reshape(n, d) for s in (21, 22, 23, 24))
    grads = oracle.attn_bwd(q, k, v, do, causal)
    eps = np.float32(1e-3)
    worst = 0.0
    for idx in (0, 1, d + 7, 3 * d + 31, (n // 2) * d + 17, (n - 1) * d + 63):
        for which in range(3):
            ten = [q.copy(), k.copy(), v.copy()]
            flat = ten[which].reshape(-1)
            orig = flat[idx]
            flat[idx] = orig + eps
            lp = oracle.attn_loss(ten[0], ten[1], ten[2], do, causal)
            flat[idx] = orig - eps
            lm = oracle.attn_loss(ten[0], ten[1], ten[2], do, causal)
            fd = np.float32((lp - lm) / (2.0 * float(eps)))
            g = grads[which].reshape(-1)[idx]
            worst = max(worst, abs(fd - g) / (1e-3 + abs(g)))
    assert worst < 5e-2, worst


def test_preprocess_equals_cpu_delta():
    """GPU definition sum_x dO*O equals the CPU's sum_j p_j dP_j (main.rs:279-287)."""
    n = 48
    q, k, v, do = (oracle.pseudo_rand(n * 64, s).reshape(n, 64) for s in (31, 32, 33, 34))
    o, _ = oracle.attn_fwd(q, k, v, True)
    delta = oracle.bwd_preprocess(do, o)
    s = (q.astype(np.float64) @ k.T.astype(np.float64)) / 8
    s = np.where(np.tril(np.ones((n, n), bool)), s, -np.inf)
    p = np.exp(s - s.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    want = (p * (do.astype(np.float64) @ v.T.astype(np.float64))).sum(1)
    assert np.abs(delta - want).max() < 1e-5


def test_batched_heads_equal_single_heads():
    q, k, v = (oracle.normal((3, 40, 64), 5, i) for i in range(3))
    o, lse = oracle.attn_fwd(q, k, v, True, threads=2)
    for h in range(3):
        o1, l1 = oracle.attn_fwd(q[h], k[h], v[h], True, threads=1)
        assert np.array_equal(o[h], o1) and np.array_equal(lse[h], l1)


def test_forward_edge_sizes():
    for n in (1, 2, 63, 65):
        q, k, v = (oracle.normal((n, 64), 9, i) for i in range(3))
        o, lse = oracle.attn_fwd(q, k, v, True)
        assert np.allclose(o[0], v[0], atol=1e-6)  # the first causal row sees only key 0
        assert np.isfinite(o).all() and np.isfinite(lse).all()
    o, lse = oracle.attn_fwd(np.zeros((0, 64), np.float32), np.zeros((0, 64), np.float32),
                             np.zeros((0, 64), np.float32), False)
    assert o.shape == (0, 64)


def test_rows_subset_matches_full():
    q, k, v = (oracle.normal((2, 100, 64), 6, i) for i in range(3))
    o, _ = oracle.attn_fwd(q, k, v, False)
    sub = oracle.attn_fwd_rows(q, k, v, False, 3, 17)
    assert np.array_equal(sub, o[:, 3::17])


# ---- 03-llm-engine pieces ---------------------------------------------------
def test_quantizers_match_golden(golden):
    rows = golden["quant_rows"]
    for i, r in enumerate(rows):
        c, s, b = oracle.quant_affine(r)
        assert np.array_equal(c, golden["quant_affine_codes"][i]), i
        assert s == golden["quant_affine_scale"][i] and b == golden["quant_affine_beta"][i], i
        c2, s2 = oracle.quant_absmax(r)
        assert np.array_equal(c2, golden["quant_absmax_codes"][i]), i
        assert s2 == golden["quant_absmax_scale"][i], i


def test_quant_affine_properties():
    x = oracle.normal((64,), 1, 0)
    c, s, b = oracle.quant_affine(x)
    assert c.min() == -128 and c.max() == 127  # the row's min and max take the end codes
    assert np.abs(c.astype(np.float32) * s + b - x).max() <= 0.5 * s * (1 + 1e-5)
    c, s, b = oracle.quant_affine(np.full(64, 0.25, np.float32))
    assert s == 1.0 and b == np.float32(128.25) and (c == -128).all()
    c2, s2 = oracle.quant_absmax(np.zeros(64, np.float32))
    assert s2 == 0.0 and (c2 == 0).all()


def test_rope_matches_golden(golden):
    for key, pos, theta in (("rope_pos37_theta1e6", 37, 1e6), ("rope_pos2047_theta1e4", 2047, 1e4)):
        x = golden["rope_in"].copy()
        oracle.rope(x, 4, 64, pos, theta)
        assert np.abs(x - golden[key]).max() < 2e-6, key


def _make_cache(ctx, n_head, n_kv_head, seed, affine=True, theta=1e6):
    qd, kd = n_head * 64, n_kv_head * 64
    rows = oracle.normal((ctx, qd + 2 * kd), seed, 0)
    kc = np.zeros((ctx, kd), np.float32)
    vc = np.zeros((ctx, kd), np.float32)
    cache = oracle.Q8Cache(ctx, n_kv_head, 64, affine)
    for t in range(ctx):
        oracle.rope_qkv_row(rows[t], t, n_head, n_kv_head, 64, theta)
        oracle.copy_kv_row(kc, vc, rows[t], t, qd, kd)
        oracle.quantize_kv_row(cache, rows[t], t, qd)
    return rows, kc, vc, cache


def test_gqa_decode_vs_float64_and_q8_distance():
    nh, nkv, ctx = 14, 2, 200
    rows, kc, vc, cache = _make_cache(ctx, nh, nkv, 3)
    q = rows[ctx - 1]
    out = oracle.gqa_decode_f32(q, kc, vc, ctx - 1, nh, nkv).reshape(nh, 64)
    for h in (0, 6, 7, 13):
        kvh = h // 7
        s = kc[:, kvh * 64:(kvh + 1) * 64].astype(np.float64) @ q[h * 64:(h + 1) * 64].astype(np.float64) / 8
        p = np.exp(s - s.max())
        p /= p.sum()
        want = p @ vc[:, kvh * 64:(kvh + 1) * 64].astype(np.float64)
        assert np.abs(out[h] - want).max() < 1e-5
    a = oracle.gqa_decode_q8(q, cache, ctx - 1, nh, 0)
    b = oracle.gqa_decode_q8(q, cache, ctx - 1, nh, 1)
    # int8 cache error, and the extra q quantisation of the reference kernel, stay small
    assert oracle.mean_rel_err(a, out.ravel()) < 3e-2
    assert oracle.mean_rel_err(b, a) < 3e-2


def test_paged_rows_equal_linear():
    nh, nkv, ctx, bs = 4, 2, 70, 16
    rows = oracle.normal((ctx, (nh + 2 * nkv) * 64), 8, 0)
    n_log = (ctx + bs - 1) // bs
    table = np.arange(n_log, dtype=np.int32)[::-1].copy() + 2  # non-identity
    slots = (n_log + 2) * bs
    lin = oracle.Q8Cache(ctx, nkv)
    pag = oracle.Q8Cache(slots, nkv)
    klin = np.zeros((ctx, nkv * 64), np.float32)
    vlin = np.zeros_like(klin)
    kpag = np.zeros((slots, nkv * 64), np.float32)
    vpag = np.zeros_like(kpag)
    for t in range(ctx):
        oracle.quantize_kv_row(lin, rows[t], t, nh * 64)
        oracle.quantize_kv_row(pag, rows[t], t, nh * 64, table, bs)
        oracle.copy_kv_row(klin, vlin, rows[t], t, nh * 64, nkv * 64)
        oracle.copy_kv_row(kpag, vpag, rows[t], t, nh * 64, nkv * 64, table, bs)
    q = rows[ctx - 1]
    assert np.array_equal(oracle.gqa_decode_q8(q, lin, ctx - 1, nh, 1),
                          oracle.gqa_decode_q8(q, pag, ctx - 1, nh, 1, table, bs))
    assert np.array_equal(oracle.gqa_decode_f32(q, klin, vlin, ctx - 1, nh, nkv),
                          oracle.gqa_decode_f32(q, kpag, vpag, ctx - 1, nh, nkv, 64, table, bs))


@pytest.mark.parametrize("quant", [False, True])
def test_split_kv_merge_equals_unsplit(quant):
    """Merging (m, l, acc) partials of disjoint key ranges reproduces unsplit attention."""
    nh, nkv, ctx = 8, 2, 333
    rows, kc, vc, cache = _make_cache(ctx, nh, nkv, 4)
    q = rows[ctx - 1]
    cuts = [0, 100, 101, 250, ctx]
    ms, ls, accs = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        m, l, acc = oracle.gqa_partial(q, a, b, nh, nkv, 64, None if quant else kc,
                                       None if quant else vc, cache if quant else None)
        ms.append(m), ls.append(l), accs.append(acc)
    merged = oracle.merge_partials(np.stack(ms), np.stack(ls), np.stack(accs)).ravel()
    want = oracle.gqa_decode_q8(q, cache, ctx - 1, nh, 0) if quant else \
        oracle.gqa_decode_f32(q, kc, vc, ctx - 1, nh, nkv)
    assert np.abs(merged - want).max() < 2e-6


def test_prefill_rows_equal_decode_rows():
    nh, nkv, ctx = 4, 2, 40
    rows, kc, vc, cache = _make_cache(ctx, nh, nkv, 12)
    stride = rows.shape[1]
    out = oracle.prefill(rows[8:], 8, ctx - 8, nh, nkv, stride, nh * 64, kcache=kc, vcache=vc)
    for i in (0, 5, ctx - 9):
        assert np.array_equal(out[i], oracle.gqa_decode_f32(rows[8 + i], kc, vc, 8 + i, nh, nkv))
    outq = oracle.prefill(rows[8:], 8, ctx - 8, nh, nkv, stride, nh * 64, cache=cache)
    assert np.array_equal(outq[3], oracle.gqa_decode_q8(rows[11], cache, 11, nh, 0))


def test_gemv_gemm_and_int8_gemv_against_float64():
    """The projection restatements against an independent float64 evaluation: gemv / gemm (fp32 and fp16 weights, with
    bias, residual accumulate) to fp32 summation accuracy, gemv_int8 against the same arithmetic written out in numpy
    (per-group activation quantisation, integer dots, per-column scales)."""
    rs = np.random.RandomState(5)
    m, k, n = 5, 96, 40
    a = oracle.normal((m, k), 61, 0)
    w = (oracle.normal((k, n), 62, 0) / np.sqrt(k)).astype(np.float32)
    b = oracle.normal((n,), 63, 0)
    want = a.astype(np.float64) @ w.astype(np.float64) + b
    assert np.abs(oracle.gemm(a, w, b) - want).max() < 1e-5
    wh = w.astype(np.float16)
    assert np.abs(oracle.gemm(a, wh, b) - (a.astype(np.float64) @ wh.astype(np.float64) + b)).max() < 1e-5
    y0 = oracle.normal((n,), 64, 0)
    assert np.abs(oracle.gemv(a[0], w, None, y0, True) - (y0 + a[0].astype(np.float64) @ w.astype(np.float64))).max() < 1e-5
    assert oracle.gemm(np.zeros((0, k), np.float32), w, b).shape == (0, n)
    # int8 weights: groups of `ag` activations share a scale amax / 127; y = (sum_g dot_g * xs_g) * scale[o] + b[o]
    w8 = rs.randint(-127, 128, size=(k, n)).astype(np.int8)
    scales = (rs.rand(n) * 0.01 + 0.001).astype(np.float32)
    x = a[1]
    for ag in (4, 8):
        acc = np.zeros(n, np.float64)
        for g0 in range(0, k, ag):
            xg = x[g0:g0 + ag]
            amax = np.float32(np.abs(xg).max())
            if amax == 0:
                continue
            codes = np.clip(np.rint(xg * (np.float32(127.0) / amax)), -127, 127).astype(np.int64)
            acc += (codes @ w8[g0:g0 + ag].astype(np.int64)) * np.float64(amax / np.float32(127.0))
        want8 = acc * scales + b
        got8 = oracle.gemv_int8(x, oracle.pack_int8_weights(w8), scales, b, ag=ag)
        assert np.abs(got8 - want8).max() < 2e-4 * max(1.0, np.abs(want8).max()), ag
