"""Generates tests/golden/attn_golden.npz: small known-answer vectors for the oracle.

The reference repository ships no golden files (its tests compare GPU output with its
Rust CPU code on seeded xorshift inputs).  These vectors come from an independent
float64 / numpy restatement of the same formulas, written without looking at
oracle/attn_oracle.c, so that the C oracle is pinned by a second implementation:

* xorshift64* uniform stream of common/src/lib.rs:67-78 (pure Python integers);
* softmax attention forward (O, natural-log LSE) and its VJP (dQ, dK, dV) in float64,
  causal and non-causal, on the reference's own seeds (1,2,3 / 11..14), N = 64;
* the affine int8 quantiser of 03-llm-engine/kernels/llm.cu:1137-1149 and the
  symmetric absmax one of :1353-1362 in numpy float32 arithmetic;
* rotate_half RoPE of 03-llm-engine/src/cpu.rs:25-37 in float64.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np

MASK = (1 << 64) - 1


def pseudo_rand(n, seed):
    out = np.empty(n, np.float32)
    s = seed
    for i in range(n):
        s ^= s >> 12
        s ^= (s << 25) & MASK
        s ^= s >> 27
        r = (s * 0x2545F4914F6CDD1D) & MASK
        out[i] = np.float32(r >> 40) / np.float32(1 << 23) - np.float32(1.0)
    return out


def attention_f64(q, k, v, causal):
    n = q.shape[0]
    s = (q.astype(np.float64) @ k.astype(np.float64).T) / 8.0
    if causal:
        s = np.where(np.tril(np.ones((n, n), bool)), s, -np.inf)
    m = s.max(axis=1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(axis=1, keepdims=True)
    p = e / l
    return p @ v.astype(np.float64), (m + np.log(l))[:, 0], p


def attention_bwd_f64(q, k, v, do, causal):
    o, _, p = attention_f64(q, k, v, causal)
    do = do.astype(np.float64)
    dp = do @ v.astype(np.float64).T
    delta = (do * o).sum(axis=1, keepdims=True)
    ds = p * (dp - delta) / 8.0
    return ds @ k.astype(np.float64), ds.T @ q.astype(np.float64), p.T @ do


def quant_affine_np(x):
    x = x.astype(np.float32)
    hi, lo = x.max(), x.min()
    scale = np.float32((hi - lo) / np.float32(255.0)) if hi > lo else np.float32(1.0)
    beta = np.float32(lo + np.float32(128.0) * scale)
    q = np.rint(((x - beta) / scale).astype(np.float32))  # rint = round half to even
    return np.clip(q, -128, 127).astype(np.int8), scale, beta


def quant_absmax_np(x):
    x = x.astype(np.float32)
    amax = np.abs(x).max()
    inv = np.float32(127.0) / amax if amax > 0 else np.float32(0.0)
    q = np.clip(np.rint((x * inv).astype(np.float32)), -127, 127).astype(np.int8)
    return q, (amax / np.float32(127.0) if amax > 0 else np.float32(0.0))


def rope_f64(x, n_heads, hd, pos, theta):
    x = x.astype(np.float64).copy()
    half = hd // 2
    for h in range(n_heads):
        for d in range(half):
            # the reference evaluates the frequency in f32: theta.powf(-2d/hd)
            freq = float(np.float32(theta) ** np.float32(-2.0 * d / hd))
            a = float(np.float32(np.float32(pos) * np.float32(freq)))
            x1, x2 = x[h * hd + d], x[h * hd + d + half]
            x[h * hd + d] = x1 * np.cos(a) - x2 * np.sin(a)
            x[h * hd + d + half] = x1 * np.sin(a) + x2 * np.cos(a)
    return x


def main():
    out = {}
    out["rand_seed1_first16"] = pseudo_rand(16, 1)
    out["rand_seed42_first16"] = pseudo_rand(16, 42)
    n = 64
    q, k, v = (pseudo_rand(n * 64, s).reshape(n, 64) for s in (1, 2, 3))
    for causal in (0, 1):
        o, lse, _ = attention_f64(q, k, v, bool(causal))
        out[f"fwd_o_c{causal}"] = o
        out[f"fwd_lse_c{causal}"] = lse
    q, k, v, do = (pseudo_rand(n * 64, s).reshape(n, 64) for s in (11, 12, 13, 14))
    for causal in (0, 1):
        dq, dk, dv = attention_bwd_f64(q, k, v, do, bool(causal))
        out[f"bwd_dq_c{causal}"] = dq
        out[f"bwd_dk_c{causal}"] = dk
        out[f"bwd_dv_c{causal}"] = dv
    rows = pseudo_rand(8 * 64, 7).reshape(8, 64) * np.float32(3.0)
    rows[3] = 0.25            # constant row: hi == lo -> scale 1
    rows[4, :] = 0.0          # all-zero row
    rows[5, 0] = 100.0        # outlier
    codes, scales, betas, scodes, sscales = [], [], [], [], []
    for r in rows:
        c, s, b = quant_affine_np(r)
        codes.append(c), scales.append(s), betas.append(b)
        c2, s2 = quant_absmax_np(r)
        scodes.append(c2), sscales.append(s2)
    out["quant_rows"] = rows
    out["quant_affine_codes"] = np.stack(codes)
    out["quant_affine_scale"] = np.array(scales, np.float32)
    out["quant_affine_beta"] = np.array(betas, np.float32)
    out["quant_absmax_codes"] = np.stack(scodes)
    out["quant_absmax_scale"] = np.array(sscales, np.float32)
    x = pseudo_rand(4 * 64, 9)
    out["rope_in"] = x
    out["rope_pos37_theta1e6"] = rope_f64(x, 4, 64, 37, 1e6)
    out["rope_pos2047_theta1e4"] = rope_f64(x, 4, 64, 2047, 1e4)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")
    out = {k: (a.astype(np.float32) if a.dtype == np.float64 else a) for k, a in out.items()}
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
