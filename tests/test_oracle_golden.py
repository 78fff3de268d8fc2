"""The CPU oracle must reproduce every golden vector the reference's own tests
hold for the hot path (tests/golden/reference_vectors.json, transcribed from
the CHECK lines by tests/golden/make_reference_vectors.py), and must agree
with the reference's in-tree CPU GEMM where that was compiled (oracle/_ref)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_vectors.json")) as f:
    CASES = {c["name"]: c for c in json.load(f)["cases"]}


def _arr(inp):
    if "splat" in inp:
        return np.full(inp["dims"], inp["splat"], np.float32)
    dt = np.int32 if inp["dtype"].startswith("i") else np.float32
    return np.array(inp["data"], dt).reshape(inp["dims"])


def _printed6(v):
    """What the upstream memref printer shows: 6 significant digits."""
    return float("%.6g" % float(v))


def _check(case, got):
    exp = case["expected"]
    got = np.asarray(got).reshape(-1)
    mode = case["compare"]
    if mode == "exact":
        if case.get("expected_rows") == "first":
            got = got[: len(exp)]
        assert got.tolist() == exp
    elif mode == "exact_all_equal":
        assert len(exp) == 1 and np.all(got == exp[0])
    elif mode == "printed6":
        assert [_printed6(x) for x in got] == exp
    elif mode == "allclose":
        assert oracle.allclose(got, np.array(exp, np.float32))
    else:
        raise AssertionError(mode)


def _run(case):
    op = case["op"]
    ins = [_arr(i) for i in case["inputs"]]
    if op in ("matmul_f32", "matmul_f32_splat"):
        return oracle.matmul_f32(ins[0], ins[1])
    if op == "matmul_f32_cinit":
        return oracle.matmul_f32(ins[0], ins[1], C_init=ins[2])
    if op == "matmul_f16_f32_truncf16":
        c = oracle.matmul_x16_f32(oracle.to_f16_bits(ins[0]), oracle.to_f16_bits(ins[1]),
                                  is_bf16=False)
        return oracle.f16_bits_to_f32(oracle.to_f16_bits(c))
    if op == "matmul_bf16_f32_cinit":
        return oracle.matmul_x16_f32(oracle.to_bf16_bits(ins[0]), oracle.to_bf16_bits(ins[1]),
                                     is_bf16=True, C_init=ins[2])
    if op == "softmax_plaidml":
        return oracle.softmax(ins[0], oracle.SOFTMAX_PLAIDML)
    if op == "reduce_all":
        return np.array([oracle.reduce_all(ins[0])])
    if op == "transpose2d":
        return oracle.transpose2d(ins[0])
    if op == "relu":
        # the PlaidML form (olt + select) and the benchmark form (ugt + select)
        # agree on every input of this vector (no -0, no NaN)
        return oracle.relu(ins[0])
    raise AssertionError(op)


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_reference_golden(name):
    case = CASES[name]
    _check(case, _run(case))


def test_loops_and_fast_matmul_are_bit_identical():
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (37, 53)).astype(np.float32)
    B = rng.uniform(-1, 1, (53, 29)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (37, 29)).astype(np.float32)
    a = oracle.matmul_f32(A, B, C0, loops=True)
    b = oracle.matmul_f32(A, B, C0, loops=False)
    assert a.tobytes() == b.tobytes()
    Ab, Bb = oracle.to_bf16_bits(A), oracle.to_bf16_bits(B)
    a = oracle.matmul_x16_f32(Ab, Bb, True, loops=True)
    b = oracle.matmul_x16_f32(Ab, Bb, True, loops=False)
    assert a.tobytes() == b.tobytes()
    rows = oracle.matmul_x16_f32_rows(Ab, Bb, 5, 7, True)
    assert rows.tobytes() == a[5:12].tobytes()


def test_matmul_is_not_fma_contracted():
    # a*b rounds to 1 before the add when mulf/addf stay separate; a fused
    # multiply-add would return -2^-26 instead of 0
    a = np.float32(1 + 2.0 ** -13)
    b = np.float32(1 - 2.0 ** -13)
    A = np.array([[a]], np.float32)
    B = np.array([[b]], np.float32)
    C0 = np.array([[-1.0]], np.float32)
    for loops in (True, False):
        assert oracle.matmul_f32(A, B, C0, loops=loops)[0, 0] == np.float32(0.0)


def test_16bit_conversions_match_numpy():
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 500),
                        rng.normal(0, 3e4, 500),
                        [0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e-8, 2.0 ** -25, 5.96e-8,
                         np.inf, -np.inf]]).astype(np.float32)
    h = oracle.to_f16_bits(x)
    with np.errstate(over="ignore"):
        assert np.array_equal(h, x.astype(np.float16).view(np.uint16))
    assert np.array_equal(oracle.f16_bits_to_f32(h), h.view(np.float16).astype(np.float32))
    allh = np.arange(65536, dtype=np.uint16)
    ours = np.array([oracle.lib().oracle_f16_to_f32(int(v)) for v in allh[::7]], np.float32)
    ref = allh[::7].view(np.float16).astype(np.float32)
    finite = ~np.isnan(ref)  # NaN payloads may be quieted on the way back through ctypes
    assert np.array_equal(ours.view(np.uint32)[finite], ref.view(np.uint32)[finite])
    assert np.all(np.isnan(ours[~finite]))
    b = oracle.to_bf16_bits(x)
    import torch
    tb = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(b, tb)


def test_relu_follows_ugt_select():
    x = np.array([np.nan, -0.0, 0.0, -1.0, 2.0, -np.inf, np.inf], np.float32)
    y = oracle.relu(x)
    assert np.isnan(y[0])
    assert y[1:].tolist() == [0.0, 0.0, 0.0, 2.0, 0.0, np.inf]
    assert not np.signbit(y[1])  # -0 -> +0: select picks the +0.0 constant


def test_silu_and_softmax_against_float64():
    rng = np.random.default_rng(2)
    x = rng.normal(0, 3, (64, 257)).astype(np.float32)
    s = oracle.silu(x)
    x64 = x.astype(np.float64)
    assert np.max(np.abs(s - x64 / (1 + np.exp(-x64))) / np.maximum(np.abs(s), 1e-30)) < 1e-6
    y = oracle.softmax(x)
    e = np.exp(x64 - x64.max(-1, keepdims=True))
    ref = e / e.sum(-1, keepdims=True)
    assert np.max(np.abs(y - ref) / ref) < 1e-5
    assert np.array_equal(y, oracle.softmax(x, oracle.SOFTMAX_PLAIDML))


def test_reductions_and_transposes():
    rng = np.random.default_rng(3)
    x = rng.uniform(0, 1, (33, 70)).astype(np.float32)
    seq = np.zeros(33, np.float32)
    for c in range(70):
        seq = (seq + x[:, c]).astype(np.float32)
    assert np.array_equal(oracle.reduce_rows(x), seq)
    assert np.array_equal(oracle.reduce_leading(x.T.copy()), seq)
    init = rng.uniform(0, 1, 33).astype(np.float32)
    seq2 = init.copy()
    for c in range(70):
        seq2 = (seq2 + x[:, c]).astype(np.float32)
    assert np.array_equal(oracle.reduce_rows(x, init), seq2)
    assert np.array_equal(oracle.transpose2d(x), x.T)
    h = rng.integers(0, 65535, (5, 9)).astype(np.uint16)
    assert np.array_equal(oracle.transpose2d(h), h.T)
    t = rng.uniform(-1, 1, (4, 5, 6)).astype(np.float32)
    for perm in [(0, 2, 1), (2, 1, 0), (1, 0, 2), (2, 0, 1)]:
        assert np.array_equal(oracle.transpose3d(t, perm), t.transpose(perm))
    # empty inputs
    assert oracle.reduce_rows(np.zeros((0, 5), np.float32)).shape == (0,)
    assert oracle.reduce_rows(np.zeros((3, 0), np.float32)).tolist() == [0, 0, 0]
    assert oracle.transpose2d(np.zeros((0, 4), np.float32)).shape == (4, 0)


def test_seeded_fill_is_reproducible_and_in_range():
    a = oracle.fill_uniform((1000,), 7, -1.0, 1.0)
    b = oracle.fill_uniform((1000,), 7, -1.0, 1.0)
    c = oracle.fill_uniform((500,), 7, -1.0, 1.0, first=500)
    assert np.array_equal(a, b) and np.array_equal(a[500:], c)
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(a.mean()) < 0.1
    assert not np.array_equal(a, oracle.fill_uniform((1000,), 8, -1.0, 1.0))


needs_ref = pytest.mark.skipif(oracle.ref_lib() is None,
                               reason="oracle/_ref not built (no reference checkout)")


@needs_ref
@pytest.mark.parametrize("is_bf16", [True, False])
def test_restatement_matches_reference_cpu_gemm_bit_for_bit(is_bf16):
    """oracle/_ref holds the reference's own _mlir_ciface_gemm (i,k,j loops in
    f32); the restatement must give the very same bits."""
    rng = np.random.default_rng(4)
    A = rng.uniform(-1, 1, (48, 96)).astype(np.float32)
    B = rng.uniform(-1, 1, (96, 40)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (48, 40)).astype(np.float32)
    conv = oracle.to_bf16_bits if is_bf16 else oracle.to_f16_bits
    Ab, Bb = conv(A), conv(B)
    ours = oracle.matmul_x16_f32(Ab, Bb, is_bf16, C_init=C0, loops=True)
    theirs = oracle.ref_gemm_x16_f32(Ab, Bb, is_bf16, C_init=C0)
    assert ours.tobytes() == theirs.tobytes()


@needs_ref
def test_reference_gemm_reproduces_its_own_golden():
    case = CASES["gemm_3x3_bf16_accf32"]
    ins = [_arr(i) for i in case["inputs"]]
    got = oracle.ref_gemm_x16_f32(oracle.to_bf16_bits(ins[0]), oracle.to_bf16_bits(ins[1]),
                                  True, C_init=ins[2])
    assert oracle.ref_lib().ref_allclose_f32(
        got.ctypes.data_as(oracle._fp),
        np.array(case["expected"], np.float32).ctypes.data_as(oracle._fp), 9) == 1


def test_one_pass_attention_recurrence_stays_within_the_budget_of_the_gpu_tests():
    """The attention kernel's arithmetic, emulated in numpy (blocks of 128 keys, running maximum in
    log2 units, un-normalised probabilities rounded to f16, division by the row sum at the end),
    against the oracle (= the reference test's CPU check, which normalises before rounding): the
    two formulations differ by 16-bit roundings only, inside the tolerances the GPU tests use, and
    both are equally far from a float64 evaluation."""
    heads, n, d, scale = 2, 384, 64, 0.5
    q, k, v = (oracle.to_f16_bits(oracle.fill_uniform((heads * n, d), 41 + i, -1.0, 1.0)) for i in range(3))
    ref = oracle.f16_bits_to_f32(oracle.attention_fwd(q, k, v, heads, scale, False))
    qf, kf, vf = (oracle.f16_bits_to_f32(x).reshape(heads, n, d) for x in (q, k, v))
    sl2 = np.float32(scale * 1.4426950408889634)
    out = np.empty((heads, n, d), np.float32)
    for h in range(heads):
        m = np.full((n, 1), -np.inf, np.float32)
        l = np.zeros((n, 1), np.float32)
        o = np.zeros((n, d), np.float32)
        for j0 in range(0, n, 128):
            s = (qf[h] @ kf[h][j0:j0 + 128].T).astype(np.float32) * sl2
            m_new = np.maximum(m, s.max(axis=1, keepdims=True))
            alpha = np.exp2(m - m_new)
            p = np.exp2(s - m_new).astype(np.float32)
            l = l * alpha + p.sum(axis=1, keepdims=True)
            o = o * alpha + p.astype(np.float16).astype(np.float32) @ vf[h][j0:j0 + 128]
            m = m_new
        out[h] = (o / l).astype(np.float16).astype(np.float32)
    out = out.reshape(heads * n, d)
    assert oracle.rel_frobenius(out, ref) <= 1e-3
    assert np.all(np.abs(out - ref) <= 2.5e-4 + 2e-3 * np.abs(ref))
    truth = np.concatenate([(lambda S: (np.exp(S - S.max(1, keepdims=True)) /
                                        np.exp(S - S.max(1, keepdims=True)).sum(1, keepdims=True)) @ vf[h].astype(np.float64))(
        (qf[h].astype(np.float64) @ kf[h].astype(np.float64).T) * scale) for h in range(heads)])
    assert np.abs(out - truth).max() <= 1.5 * np.abs(ref - truth).max() + 1e-4
