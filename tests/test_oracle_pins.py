"""Ties the C oracle's elementwise / reduce functions to the CPU loop-nest checker.

The loop-nest checker (oracle/_cpu/imex-oracle-runner) runs programs as the reference's CPU
pipeline does and is itself pinned to the CHECK lines of the reference's tests
(tests/test_reference_programs.py), among them the f16 / bf16 variants of test/Gen/PlaidML.
Here the same chains the benchmark grid uses (log, absf, addf, subf of
benchmarks/kLoopFusion/kLoopFusion.mlir.in:4-30 and the column sum of
benchmarks/kInputFusion/kInputFusion.mlir.in:29-39) run through it on seeded f16 / bf16 / f32
data, and oracle_unary / oracle_binary / oracle_reduce_leading_as — what the GPU kernels are
compared with at sizes no .mlir literal could hold — must give the same values: per-operation
rounding to the element type, ascending order of the sums."""
import os
import re
import subprocess

import numpy as np
import pytest

from __graft_entry__ import ROOT
from oracle import oracle

ORACLE_RUNNER = os.path.join(ROOT, "oracle", "_cpu", "imex-oracle-runner")
pytestmark = pytest.mark.skipif(not os.path.exists(ORACLE_RUNNER),
                                reason="oracle/_cpu/imex-oracle-runner is not built (make -C oracle cpu_runner)")

KINDS = {"f32": (oracle.DT_F32, None, None), "f16": (oracle.DT_F16, oracle.to_f16_bits, oracle.f16_bits_to_f32),
         "bf16": (oracle.DT_BF16, oracle.to_bf16_bits, oracle.bf16_bits_to_f32)}


def _dense(a):
    rows = ["[" + ", ".join(repr(float(v)) for v in r) + "]" for r in a]
    return "dense<[" + ", ".join(rows) + "]>"


PROGRAM = """
#id = affine_map<(d0, d1) -> (d0, d1)>
#t = affine_map<(d0, d1) -> (d1, d0)>
#v = affine_map<(d0, d1) -> (d0)>
module {{
func.func private @printMemref{P}(tensor<*x{T}>)
func.func @main() {{
  %x0 = arith.constant {X0} : tensor<{R}x{C}x{T}>
  %x1 = arith.constant {X1} : tensor<{R}x{C}x{T}>
  %e0 = tensor.empty() : tensor<{R}x{C}x{T}>
  %l = linalg.generic {{indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]}} ins(%x0 : tensor<{R}x{C}x{T}>) outs(%e0 : tensor<{R}x{C}x{T}>) {{
  ^bb0(%a: {T}, %o: {T}):
    %r = math.log %a : {T}
    linalg.yield %r : {T}
  }} -> tensor<{R}x{C}x{T}>
  %e1 = tensor.empty() : tensor<{R}x{C}x{T}>
  %ab = linalg.generic {{indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]}} ins(%x1 : tensor<{R}x{C}x{T}>) outs(%e1 : tensor<{R}x{C}x{T}>) {{
  ^bb0(%a: {T}, %o: {T}):
    %r = math.absf %a : {T}
    linalg.yield %r : {T}
  }} -> tensor<{R}x{C}x{T}>
  %e2 = tensor.empty() : tensor<{R}x{C}x{T}>
  %s = linalg.generic {{indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]}} ins(%l, %ab : tensor<{R}x{C}x{T}>, tensor<{R}x{C}x{T}>) outs(%e2 : tensor<{R}x{C}x{T}>) {{
  ^bb0(%a: {T}, %b: {T}, %o: {T}):
    %r = arith.addf %a, %b : {T}
    linalg.yield %r : {T}
  }} -> tensor<{R}x{C}x{T}>
  %e3 = tensor.empty() : tensor<{R}x{C}x{T}>
  %d = linalg.generic {{indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]}} ins(%s, %x0 : tensor<{R}x{C}x{T}>, tensor<{R}x{C}x{T}>) outs(%e3 : tensor<{R}x{C}x{T}>) {{
  ^bb0(%a: {T}, %b: {T}, %o: {T}):
    %r = arith.subf %a, %b : {T}
    linalg.yield %r : {T}
  }} -> tensor<{R}x{C}x{T}>
  %u = tensor.cast %d : tensor<{R}x{C}x{T}> to tensor<*x{T}>
  call @printMemref{P}(%u) : (tensor<*x{T}>) -> ()
  %zero = arith.constant 0.0 : {T}
  %ye = tensor.empty() : tensor<{C}x{T}>
  %y0 = linalg.fill ins(%zero : {T}) outs(%ye : tensor<{C}x{T}>) -> tensor<{C}x{T}>
  %y = linalg.generic {{indexing_maps = [#t, #v], iterator_types = ["parallel", "reduction"]}} ins(%s : tensor<{R}x{C}x{T}>) outs(%y0 : tensor<{C}x{T}>) {{
  ^bb0(%a: {T}, %acc: {T}):
    %r = arith.addf %a, %acc : {T}
    linalg.yield %r : {T}
  }} -> tensor<{C}x{T}>
  %yu = tensor.cast %y : tensor<{C}x{T}> to tensor<*x{T}>
  call @printMemref{P}(%yu) : (tensor<*x{T}>) -> ()
  return
}}
}}
"""


def _printed(text):
    out = []
    for m in re.finditer(r"data =\s*\n((?:[ \[].*\n?)+)", text):
        out.append(np.array([float(x) for x in re.findall(r"-?(?:\d+\.?\d*(?:e[-+]?\d+)?|inf|nan)", m.group(1))],
                            np.float64))
    return out


@pytest.mark.parametrize("kind", ["f16", "bf16", "f32"])
def test_elementwise_and_column_sum_oracles_agree_with_the_loop_nest_checker(tmp_path, kind):
    dt, to_bits, back = KINDS[kind]
    R, C = 24, 16
    x0 = oracle.fill_uniform((R, C), 41, 0.5, 4.0)
    x1 = oracle.fill_uniform((R, C), 42, -2.0, 2.0)
    if to_bits:
        x0, x1 = back(to_bits(x0)), back(to_bits(x1))
    path = tmp_path / ("chain_%s.mlir" % kind)
    path.write_text(PROGRAM.format(T=kind, P={"f32": "F32", "f16": "F16", "bf16": "BF16"}[kind], R=R, C=C,
                                   X0=_dense(x0), X1=_dense(x1)))
    r = subprocess.run([ORACLE_RUNNER, str(path), "--all-loopnests", "-e", "main"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-800:] + r.stderr[-800:]
    chain, colsum = _printed(r.stdout)
    s = oracle.binary("addf", oracle.unary("log", x0, dt), oracle.unary("absf", x1, dt), dt)
    want_chain = oracle.binary("subf", s, x0, dt).reshape(-1)
    want_sum = oracle.reduce_leading_as(s, dt)
    if to_bits:
        # six printed digits identify a 16-bit value: compare bit patterns
        assert np.array_equal(to_bits(chain.astype(np.float32)), to_bits(want_chain))
        assert np.array_equal(to_bits(colsum.astype(np.float32)), to_bits(want_sum))
    else:
        assert np.allclose(chain, want_chain, rtol=1e-5, atol=1e-6)   # printed with six digits
        assert np.allclose(colsum, want_sum, rtol=1e-5, atol=1e-6)
