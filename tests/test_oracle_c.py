"""The C restatement of the oracle agrees bit for bit with the numpy oracle (which is pinned to the
reference's fixtures)."""

import ctypes

import numpy as np
import pytest

from oracle import lqq_oracle as O
from oracle import build_oracle
from tests.helpers import random_lqq, random_tokens


@pytest.fixture(scope="module")
def clib():
    return build_oracle.load()


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


@pytest.mark.parametrize("g", [64, 128, 32])
def test_c_dequant(clib, g):
    qw = random_lqq(96, 512, g, seed=g)
    for fn in (clib.lqo_dequant_i8, clib.lqo_dequant_i8_simd):
        out = np.empty((96, 512), np.int8)
        fn(_p(qw.qweight_u4), _p(qw.s_u8), _p(qw.offset_a), _p(out), 96, 512, g)
        assert np.array_equal(out, O.dequantize_i8(qw))


def test_c_gemm_scale_and_linear(clib, golden):
    qw = random_lqq(160, 768, 64, seed=1)
    x, ascale = random_tokens(9, 768, seed=2)
    qhat = O.dequantize_i8(qw)
    acc = np.empty((9, 160), np.int32)
    clib.lqo_int_gemm(_p(x), _p(qhat), _p(acc), 9, 160, 768)
    assert np.array_equal(acc, O.int_accumulate(x, qhat))
    y = np.empty((9, 160), np.float32)
    clib.lqo_scale_f32(_p(acc), _p(ascale), _p(qw.s1), _p(y), 9, 160)
    assert np.array_equal(y.view(np.uint32), O.scale_f32(acc, ascale, qw.s1).view(np.uint32))
    # whole linear from fp32 tokens, against the golden case computed by the reference
    c = "g64_tailed"
    gq = O.LQQWeight(golden.get(c, "q_u4"), golden.get(c, "s_u8"), golden.get(c, "offset_a"),
                     golden.get(c, "s1"), 64)
    X = np.ascontiguousarray(golden.get(c, "X").astype(np.float32))
    M, K = X.shape
    out = np.empty((M, gq.N), np.float32)
    clib.lqo_w4a8_linear(_p(X), _p(gq.qweight_u4), _p(gq.s_u8), _p(gq.offset_a), _p(gq.s1), _p(out), M, gq.N, K, 64)
    assert np.array_equal(out.view(np.uint32), golden.get(c, "y_f32").view(np.uint32))


def test_c_quant_per_token(clib):
    X = O.synth_activation(7, 1000, seed=4, hot_channel_frac=0.01).astype(np.float32)
    X[3] = 0
    xq = np.empty((7, 1000), np.int8)
    sc = np.empty(7, np.float32)
    clib.lqo_quant_per_token(_p(X), _p(xq), _p(sc), 7, 1000)
    e_q, e_s = O.quantize_activation(X)
    assert np.array_equal(xq, e_q) and np.array_equal(sc.view(np.uint32), e_s.view(np.uint32))
