"""The product's packing helpers (``liquidgemm_b200.pack`` and the prepacks of ``ops``-free code) against
the fixtures computed by the reference's own ``liquidgemm/pack.py`` (tests/golden/make_golden.py), on the
CPU.  The oracle's restatements are pinned to the same fixtures in tests/test_oracle_golden.py; this file
pins the functions a user of the package actually imports (reference liquidgemm/pack.py:27-78)."""

import numpy as np
import torch

from liquidgemm_b200 import pack as P
from liquidgemm_b200.quant import LiquidQuantWeight


def _qw(golden, case):
    return LiquidQuantWeight(torch.from_numpy(golden.get(case, "q_u4")), torch.from_numpy(golden.get(case, "s_u8")),
                             torch.from_numpy(golden.get(case, "offset_a")), torch.from_numpy(golden.get(case, "s1")),
                             int(golden.get(case, "group")))


def test_pack_and_unpack_nibbles(golden):
    for case in golden.cases:
        q = torch.from_numpy(golden.get(case, "q_u4"))
        packed = P.pack_nibbles(q)
        assert packed.dtype == torch.uint8
        assert np.array_equal(packed.numpy(), golden.get(case, "nibbles"))
        assert torch.equal(P.unpack_nibbles(packed), q)


def test_pack_lanes_u32(golden):
    for case in golden.cases:
        lanes = P.pack_lanes_u32(torch.from_numpy(golden.get(case, "q_u4")))
        assert np.array_equal(lanes.numpy().astype(np.int64), golden.get(case, "lanes_u32").astype(np.int64))


def test_simd_dequant_u32_equals_the_per_element_dequant(golden):
    for case in golden.cases:
        got = P.simd_dequant_u32(_qw(golden, case))
        assert got.dtype == torch.int8
        assert np.array_equal(got.numpy(), golden.get(case, "simd_qhat").astype(np.int8))
        assert np.array_equal(got.numpy(), golden.get(case, "qhat_xor").astype(np.int8))
