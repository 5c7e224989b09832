"""GPU parity of the MXFP4 and NVFP4 routed-MoE paths against the CPU oracle, through the C ABI.

The oracle decodes the same packed bytes (src/arch/mimo_v2/moe.zig:379-416, src/arch/glm5_next/decode_kernels_ref.zig:13-65)
and applies the reference decode texts' rounding points (bf16 gate/up, bf16 SiLU product, bf16 down rows, the chain
combine); the bar for the bf16 layer output is 1e-2 relative L2.
"""
import numpy as np
import pytest

import oracle_lib as O
from moe_cases import Mxfp4Case, Nvfp4Case, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.mark.parametrize("cls,limit,shared", [(Mxfp4Case, 0.0, False), (Nvfp4Case, 10.0, True)])
def test_fp4_small_layer(cls, limit, shared):
    case = cls(512, 256, 8, 2, seed=6, shared=shared, scoring=O.SCORE_SIGMOID, max_tokens=64, routed_scale=1.0,
               limit=limit, chain=True)
    try:
        for T in (1, 5, 33, 64):
            x, logits = case.inputs(T, seed=10 + T)
            y = case.gpu_forward(x, logits)
            ids, w = case.cpu_route(logits)
            ref = case.cpu_layer(x, ids, w)
            assert rel_l2(y, ref) < TOL, (T, rel_l2(y, ref))
        # every token to the same experts: more rows than one work item holds
        T = 40
        x, _ = case.inputs(T, seed=3)
        ids = np.tile(np.array([[1, 6]], np.int32), (T, 1))
        w = np.full((T, 2), 0.5, np.float32)
        assert rel_l2(case.gpu_experts(x, ids, w), case.cpu_layer(x, ids, w)) < TOL
        assert case.status() == 0
    finally:
        case.close()


@pytest.mark.parametrize("cls,H,I,limit,shared", [(Mxfp4Case, 4096, 2048, 0.0, False), (Nvfp4Case, 6144, 2048, 10.0, True)])
def test_fp4_config_shapes(cls, H, I, limit, shared):
    # BASELINE configs 3 (MiMo shape) and 4 (GLM shape) at a reduced expert count
    case = cls(H, I, 4, 2, seed=2, shared=shared, scoring=O.SCORE_SIGMOID, max_tokens=16, routed_scale=1.0, limit=limit,
               chain=True)
    try:
        x, logits = case.inputs(6, seed=4)
        ids, w = case.gpu_route(logits)
        rid, rw = case.cpu_route(logits)
        assert (ids == rid).all()
        y = case.gpu_experts(x, ids, w)
        assert rel_l2(y, case.cpu_layer(x, rid, rw)) < TOL
        again = case.gpu_experts(x, ids, w)
        assert (y == again).all()
        one = case.gpu_experts(x[2:3], ids[2:3], w[2:3])
        assert (one[0] == y[2]).all()  # a row does not depend on the batch around it
        assert case.status() == 0
    finally:
        case.close()


def test_fp4_f32_combine_mode():
    # the same bank with the f32 combine (no chain rounding of the rows): against the oracle's unrounded f64 path
    case = Mxfp4Case(512, 256, 8, 2, seed=8, shared=False, scoring=O.SCORE_SOFTMAX, max_tokens=16, routed_scale=1.0,
                     limit=0.0, chain=False)
    try:
        x, logits = case.inputs(9, seed=2)
        y = case.gpu_forward(x, logits)
        ids, w = case.cpu_route(logits)
        assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL
    finally:
        case.close()
