"""Concat, Split, Slice, Expand and Cast on the GPU against the numpy restatement of the reference's CPU kernels: bit-exact,
over element sizes, ragged shapes (so that every copy unit from 1 to 16 bytes is taken), negative steps, empty parts, and
through the graph layer with ONNX attributes."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as onp
from refactorgraph_b200 import capi
from refactorgraph_b200.graph_builder import GraphBuilder

import _ops as ops

pytestmark = pytest.mark.gpu

NP = {torch.float32: np.float32, torch.float16: np.float16, torch.int64: np.int64, torch.uint8: np.uint8, torch.int16: np.int16, torch.float64: np.float64}


def _rand(rng, shape, dt):
    a = rng.integers(-100, 100, shape) if np.issubdtype(NP[dt], np.integer) and NP[dt] != np.uint8 else rng.integers(0, 200, shape)
    return torch.from_numpy(a.astype(NP[dt])).cuda()


@pytest.mark.parametrize("dt", [torch.float16, torch.float32, torch.uint8, torch.int64])
@pytest.mark.parametrize("shapes,axis", [([(2, 3, 8), (2, 5, 8), (2, 1, 8)], 1), ([(4, 7), (4, 9)], -1), ([(3, 16), (0, 16), (5, 16)], 0),
                                         ([(1, 2, 3, 5), (1, 2, 3, 5)], 2), ([(6,), (10,)], 0)])
def test_concat_and_split(dt, shapes, axis):
    rng = np.random.default_rng(len(shapes) + axis + 7)
    xs = [_rand(rng, s, dt) for s in shapes]
    y = ops.concat(xs, axis)
    want = onp.concat([x.cpu().numpy() for x in xs], axis)
    assert np.array_equal(y.cpu().numpy(), want)
    parts = ops.split(y, [s[axis] for s in shapes], axis)
    for got, x in zip(parts, xs):
        assert torch.equal(got, x)
    assert capi.load().rg_b200_error_state() == 0


@pytest.mark.parametrize("dt", [torch.float16, torch.float32, torch.uint8, torch.float64])
@pytest.mark.parametrize("shape,starts,steps,lengths", [((4, 10), (1, 2), (1, 3), (3, 3)), ((4, 10), (3, 9), (-1, -2), (4, 5)), ((2, 3, 16), (0, 1, 8), (1, 1, 1), (2, 2, 8)),
                                                          ((5,), (4,), (-1,), (5,)), ((3, 4, 5, 6), (0, 0, 0, 0), (1, 1, 1, 1), (3, 4, 5, 6)), ((8, 8), (0, 0), (2, 2), (0, 4))])
def test_slice(dt, shape, starts, steps, lengths):
    rng = np.random.default_rng(sum(shape))
    x = _rand(rng, shape, dt)
    y = ops.slice_(x, starts, steps, lengths)
    assert np.array_equal(y.cpu().numpy(), onp.slice_(x.cpu().numpy(), starts, steps, lengths))


def test_slice_refuses_indices_outside_the_input():
    x = torch.zeros(4, 10, dtype=torch.float16, device="cuda")
    for starts, steps, lengths in (((0, 8), (1, 1), (4, 3)), ((0, 0), (1, -1), (4, 2)), ((-1, 0), (1, 1), (2, 2))):
        rc, _ = ops.slice_(x, starts, steps, lengths, check=False)
        assert rc == capi.ERR_SHAPE


@pytest.mark.parametrize("dt", [torch.float16, torch.float32, torch.int64])
@pytest.mark.parametrize("inshape,outshape", [((1, 8), (5, 8)), ((3, 1), (3, 7)), ((4,), (2, 3, 4)), ((2, 1, 4), (2, 6, 4)), ((1,), (9,)), ((2, 3), (2, 3))])
def test_expand(dt, inshape, outshape):
    rng = np.random.default_rng(sum(outshape))
    x = _rand(rng, inshape, dt)
    y = ops.expand(x, outshape)
    assert np.array_equal(y.cpu().numpy(), onp.expand(x.cpu().numpy(), outshape))


CAST_TYPES = [torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64, torch.bool]


@pytest.mark.parametrize("src", CAST_TYPES)
@pytest.mark.parametrize("dst", CAST_TYPES)
def test_cast(src, dst):
    rng = np.random.default_rng(11)
    # values every type pair converts without leaving the target's range: 0..100, with fractions for the float sources
    base = rng.integers(0, 100, 1003).astype(np.float64)
    if src.is_floating_point:
        base = base + rng.integers(0, 4, base.shape) * 0.25
    x = torch.from_numpy(base).to(src).cuda() if src != torch.bool else torch.from_numpy(base % 3 != 0).cuda()
    y = ops.cast(x, dst)
    assert y.dtype == dst
    want = x.cpu().to(dst)           # torch on the CPU: truncation toward zero, `!= 0` for bool, round-to-nearest-even for 16-bit floats
    assert torch.equal(y.cpu(), want)


def test_graph_with_onnx_data_movement_operators():
    """The five operators through the graph layer, with the attributes ONNX gives them."""
    from refactorgraph_b200.graph_builder import F32, FP16, I64
    g = GraphBuilder()
    a = g.input("a", F32, (2, 3, 8))
    b = g.input("b", F32, (2, 5, 8))
    c = g.op("onnx::Concat", [a, b], axis=1)                                     # [2, 8, 8]
    s0, s1 = g.op("onnx::Split", [c], n_out=2, axis=-1, split=[6, 2])            # [2, 8, 6], [2, 8, 2]
    sl = g.op("onnx::Slice", [s0], starts=[7, 1], ends=[-9, 6], axes=[1, 2], steps=[-2, 2])   # rows 7,5,3,1; cols 1,3,5
    e = g.op("onnx::Expand", [s1], shape=[3, 2, 8, 2])
    h = g.op("onnx::Cast", [sl], to=int(FP16))
    k = g.op("onnx::Cast", [e], to=int(I64))
    outs = [g.output(h), g.output(k), g.output(c)]
    ex = g.compiler().compile("cuda", "flat", [])
    rng = np.random.default_rng(5)
    av = rng.standard_normal((2, 3, 8)).astype(np.float32) * 10
    bv = rng.standard_normal((2, 5, 8)).astype(np.float32) * 10
    ex.set_input(0, av)
    ex.set_input(1, bv)
    ex.run()
    cw = np.concatenate([av, bv], axis=1)
    assert np.array_equal(ex.get_output(outs[2]), cw)
    assert np.array_equal(ex.get_output(outs[0]), cw[:, 7:-9:-2, 1:6:2].astype(np.float16))
    assert np.array_equal(ex.get_output(outs[1]), np.broadcast_to(cw[:, :, 6:], (3, 2, 8, 2)).astype(np.int64))
