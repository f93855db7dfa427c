"""The sparse-convolution caller (the driver side of the reference's
examples/rgms/sparse_conv/sparse_conv.py:93-125): neighbour maps -> one relation per kernel offset
-> CSF -> ELL3D with buckets = [1] -> the half-precision RGMS operator, against the plain
gather-matmul-scatter  y[o] += x[i] @ W[offset]  that a sparse convolution stands for."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from sparsetir_b200 import sparse_conv as sc


def synthetic_maps(rng, num_offsets, n_in, n_out, fill, repeats=True):
    """torchsparse-style maps: per offset a subset of the output points, each with one input
    point; with ``repeats`` one offset also gets several pairs that end in the same output point
    and one pair listed twice."""
    sizes, maps = [], []
    for k in range(num_offsets):
        outs = np.nonzero(rng.random(n_out) < fill)[0]
        ins = rng.integers(0, n_in, size=len(outs))
        if repeats and k == num_offsets // 2 and len(outs) > 8:
            outs[1:6] = outs[0]
            ins[7], outs[7] = ins[6], outs[6]
        if k == 1:
            outs, ins = outs[:0], ins[:0]  # an offset without any pair
        sizes.append(len(outs))
        maps.append(np.stack([ins, outs], axis=1))
    return np.concatenate(maps).astype(np.int64), sizes


def gather_matmul_scatter(x, w, maps, sizes, transposed, n_out):
    y = np.zeros((n_out, w.shape[2]), np.float64)
    x64, w64 = x.astype(np.float64), w.astype(np.float64)
    off = 0
    for k, s in enumerate(sizes):
        i, o = maps[off:off + s, 0], maps[off:off + s, 1]
        off += s
        if transposed:
            i, o = o, i
        np.add.at(y, o, x64[i] @ w64[k])
    return y


def layer(seed, num_offsets, n_in, n_out, feat_in, feat_out, transposed, repeats=True, fill=0.5):
    rng = np.random.default_rng(seed)
    # the maps of a transposed layer are stored (output, input): generate them the other way round
    a, b = (n_out, n_in) if transposed else (n_in, n_out)
    maps, sizes = synthetic_maps(rng, num_offsets, a, b, fill, repeats)
    x = rng.uniform(-1, 1, size=(n_in, feat_in)).astype(np.float16)
    w = (rng.standard_normal((num_offsets, feat_in, feat_out)) / np.sqrt(feat_in)).astype(np.float16)
    return maps, sizes, x, w


@pytest.mark.parametrize("transposed", [False, True])
def test_conversion_reproduces_the_convolution_on_the_oracle(transposed):
    maps, sizes, x, w = layer(1, 7, 90, 70, 16, 24, transposed)
    buckets, m, pairs = sc.ell3d_from_maps(maps, sizes, transposed, 90, 70)
    assert m == 70 and pairs == sum(sizes) and len(buckets) == 1
    a, rows, cols, mid = buckets[0]
    assert a.shape[1:] == (128, 1) and rows.shape[1] == 128 and mid.shape == (a.shape[0],)
    assert int(a.astype(np.int64).sum()) == pairs            # every pair is one ELL row of width 1
    assert np.all(np.diff(mid) >= 0) and set(mid.tolist()) <= set(range(7)) - {1}
    got = orc.rgms_ell3d_f16(w, x, np.zeros((m, 24), np.float32),
                             [(a.astype(np.float32), rows, cols, mid)], 16, 24)
    np.testing.assert_allclose(got, gather_matmul_scatter(x, w, maps, sizes, transposed, 70), rtol=1e-2, atol=1e-3)


def test_maps_are_validated():
    maps, sizes, x, w = layer(2, 3, 20, 20, 16, 16, False)
    with pytest.raises(ValueError, match="beyond the given number"):
        sc.ell3d_from_maps(maps, sizes, False, 20, 5)
    with pytest.raises(ValueError, match="more pairs"):
        sc.ell3d_from_maps(maps, [len(maps), 1, 0], False, 20, 20)
    with pytest.raises(ValueError, match=r"\[pairs, 2\]"):
        sc.ell3d_from_maps(maps.reshape(-1), sizes, False, 20, 20)


@pytest.mark.gpu
@pytest.mark.parametrize("feat_in,feat_out,transposed,out_dtype,repeats", [
    (64, 128, False, torch.float16, True),      # tensor-core form with reductions into Y
    (64, 128, False, torch.float32, False),     # no repeated pair: the destination-stationary form
    (128, 64, True, torch.float16, True),       # a transposed layer
    (32, 96, False, torch.float32, True),       # a shape the CUDA-core transform takes
])
def test_sparse_conv_matches_gather_matmul_scatter(cuda_device, feat_in, feat_out, transposed, out_dtype, repeats):
    n_in, n_out = (5000, 4200) if not transposed else (4200, 5000)
    maps, sizes, x, w = layer(feat_in + feat_out, 27, n_in, n_out, feat_in, feat_out, transposed, repeats, fill=0.6)
    want = gather_matmul_scatter(x, w, maps, sizes, transposed, n_out)
    xd = torch.from_numpy(x).to(cuda_device)
    wd = torch.from_numpy(w).to(cuda_device)
    y = sc.sparse_conv(xd, wd, torch.from_numpy(maps).to(cuda_device), sizes, transposed, num_outputs=n_out,
                       out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert y.shape == (n_out, feat_out) and y.dtype == out_dtype
    # fp16 operands, fp32 sums: rtol 1e-2; a float16 result also rounds every addition into Y
    np.testing.assert_allclose(y.float().cpu().numpy(), want, rtol=1e-2,
                               atol=2e-2 if out_dtype == torch.float32 else 6e-2)
    # a plan is reusable: same layer, other features, accumulated into a given output
    plan = sc.SparseConvPlan(maps, sizes, transposed, n_in, n_out, device=cuda_device)
    x2 = torch.from_numpy(np.random.default_rng(9).uniform(-1, 1, size=x.shape).astype(np.float16)).to(cuda_device)
    out = torch.ones(n_out, feat_out, dtype=out_dtype, device=cuda_device)
    plan(x2, wd, out=out)
    torch.cuda.synchronize()
    want2 = 1.0 + gather_matmul_scatter(x2.cpu().numpy(), w, maps, sizes, transposed, n_out)
    np.testing.assert_allclose(out.float().cpu().numpy(), want2, rtol=1e-2,
                               atol=2e-2 if out_dtype == torch.float32 else 6e-2)
