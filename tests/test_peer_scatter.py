"""sparsetir_peer_scatter: one block stored to several destinations by one kernel.  On one GPU the
"peers" are other buffers of the same device — the kernel only sees device pointers — which covers
the address arithmetic (16-byte body, ragged head and tail, destinations out of phase with the
source); the NVLink path proper runs in the sharded bench on more than one GPU."""
import ctypes

import pytest
import torch

from sparsetir_b200 import _lib as L

pytestmark = pytest.mark.gpu


def scatter(src, dsts, device):
    arr = (ctypes.c_void_p * len(dsts))(*[d.data_ptr() for d in dsts])
    st = torch.cuda.current_stream(device).cuda_stream
    return L.load().sparsetir_peer_scatter(device.index, ctypes.c_void_p(st), ctypes.c_void_p(src.data_ptr()),
                                           src.numel() * src.element_size(), len(dsts), arr)


@pytest.mark.parametrize("numel", [1, 3, 4, 1000, 4099, 1 << 20, (1 << 22) + 7])
@pytest.mark.parametrize("src_off,dst_off", [(0, 0), (1, 1), (3, 3), (0, 2), (1, 0)])
def test_block_reaches_every_destination(cuda_device, numel, src_off, dst_off):
    g = torch.Generator(device="cpu").manual_seed(numel + 7 * src_off + dst_off)
    base = torch.randint(-2**31, 2**31 - 1, (numel + 8,), dtype=torch.int32, generator=g).to(cuda_device)
    src = base[src_off:src_off + numel]
    pads = [torch.full((numel + 16,), -7, dtype=torch.int32, device=cuda_device) for _ in range(3)]
    dsts = [p[4 + dst_off:4 + dst_off + numel] for p in pads]
    assert scatter(src, dsts, cuda_device) == 0, L.last_error()
    torch.cuda.synchronize()
    for p, d in zip(pads, dsts):
        assert torch.equal(d, src)
        # nothing outside the block was touched
        assert bool((p[:4 + dst_off] == -7).all()) and bool((p[4 + dst_off + numel:] == -7).all())


def test_argument_checks(cuda_device):
    src = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    dst = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    lib = L.load()
    st = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    arr = (ctypes.c_void_p * 1)(dst.data_ptr())
    # nothing to do
    assert lib.sparsetir_peer_scatter(cuda_device.index, st, ctypes.c_void_p(src.data_ptr()), 0, 1, arr) == 0
    assert lib.sparsetir_peer_scatter(cuda_device.index, st, ctypes.c_void_p(src.data_ptr()), 64, 0, arr) == 0
    # a byte count that is not whole words, too many peers, a null destination
    assert lib.sparsetir_peer_scatter(cuda_device.index, st, ctypes.c_void_p(src.data_ptr()), 6, 1, arr) == -1
    assert "4-byte" in L.last_error()
    assert lib.sparsetir_peer_scatter(cuda_device.index, st, ctypes.c_void_p(src.data_ptr()), 64, 99, arr) == -1
    assert "peers" in L.last_error()
    null = (ctypes.c_void_p * 1)(None)
    assert lib.sparsetir_peer_scatter(cuda_device.index, st, ctypes.c_void_p(src.data_ptr()), 64, 1, null) == -1
    assert "null" in L.last_error()


# ---- hyb SpMM that stores its rows to the peers' copies as well (sparsetir_hyb_spmm_peers)

def _hyb_case(device, n, max_deg, buckets, feat, seed):
    import numpy as np
    import test_gpu_ops as T
    from sparsetir_b200 import datagen as dg
    c = dg.csr_powerlaw(n=n, max_deg=max_deg, seed=seed)
    host, devb = T.hyb_device_buckets(c, 1, buckets, device)
    x = dg.dense_operand(seed + 1, c.n, feat)
    want = T.oracle_hyb(host, x, c.m)
    return c, devb, torch.from_numpy(x).to(device).reshape(-1), want


@pytest.mark.parametrize("feat", [32, 64, 128, 512])
@pytest.mark.parametrize("buckets", [[1, 2, 4, 8, 16, 32, 64, 128, 256, 512], [1, 2, 4], [8, 16]])
def test_hyb_spmm_peers_writes_every_copy(cuda_device, feat, buckets):
    # split rows (degrees beyond the widest bucket), narrow and wide buckets; every copy must equal
    # the plain call bit for bit, and the plain call the oracle
    import numpy as np
    import test_gpu_ops as T
    from sparsetir_b200 import ops
    c, devb, x, want = _hyb_case(cuda_device, 5000, 3000, buckets, feat, seed=len(buckets) + feat)
    y_plain = torch.zeros(c.m * feat, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(x, y_plain, devb, feat))
    y = torch.zeros(c.m * feat, device=cuda_device)
    # two "peers": buffers of this GPU, one of them the middle of a larger array
    big = torch.full((3 * c.m * feat,), 7.0, device=cuda_device)
    copies = [torch.zeros(c.m * feat, device=cuda_device), big[c.m * feat:2 * c.m * feat]]
    ops.hyb_spmm_peers(*ops.hyb_args(x, y, devb, feat, 0, peer_c=[t.data_ptr() for t in copies]))
    torch.cuda.synchronize()
    assert torch.equal(y, y_plain)
    # rows that occur in no bucket are not written anywhere: compare the rows that are
    written = np.zeros(c.m, bool)
    for _, rows, _ in devb:
        written[rows.cpu().numpy()] = True
    w = torch.from_numpy(np.repeat(written, feat)).to(cuda_device)
    for t in copies:
        assert torch.equal(t[w], y[w])
    assert bool((copies[0][~w] == 0).all()) and bool((copies[1][~w] == 7.0).all())
    assert bool((big[:c.m * feat] == 7.0).all()) and bool((big[2 * c.m * feat:] == 7.0).all())
    T.close(y, want)


def test_hyb_spmm_peers_refuses_what_it_cannot_do(cuda_device):
    from sparsetir_b200 import ops
    c, devb, x, _ = _hyb_case(cuda_device, 300, 40, [1, 2, 4, 8, 16, 32, 64], 32, seed=3)
    y = torch.zeros(c.m * 32, device=cuda_device)
    other = torch.zeros(c.m * 32, device=cuda_device)
    with pytest.raises(ops.SparseTIRError, match="one-writer"):
        ops.hyb_spmm_peers(*ops.hyb_args(x, y, devb, 32, L.HYB_ALL_ATOMIC, peer_c=[other.data_ptr()]))
    with pytest.raises(ops.SparseTIRError, match="peer"):
        ops.hyb_spmm_peers(*ops.hyb_args(x, y, devb, 32, 0, peer_c=[]))
    with pytest.raises(ops.SparseTIRError, match="aligned"):
        ops.hyb_spmm_peers(*ops.hyb_args(x, y, devb, 32, 0, peer_c=[other.data_ptr() + 4]))


# ---- SDDMM that stores its positions to the peers' copies as well (sparsetir_sddmm_peers)

@pytest.mark.parametrize("feat,with_scale", [(32, False), (64, True), (128, False), (320, True), (512, False)])
def test_sddmm_peers_writes_every_copy(cuda_device, feat, with_scale):
    # 320 and 512 features take several feature-tile passes: only the last pass's value may reach
    # the copies
    import numpy as np
    import test_gpu_ops as T
    from sparsetir_b200 import datagen as dg, ops
    c = dg.csr_lognormal(n=900, mu=3.0, sigma=1.0, max_deg=500, seed=feat)
    a = dg.dense_operand(1, c.m, feat)
    b = dg.dense_operand(2, c.n, feat)
    scale = np.random.default_rng(feat).random(c.nnz, dtype=np.float32) if with_scale else None
    plain = T.run_sddmm(c, a, b, cuda_device, scale=scale)
    out = torch.full((c.nnz,), -7.0, device=cuda_device)
    big = torch.full((c.nnz + 10,), 3.0, device=cuda_device)
    copies = [torch.full((c.nnz,), -1.0, device=cuda_device), big[5:5 + c.nnz]]  # the second 4-byte aligned only
    args = [T.dev(a.reshape(-1), cuda_device), T.dev(b.reshape(-1), cuda_device), out,
            T.dev(c.indptr, cuda_device), T.dev(c.indices, cuda_device)] + [t.data_ptr() for t in copies]
    if scale is not None:
        args.append(T.dev(scale, cuda_device))
    ops.sddmm_peers(*args)
    torch.cuda.synchronize()
    assert torch.equal(out, plain)
    for t in copies:
        assert torch.equal(t, out)
    assert bool((big[:5] == 3.0).all()) and bool((big[5 + c.nnz:] == 3.0).all())


def test_sddmm_peers_refuses_what_it_cannot_do(cuda_device):
    import test_gpu_ops as T
    from sparsetir_b200 import datagen as dg, ops
    c = dg.csr_lognormal(n=200, mu=2.0, sigma=1.0, max_deg=100, seed=1)
    feat = 20  # not a multiple of 32: no peer stores in the kernels that take it
    a, b = dg.dense_operand(1, c.m, feat), dg.dense_operand(2, c.n, feat)
    out = torch.zeros(c.nnz, device=cuda_device)
    other = torch.zeros(c.nnz, device=cuda_device)
    base = [T.dev(a.reshape(-1), cuda_device), T.dev(b.reshape(-1), cuda_device), out,
            T.dev(c.indptr, cuda_device), T.dev(c.indices, cuda_device)]
    with pytest.raises(ops.SparseTIRError, match="multiple of 32"):
        ops.sddmm_peers(*base, other.data_ptr())
    with pytest.raises(ops.SparseTIRError, match="peer"):
        ops.sddmm_peers(*base)


# ---- random shapes: the peer-storing forms against the plain calls, bit for bit

@pytest.mark.parametrize("seed", range(24))
def test_fuzz_hyb_spmm_peers_equals_plain_call(cuda_device, seed):
    import numpy as np
    import test_gpu_fuzz as F
    import test_gpu_ops as T
    from sparsetir_b200 import datagen as dg, ops
    rng = np.random.default_rng(7000 + seed)
    n = int(rng.integers(2, 3000))
    c = F.random_csr(rng, n, n)
    feat = int(rng.choice([32, 64, 96, 128, 160, 256, 512]))
    nb = int(rng.integers(1, 8))
    buckets = sorted(set(int(b) for b in rng.choice([1, 2, 4, 8, 16, 24, 32, 64, 128, 256, 512], size=nb)))
    x = T.dev(dg.dense_operand(seed, n, feat), cuda_device).reshape(-1)
    _, devb = T.hyb_device_buckets(c, 1, buckets, cuda_device)
    plain = torch.zeros(c.m * feat, device=cuda_device)
    ops.hyb_spmm(*ops.hyb_args(x, plain, devb, feat))
    y = torch.zeros(c.m * feat, device=cuda_device)
    copies = [torch.zeros(c.m * feat, device=cuda_device) for _ in range(int(rng.integers(1, 4)))]
    try:
        ops.hyb_spmm_peers(*ops.hyb_args(x, y, devb, feat, 0, peer_c=[t.data_ptr() for t in copies]))
    except ops.SparseTIRError as e:
        # a feature count that is not a whole number of the kernel's tiles (96, 160): refused
        # before any launch, nothing written
        assert "one-writer" in str(e) and feat in (96, 160)
        torch.cuda.synchronize()
        assert not bool(y.any()) and not any(bool(t.any()) for t in copies)
        return
    torch.cuda.synchronize()
    assert torch.equal(y, plain)
    for t in copies:  # rows in no bucket stay zero in all of them
        assert torch.equal(t, plain)


@pytest.mark.parametrize("seed", range(12))
def test_fuzz_sddmm_peers_equals_plain_call(cuda_device, seed):
    import numpy as np
    import test_gpu_fuzz as F
    import test_gpu_ops as T
    from sparsetir_b200 import datagen as dg, ops
    rng = np.random.default_rng(8000 + seed)
    m, n = int(rng.integers(1, 2000)), int(rng.integers(1, 2000))
    c = F.random_csr(rng, m, n)
    if c.nnz == 0:
        pytest.skip("no stored position")
    feat = int(rng.choice([32, 64, 96, 128, 256, 288, 512]))
    a, b = dg.dense_operand(seed, m, feat), dg.dense_operand(seed + 1, n, feat)
    plain = T.run_sddmm(c, a, b, cuda_device)
    out = torch.full((c.nnz,), -7.0, device=cuda_device)
    copies = [torch.full((c.nnz,), -1.0, device=cuda_device) for _ in range(int(rng.integers(1, 4)))]
    ops.sddmm_peers(T.dev(a.reshape(-1), cuda_device), T.dev(b.reshape(-1), cuda_device), out,
                    T.dev(c.indptr, cuda_device), T.dev(c.indices, cuda_device), *[t.data_ptr() for t in copies])
    torch.cuda.synchronize()
    assert torch.equal(out, plain)
    for t in copies:
        assert torch.equal(t, plain)


def test_hyb_spmm_peers_with_32_byte_lanes_selected_in_child_process(cuda_device):
    # SPARSETIR_LANE_FLOATS=8 selects 32-byte lanes for the plain call; the peer-storing form keeps
    # 16-byte lanes and must still agree with the oracle (split rows included)
    import subprocess
    import sys
    code = r'''
import os, sys
sys.path.insert(0, os.path.join(os.getcwd(), "tests"))
import numpy as np, torch
import test_gpu_ops as T
from sparsetir_b200 import datagen as dg, ops
dev = torch.device("cuda", 0)
for feat in (32, 64, 128):
    c = dg.csr_powerlaw(n=5000, max_deg=3000, seed=10 + feat)
    host, devb = T.hyb_device_buckets(c, 1, T.BK10, dev)
    xh = dg.dense_operand(1, c.n, feat)
    x = torch.from_numpy(xh).to(dev).reshape(-1)
    y = torch.zeros(c.m * feat, device=dev)
    cp = torch.zeros(c.m * feat, device=dev)
    ops.hyb_spmm_peers(*ops.hyb_args(x, y, devb, feat, 0, peer_c=[cp.data_ptr()]))
    torch.cuda.synchronize()
    assert torch.equal(y, cp)
    T.close(y, T.oracle_hyb(host, xh, c.m))
print("ok")
'''
    import os
    env = dict(os.environ, SPARSETIR_LANE_FLOATS="8")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
