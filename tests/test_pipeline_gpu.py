"""The contraction kernel's pipeline plumbing: the give-up path of its bounded waits, and that neither the
shared-memory ring geometry nor the flavour of the cross-CTA barrier arrivals changes a single bit."""
import numpy as np
import pytest
import torch

import gpu_util as G

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports(pkg, cuda):
    """A wait nobody completes runs out after its limit: the kernel returns normally, the status word holds
    the give-up record, reading it clears it, and the device is as usable as before."""
    assert pkg.cu32.read_status() == 0
    pkg.cu32.selftest_wait_giveup(G.stream(), 20000)
    word = pkg.cu32.read_status()
    assert word == (7 << 24) | (1 << 16) | 42, hex(word)
    assert "self-test gave up" in pkg.cu32.decode_status(word) and "iteration 42" in pkg.cu32.decode_status(word)
    assert pkg.cu32.read_status() == 0            # cleared by the read
    with pytest.raises(pkg.cu32.CudaException):
        pkg.cu32.selftest_wait_giveup(G.stream(), 0)
    A, B = G.rand_pm1((128, 64), 1), G.rand_pm1((64, 128), 2)
    C = G.matmul(pkg, "AB", A, B, 128, 128, 64)     # asserts a clean status itself
    assert np.isfinite(C).all()


def _cases(pkg):
    A, B = G.rand_pm1((520, 1028), 1), G.rand_pm1((1028, 388), 2)
    w = pkg.workloads.config4(N=4)
    X, W = w.X.numpy(), w.W.numpy()
    Q = np.random.default_rng(3).standard_normal((6, 256, 64)).astype(np.float32)
    Kt = np.random.default_rng(4).standard_normal((6, 512, 64)).astype(np.float32)
    At, Bt = G.rand_pm1((2052, 132), 5), G.rand_pm1((2052, 260), 6)
    return {
        "matMul": lambda: G.matmul(pkg, "AB", A, B, 520, 388, 1028),
        "conv": lambda: G.conv(pkg, "conv3D_GemmR", X, W, 1, 1, 1, 1),
        "bmmT2": lambda: G.bmm_t2(pkg, Q, Kt),
        "splitK": lambda: G.matmul_sk(pkg, "T1", At, Bt, 132, 260, 2052, 4)[0],
    }


@pytest.mark.parametrize("tile", [1, 3, 4, 5])
def test_ring_geometry_does_not_change_the_result(pkg, cuda, tile):
    """More raw slots than lo slots, two store-staging tiles: same numbers in the same order."""
    cases = _cases(pkg)
    pkg.cu32.tune("tile", tile)
    base = {k: f() for k, f in cases.items()}
    slot = (128 + {1: 128, 3: 64, 4: 128, 5: 32}[tile]) * 128          # bytes one k-block brings into a CTA
    tried = 0
    for raw, lo, bufs in [(2, 1, 1), (2, 2, 2), (3, 1, 2), (3, 2, 2), (4, 2, 1), (4, 1, 2), (5, 3, 1), (6, 3, 1), (8, 2, 1), (8, 1, 2)]:
        if 1024 + (raw + lo) * slot + bufs * 32768 > 226 * 1024:
            continue
        tried += 1
        pkg.cu32.tune("ring_raw", raw); pkg.cu32.tune("ring_lo", lo); pkg.cu32.tune("store_bufs", bufs)
        for k, f in cases.items():
            for rep in range(3):
                Y = f()
                assert np.array_equal(Y, base[k]), (tile, raw, lo, bufs, k, rep, int((Y != base[k]).sum()))
    assert tried >= 3
    # the default rings through the launch-parameter path (the base ran the compile-time path), lo tiles behind
    # their raw tiles or in a ring of their own
    pkg.cu32.tune("ring_raw", 0); pkg.cu32.tune("ring_lo", 0); pkg.cu32.tune("store_bufs", 0)
    for fixed, paired in [(0, 1), (0, 0), (1, 0)]:
        pkg.cu32.tune("ring_fixed", fixed); pkg.cu32.tune("ring_paired", paired)
        for k, f in cases.items():
            Y = f()
            assert np.array_equal(Y, base[k]), (tile, "fixed", fixed, "paired", paired, k)
    pkg.cu32.tune("ring_fixed", 1); pkg.cu32.tune("ring_paired", 1)


def test_ring_geometry_that_does_not_fit_is_refused(pkg, cuda):
    pkg.cu32.tune("tile", 4)
    pkg.cu32.tune("ring_raw", 8); pkg.cu32.tune("ring_lo", 8)
    A, B = G.dev(G.rand_pm1((256, 64), 1)), G.dev(G.rand_pm1((64, 256), 2))
    C = torch.zeros((256, 256), device="cuda")
    with pytest.raises(pkg.cu32.CudaException) as ei:
        pkg.cu32.Cuda_matMul.matMul([G.stream()], 1, A.data_ptr(), B.data_ptr(), C.data_ptr(), 256, 256, 64)
    assert ei.value.code == 1      # cudaErrorInvalidValue: nothing was launched
    torch.cuda.synchronize()
    assert bool((C == 0).all())
    pkg.cu32.tune("ring_raw", 0); pkg.cu32.tune("ring_lo", 0)
    assert pkg.cu32.read_status() == 0


def test_pair_tiles_match_the_single_cta_tile_with_either_arrive(pkg, cuda):
    """CTA-pair tiles hand operands and TMEM buffers over between two CTAs with remote barrier arrivals; the
    single-CTA tile has no such hand-over.  Same bits on the convolution, its data gradient, split-K and the
    batched form, with the default arrive and with the cluster-scope-release one."""
    cases = _cases(pkg)
    rng = np.random.default_rng(8)
    dY = rng.standard_normal((4, 14, 14, 64)).astype(np.float32)
    Wf = (rng.standard_normal((64, 3, 3, 128)) * 0.05).astype(np.float32)
    dx = pkg.cu32.Cuda_dconv3D_deltaX

    def deltax():
        ddY, dW = G.dev(dY), G.dev(Wf)
        out = G.Out(4 * 14 * 14 * 128)
        dx.dconv3D_deltaX_s1([G.stream()], 1, ddY.data_ptr(), 14, 14, dW.data_ptr(), 3, 3, out.ptr, 14, 14, 4, 128, 64, 1, 1)
        Y = out.host((4, 14, 14, 128))
        G.check_status(pkg)
        return Y
    cases["deltaX"] = deltax
    pkg.cu32.tune("tile", 2)
    base = {k: f() for k, f in cases.items()}
    for tile in (3, 4, 5):
        pkg.cu32.tune("tile", tile)
        for release in (0, 1):
            pkg.cu32.tune("arrive_release", release)
            for k, f in cases.items():
                for rep in range(4):
                    Y = f()
                    assert np.array_equal(Y, base[k]), (tile, release, k, rep, int((Y != base[k]).sum()))


def test_replicated_stores_write_every_copy(pkg, cuda):
    """cu32_matMul_replicated repeats each store of the product to further buffers (on several GPUs: the peers'
    copies of a gathered output; here all local).  Every copy equals the plain product bit for bit, canaries
    around each copy stay intact, and a request the tensor-map store path cannot serve is refused."""
    mm = pkg.cu32.Cuda_matMul
    # shapes: ragged edges; one tile; fewer rows than a tile; more tiles than CTA pairs (a block is carried to the
    # copies while the next tile is multiplied); a reduction long enough to leave the registers twice
    shapes = [(520, 388, 260), (256, 256, 64), (132, 68, 96), (2308, 2304, 160), (260, 516, 8192 + 96)]
    for form, fn in (("AB", mm.matMul_replicated), ("T2", mm.matMulT2_replicated)):
        for (N, M, K) in shapes:
            sa, sb = G.mm_shapes(form, N, M, K)
            A, B = G.rand_pm1(sa, 11), G.rand_pm1(sb, 12)
            base = G.matmul(pkg, form, A, B, N, M, K)
            dA, dB = G.dev(A), G.dev(B)
            for lazy in (1, 0):     # copies carried over from C between drains / every store repeated at once
                pkg.cu32.tune("rep_lazy", lazy)
                for n_rep in ((0, 1, 3, 7) if N * M < 1 << 20 else (2, 7)):
                    outs = [G.Out(N * M) for _ in range(n_rep + 1)]
                    fn([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), outs[0].ptr, [o.ptr for o in outs[1:]], N, M, K)
                    for i, o in enumerate(outs):
                        assert np.array_equal(o.host((N, M)), base), (form, N, M, K, lazy, n_rep, i)
                    G.check_status(pkg)
            pkg.cu32.tune("rep_lazy", 1)
    dA, dB = G.dev(G.rand_pm1((64, 64), 1)), G.dev(G.rand_pm1((64, 64), 2))
    out = G.Out(64 * 64)
    with pytest.raises(pkg.cu32.CudaException) as ei:
        mm.matMul_replicated([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, [out.ptr + 4], 64, 64, 64)
    assert ei.value.code == -4      # a copy that is not 16-byte aligned
    with pytest.raises(pkg.cu32.CudaException) as ei:
        mm.matMul_replicated([G.stream()], 1, dA.data_ptr(), dB.data_ptr(), out.ptr, [out.ptr] * 8, 64, 64, 64)
    assert ei.value.code == -8      # more than seven copies
