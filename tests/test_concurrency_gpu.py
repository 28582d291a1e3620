"""The library is called from several Java threads at once, each with its own streams
(CudaFloat32EngineBase hands every operation a stream array from a pool; Syncer threads run in the
background).  Host side: no shared mutable state without atomics.  Device side: every launch is a persistent
grid that fills the GPU, so concurrent launches take turns SM by SM and must neither deadlock nor disturb
each other's results."""
import threading

import numpy as np
import pytest

import gpu_util as G

pytestmark = pytest.mark.gpu


def test_concurrent_host_threads_on_their_own_streams(pkg, O, cuda):
    torch = cuda
    mm, cv = pkg.cu32.Cuda_matMul, pkg.cu32.Cuda_conv3D
    rng = np.random.default_rng(71)
    jobs = []
    for i in range(6):
        N, M, K = 260 + 128 * i, 516 - 64 * i, 1028 + 256 * i
        A = rng.standard_normal((N, K)).astype(np.float32)
        B = rng.standard_normal((K, M)).astype(np.float32)
        jobs.append(("mm", A, B, N, M, K))
    X = rng.standard_normal((8, 20, 20, 64)).astype(np.float32)
    W = (rng.standard_normal((72, 3, 3, 64)) * 0.05).astype(np.float32)
    jobs.append(("conv", X, W))
    jobs.append(("conv", X[:4], W))
    results, errors = {}, []

    def work(idx, job):
        try:
            torch.cuda.set_device(0)
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for rep in range(8):
                    if job[0] == "mm":
                        _, A, B, N, M, K = job
                        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
                        dC = torch.full((N, M), float("nan"), device="cuda")
                        st.synchronize()
                        mm.matMul([st.cuda_stream], 1, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), N, M, K)
                    else:
                        _, X_, W_ = job
                        n = X_.shape[0]
                        dX, dW = torch.from_numpy(X_).cuda(), torch.from_numpy(W_).cuda()
                        dCW = torch.empty(W_.size, device="cuda")
                        dC = torch.full((n, 20, 20, 72), float("nan"), device="cuda")
                        st.synchronize()
                        cv.kernel_remode(st.cuda_stream, dW.data_ptr(), dCW.data_ptr(), 3, 3, 72, 64)
                        cv.conv3D_GemmR([st.cuda_stream], 1, dX.data_ptr(), 20, 20, dW.data_ptr(), dCW.data_ptr(), 3, 3,
                                        dC.data_ptr(), 20, 20, n, 64, 72, 1, 1, 1, 1)
                    st.synchronize()
                    out = dC.cpu().numpy()
                    if rep == 0:
                        results[idx] = out
                    elif not np.array_equal(out, results[idx]):
                        errors.append((idx, rep, "result changed between repetitions"))
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append((idx, repr(e)))

    threads = [threading.Thread(target=work, args=(i, j)) for i, j in enumerate(jobs)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads), "a thread is stuck"
    assert not errors, errors
    G.check_status(pkg)
    for i, job in enumerate(jobs):
        if job[0] == "mm":
            want = O.f64.matMul(job[1], job[2])
        else:
            want = O.f64.conv3D(job[1], job[2], 20, 20, 1, 1, 1, 1)
        rep = O.report(results[i], want)
        assert rep["frob"] <= 1e-6 and rep["elem"] <= 1e-4, (i, rep)
