"""Seeded synthetic inputs for the five benchmark configurations of this path.

No dataset is involved: the shapes are the ones the headline metric is quoted on, the value
distributions are those the configurations name (uniform[-1,1], N(0,1), He-normal, ...), and
every tensor comes from its own ``torch.Generator`` seed ``20251125 + 1000*config + index``
so that a CPU oracle and a GPU run see bit-identical inputs.  Everything is FP32, dense,
row-major; ``scale`` shrinks a configuration proportionally for quick parity runs.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

BASE_SEED = 20251125


def _gen(config: int, index: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(BASE_SEED + 1000 * config + index)
    return g


def uniform_pm1(shape, config, index):
    return torch.rand(shape, generator=_gen(config, index), dtype=torch.float32) * 2.0 - 1.0


def normal(shape, config, index, std=1.0):
    return torch.randn(shape, generator=_gen(config, index), dtype=torch.float32) * std


@dataclass
class MatMulCase:
    """C[N,M] from A and B in the layout of `form` ('AB': A[N,K] B[K,M]; 'T1': A[K,N] B[K,M];
    'T2': A[N,K] B[M,K]); reference letters."""
    form: str
    N: int
    M: int
    K: int
    A: torch.Tensor
    B: torch.Tensor

    @property
    def flops(self) -> float:
        return 2.0 * self.N * self.M * self.K

    @property
    def algorithmic_bytes(self) -> float:
        return 4.0 * (self.N * self.K + self.K * self.M + self.N * self.M)


def matmul_case(form: str, N: int, M: int, K: int, config: int, dist: str = "uniform", std: float = 1.0):
    shapes = {"AB": ((N, K), (K, M)), "T1": ((K, N), (K, M)), "T2": ((N, K), (M, K))}[form]
    if dist == "uniform":
        A, B = uniform_pm1(shapes[0], config, 0), uniform_pm1(shapes[1], config, 1)
    else:
        A, B = normal(shapes[0], config, 0, std), normal(shapes[1], config, 1, std)
    return MatMulCase(form, N, M, K, A, B)


def config1():
    """FP32 matMul C = A*B, M=N=K=1024, uniform[-1,1]."""
    return matmul_case("AB", 1024, 1024, 1024, 1)


def config2(form: str = "AB", size: int = 8192):
    """FP32 matMul, one of the three forms, M=N=K=8192, uniform[-1,1]."""
    return matmul_case(form, size, size, size, 2)


def config2_ragged(form: str = "AB"):
    """Logical 8191 x 4097 x 3000 as the Java engine presents it: every dimension padded to a
    multiple of 4 with zero lanes (EngineCore.java:708-717), i.e. N=8192, M=4100, K=3000."""
    N, M, K = 8191, 4097, 3000
    Np, Mp, Kp = (N + 3) // 4 * 4, (M + 3) // 4 * 4, (K + 3) // 4 * 4
    c = matmul_case(form, N, M, K, 2, "uniform")
    rows = {"AB": ((Np, Kp), (Kp, Mp)), "T1": ((Kp, Np), (Kp, Mp)), "T2": ((Np, Kp), (Mp, Kp))}[form]
    A = torch.zeros(rows[0]); A[: c.A.shape[0], : c.A.shape[1]] = c.A
    B = torch.zeros(rows[1]); B[: c.B.shape[0], : c.B.shape[1]] = c.B
    out = MatMulCase(form, Np, Mp, Kp, A, B)
    out.logical = (N, M, K)
    return out


@dataclass
class AttentionCase:
    """Batched attention-shaped pair: S = Q K^T (batchMatMulT2), O = P V (batchMatMul)."""
    Batch: int
    L: int
    D: int
    Q: torch.Tensor
    K: torch.Tensor
    V: torch.Tensor

    @property
    def flops_each(self) -> float:
        return 2.0 * self.Batch * self.L * self.L * self.D

    @property
    def algorithmic_bytes_each(self) -> float:
        return 4.0 * (2 * self.Batch * self.L * self.D + self.Batch * self.L * self.L)


def config3(Batch: int = 1024, L: int = 512, D: int = 64):
    """Q, K, V [Batch, L, D] ~ N(0,1)."""
    return AttentionCase(Batch, L, D, normal((Batch, L, D), 3, 0), normal((Batch, L, D), 3, 1),
                         normal((Batch, L, D), 3, 2))


def softmax_rows(S: torch.Tensor, D: int) -> torch.Tensor:
    """P = softmax(S / sqrt(D)) computed once in FP32; P is then an *input* of the second
    contraction (the oracle uses the same FP32 P)."""
    return torch.softmax(S / (D ** 0.5), dim=-1)


@dataclass
class ConvCase:
    X: torch.Tensor  # [N, IH, IW, IC]
    W: torch.Tensor  # [OC, FH, FW, IC]
    sh: int
    sw: int
    ph: int
    pw: int

    @property
    def dims(self):
        N, IH, IW, IC = self.X.shape
        OC, FH, FW, _ = self.W.shape
        OH = (IH + 2 * self.ph - FH) // self.sh + 1
        OW = (IW + 2 * self.pw - FW) // self.sw + 1
        return dict(N=N, IH=IH, IW=IW, IC=IC, OC=OC, FH=FH, FW=FW, OH=OH, OW=OW)

    @property
    def flops(self) -> float:
        d = self.dims
        return 2.0 * d["N"] * d["OH"] * d["OW"] * d["OC"] * d["FH"] * d["FW"] * d["IC"]

    @property
    def algorithmic_bytes(self) -> float:
        d = self.dims
        return 4.0 * (self.X.numel() + self.W.numel() + d["N"] * d["OH"] * d["OW"] * d["OC"])


def config4(N: int = 256, HW: int = 28, IC: int = 256, OC: int = 256, F: int = 3):
    """NHWC input N(0,1); OCxFHxFWxIC filters He-normal (std sqrt(2/(F*F*IC))); stride 1, pad 1."""
    X = normal((N, HW, HW, IC), 4, 0)
    W = normal((OC, F, F, IC), 4, 1, (2.0 / (F * F * IC)) ** 0.5)
    return ConvCase(X, W, 1, 1, F // 2, F // 2)


def config5(K: int = 1048576, N: int = 512, M: int = 512):
    """Long-K weight-gradient shape: C[N,M] = A[K,N]^T B[K,M], entries 0.01*N(0,1)."""
    return matmul_case("T1", N, M, K, 5, "normal", 0.01)
