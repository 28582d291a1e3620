"""dragon-alpha-v1.2_b200: B200-native dense contractions behind Dragon-Alpha's Cu32 native API.

The directory name is not a valid Python identifier; load it with
``importlib`` under the alias ``dragon_b200`` (see ``__graft_entry__.load_package``).

Modules
-------
build    nvcc recipe for ``libdragon_cu32.so``
cu32     ctypes binding that mirrors the Java native classes ``Cuda_matMul``,
         ``Cuda_batchMatMul`` and ``Cuda_conv3D`` (same method names and argument order)
engine   host-side mirror of the parts of ``CudaFloat32EngineBase`` that call those
         natives (split-K decision, stream count, padded dimensions)
shard    one-process-per-GPU sharding of the three operator families
workloads seeded synthetic inputs of the benchmark configurations
"""
from . import build, cu32, engine, shard, workloads  # noqa: F401

__all__ = ["build", "cu32", "engine", "shard", "workloads"]
