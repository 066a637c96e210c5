"""coconet_b200: B200-native runtime for CoCoNet's fused AllReduce optimizer
step (ReduceScatter of gradients -> sliced SGD/Adam/LAMB update -> AllGather of
weights as one sm_100a kernel over NVLink peer memory).

The product is the C-ABI shared library `libcoconet_rt.so` (declared in
include/coconet_rt.h) and the DSL code generator under `dsl/`; this Python
package is a thin ctypes host layer over the library for tests and benchmarks.
There is no CPU fallback: everything raises if the library is missing.
"""
from .runtime import (  # noqa: F401
    CocoError,
    Communicator,
    HostBootstrap,
    TensorList,
    VARIANT_DSL,
    VARIANT_NCCL,
    VARIANT_OVERLAP,
    LAMB_REF_QUIRK,
    group,
    lib,
    library_path,
    rendezvous_address,
    scattered_slice_elems,
    scattered_tensor_place,
    slice_bounds,
    topology_check,
)

__all__ = [
    "CocoError", "Communicator", "HostBootstrap", "TensorList", "VARIANT_DSL", "VARIANT_NCCL", "VARIANT_OVERLAP",
    "LAMB_REF_QUIRK", "group", "lib", "library_path", "rendezvous_address", "scattered_slice_elems", "scattered_tensor_place",
    "slice_bounds", "topology_check",
]
