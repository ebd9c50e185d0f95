"""In-tree build of the native engine:  python setup.py build_ext --inplace

Produces pccl_b200/engine_c*.so next to the Python sources.  Device code is
compiled for sm_100a only (-gencode arch=compute_100a,code=sm_100a).
"""

import glob
import os

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("pccl_b200", "csrc")

sources = sorted(glob.glob(os.path.join(CSRC, "**", "*.cc"), recursive=True)
                 + glob.glob(os.path.join(CSRC, "**", "*.cu"), recursive=True))

os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")

# The verbs transport of the RDMA executor is opt-in (PCCL_RDMA=1) and needs the verbs headers.
RDMA = os.environ.get("PCCL_RDMA", "0") == "1" and os.path.exists("/usr/include/infiniband/verbs.h")
rdma_macros = [("PCCL_RDMA_ENABLED", None)] if RDMA else []
rdma_libs = ["ibverbs"] if RDMA else []

setup(
    name="pccl_b200",
    version="0.3.0",
    packages=["pccl_b200", "pccl"],
    ext_modules=[
        CUDAExtension(
            name="pccl_b200.engine_c",
            sources=sources,
            include_dirs=[os.path.join(ROOT, CSRC)],
            define_macros=rdma_macros,
            libraries=rdma_libs,
            # Link the shared libstdc++ explicitly: on images whose compiler directory holds only
            # libstdc++.a the driver would otherwise embed a second, uninitialised copy of the
            # iostream/locale state into the extension.
            extra_link_args=[p for p in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6",) if os.path.exists(p)],
            extra_compile_args={
                "cxx": ["-std=c++17", "-O2", "-fvisibility=hidden", "-Wall", "-Wno-unknown-pragmas"],
                "nvcc": ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
                         "-gencode", "arch=compute_100a,code=sm_100a"],
            },
        )
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
