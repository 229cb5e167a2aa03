"""TEST INFRASTRUCTURE. A ``Launcher`` over the reference's own card kernels, compiled for sm_100a from the
reference's sources into ``oracle/_ref/btb_kernels.fatbin`` by ``oracle/build_ref.sh``.

It does what btb's ``_Cuda.launch`` does (btb/engine/native.py:1405-1442 of btb): load the module with the driver API,
look a kernel up by name, ``cuLaunchKernel`` on the current torch stream with one ctypes value per parameter. The
GPU tests drive the same typed launcher calls against this object and against ``B200Launcher`` and compare bits.
"""

from __future__ import annotations

import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FATBIN = os.path.join(ROOT, "oracle", "_ref", "btb_kernels.fatbin")


def available() -> bool:
    return os.path.exists(FATBIN)


class RefLauncher:
    def __init__(self) -> None:
        import torch

        torch.cuda.init()
        torch.zeros(1, device="cuda")  # the primary context, current
        self.cu = C.CDLL("libcuda.so.1")
        self.cu.cuInit(0)
        data = open(FATBIN, "rb").read()
        self._image = C.create_string_buffer(data, len(data))
        self.mod = C.c_void_p()
        self._ck(self.cu.cuModuleLoadData(C.byref(self.mod), self._image), "cuModuleLoadData")
        self.fn: dict[str, C.c_void_p] = {}

    def _ck(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what}: CUDA driver error {rc}")

    def function(self, name: str) -> C.c_void_p:
        if name not in self.fn:
            f = C.c_void_p()
            self._ck(self.cu.cuModuleGetFunction(C.byref(f), self.mod, name.encode()), f"cuModuleGetFunction {name}")
            self.fn[name] = f
        return self.fn[name]

    def launch(self, name, grid, block, args, stream=None, shared=0) -> None:
        import torch

        f = self.function(name)
        vals = list(args)
        params = (C.c_void_p * len(vals))(*[C.cast(C.byref(v), C.c_void_p) for v in vals])
        s = torch.cuda.current_stream() if stream is None else stream
        self._ck(
            self.cu.cuLaunchKernel(
                f, C.c_uint(grid[0]), C.c_uint(grid[1]), C.c_uint(grid[2]), C.c_uint(block[0]), C.c_uint(block[1]),
                C.c_uint(block[2]), C.c_uint(shared), C.c_void_p(s.cuda_stream), params, None,
            ),
            f"cuLaunchKernel {name}",
        )  # fmt: skip
