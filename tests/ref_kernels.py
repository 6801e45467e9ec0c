"""Launcher for the reference's own CUDA kernels (test infrastructure only).

`make -C oracle ref` compiles crates/cuda-native-runtime/kernels/native_kernels.cu of the reference checkout,
unchanged, into oracle/_ref/native_kernels.fatbin.  This module loads that fat binary the way the reference's
runtime does (cuModuleLoadData, lookup by unmangled name: crates/cuda-native-runtime/src/runtime.rs:253-264,
367-376) and launches kernels with the reference's parameter packets: every slice is two parameters
(device pointer, u64 length), every scalar one, in order (crates/gpu-runtime/src/lib.rs:96-133); dynamic shared
memory is always 0; `cfg_1d(n)` is ceil(n / 256) blocks of 256 threads
(bins/nnue_train/src/trainer_common.rs:416-422).

Device memory is torch's (plumbing).  Nothing in the product package imports this file.
"""
from __future__ import annotations

import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FATBIN = os.path.join(ROOT, "oracle", "_ref", "native_kernels.fatbin")


def available() -> bool:
    return os.path.exists(FATBIN)


class U32(int):
    pass


class I32(int):
    pass


class U64(int):
    pass


class F32(float):
    pass


class Slice:
    """A slice argument with an explicit element count (e.g. an empty slice over a dummy allocation)."""

    def __init__(self, tensor, length):
        self.tensor, self.length = tensor, length


class RefKernels:
    def __init__(self, device: int = 0):
        import torch
        from cuda.bindings import driver as drv
        self.torch, self.drv = torch, drv
        torch.cuda.set_device(device)
        torch.zeros(1, device="cuda")          # makes the primary context current on this thread
        with open(FATBIN, "rb") as f:
            self._image = f.read()
        err, self.module = drv.cuModuleLoadData(self._image)
        self._ok(err, "cuModuleLoadData")
        self._fn = {}

    def _ok(self, err, what):
        if int(err) != 0:
            raise RuntimeError("%s failed: %s" % (what, err))

    def function(self, name):
        if name not in self._fn:
            err, fn = self.drv.cuModuleGetFunction(self.module, name.encode())
            self._ok(err, "cuModuleGetFunction(%s)" % name)
            self._fn[name] = fn
        return self._fn[name]

    def launch(self, name, grid, block, *args, stream=0):
        """args: torch tensors (passed as pointer + element count) or U32 / I32 / U64 / F32 scalars."""
        vals = []
        for a in args:
            if isinstance(a, self.torch.Tensor):
                assert a.is_cuda and a.is_contiguous()
                vals.append(C.c_void_p(a.data_ptr()))
                vals.append(C.c_ulonglong(a.numel()))
            elif isinstance(a, Slice):
                vals.append(C.c_void_p(a.tensor.data_ptr()))
                vals.append(C.c_ulonglong(a.length))
            elif isinstance(a, U32):
                vals.append(C.c_uint(int(a)))
            elif isinstance(a, I32):
                vals.append(C.c_int(int(a)))
            elif isinstance(a, U64):
                vals.append(C.c_ulonglong(int(a)))
            elif isinstance(a, F32):
                vals.append(C.c_float(float(a)))
            else:
                raise TypeError("untyped kernel argument %r" % (a,))
        ptrs = (C.c_void_p * len(vals))(*[C.addressof(v) for v in vals])
        g = tuple(grid) + (1,) * (3 - len(tuple(grid))) if not isinstance(grid, int) else (grid, 1, 1)
        b = tuple(block) + (1,) * (3 - len(tuple(block))) if not isinstance(block, int) else (block, 1, 1)
        err, = self.drv.cuLaunchKernel(self.function(name), g[0], g[1], g[2], b[0], b[1], b[2], 0, stream,
                                       C.addressof(ptrs), 0)
        self._ok(err, "cuLaunchKernel(%s)" % name)

    def launch_1d(self, name, n, *args, stream=0):
        self.launch(name, (n + 255) // 256, 256, *args, stream=stream)

    # ---- the reference's launch sequences ------------------------------------------------------------------
    def sparse_ft_forward(self, weight, indices, nnz, out, B, F, N, A, name="sparse_ft_forward"):
        # trainer_layerstack.rs:2215-2244: 1 thread = 4 outputs
        self.launch_1d(name, B * F // 4, weight, indices, nnz, out, U32(B), U32(F), U32(N), U32(A))

    def inverse_index(self, indices, nnz, B, A, N):
        """build_feature_counts -> 3 scan kernels -> scatter_positions (trainer_layerstack.rs:3736-3830).
        Returns (positions, offsets)."""
        t = self.torch
        counts = t.zeros(N, dtype=t.int32, device="cuda")
        ctr = t.zeros(N, dtype=t.int32, device="cuda")
        offsets = t.zeros(N + 1, dtype=t.int32, device="cuda")
        blocks = (N + 1023) // 1024
        block_sums = t.zeros(blocks, dtype=t.int32, device="cuda")
        block_offsets = t.zeros(blocks + 1, dtype=t.int32, device="cuda")
        positions = t.zeros(B * A, dtype=t.int32, device="cuda")
        self.launch_1d("build_feature_counts", B * A, indices, nnz, counts, U32(B), U32(A), U32(N))
        self.launch("prefix_sum_block_local", blocks, 1024, counts, offsets, block_sums, U32(N))
        self.launch("exclusive_prefix_sum_small", 1, 1024, block_sums, block_offsets, U32(blocks))
        self.launch("prefix_sum_add_block_offset", blocks, 1024, offsets, block_offsets, U32(N), U32(blocks))
        self.launch_1d("scatter_positions", B * A, indices, nnz, offsets, ctr, positions, U32(B), U32(A), U32(N))
        return positions, offsets

    def ft_backward(self, dft_list, idx_list, nnz, B, A, N, F, grad, suffix="", extra=()):
        """Phase D of the reference: the first perspective overwrites, the others add (atomics)."""
        for i, (dft, idx) in enumerate(zip(dft_list, idx_list)):
            positions, offsets = self.inverse_index(idx, nnz, B, A, N)
            name = ("gather_and_sum_per_feature_overwrite" if i == 0 else "gather_and_sum_per_feature_add") + suffix
            self.launch(name, (N, F // 128), 128, dft, positions, offsets, grad, U32(N), U32(F), *extra)

    def sync(self):
        self.torch.cuda.synchronize()
