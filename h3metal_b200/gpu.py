"""Python side of the B200 runtime (libh3b200.so): buffers, typed views, ordered launches, wait and profiling.

Keeps the names and meanings of the reference's h3metal/gpu.py (`Gpu` :179-265, `Tensor` :121-157, `Buffer`
:109-118, `Kernel` :167-176, `GpuError` :94, `pack` :304) for the quantised-linear path, so that code written
against that module keeps working:

* launches are asynchronous and ordered; results are valid after `Gpu.wait()`, which returns the GPU seconds of
  the work since the previous wait;
* `Gpu.empty()` is zero-filled; `Gpu.upload()` copies a NumPy array to the device;
* errors of the native library surface as `GpuError` carrying its thread-local message.

What differs, because a B200 has its own memory instead of Apple's shared storage: `Tensor.numpy()` synchronises
and returns a host COPY (the reference returns a live view of shared memory), and `Gpu.kernel()` / `Gpu.launch()`
accept only the two kernels of this path, ("gemm.metal", "gemm") in its int8 format with the storing epilogue and
("ops.metal", "rot_q8"), which they route to the ahead-of-time compiled CUDA entry points. Device memory, streams
and host<->device copies are PyTorch's (plumbing only); every computation is in the native library. There is no
CPU fallback: if the library is missing or the device is not a B200, constructing `Gpu` raises.
"""

from __future__ import annotations

import ctypes
import math
import os
import struct
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

H3B_F32, H3B_F16, H3B_BF16, H3B_I8, H3B_I32 = 0, 1, 2, 3, 4
_ABI_DTYPE = {"f32": H3B_F32, "f16": H3B_F16, "bf16": H3B_BF16, "i8": H3B_I8, "i32": H3B_I32}
_METAL_T = {"half": "f16", "bfloat": "bf16", "float": "f32"}


class GpuError(RuntimeError):
    pass


def _find_library() -> str:
    for cand in (os.environ.get("H3B200_LIB", ""), os.path.join(_HERE, "libh3b200.so")):
        if cand and os.path.exists(cand):
            return os.path.abspath(cand)
    raise GpuError("libh3b200.so not found: build it with `python -m h3metal_b200.build` (needs nvcc); "
                   "there is no CPU fallback for this path")


# name -> (restype, argtypes): every symbol include/h3b200.h declares
def _signatures():
    vp, u64, i32, i64, cp, dbl = (ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_int64, ctypes.c_char_p,
                                  ctypes.c_double)
    return {
        "h3b_last_error": (cp, []),
        "h3b_open": (vp, [i32]),
        "h3b_close": (None, [vp]),
        "h3b_device_name": (cp, [vp]),
        "h3b_recommended_working_set": (u64, [vp]),
        "h3b_max_buffer_length": (u64, [vp]),
        "h3b_sm_count": (i32, [vp]),
        "h3b_set_stream": (i32, [vp, vp]),
        "h3b_use_own_stream": (i32, [vp]),
        "h3b_set_launch_overlap": (i32, [vp, i32]),
        "h3b_rot_q8": (i32, [vp, vp, i32, i64, vp, vp, i32, i32, i32, i32, i32]),
        "h3b_norm_mod_q8": (i32, [vp, vp, i64, vp, i64, vp, vp, vp, i32, i32, i32, ctypes.c_float, i32, i32, vp, vp]),
        "h3b_rot_amax": (i32, [vp, vp, i32, i64, vp, i32, i32, i32, i32]),
        "h3b_rot_q8_given_amax": (i32, [vp, vp, i32, i64, vp, vp, i32, i32, i32, i32]),
        "h3b_rot_amax_push": (i32, [vp, vp, i32, i64, ctypes.POINTER(vp), i32, i32, i32, i32, i32]),
        "h3b_rot_q8_given_amax_slots": (i32, [vp, vp, i32, i64, vp, vp, i64, i32, vp, i32, i32, i32, i32]),
        "h3b_dequant_i32": (i32, [vp, vp, i64, vp, vp, vp, vp, i32, i64, i32, i32]),
        "h3b_gemm_w8a8": (i32, [vp, vp, i64, vp, i64, vp, vp, vp, vp, i32, i64, i32, i32, i32, vp, i64, vp, i64, i32,
                                vp]),
        "h3b_gemm_w8a8_gated": (i32, [vp, vp, i64, vp, i64, vp, vp, vp, vp, i64, i32, i32, i32, vp, vp, i64, vp, i64, vp, i64,
                                      i32, vp]),
        "h3b_gemm_w8a8_lora_noalloc": (i32, [vp, vp, i64, vp, i64, vp, vp, vp, vp, i32, i64, i32, i32, i32, vp, i64, vp,
                                             vp, i64, i32, vp]),
        "h3b_peer_alloc": (vp, [vp, u64]),
        "h3b_peer_free": (i32, [vp, vp]),
        "h3b_peer_export": (i32, [vp, vp, ctypes.c_char_p]),
        "h3b_peer_import": (vp, [vp, ctypes.c_char_p]),
        "h3b_peer_unmap": (i32, [vp, vp]),
        "h3b_peer_sync": (i32, [vp, ctypes.POINTER(vp), i32, i32, ctypes.c_uint32, i32]),
        "h3b_gemm_w8a8_push": (i32, [vp, vp, i64, vp, i64, vp, vp, ctypes.POINTER(vp), i32, i32, i32, i64, i32, i32, i32]),
        "h3b_reduce_dequant": (i32, [vp, vp, i64, i64, i32, i32, vp, vp, vp, ctypes.POINTER(vp), i32, i32, i64, i32, i32,
                                     i32]),
        "h3b_reduce_dequant_low": (i32, [vp, vp, i64, i64, i32, i32, vp, vp, vp, vp, i64, ctypes.POINTER(vp), i32, i32, i64, i32,
                                         i32, i32, vp, vp, i64]),
        "h3b_reduce_dequant_gated": (i32, [vp, vp, i64, i64, i32, i32, vp, vp, vp, vp, i64, i32, i32, i32, vp, vp, i64]),
        "h3b_gemm_tile_n": (i32, [vp, i32, i32]),
        "h3b_gemm_set_policy": (i32, [vp, i32, i32, i32]),
        "h3b_gemm_set_store_mode": (i32, [vp, i32]),
        "h3b_rot_set_policy": (i32, [vp, i32, i32, i32]),
        "h3b_selftest_expire_wait": (i32, [vp]),
        "h3b_mma_rate_probe": (i32, [vp, i32, i32, ctypes.POINTER(dbl)]),
        "h3b_commit": (None, [vp]),
        "h3b_wait": (dbl, [vp]),
        "h3b_set_profile": (None, [vp, i32]),
        "h3b_profile_take": (i32, [vp, ctypes.POINTER(dbl), i32]),
        "h3b_launch_count": (u64, [vp]),
    }


def _load():
    lib = ctypes.CDLL(_find_library())
    for name, (res, args) in _signatures().items():
        f = getattr(lib, name)
        f.restype = res
        f.argtypes = args
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _err() -> str:
    return lib().h3b_last_error().decode()


_NP = {
    "f32": np.float32, "f16": np.float16, "bf16": np.uint16, "i8": np.int8, "u8": np.uint8,
    "i32": np.int32, "u32": np.uint32, "i16": np.int16, "u16": np.uint16,
}
_SIZE = {"f32": 4, "f16": 2, "bf16": 2, "i8": 1, "u8": 1, "i32": 4, "u32": 4, "i16": 2, "u16": 2}


def _torch():
    import torch
    return torch


def _torch_dtype(dtype: str):
    t = _torch()
    return {"f32": t.float32, "f16": t.float16, "bf16": t.bfloat16, "i8": t.int8, "u8": t.uint8, "i32": t.int32,
            "i16": t.int16, "u16": t.uint16, "u32": t.uint32}[dtype]


@dataclass
class Buffer:
    """Device memory: `handle` is the device address, `owner` the torch tensor that keeps it alive."""
    handle: int
    nbytes: int
    owner: object = None


@dataclass
class Tensor:
    """A typed view of (part of) a device buffer."""
    buf: Buffer
    offset: int
    shape: tuple
    dtype: str
    strides: tuple = field(default=None)  # in elements; None = contiguous

    @property
    def nbytes(self) -> int:
        return int(math.prod(self.shape) * _SIZE[self.dtype])

    @property
    def ptr(self) -> int:
        return self.buf.handle + self.offset

    def arg(self):
        return (self.buf.handle, self.offset)

    def torch(self):
        """The same memory as a torch tensor (no copy). bf16 views are torch.bfloat16."""
        raw = self.buf.owner.view(_torch().uint8).reshape(-1)
        flat = raw[self.offset:self.offset + self.nbytes]
        return flat.view(_torch_dtype(self.dtype)).reshape(self.shape)

    def numpy(self) -> np.ndarray:
        """A host copy of the data, taken after the device has finished the work launched so far.

        bf16 comes back as uint16 bit patterns, as in the reference."""
        t = self.torch()
        if self.dtype == "bf16":
            t = t.view(_torch().int16)
        elif self.dtype in ("u16", "u32"):
            t = t.view({"u16": _torch().int16, "u32": _torch().int32}[self.dtype])
        host = t.cpu().numpy()  # synchronises with the stream that wrote it
        return host.view(_NP[self.dtype]).reshape(self.shape)

    def view(self, shape, dtype=None, offset_elems=0):
        dtype = dtype or self.dtype
        return Tensor(self.buf, self.offset + int(offset_elems * _SIZE[self.dtype]), tuple(shape), dtype)

    def row(self, start: int, count: int):
        """Rows [start, start + count) of a 2-D (or higher) contiguous tensor."""
        per = int(math.prod(self.shape[1:]))
        return Tensor(self.buf, self.offset + int(start * per * _SIZE[self.dtype]), (count,) + tuple(self.shape[1:]),
                      self.dtype)


class Kernel:
    """One of the path's two kernels with the specialisation macros the caller asked for."""

    SUPPORTED = {("gemm.metal", "gemm"), ("ops.metal", "rot_q8"), ("ops.metal", "norm_mod_q8")}

    def __init__(self, gpu: "Gpu", file: str, fn: str, macros: dict | None = None):
        if (file, fn) not in self.SUPPORTED:
            raise GpuError(f"kernel {file}:{fn} is not part of the int8 linear path this library implements")
        self.file, self.fn, self.macros = file, fn, dict(macros or {})
        ms = ";".join(f"{k}={v}" for k, v in sorted(self.macros.items()))
        self.name = f"{file}:{fn}({ms})"
        self.max_threads = 1024


class Gpu:
    def __init__(self, kernel_dir: str | None = None, device: int | None = None):
        """kernel_dir is accepted for signature compatibility and ignored (kernels are compiled ahead of time).
        device defaults to LOCAL_RANK, else the current torch CUDA device."""
        torch = _torch()
        if not torch.cuda.is_available():
            raise GpuError("no CUDA device: this library runs on B200 (sm_100a) only and has no CPU fallback")
        if device is None:
            device = int(os.environ["LOCAL_RANK"]) if "LOCAL_RANK" in os.environ else torch.cuda.current_device()
        self.device_index = int(device)
        self.torch_device = torch.device("cuda", self.device_index)
        torch.cuda.set_device(self.torch_device)
        torch.zeros(1, device=self.torch_device)  # make sure the primary context exists before the library opens it
        self.ctx = lib().h3b_open(self.device_index)
        if not self.ctx:
            raise GpuError(_err())
        self.device = lib().h3b_device_name(self.ctx).decode()
        self.working_set = lib().h3b_recommended_working_set(self.ctx)
        self.max_buffer = lib().h3b_max_buffer_length(self.ctx)
        self.sm_count = lib().h3b_sm_count(self.ctx)
        self.rot_block = 256  # rotation block used when rot_q8 is launched through the generic launch()
        self.lora_t_split = 4  # ops.gemm may split K of a LoRA term's input-side product this many ways (0 = never)
        self._kernels = {}
        self.names = []
        self.use_stream(None)

    # -- streams --------------------------------------------------------------------------------------------------
    def use_stream(self, stream=None):
        """Launch on `stream` (a torch.cuda.Stream); None = torch's current stream of this device, so that kernels
        are ordered with the uploads and allocations torch does for this object."""
        torch = _torch()
        self.stream = stream if stream is not None else torch.cuda.current_stream(self.torch_device)
        if lib().h3b_set_stream(self.ctx, ctypes.c_void_p(self.stream.cuda_stream)):
            raise GpuError(_err())

    def set_launch_overlap(self, on: bool):
        """Programmatic dependent launch of the path's kernels (on by default): a kernel's set-up overlaps the tail
        of the kernel before it; every kernel still waits for its predecessor before touching global memory."""
        self._check(lib().h3b_set_launch_overlap(self.ctx, 1 if on else 0))

    def kernel(self, file: str, fn: str, **macros) -> Kernel:
        key = (file, fn, tuple(sorted(macros.items())))
        k = self._kernels.get(key)
        if k is None:
            k = Kernel(self, file, fn, macros)
            self._kernels[key] = k
        return k

    # -- memory ---------------------------------------------------------------------------------------------------
    def buffer(self, nbytes: int) -> Buffer:
        torch = _torch()
        n = max(1, int(nbytes))
        with torch.cuda.stream(self.stream):
            t = torch.zeros(n, dtype=torch.uint8, device=self.torch_device)
        return Buffer(t.data_ptr(), int(nbytes), owner=t)

    def empty(self, shape, dtype="f32") -> Tensor:
        shape = tuple(int(s) for s in shape)
        nbytes = int(math.ceil(math.prod(shape) * _SIZE[dtype]))
        return Tensor(self.buffer(nbytes), 0, shape, dtype)

    def upload(self, arr: np.ndarray, dtype: str | None = None) -> Tensor:
        torch = _torch()
        if dtype is None:
            dtype = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.int8): "i8",
                     np.dtype(np.uint8): "u8", np.dtype(np.int32): "i32", np.dtype(np.uint32): "u32",
                     np.dtype(np.uint16): "bf16", np.dtype(np.int16): "i16"}[arr.dtype]
        host = np.ascontiguousarray(arr)
        if not host.flags.writeable:  # e.g. a view of a read-only file mapping: torch wants a writable source
            host = host.copy()
        raw = torch.from_numpy(host.view(np.uint8).reshape(-1))
        with torch.cuda.stream(self.stream):
            dev = raw.to(self.torch_device)
        return Tensor(Buffer(dev.data_ptr(), host.nbytes, owner=dev), 0, tuple(arr.shape), dtype)

    def wrap(self, t, dtype: str | None = None) -> Tensor:
        """A Tensor over the memory of a contiguous torch CUDA tensor (no copy)."""
        torch = _torch()
        if not t.is_cuda or t.device.index != self.device_index or not t.is_contiguous():
            raise GpuError("wrap: need a contiguous tensor on this Gpu's device")
        if dtype is None:
            dtype = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16", torch.int8: "i8",
                     torch.uint8: "u8", torch.int32: "i32", torch.int16: "i16"}[t.dtype]
        return Tensor(Buffer(t.data_ptr(), t.numel() * t.element_size(), owner=t), 0, tuple(t.shape), dtype)

    # -- native entry points ----------------------------------------------------------------------------------------
    def _check(self, rc: int):
        if rc:
            raise GpuError(_err())

    def rot_q8_native(self, x: Tensor, x_stride: int, out: Tensor, sa: Tensor | None, M: int, D: int, block: int,
                      mode: int, out_hr: bool, name: str = "rot_q8"):
        if x.dtype not in ("bf16", "f16", "f32"):
            raise ValueError(f"rot_q8 input type {x.dtype}")
        self._check(lib().h3b_rot_q8(self.ctx, x.ptr, _ABI_DTYPE[x.dtype], x_stride, out.ptr,
                                      sa.ptr if sa is not None else None, M, D, block, mode, int(out_hr)))
        if self._profile:
            self.names.append(name)

    def norm_mod_q8_native(self, x: Tensor, x_stride: int, mod: Tensor, mod_stride: int, rtype: Tensor, out: Tensor,
                           sa: Tensor | None, M: int, D: int, block: int, eps: float, ln: bool, out_kind: int,
                           y: Tensor | None, post: Tensor | None, name: str = "norm_mod_q8"):
        p = lambda t: t.ptr if t is not None else None  # noqa: E731
        self._check(lib().h3b_norm_mod_q8(self.ctx, x.ptr, x_stride, mod.ptr, mod_stride, rtype.ptr, out.ptr, p(sa), M, D,
                                           block, eps, int(ln), out_kind, p(y), p(post)))
        if self._profile:
            self.names.append(name)

    def rot_amax_native(self, x: Tensor, x_stride: int, amax: Tensor, M: int, D: int, block: int, mode: int):
        self._check(lib().h3b_rot_amax(self.ctx, x.ptr, _ABI_DTYPE[x.dtype], x_stride, amax.ptr, M, D, block, mode))
        if self._profile:
            self.names.append("rot_amax")

    def rot_q8_given_amax_native(self, x: Tensor, x_stride: int, out: Tensor, amax_to_scale: Tensor, M: int, D: int,
                                 block: int, mode: int):
        self._check(lib().h3b_rot_q8_given_amax(self.ctx, x.ptr, _ABI_DTYPE[x.dtype], x_stride, out.ptr,
                                                 amax_to_scale.ptr, M, D, block, mode))
        if self._profile:
            self.names.append("rot_q8_given_amax")

    def rot_amax_push_native(self, x: Tensor, x_stride: int, dst, M: int, D: int, block: int, mode: int):
        """This shard's row maxima stored to dst[q] (an address per GPU: this GPU's slot in GPU q's table)."""
        self._check(lib().h3b_rot_amax_push(self.ctx, x.ptr, _ABI_DTYPE[x.dtype], x_stride, self._ptr_array(dst), len(dst), M,
                                            D, block, mode))
        if self._profile:
            self.names.append("rot_amax(push)")

    def rot_q8_given_amax_slots_native(self, x: Tensor, x_stride: int, out: Tensor, slots_ptr: int, slot_stride: int,
                                       world: int, scale: Tensor, M: int, D: int, block: int, mode: int):
        self._check(lib().h3b_rot_q8_given_amax_slots(self.ctx, x.ptr, _ABI_DTYPE[x.dtype], x_stride, out.ptr,
                                                       ctypes.c_void_p(slots_ptr), slot_stride, world, scale.ptr, M, D, block,
                                                       mode))
        if self._profile:
            self.names.append("rot_q8_given_amax(slots)")

    def dequant_native(self, acc: Tensor, acc_stride: int, sa: Tensor, sw: Tensor, bias: Tensor | None, out: Tensor,
                       c_stride: int, M: int, N: int):
        self._check(lib().h3b_dequant_i32(self.ctx, acc.ptr, acc_stride, sa.ptr, sw.ptr,
                                           bias.ptr if bias is not None else None, out.ptr, _ABI_DTYPE[out.dtype],
                                           c_stride, M, N))
        if self._profile:
            self.names.append("dequant")

    def gemm_native(self, a: Tensor, a_stride: int, w: Tensor, w_stride: int, sw: Tensor | None, sa: Tensor | None,
                    bias: Tensor | None, out: Tensor, out_dtype: str, c_stride: int, M: int, N: int, K: int,
                    lt: Tensor | None = None, t_stride: int = 0, lb: Tensor | None = None, b_stride: int = 0,
                    R: int = 0, ranges_ptr: int | None = None, name: str = "gemm"):
        p = lambda t: t.ptr if t is not None else None  # noqa: E731
        self._check(lib().h3b_gemm_w8a8(self.ctx, a.ptr, a_stride, w.ptr, w_stride, p(sw), p(sa), p(bias), out.ptr,
                                         _ABI_DTYPE[out_dtype], c_stride, M, N, K, p(lt), t_stride, p(lb), b_stride,
                                         R, ranges_ptr))
        if self._profile:
            self.names.append(name)

    def gemm_gated_native(self, a: Tensor, a_stride: int, w: Tensor, w_stride: int, sw: Tensor, sa: Tensor,
                          bias: Tensor | None, x: Tensor, c_stride: int, M: int, N: int, K: int, rtype: Tensor,
                          gate: Tensor, g_stride: int, lt: Tensor | None = None, t_stride: int = 0,
                          lb: Tensor | None = None, b_stride: int = 0, R: int = 0, ranges_ptr: int | None = None,
                          name: str = "gemm(epi1)"):
        p = lambda t: t.ptr if t is not None else None  # noqa: E731
        self._check(lib().h3b_gemm_w8a8_gated(self.ctx, a.ptr, a_stride, w.ptr, w_stride, sw.ptr, sa.ptr, p(bias), x.ptr,
                                               c_stride, M, N, K, rtype.ptr, gate.ptr, g_stride, p(lt), t_stride, p(lb),
                                               b_stride, R, ranges_ptr))
        if self._profile:
            self.names.append(name)

    # -- row-parallel layers: peer-mapped memory, rendezvous, push and the owner's reduction ------------------------------
    def peer_alloc(self, nbytes: int) -> Tensor:
        """Zero-filled device memory that other processes can map (u8 [nbytes])."""
        ptr = lib().h3b_peer_alloc(self.ctx, int(nbytes))
        if not ptr:
            raise GpuError(_err())
        return self.wrap_ptr(int(ptr), int(nbytes))

    def wrap_ptr(self, ptr: int, nbytes: int) -> Tensor:
        """A u8 Tensor over raw device memory this process can address (its own or a peer mapping); not owned."""
        torch = _torch()

        class _Raw:
            __cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 2}
        t = torch.as_tensor(_Raw(), device=self.torch_device)
        return Tensor(Buffer(int(ptr), int(nbytes), owner=t), 0, (int(nbytes),), "u8")

    def peer_free(self, ptr: int):
        self._check(lib().h3b_peer_free(self.ctx, ctypes.c_void_p(ptr)))

    def peer_export(self, ptr: int) -> bytes:
        handle = ctypes.create_string_buffer(64)
        self._check(lib().h3b_peer_export(self.ctx, ctypes.c_void_p(ptr), handle))
        return handle.raw

    def peer_import(self, handle: bytes) -> int:
        ptr = lib().h3b_peer_import(self.ctx, ctypes.create_string_buffer(bytes(handle), 64))
        if not ptr:
            raise GpuError(_err())
        return int(ptr)

    def peer_unmap(self, ptr: int):
        self._check(lib().h3b_peer_unmap(self.ctx, ctypes.c_void_p(ptr)))

    @staticmethod
    def _ptr_array(ptrs):
        return (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])

    def peer_sync_native(self, flags, rank: int, world: int, epoch: int, mode: int = 0):
        self._check(lib().h3b_peer_sync(self.ctx, self._ptr_array(flags), rank, world, epoch & 0xFFFFFFFF, mode))
        if self._profile:
            self.names.append("peer_sync")

    def gemm_push_native(self, a: Tensor, a_stride: int, w: Tensor, w_stride: int, sw: Tensor | None, sa: Tensor | None,
                         slots, rows_per_gpu: int, stage_dtype: str, stage_stride: int, M: int, N: int, K: int):
        p = lambda t: t.ptr if t is not None else None  # noqa: E731
        self._check(lib().h3b_gemm_w8a8_push(self.ctx, a.ptr, a_stride, w.ptr, w_stride, p(sw), p(sa),
                                              self._ptr_array(slots), len(slots), rows_per_gpu, _ABI_DTYPE[stage_dtype],
                                              stage_stride, M, N, K))
        if self._profile:
            self.names.append("gemm(push)")

    def reduce_dequant_native(self, stage_ptr: int, slot_stride: int, stage_stride: int, stage_dtype: str, world: int,
                              sa_ptr: int | None, sw: Tensor | None, bias: Tensor | None, outs, out_dtype: str,
                              c_stride: int, rows: int, N: int, row0: int = 0):
        p = lambda t: t.ptr if t is not None else None  # noqa: E731
        self._check(lib().h3b_reduce_dequant(self.ctx, ctypes.c_void_p(stage_ptr), slot_stride, stage_stride,
                                              _ABI_DTYPE[stage_dtype], world, ctypes.c_void_p(sa_ptr) if sa_ptr else None,
                                              p(sw), p(bias), self._ptr_array(outs), len(outs), _ABI_DTYPE[out_dtype],
                                              c_stride, rows, N, row0))
        if self._profile:
            self.names.append("reduce_dequant")

    def reduce_dequant_low_native(self, stage_ptr: int, slot_stride: int, stage_stride: int, stage_dtype: str, world: int,
                                  sa_ptr: int | None, sw: Tensor | None, bias: Tensor | None, low: Tensor, low_stride: int,
                                  outs, out_dtype: str, c_stride: int, rows: int, N: int, row0: int = 0,
                                  rtype_ptr: int | None = None, gate: Tensor | None = None, g_stride: int = 0):
        """The owner's reduction with a low-rank term added after the bias; with gate, outs = [X] and the result is
        accumulated into the fp32 residual stream."""
        p = lambda t: t.ptr if t is not None else None  # noqa: E731
        self._check(lib().h3b_reduce_dequant_low(self.ctx, ctypes.c_void_p(stage_ptr), slot_stride, stage_stride,
                                                  _ABI_DTYPE[stage_dtype], world,
                                                  ctypes.c_void_p(sa_ptr) if sa_ptr else None, p(sw), p(bias), low.ptr,
                                                  low_stride, self._ptr_array(outs), len(outs), _ABI_DTYPE[out_dtype],
                                                  c_stride, rows, N, row0,
                                                  ctypes.c_void_p(rtype_ptr) if rtype_ptr else None, p(gate), g_stride))
        if self._profile:
            self.names.append("reduce_dequant(low)")

    def reduce_dequant_gated_native(self, stage_ptr: int, slot_stride: int, stage_stride: int, stage_dtype: str, world: int,
                                    sa_ptr: int | None, sw: Tensor | None, bias: Tensor | None, x: Tensor, c_stride: int,
                                    rows: int, N: int, row0: int, rtype_ptr: int, gate: Tensor, g_stride: int):
        p = lambda t: t.ptr if t is not None else None  # noqa: E731
        self._check(lib().h3b_reduce_dequant_gated(self.ctx, ctypes.c_void_p(stage_ptr), slot_stride, stage_stride,
                                                    _ABI_DTYPE[stage_dtype], world,
                                                    ctypes.c_void_p(sa_ptr) if sa_ptr else None, p(sw), p(bias), x.ptr,
                                                    c_stride, rows, N, row0, ctypes.c_void_p(rtype_ptr), gate.ptr, g_stride))
        if self._profile:
            self.names.append("reduce_dequant(epi1)")

    def gemm_tile_n(self, N: int, lora: bool) -> int:
        return lib().h3b_gemm_tile_n(self.ctx, N, int(lora))

    def set_store_mode(self, mode: int = 0):
        """How CTA pairs write 16-bit outputs: 1 staged through shared memory and TMA stores whenever possible,
        -1 direct stores from registers, 0 automatic (staged for short launches with K <= 4096 and for M >= 49152)."""
        self._check(lib().h3b_gemm_set_store_mode(self.ctx, mode))

    def set_policy(self, tile_n: int = 0, band: int = 0, rot_threads: int = 0, rot_stages: int = 0, pair: int = 0,
                   rot_chunk: int = 0):
        """Overrides of the library's own choices (0 = automatic), for tuning sweeps and for tests that want a
        particular kernel variant. rot_stages = -1 selects the register-fed rotate+quantise kernel; pair = -1 / 1 keeps
        the product off / on CTA pairs; rot_chunk = 32 / 64 sets the channels per thread of the TMA-fed kernel."""
        self._check(lib().h3b_gemm_set_policy(self.ctx, tile_n, band, pair))
        self._check(lib().h3b_rot_set_policy(self.ctx, rot_threads, rot_stages, rot_chunk))

    # -- execution ------------------------------------------------------------------------------------------------
    def launch(self, k: Kernel, grid, threads, args, params: bytes = b"", params_index: int | None = None,
               tg_mem: int = 0):
        """The reference's generic dispatch, for its two kernels of this path: decodes the macros and the
        parameter block (kernels/params.h:7-16,25-29) and the buffer order (kernels/gemm.metal:117-128,
        kernels/ops.metal:274-277) and calls the native entry point. grid / threads / tg_mem are ignored."""
        if (k.file, k.fn) == ("ops.metal", "rot_q8"):
            M, D, x_stride, mode = struct.unpack("<4i", params)
            x, out, sa = (list(args) + [None, None])[:3]
            in_t = _METAL_T.get(str(k.macros.get("IN_T", "bfloat")), x.dtype)
            if in_t != x.dtype:
                x = x.view(x.shape, in_t)
            self.rot_q8_native(x, x_stride, out, sa, M, D, self.rot_block, mode, bool(int(k.macros.get("OUT_HR", 0))),
                               name=k.name)
            return
        if (k.file, k.fn) == ("ops.metal", "norm_mod_q8"):
            M, D, x_stride, mod_stride, eps = struct.unpack("<4if", params)
            x, mod, rtype, out, sa, _params, y, post = (list(args) + [None] * 8)[:8]
            mac = k.macros
            kind = 1 if int(mac.get("OUT_F", 0)) else 2 if int(mac.get("OUT_H", 0)) else 3 if int(mac.get("OUT_HR", 0)) else 0
            self.norm_mod_q8_native(x, x_stride, mod, mod_stride, rtype, out, sa, M, D, self.rot_block, eps,
                                    bool(int(mac.get("LN", 0))), kind, y if int(mac.get("POST", 0)) else None,
                                    post if int(mac.get("POST", 0)) else None, name=k.name)
            return
        mac = k.macros
        if int(mac.get("WFMT", 1)) != 1:
            raise GpuError("gemm: only the int8 weight format (WFMT 1) exists here")
        epi1 = int(mac.get("EPI", 0)) == 1
        M, N, K, a_stride, c_stride, w_stride, _groups, _g_stride = struct.unpack("<8i", params)
        a, w, sw, sa, out, bias = (list(args) + [None] * 6)[:6]
        out_dtype = _METAL_T[str(mac.get("OUT_T", "half"))]
        lt = lb = None
        R = 0
        ranges_ptr = None
        if int(mac.get("LORA", 0)):
            lt, lb, lr = args[9], args[10], args[11]
            tn = int(mac.get("TN", 128))
            if tn != self.gemm_tile_n(N, True):
                raise GpuError(f"gemm: the low-rank range table is for {tn}-column tiles; this library uses "
                               f"{self.gemm_tile_n(N, True)} for N={N} (build it with LowRank.table(gpu, that width))")
            # T's and B's row strides lead the table. A table built by LowRank.table() carries them on the host; only
            # a table from elsewhere is read back from the device (a blocking copy).
            head = getattr(lr, "host_head", None)
            if head is None:
                head = lr.numpy()[:2]
            R = int(head[0])
            ranges_ptr = lr.ptr + 8
            lora_args = (lt, int(head[0]), lb, int(head[1]), R, ranges_ptr)
        else:
            lora_args = (None, 0, None, 0, 0, None)
        b = bias if int(mac.get("HAS_BIAS", 0)) else None
        if epi1:
            self.gemm_gated_native(a, a_stride, w, w_stride, sw, sa, b, out, c_stride, M, N, K, args[6], args[7],
                                   _g_stride, *lora_args, name=k.name)
        else:
            self.gemm_native(a, a_stride, w, w_stride, sw, sa, b, out, out_dtype, c_stride, M, N, K, *lora_args,
                             name=k.name)

    _profile = False

    def commit(self):
        lib().h3b_commit(self.ctx)

    def wait(self) -> float:
        dt = lib().h3b_wait(self.ctx)
        if dt < 0:
            raise GpuError(_err())
        return dt

    def profile(self, on: bool):
        lib().h3b_set_profile(self.ctx, 1 if on else 0)
        self._profile = on
        self.names = []

    def profile_take(self):
        out = (ctypes.c_double * 100000)()
        n = lib().h3b_profile_take(self.ctx, out, 100000)
        names, self.names = self.names[:n], self.names[n:]
        return list(zip(names, out[:n]))

    def mma_rate_probe(self, pair: bool = False, iters: int = 40000) -> dict:
        """Issue rate of the int8 tensor pipe from operands resident in shared memory (no TMA, no epilogue): the
        measured ceiling of the product, as the reference measures its matrix units (bench/hw/mma_rate.py:9-24).
        Blocking; one launch of about iters x 0.3 microseconds."""
        out = (ctypes.c_double * 5)()
        self._check(lib().h3b_mma_rate_probe(self.ctx, int(pair), int(iters), out))
        return {"seconds": out[0], "cycles": out[1], "ops_per_clk_per_sm": out[2], "tops": out[3], "ctas": int(out[4])}

    @property
    def launch_count(self) -> int:
        return int(lib().h3b_launch_count(self.ctx))

    def close(self):
        if self.ctx:
            lib().h3b_close(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def pack(fmt: str, *vals) -> bytes:
    return struct.pack("<" + fmt, *vals)
