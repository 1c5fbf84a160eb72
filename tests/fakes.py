"""A host-only stand-in for h3metal_b200.gpu.Gpu: holds NumPy arrays and records native calls. Lets the CPU tests
exercise the launchers' host logic (padding, strides, the two-step LoRA sequence, error behaviour) without a GPU."""
import numpy as np

from h3metal_b200 import gpu as gpu_mod


class HostBuffer:
    def __init__(self, arr):
        self.arr = arr
        self.handle = arr.ctypes.data
        self.nbytes = arr.nbytes
        self.owner = arr


class HostTensor(gpu_mod.Tensor):
    def numpy(self):
        n = int(np.prod(self.shape))
        size = gpu_mod._SIZE[self.dtype]
        raw = self.buf.arr.view(np.uint8).reshape(-1)[self.offset:self.offset + n * size]
        return raw.view(gpu_mod._NP[self.dtype]).reshape(self.shape)

    def view(self, shape, dtype=None, offset_elems=0):
        dtype = dtype or self.dtype
        return HostTensor(self.buf, self.offset + int(offset_elems * gpu_mod._SIZE[self.dtype]), tuple(shape), dtype)


class RecordingGpu:
    def __init__(self, tile_n=None):
        self.calls = []
        self._tile_n = tile_n
        self._profile = False

    def empty(self, shape, dtype="f32"):
        shape = tuple(int(s) for s in shape)
        arr = np.zeros(max(1, int(np.prod(shape)) * gpu_mod._SIZE[dtype]), np.uint8)
        return HostTensor(HostBuffer(arr), 0, shape, dtype)

    def upload(self, arr, dtype=None):
        arr = np.ascontiguousarray(arr)
        dtype = dtype or {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.int8): "i8",
                          np.dtype(np.int32): "i32", np.dtype(np.uint16): "bf16"}[arr.dtype]
        t = self.empty(arr.shape, dtype)
        t.numpy()[...] = arr.view(gpu_mod._NP[dtype]).reshape(t.shape)
        return t

    def gemm_tile_n(self, N, lora):
        if self._tile_n:
            return self._tile_n
        return 32 if N <= 32 else 64 if N <= 64 else 128 if N <= 128 else 256 if (N % 256 == 0 or N >= 2048) else 128

    def gemm_native(self, a, a_stride, w, w_stride, sw, sa, bias, out, out_dtype, c_stride, M, N, K, lt=None,
                    t_stride=0, lb=None, b_stride=0, R=0, ranges_ptr=None, name="gemm"):
        self.calls.append(dict(kind="gemm", a=a, a_stride=a_stride, w=w, w_stride=w_stride, sw=sw, sa=sa, bias=bias,
                               out=out, out_dtype=out_dtype, c_stride=c_stride, M=M, N=N, K=K, lt=lt,
                               t_stride=t_stride, lb=lb, b_stride=b_stride, R=R, ranges_ptr=ranges_ptr))

    def rot_q8_native(self, x, x_stride, out, sa, M, D, block, mode, out_hr, name="rot_q8"):
        self.calls.append(dict(kind="rot_q8", x=x, x_stride=x_stride, out=out, sa=sa, M=M, D=D, block=block,
                               mode=mode, out_hr=out_hr))
