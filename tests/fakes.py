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
                          np.dtype(np.int32): "i32", np.dtype(np.uint16): "bf16", np.dtype(np.uint8): "u8"}[arr.dtype]
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

    def gemm_gated_native(self, a, a_stride, w, w_stride, sw, sa, bias, x, c_stride, M, N, K, rtype, gate, g_stride,
                          lt=None, t_stride=0, lb=None, b_stride=0, R=0, ranges_ptr=None, name="gemm(epi1)"):
        self.calls.append(dict(kind="gemm_gated", a=a, a_stride=a_stride, w=w, w_stride=w_stride, bias=bias, out=x,
                               c_stride=c_stride, M=M, N=N, K=K, g_stride=g_stride, lt=lt, R=R))

    def norm_mod_q8_native(self, x, x_stride, mod, mod_stride, rtype, out, sa, M, D, block, eps, ln, out_kind, y, post,
                           name="norm_mod_q8"):
        self.calls.append(dict(kind="norm_mod_q8", x=x, x_stride=x_stride, mod=mod, mod_stride=mod_stride, rtype=rtype,
                               out=out, sa=sa, M=M, D=D, block=block, eps=eps, ln=ln, out_kind=out_kind, y=y, post=post))

    def rot_q8_native(self, x, x_stride, out, sa, M, D, block, mode, out_hr, name="rot_q8"):
        self.calls.append(dict(kind="rot_q8", x=x, x_stride=x_stride, out=out, sa=sa, M=M, D=D, block=block,
                               mode=mode, out_hr=out_hr))


def _host_torch(self):
    """The same host memory as a torch CPU tensor (so that gloo collectives act on it in place)."""
    import torch
    arr = self.numpy()
    if self.dtype == "bf16":
        return torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(arr)


HostTensor.torch = _host_torch


class OracleBackedGpu(RecordingGpu):
    """Executes the native calls with the CPU oracle, on host arrays. Lets the multi-rank orchestration of
    h3metal_b200.parallel run under gloo without a GPU; the arithmetic is the oracle's, the sequencing (which
    shard, which collective, which epilogue) is the product's."""

    def _rows(self, t, rows, cols, stride, dtype):
        flat = t.buf.arr.view(np.uint8).reshape(-1)[t.offset:].view(gpu_mod._NP[dtype])[:(rows - 1) * stride + cols]
        return np.lib.stride_tricks.as_strided(flat, (rows, cols), (stride * flat.itemsize, flat.itemsize))

    def _rotated(self, x, x_stride, M, D, block, mode):
        from oracle import rotq8_ref
        cols = 2 * D if mode == 1 else D
        mat = self._rows(x, M, cols, x_stride, x.dtype)
        xf = rotq8_ref._as_f32_input(mat, x.dtype)
        val = xf[:, :D]
        if mode == 1:
            val = (val * rotq8_ref.silu_f32(xf[:, D:2 * D])).astype(np.float32)
        return (rotq8_ref.fwht_blocks_f32(val, block) * rotq8_ref.normaliser(block)).astype(np.float32)

    def rot_q8_native(self, x, x_stride, out, sa, M, D, block, mode, out_hr, name="rot_q8"):
        v = self._rotated(x, x_stride, M, D, block, mode)
        amax = np.abs(v).max(axis=1)
        self._quantise(v, amax, out, sa, M, D)

    def rot_amax_native(self, x, x_stride, amax, M, D, block, mode):
        amax.numpy().reshape(-1)[:M] = np.abs(self._rotated(x, x_stride, M, D, block, mode)).max(axis=1)

    def rot_q8_given_amax_native(self, x, x_stride, out, amax_to_scale, M, D, block, mode):
        v = self._rotated(x, x_stride, M, D, block, mode)
        self._quantise(v, amax_to_scale.numpy().reshape(-1)[:M].copy(), out, amax_to_scale, M, D)

    def _quantise(self, v, amax, out, sa, M, D):
        scale = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
        rs = (np.float32(1.0) / scale).astype(np.float32)
        q = np.rint((v * rs[:, None]).astype(np.float32)).astype(np.int32).astype(np.int8)
        self._rows(out, M, D, D, "i8")[...] = q
        sa.numpy().reshape(-1)[:M] = scale

    def gemm_native(self, a, a_stride, w, w_stride, sw, sa, bias, out, out_dtype, c_stride, M, N, K, lt=None,
                    t_stride=0, lb=None, b_stride=0, R=0, ranges_ptr=None, name="gemm"):
        from oracle import gemm_ref
        assert lt is None, "the fake does not carry the low-rank term"
        acc = gemm_ref.int32_product(self._rows(a, M, K, a_stride, "i8"), self._rows(w, N, K, w_stride, "i8"))
        dst = self._rows(out, M, N, c_stride, out_dtype)
        if out_dtype == "i32":
            dst[...] = acc
            return
        v = gemm_ref.epilogue_q8(acc, sa.numpy().reshape(-1)[:M], sw.numpy().reshape(-1)[:N],
                                 bias.numpy().reshape(-1)[:N] if bias is not None else None)
        dst[...] = gemm_ref.store_as(v, out_dtype)

    def dequant_native(self, acc, acc_stride, sa, sw, bias, out, c_stride, M, N):
        from oracle import gemm_ref
        v = gemm_ref.epilogue_q8(self._rows(acc, M, N, acc_stride, "i32"), sa.numpy().reshape(-1)[:M],
                                 sw.numpy().reshape(-1)[:N], bias.numpy().reshape(-1)[:N] if bias is not None else None)
        self._rows(out, M, N, c_stride, out.dtype)[...] = gemm_ref.store_as(v, out.dtype)
