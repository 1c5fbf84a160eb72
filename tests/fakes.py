"""A host-only stand-in for h3metal_b200.gpu.Gpu: holds NumPy arrays and records native calls. Lets the CPU tests
exercise the launchers' host logic (padding, strides, the two-step LoRA sequence, error behaviour) without a GPU."""
import os

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
        acc = gemm_ref.int32_product(self._rows(a, M, K, a_stride, "i8"), self._rows(w, N, K, w_stride, "i8"))
        dst = self._rows(out, M, N, c_stride, out_dtype)
        if out_dtype == "i32":
            dst[...] = acc
            return
        low = None
        if lt is not None:  # T B'^T as the oracle forms it (fp16 inputs, wide accumulation; gemm_ref.lora_low)
            T = self._rows(lt, M, R, t_stride, "f16").astype(np.float64)
            low = (T @ self._rows(lb, N, R, b_stride, "f16").astype(np.float64).T).astype(np.float32)
        v = gemm_ref.epilogue_q8(acc, sa.numpy().reshape(-1)[:M], sw.numpy().reshape(-1)[:N],
                                 bias.numpy().reshape(-1)[:N] if bias is not None else None, low)
        dst[...] = gemm_ref.store_as(v, out_dtype)

    def dequant_native(self, acc, acc_stride, sa, sw, bias, out, c_stride, M, N):
        from oracle import gemm_ref
        v = gemm_ref.epilogue_q8(self._rows(acc, M, N, acc_stride, "i32"), sa.numpy().reshape(-1)[:M],
                                 sw.numpy().reshape(-1)[:N], bias.numpy().reshape(-1)[:N] if bias is not None else None)
        self._rows(out, M, N, c_stride, out.dtype)[...] = gemm_ref.store_as(v, out.dtype)


class SharedPeerGpu(OracleBackedGpu):
    """Adds the peer-memory natives on files mapped by every rank, so that gloo ranks (processes) can play the GPUs of
    a row-parallel layer: a "device address" is the address of the mapping in this process, exactly as a CUDA IPC
    mapping has a different address in every process. The rendezvous is a gloo barrier."""

    def __init__(self, group=None, tile_n=None, sync_limit_s=20.0):
        super().__init__(tile_n)
        self.group = group
        self._regions = []  # (address, nbytes, uint8 array, path or None)
        self.sync_limit_s = sync_limit_s  # how long a rendezvous polls before it gives up (the device's is ~1 s)
        self.drop_signals = 0             # the next n rendezvous of this rank signal nobody (a message that is lost)
        self.status = 0                   # the context's status word: 7 after a rendezvous that ran out

    def _register(self, arr, path=None):
        self._regions.append((arr.ctypes.data, arr.nbytes, arr, path))
        return arr.ctypes.data

    def _bytes(self, ptr, nbytes):
        for start, size, arr, _ in self._regions:
            if start <= ptr and ptr + nbytes <= start + size:
                return arr[ptr - start:ptr - start + nbytes]
        raise KeyError(f"address {ptr:#x} (+{nbytes}) is not in a known buffer")

    def empty(self, shape, dtype="f32"):
        t = super().empty(shape, dtype)
        self._register(t.buf.arr)
        return t

    def wait(self):
        """Like the library's h3b_wait: reports a device-side give-up once, clears it, and the context stays usable."""
        if self.status:
            code, self.status = self.status, 0
            raise gpu_mod.GpuError(f"GPU kernel gave up: status {code}: rendezvous of a row-parallel layer timed out: "
                                   f"another GPU did not signal")
        return 0.0

    def peer_alloc(self, nbytes):
        import tempfile
        fd, path = tempfile.mkstemp(prefix="h3b_peer_")
        os.close(fd)
        arr = np.memmap(path, dtype=np.uint8, mode="w+", shape=(int(nbytes),))
        self._register(arr, path)
        return HostTensor(HostBuffer(arr), 0, (int(nbytes),), "u8")

    def peer_export(self, ptr):
        return next(path for start, _, _, path in self._regions if start == ptr).encode()

    def peer_import(self, handle):
        arr = np.memmap(bytes(handle).decode(), dtype=np.uint8, mode="r+")
        return self._register(arr)

    def peer_unmap(self, ptr):
        self._regions = [r for r in self._regions if r[0] != ptr]

    def peer_free(self, ptr):
        path = next(path for start, _, _, path in self._regions if start == ptr)
        self.peer_unmap(ptr)
        os.unlink(path)

    def peer_sync_native(self, flags, rank, world, epoch, mode=0):
        """The device protocol on the file-backed blocks: store `epoch` into word `rank` of every rank's flag array,
        then poll this rank's own array until every word has reached `epoch` - for a bounded time, after which the
        status word gets code 7 and the call returns (peer_sync_kernel in csrc/peer.cu)."""
        import time
        assert mode == 0 and len(flags) == world
        if self.drop_signals > 0:
            self.drop_signals -= 1
        else:
            for q in range(world):
                self._bytes(flags[q], 4 * world).view(np.uint32)[rank] = epoch
        mine = self._bytes(flags[rank], 4 * world).view(np.uint32)
        t0 = time.monotonic()
        while any(int(np.int32(np.uint32(int(mine[q]) - epoch & 0xFFFFFFFF))) < 0 for q in range(world)):
            if time.monotonic() - t0 > self.sync_limit_s:
                if not self.status:
                    self.status = 7
                return
            time.sleep(0.0005)

    def rot_amax_push_native(self, x, x_stride, dst, M, D, block, mode):
        amax = np.abs(self._rotated(x, x_stride, M, D, block, mode)).max(axis=1).astype(np.float32)
        for ptr in dst:
            self._bytes(ptr, M * 4).view(np.float32)[...] = amax

    def rot_q8_given_amax_slots_native(self, x, x_stride, out, slots_ptr, slot_stride, world, scale, M, D, block, mode):
        table = self._bytes(slots_ptr, ((world - 1) * slot_stride + M) * 4).view(np.float32)
        amax = np.max([table[s * slot_stride:s * slot_stride + M] for s in range(world)], axis=0)
        self._quantise(self._rotated(x, x_stride, M, D, block, mode), amax.copy(), out, scale, M, D)

    def gemm_push_native(self, a, a_stride, w, w_stride, sw, sa, slots, rows_per_gpu, stage_dtype, stage_stride, M, N, K):
        from oracle import gemm_ref
        assert M == rows_per_gpu * len(slots) and stage_stride == N
        acc = gemm_ref.int32_product(self._rows(a, M, K, a_stride, "i8"), self._rows(w, N, K, w_stride, "i8"))
        for o, slot in enumerate(slots):
            part = acc[o * rows_per_gpu:(o + 1) * rows_per_gpu]
            if stage_dtype == "i32":
                self._bytes(slot, part.size * 4).view(np.int32).reshape(part.shape)[...] = part
            else:
                v = gemm_ref.epilogue_q8(part, sa.numpy().reshape(-1)[o * rows_per_gpu:(o + 1) * rows_per_gpu],
                                         sw.numpy().reshape(-1)[:N], None)
                self._bytes(slot, part.size * 2).view(np.uint16).reshape(part.shape)[...] = gemm_ref.store_as(v, "bf16")

    def reduce_dequant_gated_native(self, stage_ptr, slot_stride, stage_stride, stage_dtype, world, sa_ptr, sw, bias, x,
                                    c_stride, rows, N, row0, rtype_ptr, gate, g_stride):
        from oracle import gemm_ref
        if self.status:
            return  # as reduce_dequant_kernel: nothing is stored after a kernel before it gave up
        v = self._reduced(stage_ptr, stage_dtype, world, sa_ptr, sw, bias, rows, N)
        X = x.numpy().reshape(-1)[:rows * N].reshape(rows, N)
        types = self._bytes(rtype_ptr, rows)
        table = gate.numpy().reshape(-1, g_stride)[:, :N]
        X[...] = gemm_ref.accumulate_gated(X, v, table, types)

    def reduce_dequant_low_native(self, stage_ptr, slot_stride, stage_stride, stage_dtype, world, sa_ptr, sw, bias, low,
                                  low_stride, outs, out_dtype, c_stride, rows, N, row0=0, rtype_ptr=None, gate=None,
                                  g_stride=0):
        from oracle import gemm_ref
        assert low_stride == N
        if self.status:
            return
        term = low.numpy().reshape(-1)[:rows * N].reshape(rows, N)
        v = self._reduced(stage_ptr, stage_dtype, world, sa_ptr, sw, bias, rows, N, term)
        if gate is not None:
            X = self._bytes(outs[0], rows * N * 4).view(np.float32).reshape(rows, N)
            table = gate.numpy().reshape(-1, g_stride)[:, :N]
            X[...] = gemm_ref.accumulate_gated(X, v, table, self._bytes(rtype_ptr, rows))
            return
        self._store_rows(gemm_ref.store_as(v, out_dtype), outs, out_dtype, rows, N, row0)

    def reduce_dequant_native(self, stage_ptr, slot_stride, stage_stride, stage_dtype, world, sa_ptr, sw, bias, outs,
                              out_dtype, c_stride, rows, N, row0=0):
        from oracle import gemm_ref
        assert stage_stride == N and c_stride == N and slot_stride == rows * N
        if self.status:
            return  # as reduce_dequant_kernel: nothing is stored after a kernel before it gave up
        v = self._reduced(stage_ptr, stage_dtype, world, sa_ptr, sw, bias, rows, N)
        self._store_rows(gemm_ref.store_as(v, out_dtype), outs, out_dtype, rows, N, row0)

    def _store_rows(self, bits, outs, out_dtype, rows, N, row0):
        osize = gpu_mod._SIZE[out_dtype]
        for o in outs:
            dst = self._bytes(o + row0 * N * osize, rows * N * osize)
            dst.view(gpu_mod._NP[out_dtype]).reshape(rows, N)[...] = bits

    def _reduced(self, stage_ptr, stage_dtype, world, sa_ptr, sw, bias, rows, N, low=None):
        from oracle import bf16_bits_to_f32, gemm_ref
        esize = 4 if stage_dtype == "i32" else 2
        stage = self._bytes(stage_ptr, world * rows * N * esize)
        b = bias.numpy().reshape(-1)[:N] if bias is not None else None
        if stage_dtype == "i32":
            acc = stage.view(np.int32).reshape(world, rows, N).sum(axis=0, dtype=np.int32)
            return gemm_ref.epilogue_q8(acc, self._bytes(sa_ptr, rows * 4).view(np.float32), sw.numpy().reshape(-1)[:N], b,
                                        low)
        assert low is None
        parts = bf16_bits_to_f32(stage.view(np.uint16).reshape(world, rows, N))
        v = np.zeros((rows, N), np.float32)
        for s in range(world):
            v = (v + parts[s]).astype(np.float32)
        if b is not None:
            v = (v + b[None, :]).astype(np.float32)
        return v
