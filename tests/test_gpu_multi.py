"""One process per GPU, NCCL for the plumbing: the sharded layers of h3metal_b200.parallel against the single-GPU
result, including the row-parallel variants that push their partials through peer-mapped memory. The two-GPU case is
skipped on a box with one GPU (the CPU suite covers the orchestration with gloo); the one-rank case runs anywhere."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["H3B_ROOT"])
import oracle
from oracle import gemm_ref
from h3metal_b200 import ops, parallel
from h3metal_b200.gpu import Gpu

rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
g = Gpu(device=rank)
M, D, F, B = 1024, 1024, 2048, 128
rng = np.random.default_rng(5)
x = oracle.bf16_round_bits((rng.standard_normal((M, D)) * 2).astype(np.float32))
w_up = rng.integers(-127, 128, size=(2 * F, D), dtype=np.int8); s_up = rng.uniform(1e-3, 2e-3, size=2 * F).astype(np.float32)
b_up = (rng.standard_normal(2 * F) * 0.01).astype(np.float32)
w_dn = rng.integers(-127, 128, size=(D, F), dtype=np.int8); s_dn = rng.uniform(1e-3, 2e-3, size=D).astype(np.float32)
b_dn = (rng.standard_normal(D) * 0.01).astype(np.float32)
up = parallel.ColumnParallelLinear(g, None, w_up, s_up, b_up, M, block=B, splits=[F, F])
down = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=B, swiglu_in=True)
h_local = up(g.upload(x, "bf16"))
y = down(h_local)
g.wait()
# single-GPU result with the same kernels
full_up = ops.QWeight("q8", g.upload(w_up), g.upload(s_up), 2 * F, D, bias=g.upload(b_up))
full_dn = ops.QWeight("q8", g.upload(w_dn), g.upload(s_dn), D, F, bias=g.upload(b_dn))
a8, sa, h = g.empty((M, D), "i8"), g.empty((M,), "f32"), g.empty((M, 2 * F), "bf16")
ops.rot_q8(g, g.upload(x, "bf16"), a8, sa, M, D, block=B); ops.gemm(g, a8, full_up, h, M, sa=sa, tile=(128, 32, 4))
a8b, sab, y1 = g.empty((M, F), "i8"), g.empty((M,), "f32"), g.empty((M, D), "bf16")
ops.rot_q8(g, h, a8b, sab, M, F, swiglu=True, block=B); ops.gemm(g, a8b, full_dn, y1, M, sa=sab, tile=(128, 32, 4))
g.wait()
hh = h.numpy(); want_local = np.concatenate([hh[:, a:b] for a, b in up.slices], axis=1)
assert np.array_equal(h_local.numpy(), want_local), "column-parallel output"
assert np.array_equal(down.sa.numpy(), sab.numpy()), "whole-row scales"
half = F // world
assert np.array_equal(down.a8.numpy(), a8b.numpy()[:, rank * half:(rank + 1) * half]), "K-shard codes"
assert np.array_equal(y.numpy(), y1.numpy()), "row-parallel output"
r0 = rank * (M // world)
for reduce, scatter in (("int32", True), ("push", False), ("push", True), ("push_bf16", False), ("push_bf16", True)):
    layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=B, swiglu_in=True, reduce=reduce, scatter=scatter)
    for call in range(3):  # staging buffers alternate and are reused
        yp = layer(h_local)
        g.wait()
        want = y1.numpy()[r0:r0 + M // world] if scatter else y1.numpy()
        if reduce == "push_bf16":
            a, b = oracle.bf16_bits_to_f32(yp.numpy()), oracle.bf16_bits_to_f32(want)
            rel = np.linalg.norm(a - b) / np.linalg.norm(b)
            assert rel < 5e-3, (reduce, scatter, call, rel)
        else:
            assert np.array_equal(yp.numpy(), want), (reduce, scatter, call)
    layer.close()
# column-parallel with a LoRA term (B's rows follow the weight's): this rank's columns of the single-GPU result
A_l = (rng.standard_normal((32, D)) / np.sqrt(D)).astype(np.float32)
B_l = (rng.standard_normal((2 * F, 32)) * 0.5).astype(np.float32)
up_l = parallel.ColumnParallelLinear(g, None, w_up, s_up, b_up, M, block=B, splits=[F, F], lora=(A_l, B_l))
h_lora_local = up_l(g.upload(x, "bf16"))
full_l = ops.QWeight("q8", g.upload(w_up), g.upload(s_up), 2 * F, D, bias=g.upload(b_up),
                     low=ops.low_rank(g, A_l, B_l, ops.Scratch(g)))
h_lora = g.empty((M, 2 * F), "bf16")
ops.gemm(g, a8, full_l, h_lora, M, sa=sa, tile=(128, 32, 4))
g.wait()
hl = h_lora.numpy()
assert not np.array_equal(hl, hh), "the LoRA term changes the output"
assert np.array_equal(h_lora_local.numpy(), np.concatenate([hl[:, a:b] for a, b in up_l.slices], axis=1)), "column-parallel LoRA"
# the same layer accumulating into this rank's rows of an fp32 residual stream (the reference's epilogue 1)
rows = M // world
rng2 = np.random.default_rng(77)
x_stream = rng2.standard_normal((M, D)).astype(np.float32)
types = rng2.integers(0, 3, size=M).astype(np.uint8)
gates = rng2.standard_normal((3, D)).astype(np.float32)
X1 = g.upload(x_stream)
ops.gemm(g, a8b, full_dn, X1, M, sa=sab, epi=1, rtype=g.upload(types), gate=g.upload(gates), g_stride=D, tile=(128, 32, 4))
layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=B, swiglu_in=True, reduce="push", scatter=True)
X = g.upload(x_stream[r0:r0 + rows])
layer.accumulate_gated(h_local, X, g.upload(types[r0:r0 + rows]), g.upload(gates), D)
g.wait()
assert np.array_equal(X.numpy(), X1.numpy()[r0:r0 + rows]), "gated accumulate on the owner's rows"
layer.close()
# a LoRA term on the row-parallel layer: T of the owner's rows is one GPU's T bit for bit (exact int32 partial sums
# over the K shards); the output differs from one GPU's only by where the term's fp32 MMAs ran
A_d = (rng.standard_normal((40, F)) / np.sqrt(F)).astype(np.float32)
B_d = (rng.standard_normal((D, 40)) * 0.5).astype(np.float32)
scr = ops.Scratch(g)
full_dl = ops.QWeight("q8", g.upload(w_dn), g.upload(s_dn), D, F, bias=g.upload(b_dn), low=ops.low_rank(g, A_d, B_d, scr))
y_l1 = g.empty((M, D), "bf16")
ops.gemm(g, a8b, full_dl, y_l1, M, sa=sab, tile=(128, 32, 4))
g.wait()
T1 = scr.t.view((M, 64)).numpy().copy()
assert not np.array_equal(y_l1.numpy(), y1.numpy()), "the LoRA term changes the output"
layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=B, swiglu_in=True, reduce="push", lora=(A_d, B_d))
for call in range(2):
    y_l = layer(h_local)
    g.wait()
    assert np.array_equal(layer.t_rows.numpy(), T1[r0:r0 + rows]), "T of the owner's rows"
    a, b = oracle.bf16_bits_to_f32(y_l.numpy()), oracle.bf16_bits_to_f32(y_l1.numpy())
    rel = np.linalg.norm(a - b) / np.linalg.norm(b)
    assert rel <= 1e-5, ("row-parallel LoRA", call, rel)
layer.close()
dist.barrier(); dist.destroy_process_group()
print(f"rank {rank} ok")
'''


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_sharded_layers_match_one_gpu_bit_for_bit(tmp_path, world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), H3B_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {rank} ok" in out, out[-2000:]
