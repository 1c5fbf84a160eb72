"""Row-parallel push on ONE GPU: the p ranks of a K-sharded layer are played one after the other by one process,
with every "peer" block a local allocation. Signals are sent first (mode 1) and waited for afterwards (mode 2), so
no kernel ever waits for a kernel that has not run. Checks the push epilogue (tile -> owner slot, transposed
stores), the owner's reduction and the bounded rendezvous through the C ABI against the single-GPU product and the
oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from h3metal_b200.gpu import Gpu
    g = Gpu()
    yield g
    g.close()


def _case(rng, M, N, K):
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sa = rng.uniform(0.01, 0.03, size=M).astype(np.float32)
    sw = rng.uniform(1e-3, 2e-3, size=N).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    return a, w, sa, sw, bias


@pytest.mark.parametrize("world,M,N,K,stage", [
    (1, 256, 256, 512, "i32"), (2, 512, 384, 1024, "i32"), (4, 1024, 4096, 2048, "i32"), (8, 1024, 256, 1024, "i32"),
    (2, 512, 384, 1024, "bf16"), (4, 512, 2048, 1024, "bf16"),
])
def test_pushed_partials_reduce_to_the_single_gpu_product(gpu, world, M, N, K, stage):
    from oracle import gemm_ref
    from h3metal_b200.parallel import push_layout
    rng = np.random.default_rng(world * 100 + N)
    a, w, sa, sw, bias = _case(rng, M, N, K)
    rows, slot_bytes, stage_bytes, out_off, total = push_layout(M, N, world, stage, "bf16")
    esize = 4 if stage == "i32" else 2
    blocks = [gpu.peer_alloc(256 + total) for _ in range(world)]
    base = [b.ptr for b in blocks]
    d_sa, d_sw, d_bias = gpu.upload(sa), gpu.upload(sw), gpu.upload(bias)
    kp = K // world
    shards = [(gpu.upload(np.ascontiguousarray(a[:, r * kp:(r + 1) * kp])),
               gpu.upload(np.ascontiguousarray(w[:, r * kp:(r + 1) * kp]))) for r in range(world)]
    for call in range(3):  # three calls: both staging buffers are used and reused
        buf = (call % 2) * stage_bytes
        for r in range(world):  # rank r: product over its K shard, pushed to every owner's slot r
            slots = [base[o] + 256 + buf + r * slot_bytes for o in range(world)]
            gpu.gemm_push_native(shards[r][0], kp, shards[r][1], kp, d_sw, d_sa, slots, rows, stage, N, M, N, kp)
            gpu.peer_sync_native(base, r, world, call * 2 + 1, mode=1)
        for o in range(world):  # owner o: wait (already satisfied), sum its rows, store them into every output
            gpu.peer_sync_native(base, o, world, call * 2 + 1, mode=2)
            outs = [base[q] + 256 + out_off for q in range(world)]
            gpu.reduce_dequant_native(base[o] + 256 + buf, slot_bytes // esize, N, stage, world, d_sa.ptr + 4 * o * rows,
                                      d_sw, d_bias, outs, "bf16", N, rows, N, row0=o * rows)
        gpu.wait()
        acc = gemm_ref.int32_product(a, w)
        want = gemm_ref.store_as(gemm_ref.epilogue_q8(acc, sa, sw, bias), "bf16")
        for q in range(world):
            got = blocks[q].view((M, N), "bf16", offset_elems=256 + out_off).numpy()
            if stage == "i32":
                assert np.array_equal(got, want), f"call {call}, output copy {q}"
            else:
                from oracle import bf16_bits_to_f32
                g32, w32 = bf16_bits_to_f32(got), bf16_bits_to_f32(want)
                rel = np.linalg.norm(g32 - w32) / np.linalg.norm(w32)
                assert rel < 5e-3, (call, q, rel)  # approximate variant: partials are rounded to bf16 before the sum
    for b in blocks:
        gpu.peer_free(b.ptr)


def test_int32_slots_hold_the_partial_accumulators(gpu):
    """The staged values themselves: slot r of owner o = rows of o of A[:, shard r] W[:, shard r]^T, exactly."""
    from oracle import gemm_ref
    world, M, N, K = 2, 256, 320, 512
    rng = np.random.default_rng(11)
    a, w, sa, sw, _ = _case(rng, M, N, K)
    rows, kp = M // world, K // world
    blocks = [gpu.peer_alloc(world * rows * N * 4) for _ in range(world)]
    d_sa, d_sw = gpu.upload(sa), gpu.upload(sw)
    for r in range(world):
        slots = [blocks[o].ptr + r * rows * N * 4 for o in range(world)]
        gpu.gemm_push_native(gpu.upload(np.ascontiguousarray(a[:, r * kp:(r + 1) * kp])), kp,
                             gpu.upload(np.ascontiguousarray(w[:, r * kp:(r + 1) * kp])), kp, d_sw, d_sa, slots, rows, "i32",
                             N, M, N, kp)
    gpu.wait()
    for o in range(world):
        got = blocks[o].view((world, rows, N), "i32").numpy()
        for r in range(world):
            want = gemm_ref.int32_product(a[o * rows:(o + 1) * rows, r * kp:(r + 1) * kp], w[:, r * kp:(r + 1) * kp])
            assert np.array_equal(got[r], want), (o, r)
    for b in blocks:
        gpu.peer_free(b.ptr)


def test_gated_reduction_matches_the_single_gpu_gated_product(gpu):
    """Owner-side reduction with the reference's epilogue 1: bit-identical to h3b_gemm_w8a8_gated on the whole K."""
    world, M, N, K = 2, 512, 768, 1024
    rng = np.random.default_rng(17)
    a, w, sa, sw, bias = _case(rng, M, N, K)
    x0 = rng.standard_normal((M, N)).astype(np.float32)
    types = rng.integers(0, 4, size=M).astype(np.uint8)
    gates = rng.standard_normal((4, N)).astype(np.float32)
    d_sa, d_sw, d_bias, d_gate, d_types = gpu.upload(sa), gpu.upload(sw), gpu.upload(bias), gpu.upload(gates), gpu.upload(types)
    want = gpu.upload(x0)
    gpu.gemm_gated_native(gpu.upload(a), K, gpu.upload(w), K, d_sw, d_sa, d_bias, want, N, M, N, K, d_types, d_gate, N)
    rows, kp = M // world, K // world
    blocks = [gpu.peer_alloc(world * rows * N * 4) for _ in range(world)]
    for r in range(world):
        slots = [blocks[o].ptr + r * rows * N * 4 for o in range(world)]
        gpu.gemm_push_native(gpu.upload(np.ascontiguousarray(a[:, r * kp:(r + 1) * kp])), kp,
                             gpu.upload(np.ascontiguousarray(w[:, r * kp:(r + 1) * kp])), kp, d_sw, d_sa, slots, rows, "i32",
                             N, M, N, kp)
    got = []
    for o in range(world):
        X = gpu.upload(x0[o * rows:(o + 1) * rows])
        gpu.reduce_dequant_gated_native(blocks[o].ptr, rows * N, N, "i32", world, d_sa.ptr + 4 * o * rows, d_sw, d_bias, X, N,
                                        rows, N, 0, d_types.ptr + o * rows, d_gate, N)
        got.append(X)
    gpu.wait()
    from oracle import gemm_ref
    ref = gemm_ref.accumulate_gated(x0, gemm_ref.epilogue_q8(gemm_ref.int32_product(a, w), sa, sw, bias), gates, types)
    assert np.array_equal(want.numpy(), ref)
    assert np.array_equal(np.concatenate([x.numpy() for x in got]), ref)
    for b in blocks:
        gpu.peer_free(b.ptr)


@pytest.mark.parametrize("world,swiglu", [(2, False), (4, True)])
def test_row_maxima_through_slots_give_the_whole_row_scale(gpu, world, swiglu):
    """K-sharded rotate+quantise with the maxima exchanged through per-rank slots: codes and scales of every shard
    equal the corresponding columns of the unsharded kernel's result, bit for bit."""
    import oracle
    from h3metal_b200 import ops
    M, D, block = 300, 2048, 128
    rng = np.random.default_rng(world)
    cols = 2 * D if swiglu else D
    x = oracle.bf16_round_bits((rng.standard_normal((M, cols)) * 2).astype(np.float32))
    full_q, full_s = gpu.empty((M, D), "i8"), gpu.empty((M,), "f32")
    ops.rot_q8(gpu, gpu.upload(x, "bf16"), full_q, full_s, M, D, swiglu=swiglu, block=block)
    dp = D // world
    tables = [gpu.peer_alloc(world * M * 4) for _ in range(world)]  # one table of `world` slots per rank
    shards = []
    for r in range(world):  # value | gate columns of this rank's K shard, side by side
        parts = [x[:, r * dp:(r + 1) * dp]] + ([x[:, D + r * dp:D + (r + 1) * dp]] if swiglu else [])
        shards.append(gpu.upload(np.ascontiguousarray(np.concatenate(parts, axis=1)), "bf16"))
        gpu.rot_amax_push_native(shards[r], 2 * dp if swiglu else dp, [t.ptr + r * M * 4 for t in tables], M, dp, block,
                                 1 if swiglu else 0)
    gpu.wait()
    want_q, want_s = full_q.numpy(), full_s.numpy()
    for r in range(world):
        q, s = gpu.empty((M, dp), "i8"), gpu.empty((M,), "f32")
        gpu.rot_q8_given_amax_slots_native(shards[r], 2 * dp if swiglu else dp, q, tables[r].ptr, M, world, s, M, dp, block,
                                           1 if swiglu else 0)
        gpu.wait()
        assert np.array_equal(s.numpy(), want_s), r
        assert np.array_equal(q.numpy(), want_q[:, r * dp:(r + 1) * dp]), r
    for t in tables:
        gpu.peer_free(t.ptr)


def test_rendezvous_gives_up_when_a_rank_never_signals(gpu):
    """A wait for a flag nobody sets must run out (about a second), surface at wait() and leave the context usable."""
    from h3metal_b200.gpu import GpuError
    block = gpu.peer_alloc(256)
    gpu.peer_sync_native([block.ptr, block.ptr], 0, 2, 5, mode=2)
    with pytest.raises(GpuError, match="did not signal"):
        gpu.wait()
    gpu.peer_sync_native([block.ptr], 0, 1, 6, mode=0)  # signal and wait on one GPU with one rank: completes
    assert gpu.wait() >= 0.0
    gpu.peer_free(block.ptr)


def test_push_rejects_bad_arguments(gpu):
    from h3metal_b200.gpu import GpuError
    a, w = gpu.empty((256, 128), "i8"), gpu.empty((64, 128), "i8")
    block = gpu.peer_alloc(256 * 64 * 4)
    with pytest.raises(GpuError, match="multiple of 128"):
        gpu.gemm_push_native(a, 128, w, 128, None, None, [block.ptr, block.ptr], 64, "i32", 64, 128, 64, 128)
    with pytest.raises(GpuError, match="rows_per_gpu x world"):
        gpu.gemm_push_native(a, 128, w, 128, None, None, [block.ptr], 128, "i32", 64, 256, 64, 128)
    gpu.peer_free(block.ptr)
