"""Multi-rank orchestration of h3metal_b200.parallel on CPU: two gloo ranks, kernels replaced by the oracle
(tests/fakes.py: OracleBackedGpu). Checks the sharding plans and that every strategy reproduces the single-rank
result bit for bit (row-parallel: whole-row scales through the MAX all-reduce, exact int32 SUM all-reduce)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle import gemm_ref
from h3metal_b200 import parallel

WORLD = 2
M, D, F, BLOCK = 256, 512, 1024, 128


def test_shard_plans():
    assert parallel.shard_bounds(1024, 1, 4, 128) == (256, 512)
    with pytest.raises(ValueError):
        parallel.shard_bounds(1000, 0, 4, 128)
    # q | k | v fused output: each rank takes its share of every third
    assert parallel.column_slices(3 * 512, [512, 512, 512], 1, 2) == [(256, 512), (768, 1024), (1280, 1536)]
    # value | gate: matching halves
    assert parallel.column_slices(2 * 1024, [1024, 1024], 0, 2) == [(0, 512), (1024, 1536)]
    with pytest.raises(ValueError):
        parallel.column_slices(100, [60, 30], 0, 2)
    # peer block of a push layer: two staging buffers of `world` slots, then the gathered output
    assert parallel.push_layout(1024, 512, 4, "i32", "bf16") == (256, 256 * 512 * 4, 4 * 256 * 512 * 4, 2 * 1024 * 512 * 4,
                                                                  2 * 1024 * 512 * 4 + 1024 * 512 * 2)
    assert parallel.push_layout(1024, 512, 4, "bf16", None)[4] == 2 * 1024 * 512 * 2
    with pytest.raises(ValueError):
        parallel.push_layout(384, 512, 2, "i32", None)  # 192 rows per rank: not whole 128-row tiles
    a = np.arange(12).reshape(6, 2)
    assert parallel.take_rows(a, [(0, 1), (4, 6)]).tolist() == [[0, 1], [8, 9], [10, 11]]


def _inputs():
    rng = np.random.default_rng(7)
    x = oracle.bf16_round_bits((rng.standard_normal((M, D)) * 2).astype(np.float32))
    w_up = rng.integers(-127, 128, size=(2 * F, D), dtype=np.int8)       # value | gate, column-parallel
    s_up = rng.uniform(1e-3, 2e-3, size=2 * F).astype(np.float32)
    b_up = (rng.standard_normal(2 * F) * 0.01).astype(np.float32)
    w_dn = rng.integers(-127, 128, size=(D, F), dtype=np.int8)           # row-parallel, fed by swiglu
    s_dn = rng.uniform(1e-3, 2e-3, size=D).astype(np.float32)
    b_dn = (rng.standard_normal(D) * 0.01).astype(np.float32)
    return x, (w_up, s_up, b_up), (w_dn, s_dn, b_dn)


def _adapter(rank=24):
    """A rank-24 adapter of the down projection (A in the rotated input space), rounded up to 32 ranks when stored."""
    rng = np.random.default_rng(11)
    A_l = (rng.standard_normal((rank, F)) / np.sqrt(F)).astype(np.float32)
    B_l = (rng.standard_normal((D, rank)) * 0.5).astype(np.float32)
    return A_l, B_l


def _single_rank_reference():
    x, (w_up, s_up, b_up), (w_dn, s_dn, b_dn) = _inputs()
    q, s = oracle.rot_q8_rows(x, D, block=BLOCK)
    h, _, _ = gemm_ref.gemm_q8(q, w_up, s, s_up, b_up, None, "bf16")
    q2, s2 = oracle.rot_q8_rows(h, F, block=BLOCK, swiglu=True)
    y, _, acc = gemm_ref.gemm_q8(q2, w_dn, s2, s_dn, b_dn, None, "bf16")
    return h, q2, s2, y


def _worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        from tests.fakes import SharedPeerGpu
        g = SharedPeerGpu()
        x, (w_up, s_up, b_up), (w_dn, s_dn, b_dn) = _inputs()
        up = parallel.ColumnParallelLinear(g, None, w_up, s_up, b_up, M, block=BLOCK, splits=[F, F])
        down = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True)
        h_local = up(g.upload(x, "bf16"))
        y = down(h_local)
        down_rs = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, scatter=True)
        y_rows = down_rs(h_local)
        down_f32 = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, reduce="f32")
        y_fast = down_f32(h_local)
        pushed = {}
        for reduce, scatter in (("push", False), ("push", True), ("push_bf16", False), ("push_bf16", True)):
            layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, reduce=reduce,
                                               scatter=scatter)
            outs = [layer(h_local).numpy().copy() for _ in range(3)]  # three calls: both staging buffers, reused
            assert all(np.array_equal(o, outs[0]) for o in outs)
            pushed[(reduce, scatter)] = outs[0]
            layer.close()
        # the same layer accumulating into this rank's rows of an fp32 residual stream (the reference's epilogue 1)
        rows = M // WORLD
        rng2 = np.random.default_rng(99)
        x_stream = rng2.standard_normal((M, D)).astype(np.float32)
        types = rng2.integers(0, 3, size=M).astype(np.uint8)
        gates = rng2.standard_normal((3, D)).astype(np.float32)
        layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, reduce="push", scatter=True)
        X = g.upload(x_stream[rank * rows:(rank + 1) * rows])
        layer.accumulate_gated(h_local, X, g.upload(types[rank * rows:(rank + 1) * rows]), g.upload(gates), D)
        gated = X.numpy().copy()
        layer.close()
        # a low-rank term on the row-parallel layer: T's partial sums pushed and reduced like the main product's
        A_l, B_l = _adapter()
        layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, reduce="push",
                                           lora=(A_l, B_l))
        y_lora = [layer(h_local).numpy().copy() for _ in range(2)]
        t_rows = layer.t_rows.numpy().copy()
        layer.close()
        layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, reduce="push",
                                           scatter=True, lora=(A_l, B_l))
        X = g.upload(x_stream[rank * rows:(rank + 1) * rows])
        layer.accumulate_gated(h_local, X, g.upload(types[rank * rows:(rank + 1) * rows]), g.upload(gates), D)
        gated_lora = X.numpy().copy()
        layer.close()
        with pytest.raises(ValueError):
            parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, reduce="int32",
                                       lora=(A_l, B_l))
        tok = parallel.TokenShardedLinear(g, None, parallel.ops.QWeight("q8", g.upload(w_up), g.upload(s_up), 2 * F, D,
                                                                         bias=g.upload(b_up)), M, block=BLOCK)
        h_tok = tok(g.upload(x[tok.m0:tok.m0 + tok.rows], "bf16"))
        results[rank] = dict(slices=up.slices, h_local=h_local.numpy().copy(), a8=down.a8.numpy().copy(),
                             sa=down.sa.numpy().copy(), y=y.numpy().copy(), y_rows=(down_rs.r0, y_rows.numpy().copy()), y_fast=y_fast.numpy().copy(),
                             tok=(tok.m0, tok.rows, h_tok.numpy().copy()), pushed=pushed, gated=gated, y_lora=y_lora,
                             t_rows=t_rows, gated_lora=gated_lora)
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_one_rank_bit_for_bit():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(port, results), nprocs=WORLD, join=True)
    h, q2, s2, y = _single_rank_reference()
    half = F // WORLD
    for rank in range(WORLD):
        r = results[rank]
        # column-parallel: this rank's value and gate slices, side by side
        assert r["slices"] == [(rank * half, (rank + 1) * half), (F + rank * half, F + (rank + 1) * half)]
        want_local = np.concatenate([h[:, a:b] for a, b in r["slices"]], axis=1)
        assert np.array_equal(r["h_local"], want_local)
        # row-parallel: codes of this K shard quantised with the WHOLE row's scale; exact output on every rank
        assert np.array_equal(r["a8"], q2[:, rank * half:(rank + 1) * half])
        assert np.array_equal(r["sa"], s2)
        assert np.array_equal(r["y"], y)
        r0, y_rows = r["y_rows"]  # reduce-scatter: this rank's rows of the same exact result
        assert r0 == rank * M // WORLD and np.array_equal(y_rows, y[r0:r0 + M // WORLD])
        # approximate variant (fp32 partials): inside the path's 1e-3 bound
        got = oracle.bf16_bits_to_f32(r["y_fast"]).astype(np.float64)
        want = oracle.bf16_bits_to_f32(y).astype(np.float64)
        assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3
        # push variants: partials through (here: file-backed) peer memory; exact for int32 staging
        for (reduce, scatter), got in r["pushed"].items():
            want_rows = y[r0:r0 + M // WORLD] if scatter else y
            if reduce == "push":
                assert np.array_equal(got, want_rows), (reduce, scatter)
            else:
                a, b = oracle.bf16_bits_to_f32(got).astype(np.float64), oracle.bf16_bits_to_f32(want_rows).astype(np.float64)
                assert np.linalg.norm(a - b) / np.linalg.norm(b) <= 5e-3, (reduce, scatter)
        # gated accumulate on the rank's own rows: X += gate[type] * (product + bias), fp32, from the exact int32 sum
        rng2 = np.random.default_rng(99)
        x_stream = rng2.standard_normal((M, D)).astype(np.float32)
        types = rng2.integers(0, 3, size=M).astype(np.uint8)
        gates = rng2.standard_normal((3, D)).astype(np.float32)
        acc = gemm_ref.int32_product(q2, _inputs()[2][0])
        v = gemm_ref.epilogue_q8(acc, s2, _inputs()[2][1], _inputs()[2][2])
        want_x = gemm_ref.accumulate_gated(x_stream, v, gates, types)
        assert np.array_equal(r["gated"], want_x[r0:r0 + M // WORLD])
        # low-rank term on the row-parallel layer: T of the rank's rows equals one GPU's T bit for bit (exact int32
        # partial sums), and so does the output, the term joining after the bias as in the product's own epilogue
        term = gemm_ref.low_rank_ref(*_adapter())
        T = gemm_ref.lora_T(q2, s2, term)
        assert np.array_equal(r["t_rows"], T[r0:r0 + M // WORLD])
        y_term, v_term, _ = gemm_ref.gemm_q8(q2, _inputs()[2][0], s2, _inputs()[2][1], _inputs()[2][2], term, "bf16")
        assert all(np.array_equal(o, y_term) for o in r["y_lora"])
        assert not np.array_equal(y_term, y)  # the term is there
        want_x = gemm_ref.accumulate_gated(x_stream, v_term, gates, types)
        assert np.array_equal(r["gated_lora"], want_x[r0:r0 + M // WORLD])
        # token-sharded: rows of the full result
        m0, rows, h_tok = r["tok"]
        assert (m0, rows) == (rank * M // WORLD, M // WORLD) and np.array_equal(h_tok, h[m0:m0 + rows])


def _late_rank_worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        from h3metal_b200.gpu import GpuError
        from tests.fakes import SharedPeerGpu
        g = SharedPeerGpu(sync_limit_s=1.0)
        x, (w_up, s_up, b_up), (w_dn, s_dn, b_dn) = _inputs()
        up = parallel.ColumnParallelLinear(g, None, w_up, s_up, b_up, M, block=BLOCK, splits=[F, F])
        # float inputs make the layer exchange its row maxima through the process group, so the only rendezvous of a
        # call are the two around the owner's reduction
        h32 = g.upload(oracle.bf16_bits_to_f32(up(g.upload(x, "bf16")).numpy()))
        layer = parallel.RowParallelLinear(g, None, w_dn, s_dn, b_dn, M, block=BLOCK, swiglu_in=True, reduce="push")
        first = layer(h32).numpy().copy()
        g.wait()
        layer.out.numpy()[...] = 0
        dist.barrier()
        # second step: rank 1 never joins it (a rank that stalled on the host between steps). Rank 0 runs its half
        # alone: the quantiser's scales are given (the MAX exchange is a host-side collective that would simply
        # block), so it goes straight to the product, the rendezvous and the reduction.
        error = None
        if rank == 0:
            layer._push(g, layer.wt)
            try:
                g.wait()
            except GpuError as e:
                error = str(e)
        dist.barrier()
        after_failure = layer.out.numpy().copy()
        layer.recover()
        third = layer(h32).numpy().copy()
        g.wait()
        results[rank] = dict(first=first, error=error, after_failure=after_failure, third=third, rows=layer.rows)
        layer.close()
    finally:
        dist.destroy_process_group()


def test_row_parallel_layer_when_one_rank_never_arrives():
    """What a pushed row-parallel layer returns and raises when a rank never reaches the rendezvous (made on the host:
    rank 1 sits the step out; the fake's poll is bounded like the device's). The rank that waited in vain reports the
    give-up at wait(); its reduction stored nothing - no rank's output received sums over staging that was never
    filled - and after recover() on both ranks the layer computes the right result again."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(_late_rank_worker, args=(port, results), nprocs=WORLD, join=True)
    _, _, _, y = _single_rank_reference()
    for rank in range(WORLD):
        r = results[rank]
        assert np.array_equal(r["first"], y), "before the failure"
        assert not r["after_failure"].any(), "a reduction behind a rendezvous that ran out must store nothing"
        assert np.array_equal(r["third"], y), "after recover()"
    assert results[0]["error"] is not None and "did not signal" in results[0]["error"]
    assert results[1]["error"] is None
