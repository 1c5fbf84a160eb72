"""The five benchmark configurations end to end on one GPU (rotate + quantise, then the product with bias and LoRA)
against the oracle on the same seeded inputs. Small configurations are compared whole; for the large ones the GPU
runs the full size and the oracle checks a sample of rows (the path is row-independent), as the reference's tests
do at real model shapes (tests/test_gemm.py:139-140)."""
import numpy as np
import pytest

import oracle
from oracle import gemm_ref
from h3metal_b200 import ops, workloads
from h3metal_b200.linear import upload_weight
from tests.conftest import rel_fro

pytestmark = pytest.mark.gpu


def _check_layer(gpu, cfg, spec, M, seed, rows, cpu_weights):
    """Runs one linear of `cfg` at M rows on the GPU and checks `rows` of it against the oracle."""
    import torch
    rng = np.random.default_rng(seed)
    K, N, block = spec.K, spec.N, cfg.block
    m_pad = ops.pad_rows(M)
    in_cols = 2 * K if spec.swiglu_in else K
    if cpu_weights:
        codes, scales = workloads.weight_np(rng, N, K, block)
        bias = workloads.bias_np(rng, N) if cfg.bias else None
        xh = workloads.activations_np(rng, m_pad, in_cols, cfg.n_outliers(K))
        X = gpu.upload(xh, "bf16")
        wt = upload_weight(gpu, codes, scales, bias)
    else:
        gen = torch.Generator(device=gpu.torch_device)
        gen.manual_seed(seed)
        codes_t, scales_t = workloads.weight_torch(gen, N, K, gpu.torch_device)
        bias_t = torch.randn(N, generator=gen, device=gpu.torch_device) * 0.01 if cfg.bias else None
        x_t = workloads.activations_torch(gen, m_pad, in_cols, cfg.n_outliers(K), gpu.torch_device)
        X = gpu.wrap(x_t)
        wt = upload_weight(gpu, codes_t, scales_t, bias_t)
        codes, scales = codes_t.cpu().numpy(), scales_t.cpu().numpy()
        bias = bias_t.cpu().numpy() if bias_t is not None else None
        xh = x_t[torch.as_tensor(rows, device=x_t.device)].view(torch.int16).cpu().numpy().view(np.uint16)
    term = None
    if cfg.lora_rank:
        A_l, B_l = workloads.lora_np(rng, cfg.lora_rank, K, N, block)
        wt.low = ops.low_rank(gpu, A_l, B_l, ops.Scratch(gpu))
        term = gemm_ref.low_rank_ref(A_l, B_l)
    a8, sa = gpu.empty((m_pad, K), "i8"), gpu.empty((m_pad,), "f32")
    out = gpu.empty((m_pad, N), "bf16")
    ops.rot_q8(gpu, X, a8, sa, M, K, swiglu=spec.swiglu_in, block=block)
    ops.gemm(gpu, a8, wt, out, M, sa=sa, tile=(128, 32, 4))
    gpu.wait()

    idx = torch.as_tensor(rows, device=gpu.torch_device)
    got_q = a8.torch()[idx].cpu().numpy()
    got_s = sa.torch()[idx].cpu().numpy()
    got_out = out.torch()[idx].view(torch.int16).cpu().numpy().view(np.uint16)
    x_rows = xh[rows] if cpu_weights else xh
    q, s = oracle.rot_q8_rows(x_rows, K, block=block, swiglu=spec.swiglu_in)
    diff = np.abs(got_q.astype(np.int32) - q.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() <= 1e-4, f"{cfg.name}/{spec.name}: codes"
    if not spec.swiglu_in:
        assert diff.max() == 0 and np.array_equal(got_s, s)
    assert np.abs(got_s.view(np.int32).astype(np.int64) - s.view(np.int32).astype(np.int64)).max() <= 3  # ulps (measured worst case, swiglu rows)
    # the product is checked on the GPU's own codes so that a one-step code difference cannot hide in it
    stored, v, _ = gemm_ref.gemm_q8(got_q, codes, got_s, scales, bias, term, "bf16")
    if term is None:
        assert np.array_equal(got_out, stored), f"{cfg.name}/{spec.name}: stored bf16 values"
    assert rel_fro(oracle.bf16_bits_to_f32(got_out), oracle.bf16_bits_to_f32(stored)) <= 1e-3
    # and against the oracle's own codes: the end-to-end acceptance bound
    stored2, _, _ = gemm_ref.gemm_q8(q, codes, s, scales, bias, term, "bf16")
    assert rel_fro(oracle.bf16_bits_to_f32(got_out), oracle.bf16_bits_to_f32(stored2)) <= 1e-3


def _rows(M, n, seed=0):
    return np.unique(np.r_[0:8, M - 8:M, np.random.default_rng(seed).integers(0, M, n)])


def test_config0_whole(gpu):
    cfg = workloads.CONFIGS[0]
    _check_layer(gpu, cfg, cfg.layers[0], cfg.M, 0, np.arange(0, cfg.M, 7), cpu_weights=True)


@pytest.mark.parametrize("layer", range(4))
def test_config1_zimage_block(gpu, layer):
    cfg = workloads.CONFIGS[1]
    _check_layer(gpu, cfg, cfg.layers[layer], cfg.M, 10 + layer, _rows(cfg.M, 48), cpu_weights=False)


@pytest.mark.parametrize("layer", range(4))
def test_config2_flux2_block_with_lora(gpu, layer):
    cfg = workloads.CONFIGS[2]
    _check_layer(gpu, cfg, cfg.layers[layer], cfg.M, 20 + layer, _rows(cfg.M, 48), cpu_weights=False)


@pytest.mark.parametrize("layer", [2, 3])
def test_config2_with_the_reference_swiglu_mlp(gpu, layer):
    """The FLUX.2 block's MLP as the reference runs it (h3metal/flux2.py:142-144; shapes of tests/test_gemm.py:121-124):
    fc1 3072 -> 18432, the SwiGLU quantiser, fc2 9216 -> 3072, with the rank-32 term."""
    cfg = workloads.CONFIGS[5]
    _check_layer(gpu, cfg, cfg.layers[layer], cfg.M, 50 + layer, _rows(cfg.M, 48), cpu_weights=False)


@pytest.mark.parametrize("layer", range(4))
def test_config3_33b_block(gpu, layer):
    cfg = workloads.CONFIGS[3]
    _check_layer(gpu, cfg, cfg.layers[layer], cfg.M, 30 + layer, _rows(cfg.M, 24), cpu_weights=False)


@pytest.mark.parametrize("layer", range(4))
def test_config4_stress_rows_with_lora(gpu, layer):
    """M = 66560 rows with a rank-64 term, every layer at full size (the two widest write 2.4 and 4.4 GB of output):
    whatever the benchmark times has been checked at its real shape first, as the reference insists for its own
    sweeps (docs/design.md:59-69)."""
    import torch
    cfg = workloads.CONFIGS[4]
    _check_layer(gpu, cfg, cfg.layers[layer], cfg.M, 40 + layer, _rows(cfg.M, 24), cpu_weights=False)
    torch.cuda.empty_cache()


@pytest.mark.parametrize("K", [3072, 6144, 16384])
@pytest.mark.parametrize("block", [64, 128, 256])
def test_config4_sweep_blocks(gpu, K, block):
    """The K x block sweep of the stress configuration (N = 6144), at a reduced row count."""
    cfg = workloads.Config("sweep", 1024, (workloads.Linear("lin", K, 6144),), block=block)
    _check_layer(gpu, cfg, cfg.layers[0], cfg.M, K + block, _rows(cfg.M, 16), cpu_weights=False)
