"""The steps either side of the product (activation quantisation, dequantising bfloat16 output) on the GPU against
their CPU restatement, bit for bit.  The integer product inside is checked against the oracle as everywhere else."""
import os
import sys

import numpy as np
import pytest

import oracle_lib
import ternixengine_b200 as tb

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import bitnet_scaling_oracle as scaling  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1, 2560), (37, 4099), (256, 8192), (5, 3)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_quantize_rows_matches_restatement(shape, dtype):
    import torch
    rng = np.random.default_rng(shape[0] + shape[1])
    x = (rng.standard_normal(shape) * rng.uniform(0.01, 30.0, size=(shape[0], 1))).astype(np.float32)
    x[0, 0] = 0.0
    if shape[0] > 2:
        x[2, :] = 0.0                                        # an all-zero row
    xt = torch.from_numpy(x).cuda().to(getattr(torch, dtype))
    x_ref = xt.float().cpu().numpy()                         # what the kernel really sees
    q, s = tb.quantize_rows(xt)
    q_ref, s_ref = scaling.quantize_rows(x_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))


@pytest.mark.parametrize("shape", [(512, 1024, 2048), (300, 2064, 832), (1, 2560, 6912), (32, 4096, 1024), (7, 129, 4)])
def test_matmul_dequant_bf16(shape):
    """Fused epilogue (large M) and the unfused fallback: the same bits as the restatement on the exact product."""
    import torch
    m, k, n = shape
    a = tb.synth_activations((m, k), 3 * m + k)
    wp = tb.synth_packed_weights(k, n, 5 * n + 1)
    c = oracle_lib.matmul(a, wp)
    row_scale = np.random.default_rng(m).uniform(1e-3, 0.2, size=m).astype(np.float32)
    w_scale = 0.0371
    expect = scaling.dequant_bf16_bits(c, row_scale, w_scale)
    wide = torch.full((m, n + 8), 7.0, dtype=torch.bfloat16, device="cuda")
    twin = torch.zeros((m, n + 8), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = tb.matmul_dequant(torch.from_numpy(a).cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(row_scale).cuda(),
                            w_scale, out=wide[:, :n], status=status, extra_dest_ptrs=(twin.data_ptr(),))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = out.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, expect), f"{int((got != expect).sum())} of {got.size} bf16 outputs differ"
    assert bool((wide[:, n:] == 7.0).all())
    assert np.array_equal(twin[:, :n].contiguous().view(torch.int16).cpu().numpy().view(np.uint16), expect)


def test_quantize_then_matmul_dequant_end_to_end():
    """float activations -> int8 -> exact ternary product -> bf16, close to the float product within the
    quantisation error the recipe implies (|error| <= 0.5 * row_scale * w_scale * sum_k |w| per output)."""
    import torch
    m, k, n = 256, 2560, 2560
    rng = np.random.default_rng(0)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = tb.synth_weights(k, n, 9)
    xt = torch.from_numpy(x).cuda()
    q, s = tb.quantize_rows(xt)
    y = tb.matmul_dequant(q, torch.from_numpy(tb.pack_ternary(w)).cuda(), s, 0.5).float().cpu().numpy()
    exact = (x.astype(np.float64) @ w.astype(np.float64)) * 0.5
    bound = 0.5 * s.cpu().numpy()[:, None].astype(np.float64) * 0.5 * np.abs(w).sum(axis=0)[None, :] + \
        np.abs(exact) * 2.0 ** -8 + 1e-6
    assert (np.abs(y - exact) <= bound).all()
