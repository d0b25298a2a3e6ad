"""The 8-bit oracle (oracle/q8_oracle.c) against fixtures made by the reference's own Python functions and the
torch comparators of its unit tests (tests/golden/make_q8_golden.py).  CPU only."""
import os

import numpy as np
import pytest

from oracle import q8_oracle as q8o

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _ulp_bf16(v):
    """Spacing of bf16 at |v| (fp32 array)."""
    e = np.floor(np.log2(np.maximum(np.abs(v), 2.0 ** -126)))
    return np.exp2(e - 7)


def test_fp8_tables_match_torch():
    torch = pytest.importorskip("torch")
    allb = torch.arange(256, dtype=torch.uint8)
    for dt, table in ((torch.float8_e4m3fn, q8o.e4m3_table()), (torch.float8_e5m2, q8o.e5m2_table())):
        ref = allb.view(dt).float().numpy()
        assert np.array_equal(np.isnan(ref), np.isnan(table))
        ok = ~np.isnan(ref)
        assert np.array_equal(ref[ok], table[ok])


def test_e4m3_encode_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-3, 0.02, 1.0, 50.0, 300.0)])
    table = q8o.e4m3_table()
    finite = table[~np.isnan(table)]
    mids = (np.sort(finite)[:-1] + np.sort(finite)[1:]) / 2          # every tie point
    vals = np.clip(np.concatenate([vals, mids.astype(np.float32), finite, [448.0, -448.0, 0.0]]), -448, 448).astype(np.float32)
    ref = torch.from_numpy(vals).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = q8o.f32_to_e4m3(vals)
    same = got == ref
    # +0 / -0 of a zero result may differ in sign handling only if the input was a signed zero; compare values
    assert np.array_equal(table[got[~same]], table[ref[~same]])


@pytest.mark.parametrize("tag", ["bf16", "fp16"])
def test_quantisers_match_reference_functions(tag):
    g = np.load(os.path.join(GOLD, "q8_quant.npz"))
    x = g[f"x_{tag}"]
    bf = tag == "bf16"
    # the fixtures were made on a CPU, where a division by a python number divides
    q, s = q8o.quantize(x, bf, q8o.QUANT_FP8_PER_TENSOR, host_scalar_reciprocal=False)
    assert np.array_equal(s, g[f"pt_s_{tag}"]) and np.array_equal(q, g[f"pt_q_{tag}"])
    q, s = q8o.quantize(x, bf, q8o.QUANT_FP8_PER_TOKEN, host_scalar_reciprocal=False)
    assert np.array_equal(s, g[f"tok_s_{tag}"]) and np.array_equal(q, g[f"tok_q_{tag}"])
    q, _ = q8o.quantize(x, bf, q8o.QUANT_FP8_STATIC, static_scale=float(g["static_scale"][0]))
    assert np.array_equal(q, g[f"st_q_{tag}"])
    q, s = q8o.quantize(x, bf, q8o.QUANT_INT8_PER_TENSOR, weight_scale=float(g["sq_weight_scale"][0]),
                        host_scalar_reciprocal=False)
    assert np.array_equal(q, g[f"sq_q_{tag}"])
    assert s[0] == g[f"sq_s_{tag}"][0] and s[1] == g[f"sq_alpha_{tag}"][0]


def test_reciprocal_rule_differs_only_by_scale_rounding():
    """The GPU rule (multiply by the fp32 reciprocal) gives the same scale as a division except on rare inputs; on
    these fixtures they agree, and the rule is exercised at a value where they do not."""
    g = np.load(os.path.join(GOLD, "q8_quant.npz"))
    for tag in ("bf16", "fp16"):
        _, s0 = q8o.quantize(g[f"x_{tag}"], tag == "bf16", q8o.QUANT_FP8_PER_TOKEN, host_scalar_reciprocal=False)
        _, s1 = q8o.quantize(g[f"x_{tag}"], tag == "bf16", q8o.QUANT_FP8_PER_TOKEN, host_scalar_reciprocal=True)
        assert np.max(np.abs(s0 - s1) / s0) < 2 ** -7


def test_int8_gemm_exact_and_unit_test_comparator():
    g = np.load(os.path.join(GOLD, "q8_int8_gemm.npz"))
    acc = q8o.gemm_acc(g["x"], g["w"], q8o.KIND_INT8)
    assert np.array_equal(acc, g["acc"].astype(np.float32))           # |acc| < 2^24: exact in fp32
    y = q8o.tensorwise(g["x"], g["w"], g["bias"], float(g["alpha"][0]), 1.0, out_bf16=False, kind=q8o.KIND_INT8)
    y = y.view(np.float16).astype(np.float32)
    # fp32 restatement of alpha * acc + bias, one rounding to fp16
    want = (np.float32(g["alpha"][0]) * g["acc"].astype(np.float64) + g["bias"].astype(np.float64)).astype(np.float16)
    assert np.max(np.abs(y - want.astype(np.float32))) <= np.max(np.spacing(np.abs(want)).astype(np.float32))
    assert np.mean(y != want.astype(np.float32)) < 1e-3
    # the reference's unit test: allclose(fp16 nn.Linear on dequantised operands, atol=0.1)
    assert np.allclose(y, g["y_fp16_linear"].astype(np.float32), atol=0.1)


def test_fp8_tensorwise_matches_scaled_mm():
    g = np.load(os.path.join(GOLD, "q8_fp8_gemm.npz"))
    y = q8o.tensorwise(g["a"], g["b"], None, float(g["alpha"][0]), 1.0, out_bf16=True)
    got, want = q8o.bf16_bits_to_f32(y), q8o.bf16_bits_to_f32(g["scaled_mm"])
    # the comparator accumulates in fp32: allow its rounding noise on top of one bf16 step
    slack = 1e-6 * float(g["alpha"][0]) * q8o.gemm_abs(g["a"], g["b"], q8o.KIND_E4M3)
    assert np.all(np.abs(got - want) <= _ulp_bf16(want) + slack)
    assert np.mean(got != want) < 0.01
    yb = q8o.tensorwise(g["a"], g["b"], (g["bias"], "bf16"), float(g["alpha"][0]), 1.0, out_bf16=True)
    gotb, wantb = q8o.bf16_bits_to_f32(yb), q8o.bf16_bits_to_f32(g["scaled_mm_bias"])
    # the comparator rounds to bf16 before adding the bias (two roundings), the kernel semantics round once
    assert np.all(np.abs(gotb - wantb) <= 2 * _ulp_bf16(np.maximum(np.abs(wantb), np.abs(want))))
    # the reference's unit test tolerance
    assert np.allclose(gotb, wantb, atol=0.25)


def test_fp8_rowwise_matches_float64_product():
    g = np.load(os.path.join(GOLD, "q8_fp8_gemm.npz"))
    y = q8o.rowwise(g["a"], g["b"], None, g["row_sa"], g["row_sb"])
    got, want = q8o.bf16_bits_to_f32(y), g["row_f64"]
    assert np.all(np.abs(got - want) <= 0.51 * _ulp_bf16(want) + 1e-6 * np.abs(want))


@pytest.mark.parametrize("kind", ["tensor", "token"])
def test_module_forward_matches_reference_dequant_path(kind):
    """quantise (oracle) -> GEMM (oracle) against the reference's FP8DynamicLinear forward in its
    dequantise-and-matmul mode: same quantised operands, bf16 matmul arithmetic there, so a loose bound."""
    g = np.load(os.path.join(GOLD, "q8_fp8_gemm.npz"))
    x = g["mod_x"].reshape(-1, 256)
    ws = g[f"mod_ws_{kind}"]
    if kind == "tensor":
        q, s = q8o.quantize(x, True, q8o.QUANT_FP8_PER_TENSOR, host_scalar_reciprocal=False)
        y = q8o.tensorwise(q, g["b"], (g["bias"], "bf16"), float(np.float32(ws[0]) * s[0]), 1.0, out_bf16=True)
    else:
        q, s = q8o.quantize(x, True, q8o.QUANT_FP8_PER_TOKEN, host_scalar_reciprocal=False)
        y = q8o.rowwise(q, g["b"], (g["bias"], "bf16"), s, ws.reshape(-1))
    got = q8o.bf16_bits_to_f32(y)
    want = q8o.bf16_bits_to_f32(g[f"mod_y_{kind}"]).reshape(got.shape)
    err = np.max(np.abs(got - want)) / np.max(np.abs(want))
    assert err < 2e-2, err
