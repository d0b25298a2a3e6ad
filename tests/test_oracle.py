"""The numpy oracle against fixtures produced by the reference's own functions
(tests/golden/make_golden.py).  CPU only."""
import hashlib
import os

import numpy as np
import pytest

from oracle import awq_oracle as orc


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_nibble_order_tables():
    # slot i of a word holds logical channel ORDER[i]; REV is its inverse.
    for j in range(8):
        assert orc.AWQ_ORDER[orc.AWQ_REVERSE_ORDER[j]] == j
    word = 0
    for slot, logical in enumerate(orc.AWQ_ORDER):
        word |= logical << (4 * slot)
    got = orc.unpack_logical(np.array([[word]], dtype=np.uint32).view(np.int32))
    assert got.tolist() == [[0, 1, 2, 3, 4, 5, 6, 7]]


def test_pack_unpack_roundtrip():
    rng = np.random.default_rng(3)
    v = rng.integers(0, 16, size=(37, 64))
    assert np.array_equal(orc.unpack_logical(orc.pack_logical(v)), v)
    with pytest.raises(ValueError):
        orc.pack_logical(np.full((1, 8), 16))


def test_dequant_bit_exact_small(golden_dir):
    g = _load(golden_dir, "awq_small.npz")
    W = orc.dequantize(g["qweight"], g["qzeros"], g["scales"], int(g["group_size"]))
    assert np.array_equal(W.view(np.uint16), g["W"].view(np.uint16))


def test_dequant_bit_exact_all_pairs(golden_dir):
    g = _load(golden_dir, "awq_all_pairs.npz")
    assert np.array_equal(orc.unpack_logical(g["qweight"]), g["q"])
    assert np.array_equal(orc.unpack_logical(g["qzeros"]), g["z"])
    W = orc.dequantize(g["qweight"], g["qzeros"], g["scales"], int(g["group_size"]))
    assert np.array_equal(W.view(np.uint16), g["W_bits"])
    # every (q, z) pair occurs
    pairs = set(zip(g["q"][:128].ravel().tolist(), np.repeat(g["z"][:1], 128, 0).ravel().tolist()))
    assert len(pairs) == 256


def test_quantise_and_pack_match_reference(golden_dir):
    g = _load(golden_dir, "awq_small.npz")
    G = int(g["group_size"])
    w_fake, s_nk, z_nk = orc.rtn_quantize(g["w"], G)
    assert np.array_equal(w_fake.view(np.uint16), g["w_fake"].view(np.uint16))
    assert np.array_equal(s_nk.T.view(np.uint16), g["scales_kn"].view(np.uint16))
    assert np.array_equal(z_nk.T.astype(np.float16), g["zeros_kn"])
    qw, qz, sc = orc.pack_linear(w_fake, np.ascontiguousarray(s_nk.T),
                                 np.ascontiguousarray(z_nk.T), G)
    assert np.array_equal(qw, g["qweight"])
    assert np.array_equal(qz, g["qzeros"])
    assert np.array_equal(sc.view(np.uint16), g["scales"].view(np.uint16))


def test_forward_small(golden_dir):
    g = _load(golden_dir, "awq_small.npz")
    y = orc.linear_forward(g["x"], g["qweight"], g["qzeros"], g["scales"], int(g["group_size"]))
    ref = g["y"]                      # reference returns [1, M, N] for 2-D input
    assert ref.shape == (1,) + y.shape
    # accumulation order of the reference's BLAS call is unspecified: 1e-3 of max|ref|
    assert orc.max_normalised_error(y, ref[0]) <= 1e-3


def test_forward_bias_3d(golden_dir):
    g = _load(golden_dir, "awq_bias_3d.npz")
    G = int(g["group_size"])
    y3 = orc.linear_forward(g["x3"], g["qweight"], g["qzeros"], g["scales"], G, g["bias"])
    assert y3.shape == g["y3"].shape
    assert orc.max_normalised_error(y3, g["y3"]) <= 1e-3
    assert tuple(g["ybf_shape"]) == (1, 5, 64)
    assert tuple(g["y_empty_shape"]) == (0, 64)


def test_config1_generator_and_forward(golden_dir):
    g = _load(golden_dir, "awq_config1_slice.npz")
    K, N, M, G = int(g["K"]), int(g["N"]), int(g["M"]), int(g["group_size"])
    qw, qz, sc = orc.make_awq_tensors(K, N, G, seed=int(g["seed"]))
    assert hashlib.sha256(qw.tobytes()).digest() == g["qweight_sha256"].tobytes()
    W = orc.dequantize(qw, qz, sc, G)
    assert hashlib.sha256(W.tobytes()).digest() == g["W_sha256"].tobytes()
    assert np.array_equal(W[:, :64].view(np.uint16), g["W_cols_0_64"].view(np.uint16))
    x = orc.make_activations(M, K, seed=int(g["seed"]))
    y = orc.linear_forward(x, qw, qz, sc, G)
    assert orc.max_normalised_error(y, g["y"][0]) <= 1e-3


# ---- the C restatement (used as the timed CPU baseline) ----------------------------------
def test_c_oracle_matches_goldens(golden_dir):
    from oracle import c_oracle
    g = _load(golden_dir, "awq_all_pairs.npz")
    W = c_oracle.dequantize(g["qweight"], g["qzeros"], g["scales"], int(g["group_size"]))
    assert np.array_equal(W.view(np.uint16), g["W_bits"])
    g = _load(golden_dir, "awq_small.npz")
    G = int(g["group_size"])
    assert np.array_equal(c_oracle.dequantize(g["qweight"], g["qzeros"], g["scales"], G).view(np.uint16),
                          g["W"].view(np.uint16))
    y = c_oracle.linear_forward(g["x"], g["qweight"], g["qzeros"], g["scales"], G)
    assert orc.max_normalised_error(y, g["y"][0]) <= 1e-3
    g = _load(golden_dir, "awq_bias_3d.npz")
    y3 = c_oracle.linear_forward(g["x3"], g["qweight"], g["qzeros"], g["scales"], int(g["group_size"]), g["bias"])
    assert orc.max_normalised_error(y3, g["y3"]) <= 1e-3
    assert c_oracle.threads() >= 1


def _ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in fp16 representable values (sign-magnitude bits mapped onto a line)."""
    def line(v):
        u = v.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(line(a) - line(b))


def test_gated_epilogue_restatement_matches_torch():
    """The epilogue restatements against the tensor operations the reference's layers run on fp16 tensors
    (torch's own CPU kernels): SiLU(gate) * up and the residual add."""
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(11)
    gate = (rng.standard_normal((64, 512)) * 3).astype(np.float16)
    up = (rng.standard_normal((64, 512)) * 2).astype(np.float16)
    ref = (F.silu(torch.from_numpy(gate)) * torch.from_numpy(up)).numpy()
    got = orc.silu_mul(gate, up)
    d = _ulp_distance(got, ref)
    # the last place of exp() is not part of the contract: SiLU may differ by one fp16 place on a few
    # elements, which the product can turn into two
    assert d.max() <= 2 and (d != 0).mean() < 1e-3
    res = (rng.standard_normal((64, 512))).astype(np.float16)
    assert np.array_equal(orc.add_residual(got, res).view(np.uint16),
                          (torch.from_numpy(got) + torch.from_numpy(res)).numpy().view(np.uint16))


def test_interleave_columns_restatement():
    rng = np.random.default_rng(12)
    a, b = rng.integers(0, 16, size=(5, 64)), rng.integers(0, 16, size=(5, 64))
    out = orc.unpack_logical(orc.interleave_columns(orc.pack_logical(a), orc.pack_logical(b)))
    assert np.array_equal(out[:, 0::2], a) and np.array_equal(out[:, 1::2], b)
