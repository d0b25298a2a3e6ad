"""The checkpoint reader / writer: the container format against the `safetensors` package where it is
installed, and the fill of a model's quantized linears.  CPU only (the repack step is skipped for CPU modules)."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

from llmrqt_sdv1_b200 import AWQLinear_GEMM, checkpoint
from oracle import awq_oracle as orc


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.norm = nn.LayerNorm(256)
        self.proj = AWQLinear_GEMM(4, 128, 256, 64, True, "cpu")
        self.head = nn.Linear(64, 8, bias=False)


def _filled_block(seed):
    blk = _Block()
    qw, qz, sc = orc.make_awq_tensors(256, 64, 128, seed=seed)
    blk.proj.qweight, blk.proj.qzeros, blk.proj.scales = torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc)
    blk.proj.bias = torch.randn(64, generator=torch.Generator().manual_seed(seed)).half()
    return blk.half()


def test_round_trip_and_strictness(tmp_path):
    src = _filled_block(1)
    path = os.path.join(tmp_path, "model.safetensors")
    checkpoint.save_checkpoint(src.state_dict(), path, metadata={"format": "pt"})
    header, start = checkpoint.read_header(path)
    assert set(header) == set(src.state_dict()) and start % 8 == 0
    assert header["proj.qweight"] == {"dtype": "I32", "shape": [256, 8], "data_offsets": header["proj.qweight"]["data_offsets"]}
    dst = _filled_block(2)
    report = checkpoint.load_checkpoint(dst, path)
    assert not report["missing"] and not report["unexpected"]
    for k, v in src.state_dict().items():
        assert torch.equal(dst.state_dict()[k], v), k
    # a directory of shards, a float32 destination (cast), and the strict / non-strict reports
    os.makedirs(os.path.join(tmp_path, "shards"))
    sd = src.state_dict()
    names = sorted(sd)
    checkpoint.save_checkpoint({k: sd[k] for k in names[:3]}, os.path.join(tmp_path, "shards", "a.safetensors"))
    checkpoint.save_checkpoint({k: sd[k] for k in names[3:]}, os.path.join(tmp_path, "shards", "b.safetensors"))
    dst = _filled_block(3)
    dst.norm.float()
    checkpoint.load_checkpoint(dst, os.path.join(tmp_path, "shards"))
    assert torch.equal(dst.norm.weight, sd["norm.weight"].float()) and torch.equal(dst.proj.qzeros, sd["proj.qzeros"])
    checkpoint.save_checkpoint({"proj.qweight": sd["proj.qweight"], "extra": torch.zeros(3)}, path)
    with pytest.raises(KeyError):
        checkpoint.load_checkpoint(_filled_block(4), path)
    report = checkpoint.load_checkpoint(_filled_block(4), path, strict=False)
    assert report["unexpected"] == ["extra"] and "proj.scales" in report["missing"] and report["loaded"] == ["proj.qweight"]
    checkpoint.save_checkpoint({"proj.qweight": torch.zeros((4, 4), dtype=torch.int32)}, path)
    with pytest.raises(ValueError):
        checkpoint.load_checkpoint(_filled_block(4), path, strict=False)


def test_container_agrees_with_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    state = {"a.qweight": torch.randint(-2**31, 2**31 - 1, (16, 4), dtype=torch.int64).to(torch.int32),
             "a.scales": torch.randn(2, 32).half(), "b": torch.randn(5, 3).bfloat16(), "c": torch.arange(7, dtype=torch.uint8),
             "empty": torch.zeros((0, 4)), "scalar": torch.tensor(3.5)}
    mine, theirs = os.path.join(tmp_path, "mine.safetensors"), os.path.join(tmp_path, "theirs.safetensors")
    checkpoint.save_checkpoint(state, mine)
    back = st.load_file(mine)
    assert set(back) == set(state)
    for k in state:
        assert back[k].dtype == state[k].dtype and torch.equal(back[k], state[k]), k
    st.save_file(state, theirs)
    got = dict(checkpoint.iter_tensors(theirs))
    assert set(got) == set(state)
    for k in state:
        assert got[k].dtype == state[k].dtype and torch.equal(got[k], state[k]), k
    assert [n for n, _ in checkpoint.iter_tensors(theirs, names=["b"])] == ["b"]


def test_malformed_files_are_rejected(tmp_path):
    path = os.path.join(tmp_path, "bad.safetensors")
    with open(path, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(ValueError):
        checkpoint.read_header(path)
    with open(path, "wb") as f:
        f.write((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(ValueError):
        checkpoint.read_header(path)
    import json
    hdr = json.dumps({"t": {"dtype": "F16", "shape": [4], "data_offsets": [0, 6]}}).encode()
    with open(path, "wb") as f:
        f.write(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 6)
    with pytest.raises(ValueError):
        checkpoint.read_header(path)
    with pytest.raises(FileNotFoundError):
        checkpoint.checkpoint_files(str(tmp_path / "nothing_here") if os.makedirs(tmp_path / "nothing_here") is None else "")
