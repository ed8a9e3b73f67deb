"""CPU: the safetensors reader/writer of the checkpoint ingest against the safetensors package,
and its refusal of malformed files."""
import json
import os
import struct

import pytest
import torch

from moe_gen_b200 import ingest
from oracle import moe_oracle as O


def _tensors():
    g = torch.Generator().manual_seed(5)
    return {
        "model.layers.3.mlp.gate.weight": torch.randn(8, 64, generator=g).to(torch.bfloat16),
        "model.layers.3.mlp.gate.e_score_correction_bias": torch.randn(8, generator=g),
        "model.layers.3.mlp.experts.0.up_proj.weight": torch.randn(128, 64, generator=g).to(torch.float8_e4m3fn),
        "model.layers.3.mlp.experts.0.up_proj.weight_scale_inv": torch.rand(1, 1, generator=g),
        "empty": torch.empty(0, 4, dtype=torch.bfloat16),
    }


def test_written_file_is_read_back_and_by_the_safetensors_package(tmp_path):
    path = str(tmp_path / "a.safetensors")
    t = _tensors()
    ingest.write_safetensors(path, t, metadata={"format": "pt"})
    f = ingest.SafetensorsFile(path)
    assert set(f.tensors) == set(t)
    for name, want in t.items():
        got = f.tensor(name)
        assert got.dtype == want.dtype and got.shape == want.shape
        assert torch.equal(got.view(torch.uint8), want.contiguous().view(torch.uint8))
        assert f.raw(name).size == want.numel() * want.element_size()
    f.close()
    st = pytest.importorskip("safetensors.torch")
    theirs = st.load_file(path)
    for name, want in t.items():
        assert torch.equal(theirs[name].view(torch.uint8), want.contiguous().view(torch.uint8))


def test_files_of_the_safetensors_package_are_read(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    path = str(tmp_path / "b.safetensors")
    t = {k: v for k, v in _tensors().items() if v.numel()}
    st.save_file(t, path)
    f = ingest.SafetensorsFile(path)
    for name, want in t.items():
        assert torch.equal(f.tensor(name).view(torch.uint8), want.contiguous().view(torch.uint8))
    f.close()


def test_malformed_files_are_refused(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        ingest.SafetensorsFile(str(p))
    p = tmp_path / "len.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError):
        ingest.SafetensorsFile(str(p))
    hdr = json.dumps({"x": {"dtype": "BF16", "shape": [4, 4], "data_offsets": [0, 8]}}).encode()
    p = tmp_path / "span.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(ValueError):                      # 4x4 bf16 needs 32 bytes, the entry spans 8
        ingest.SafetensorsFile(str(p))
    hdr = json.dumps({"x": {"dtype": "BF16", "shape": [4, 4], "data_offsets": [0, 32]}}).encode()
    p = tmp_path / "past_end.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(ValueError):
        ingest.SafetensorsFile(str(p))
    hdr = json.dumps({"x": {"dtype": "C64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    p = tmp_path / "dtype.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(ValueError):
        ingest.SafetensorsFile(str(p))


def test_checkpoint_finds_tensors_across_shards_and_through_the_index(tmp_path):
    spec = O.LayerSpec(128, 128, 4, 2, 128, 1, 1, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_FP8_BLOCK128, O.COMBINE_FP32)
    _, W = O.make_inputs(spec, 4, 1)
    experts = [(W.q_gate[e], W.q_up[e], W.q_down[e]) for e in range(4)]
    ingest.export_moe_layer(str(tmp_path / "model-00001-of-00002.safetensors"), 7, W.gate_w, W.bias, experts[:2])
    # second shard: experts 2 and 3 under their own numbers
    gate_n, bias_n, exp_n, mats, shared_n = ingest.NAMING["deepseek"]
    second = {}
    for e in (2, 3):
        for m, (q, s) in zip(mats, experts[e]):
            n = exp_n.format(p="model.layers.7", e=e, m=m)
            second[n + ".weight"], second[n + ".weight_scale_inv"] = q, s
    ingest.write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), second)
    ck = ingest.Checkpoint(str(tmp_path))
    n3 = "model.layers.7.mlp.experts.3.down_proj.weight"
    assert n3 in ck and os.path.basename(ck.file_of(n3).path) == "model-00002-of-00002.safetensors"
    assert torch.equal(ck.file_of(n3).tensor(n3).view(torch.uint8), W.q_down[3][0].view(torch.uint8))
    with pytest.raises(KeyError):
        ck.file_of("model.layers.7.mlp.experts.9.down_proj.weight")
    ck.close()
    # with an index file only the named shard is opened
    wm = {n3: "model-00002-of-00002.safetensors"}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    ck = ingest.Checkpoint(str(tmp_path))
    assert n3 in ck and "model.layers.7.mlp.gate.weight" not in ck
    assert list(ck._files) == []
    ck.file_of(n3)
    assert len(ck._files) == 1
    ck.close()
