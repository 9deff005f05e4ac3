"""Checkpoint shard format: .bin + .json round trip, validation, and loading a model from it."""
import json
import os

import pytest
import torch

from batchgen_b200.ckpt.converter import (ConvertedCheckpoint, convert_dir, convert_shard, save_model_checkpoint,
                                          validate_dir)
from batchgen_b200.config import EngineConfig, get_model_config
from batchgen_b200.models import build_model
from batchgen_b200.models.weights import WeightSource
from batchgen_b200.runtime.engine import Engine
from batchgen_b200.runtime.sequence import SamplingParams


def test_shard_layout_is_back_to_back(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.float32).view(2, 3), "b": torch.ones(5, dtype=torch.bfloat16),
               "c": torch.zeros(0, dtype=torch.int32), "d": torch.tensor([1, 2, 3], dtype=torch.uint8)}
    src = tmp_path / "model-00001.pt"
    torch.save(tensors, src)
    meta_path = convert_shard(str(src), str(tmp_path / "out"))
    meta = json.load(open(meta_path))
    assert meta["file_name"] == "model-00001.bin"
    sd = meta["state_dict"]
    assert list(sd) == ["a", "b", "c", "d"]
    assert sd["a"] == {"dtype": "float32", "shape": [2, 3], "offset": 0, "byte_size": 24}
    assert sd["b"]["offset"] == 24 and sd["b"]["byte_size"] == 10 and sd["d"]["offset"] == 34
    assert meta["total_byte_size"] == 37 == os.path.getsize(tmp_path / "out" / "model-00001.bin")
    raw = open(tmp_path / "out" / "model-00001.bin", "rb").read()
    assert torch.frombuffer(bytearray(raw[:24]), dtype=torch.float32).tolist() == list(range(6))
    assert validate_dir(str(tmp_path / "out")) == 4
    ck = ConvertedCheckpoint(str(tmp_path / "out"))
    for k, v in tensors.items():
        assert torch.equal(ck.get(k), v)


def test_validation_catches_truncation(tmp_path):
    torch.save({"a": torch.ones(8)}, tmp_path / "s.pt")
    convert_shard(str(tmp_path / "s.pt"), str(tmp_path / "o"))
    with open(tmp_path / "o" / "s.bin", "r+b") as f:
        f.truncate(10)
    with pytest.raises(ValueError):
        validate_dir(str(tmp_path / "o"))


def test_model_from_converted_checkpoint_generates_same_tokens(tmp_path):
    cfg = get_model_config("tiny-deepseek-v3")
    src = WeightSource(seed=3)
    save_model_checkpoint(cfg, src, str(tmp_path / "hf"), shard_layers=1)
    metas = convert_dir(str(tmp_path / "hf"), str(tmp_path / "conv"), workers=2)
    assert len(metas) >= 2 and validate_dir(str(tmp_path / "conv")) > 50
    ck = ConvertedCheckpoint(str(tmp_path / "conv"))
    ecfg = EngineConfig(page_size=16, initial_gpu_page_buffer=2, extension_gpu_page_buffer=1, decision_frequency_pages=1)
    prompts = [torch.randint(2, cfg.vocab_size, (20,), generator=torch.Generator().manual_seed(i)).tolist() for i in range(3)]
    params = SamplingParams(max_new_tokens=6, ignore_eos=True)
    a = Engine(build_model(cfg, seed=3), ecfg, num_gpu_pages=32).generate(prompts, params)
    b = Engine(build_model(cfg, seed=999, loader=ck.loader()), ecfg, num_gpu_pages=32).generate(prompts, params)
    assert a == b


def test_published_tensor_names_of_mixtral_and_qwen2_moe_are_found():
    """A checkpoint that uses the families' own names (Mixtral: block_sparse_moe.experts.N.w1/w2/w3 and
    block_sparse_moe.gate; Qwen2-MoE: mlp.shared_expert.*) loads into the same model as the builder's names."""
    import torch
    from batchgen_b200.config import get_model_config
    from batchgen_b200.models import build_model
    from batchgen_b200.models.checkpoint_names import candidates
    from batchgen_b200.models.weights import WeightSource, checkpoint_tensor_specs
    for preset in ("tiny-mixtral", "tiny-qwen2-moe"):
        cfg = get_model_config(preset)
        seeded = WeightSource(seed=3)
        published = {}
        renamed = 0
        for name, shape, kind, _ in checkpoint_tensor_specs(cfg):
            alts = candidates(cfg, name)
            renamed += bool(alts)
            published[alts[0] if alts else name] = seeded.get(name, shape, kind)
        assert renamed > 0
        looked_up = []

        def loader(name, shape):
            looked_up.append(name)
            return published.get(name)

        a = build_model(cfg, seed=3)
        b = build_model(cfg, seed=99, loader=loader)          # another seed: every tensor must come from the loader
        for la, lb in zip(a.w.layers, b.w.layers):
            assert torch.equal(la.experts.w13, lb.experts.w13) and torch.equal(la.router_w, lb.router_w)
            if la.w13 is not None:
                assert torch.equal(la.w13.w, lb.w13.w)
        assert torch.equal(a.w.embed, b.w.embed)
