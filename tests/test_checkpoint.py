"""SafeTensors records of NVFP4 parameters: round trip, axis-0 shards by byte span, the
reference's rejection rules (crates/nml-checkpoint/src/lib.rs:569-620)."""
import json

import numpy as np
import pytest
import torch

from helpers import make_weight


def parameter(name, triple, width):
    from nml_b200 import ops
    payload, scales, g = triple
    return ops.NvFp4Parameter.nvfp4(name, tuple(payload.shape[:-1]) + (width,), torch.bfloat16,
                                    torch.from_numpy(payload), torch.from_numpy(scales),
                                    torch.tensor(float(g)))


def test_round_trip_shards_and_index(tmp_path):
    from nml_b200 import checkpoint
    experts = parameter("layers.0.mlp.experts.gate_up_proj", make_weight(1, (8, 12, 48)), 48)
    head = parameter("lm_head.weight", make_weight(2, (64, 80)), 80)
    norm = torch.ones(48, dtype=torch.bfloat16)
    checkpoint.save_nvfp4(tmp_path / "model-00001-of-00002.safetensors", {experts.name: experts},
                          {"norm.weight": norm})
    checkpoint.save_nvfp4(tmp_path / "model-00002-of-00002.safetensors", {head.name: head})
    weight_map = {}
    for file, names in (("model-00001-of-00002.safetensors",
                         [f"{experts.name}.{c}" for c in checkpoint.COMPONENTS] + ["norm.weight"]),
                        ("model-00002-of-00002.safetensors",
                         [f"{head.name}.{c}" for c in checkpoint.COMPONENTS])):
        weight_map.update({name: file for name in names})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    for source in (tmp_path, ):
        ckpt = checkpoint.NvFp4Checkpoint(source)
        assert ckpt.nvfp4_bases() == sorted([experts.name, head.name])
        full = ckpt.load(experts.name, (8, 12, 48), torch.bfloat16)
        assert torch.equal(full.payload, experts.payload)
        assert torch.equal(full.block_scales, experts.block_scales)
        assert full.global_scale.item() == experts.global_scale.item()
        for rank in range(4):  # expert-parallel shards
            shard = ckpt.load_shard(experts.name, (8, 12, 48), torch.bfloat16, rank, 4)
            assert shard.shape == (2, 12, 48)
            assert torch.equal(shard.payload, experts.payload[2 * rank:2 * rank + 2])
            assert torch.equal(shard.block_scales, experts.block_scales[2 * rank:2 * rank + 2])
        columns = ckpt.load_rows(head.name, (64, 80), torch.bfloat16, 16, 48)  # head columns
        assert torch.equal(columns.payload, head.payload[16:48])
        assert torch.equal(ckpt.load_dense("norm.weight"), norm)


def test_rejections(tmp_path):
    from nml_b200 import checkpoint
    from safetensors.torch import save_file
    good = parameter("w", make_weight(3, (4, 32)), 32)
    save_file({"w.payload": good.payload, "w.block_scales": good.block_scales,
               "v.payload": good.payload.clone(),
               "u.payload": good.payload.to(torch.int8),
               "u.block_scales": good.block_scales.clone(),
               "u.global_scale": torch.tensor(1.0)}, str(tmp_path / "bad.safetensors"))
    ckpt = checkpoint.NvFp4Checkpoint(tmp_path / "bad.safetensors")
    with pytest.raises(checkpoint.CheckpointError, match="only 2 of its 3"):
        ckpt.load("w", (4, 32), torch.bfloat16)
    with pytest.raises(checkpoint.CheckpointError, match="only 1 of its 3"):
        ckpt.load("v", (4, 32), torch.bfloat16)
    with pytest.raises(checkpoint.CheckpointError, match="must be U8"):
        ckpt.load("u", (4, 32), torch.bfloat16)
    with pytest.raises(checkpoint.CheckpointError, match="missing tensor"):
        ckpt.load("nothing", (4, 32), torch.bfloat16)
    checkpoint.save_nvfp4(tmp_path / "ok.safetensors", {"w": good})
    ok = checkpoint.NvFp4Checkpoint(tmp_path / "ok.safetensors")
    with pytest.raises(checkpoint.CheckpointError, match="expected shape"):
        ok.load("w", (4, 64), torch.bfloat16)
    with pytest.raises(checkpoint.CheckpointError, match="does not divide"):
        ok.load_shard("w", (4, 32), torch.bfloat16, 0, 3)
    with pytest.raises(checkpoint.CheckpointError, match="ambiguous"):
        checkpoint.save_nvfp4(tmp_path / "two.safetensors",
                              {"a": good, "b": parameter("b", make_weight(3, (4, 32)), 32)})
        checkpoint.NvFp4Checkpoint(tmp_path / "two.safetensors").load(
            "a", (4, 32), torch.bfloat16, aliases=("b",))


def test_loaded_parameter_decodes_like_the_source(tmp_path):
    import oracle
    from nml_b200 import checkpoint
    triple = make_weight(4, (6, 40))
    checkpoint.save_nvfp4(tmp_path / "m.safetensors", {"t": parameter("t", triple, 40)})
    loaded = checkpoint.NvFp4Checkpoint(tmp_path / "m.safetensors").load("t", (6, 40),
                                                                         torch.bfloat16)
    decoded = oracle.dequantize_tensor(loaded.payload.numpy(), loaded.block_scales.numpy(),
                                       np.float32(loaded.global_scale.item()), 40)
    assert np.array_equal(decoded, oracle.dequantize_tensor(*triple, 40))
