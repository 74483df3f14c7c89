"""Host logic of the checkpoint helpers: the reference's dictionary keys, validation, and rebuilding a
layer from packed buffers (no GPU: the buffers are made up, nothing is computed)."""
import pytest
import torch

from arcquant_b200 import checkpoint
from arcquant_b200.llama_layer import LlamaLayerConfig, PackedLinear, QLlamaDecoderLayerTP


def _ref_dicts(hidden=256, ffn=512, layer=3):
    g = torch.Generator().manual_seed(0)
    ri, sn = {}, {}
    for block, proj, n in (("self_attn", "q_proj", hidden), ("self_attn", "o_proj", hidden), ("mlp", "up_proj", hidden),
                           ("mlp", "down_proj", ffn)):
        key = f"layers.{layer}.{block}.{proj}.input"
        ri[key] = torch.randperm(n, generator=g)
        sn[key] = 64
    return ri, sn


def test_reference_keys_map_to_the_fused_linears():
    ri, sn = _ref_dicts()
    idx = checkpoint.layer_indices_from_reference(ri, 3)
    ke = checkpoint.layer_select_nums_from_reference(sn, 3)
    assert set(idx) == set(ke) == {"q", "o", "up", "down"}
    assert idx["down"].dtype == torch.int16 and idx["down"].numel() == 512
    assert torch.equal(idx["q"].long(), ri["layers.3.self_attn.q_proj.input"])
    with pytest.raises(KeyError):
        checkpoint.layer_indices_from_reference(ri, 4)
    bad = dict(ri)
    bad["layers.3.mlp.up_proj.input"] = torch.zeros(256, dtype=torch.int64)
    with pytest.raises(ValueError):
        checkpoint.layer_indices_from_reference(bad, 3)
    sn["layers.3.mlp.up_proj.input"] = 50
    with pytest.raises(ValueError):
        checkpoint.layer_select_nums_from_reference(sn, 3)


def _fake_packed(rows, kq, ke, prefix):
    k_eff = kq + ke
    return {prefix + "W": torch.zeros((rows, k_eff // 2), dtype=torch.uint8),
            prefix + "SFW": torch.zeros(((rows // 128 + 1) * 128 * k_eff // 16,), dtype=torch.uint8),
            prefix + "scale": torch.tensor(0.5), prefix + "index": torch.arange(kq, dtype=torch.int16),
            prefix + "select_num_t": torch.tensor(ke, dtype=torch.int32)}


def test_layer_is_rebuilt_from_packed_buffers_and_round_trips(tmp_path):
    cfg = LlamaLayerConfig(hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, select_num=64)
    state = {"ln1": torch.ones(256, dtype=torch.bfloat16), "ln2": torch.ones(256, dtype=torch.bfloat16)}
    state.update(_fake_packed((4 + 2 * 2) * 64, 256, 64, "qkv."))
    state.update(_fake_packed(2 * 512, 256, 64, "gate_up."))
    state.update(_fake_packed(256, 256, 64, "o."))
    state.update(_fake_packed(256, 512, 64, "down."))
    layer = QLlamaDecoderLayerTP.from_packed(cfg, state, device="cpu")
    assert layer.down.select_num == 64 and layer.qkv.W.shape == (512, 160)
    sd = layer.state_dict()
    assert set(sd) == set(state) | {"fuse_swiglu_t"}           # a state without the flag: [gate | up] halves
    assert int(sd["fuse_swiglu_t"]) == 0 and not layer.fuse_swiglu
    path = str(tmp_path / "layer.pt")
    checkpoint.save_packed_layer(layer, path)
    again = checkpoint.load_packed_layer(cfg, path, device="cpu")
    for k, v in again.state_dict().items():
        assert torch.equal(v, sd[k])
    # a state saved for another tensor-parallel degree is refused
    with pytest.raises(ValueError):
        QLlamaDecoderLayerTP.from_packed(cfg, state, tp_rank=0, tp_size=2, device="cpu")
    del state["o.SFW"]
    with pytest.raises(KeyError):
        PackedLinear.from_packed(state, "o.")
