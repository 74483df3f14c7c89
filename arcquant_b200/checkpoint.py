"""Reading the reference's calibration artefacts and saving / loading packed layers.

The reference stores, per model, two dictionaries produced by its calibration scripts
(``./saved/<model>_reorder_index_<dataset>.pt`` and ``./saved/<model>_select_num_<dataset>.pt``), keyed
``layers.{i}.{self_attn|mlp}.{proj}.input`` (model/model_utils.py:39-43 of ARCQuant): the channel order
of the input of each projection and the number of residual channels.  q/k/v share the order of
``q_proj``, gate/up the order of ``up_proj``.  This module maps those keys onto the fused linears of
`QLlamaDecoderLayerTP` and saves / restores a layer's packed state (codes, block scales, per-tensor
scale, int16 order, KE, norm gains) so that loading does not re-quantize bf16 weights.
"""
from __future__ import annotations

import torch

KEY = "layers.{}.{}.{}.input"
_SITES = {"q": ("self_attn", "q_proj"), "o": ("self_attn", "o_proj"), "up": ("mlp", "up_proj"),
          "down": ("mlp", "down_proj")}


def layer_indices_from_reference(reorder_index: dict, layer_idx: int) -> dict:
    """{'q','o','up','down'} -> int16 channel order of layer `layer_idx`, from the reference's dictionary."""
    out = {}
    for name, (block, proj) in _SITES.items():
        key = KEY.format(layer_idx, block, proj)
        if key not in reorder_index:
            raise KeyError(f"reference reorder index has no entry '{key}'")
        idx = torch.as_tensor(reorder_index[key]).to(torch.int64).reshape(-1)
        n = idx.numel()
        if n > 32752 or not torch.equal(torch.sort(idx).values, torch.arange(n)):
            raise ValueError(f"'{key}' is not a permutation of 0..{n - 1} that fits int16")
        out[name] = idx.to(torch.int16)
    return out


def layer_select_nums_from_reference(select_nums: dict, layer_idx: int) -> dict:
    """{'q','o','up','down'} -> KE of layer `layer_idx` (multiples of 64 in the reference; 16 is the
    granularity the kernels need)."""
    out = {}
    for name, (block, proj) in _SITES.items():
        key = KEY.format(layer_idx, block, proj)
        if key not in select_nums:
            raise KeyError(f"reference select_num has no entry '{key}'")
        ke = int(select_nums[key])
        if ke < 0 or ke % 16:
            raise ValueError(f"'{key}': select_num {ke} is not a non-negative multiple of 16")
        out[name] = ke
    return out


def save_packed_layer(layer, path: str) -> None:
    """state_dict of a packed layer (uint8 codes and scales, fp32 scalars, int16 orders, bf16 gains)."""
    torch.save({k: v.detach().cpu() for k, v in layer.state_dict().items()}, path)


def load_packed_layer(cfg, path: str, tp_rank: int = 0, tp_size: int = 1, group=None, device="cuda"):
    from .llama_layer import QLlamaDecoderLayerTP

    state = torch.load(path, map_location="cpu")
    return QLlamaDecoderLayerTP.from_packed(cfg, state, tp_rank, tp_size, group, device)
