"""Static per-(layer, KV head) scales: the file format and lookups of the reference's vllm_int8/static_scales.py:9-75.

The file is a torch-saved dict with fp32 tensors `k_scale` and `v_scale` of shape [num_layers, Hkv] (what the
reference's calibration script writes, scripts/04_calibrate_static_scale.py:57-65).  A layer's row is found from the
layer index inside its vLLM name ("model.layers.12.self_attn.attn" -> 12).
"""

from __future__ import annotations

import re
from typing import Optional, Tuple

import torch

_SCALES: Optional[dict] = None
_LAYER_RE = re.compile(r"layers\.(\d+)")


def set_static_scales(k_scale: torch.Tensor, v_scale: torch.Tensor) -> None:
    """Install scales that are already in memory ([num_layers, Hkv] each)."""
    global _SCALES
    assert k_scale.ndim == 2 and k_scale.shape == v_scale.shape
    _SCALES = {"k_scale": k_scale.detach().float().cpu(), "v_scale": v_scale.detach().float().cpu()}


def load_static_scales(path: str) -> None:
    data = torch.load(path, map_location="cpu")
    set_static_scales(data["k_scale"], data["v_scale"])


def clear_static_scales() -> None:
    global _SCALES
    _SCALES = None


def extract_layer_idx(layer_name: str) -> int:
    found = _LAYER_RE.search(layer_name)
    if found is None:
        raise RuntimeError(f"Cannot extract layer index from {layer_name}")
    return int(found.group(1))


def get_layer_scales(layer_name: str, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """(k_scale, v_scale) of the layer as contiguous fp32 [Hkv] tensors on `device`."""
    if _SCALES is None:
        raise RuntimeError("Call load_static_scales() first.")
    idx = extract_layer_idx(layer_name)
    pick = lambda name: _SCALES[name][idx].to(device=device, dtype=torch.float32).contiguous()
    return pick("k_scale"), pick("v_scale")
