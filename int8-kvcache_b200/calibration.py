"""Static scale calibration from K/V dumps.

The reference calibrates by running Qwen2.5-7B over 40 prompts and keeping, per layer and KV head, the running
absolute maximum of K and of V; scale = max(amax / 127, 1e-6) (scripts/04_calibrate_static_scale.py:25-65).  The
model run itself is outside this package; this module is the accumulation and the file format, fed with K/V tensors
that the caller collected (for instance dumps in the layout of the reference's outputs/kv_sample.pt:
{layer_index: {"k": [N, Hkv, T, D], "v": [N, Hkv, T, D]}}).
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch


class ScaleCalibrator:
    """Running per-(layer, KV head) absolute maxima of K and V."""

    def __init__(self, num_layers: int, num_kv_heads: int):
        self.k_amax = torch.zeros(num_layers, num_kv_heads, dtype=torch.float32)
        self.v_amax = torch.zeros_like(self.k_amax)

    def observe(self, layer: int, k: torch.Tensor, v: torch.Tensor, head_axis: int = 1) -> None:
        """k, v: any float tensors whose `head_axis` is the KV-head axis ([N, Hkv, T, D] by default)."""
        for amax, x in ((self.k_amax, k), (self.v_amax, v)):
            dims = tuple(d for d in range(x.ndim) if d != head_axis % x.ndim)
            amax[layer] = torch.maximum(amax[layer], x.detach().float().abs().amax(dim=dims).cpu())

    def observe_dump(self, dump: Mapping[int, Mapping[str, torch.Tensor]]) -> None:
        for layer, kv in dump.items():
            self.observe(int(layer), kv["k"], kv["v"])

    def scales(self) -> Dict[str, torch.Tensor]:
        """The dict the reference saves: k_scale, v_scale, k_amax, v_amax, each [num_layers, Hkv] fp32."""
        return {
            "k_scale": (self.k_amax / 127.0).clamp_min(1e-6),
            "v_scale": (self.v_amax / 127.0).clamp_min(1e-6),
            "k_amax": self.k_amax.clone(),
            "v_amax": self.v_amax.clone(),
        }

    def save(self, path: str) -> None:
        torch.save(self.scales(), path)
