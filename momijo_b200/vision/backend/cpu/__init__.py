"""Host kernels under the reference's names (legacy/src/momijo/vision/backend/cpu/*.mojo and its ``simd``
sub-package). They are the oracles of the CUDA pixel kernels: plain integer arithmetic on packed HWC
uint8 tensors, always computed on the host. The ``*_simd`` and ``*_tiled`` names give the same results as
the scalar ones (in the reference they differ only in loop structure)."""
from __future__ import annotations

import torch


def clamp_i32(x: int, lo: int, hi: int) -> int:
    return lo if x < lo else (hi if x > hi else x)


def rgb_to_gray_u8_hwc(src: torch.Tensor) -> torch.Tensor:
    """(299 R + 587 G + 114 B) // 1000 per pixel -> [H, W, 1]; images with fewer than three channels come
    back as a packed copy (legacy/src/momijo/vision/backend/cpu/convert_color_cpu.mojo:17-50)."""
    t = src.cpu()
    if t.shape[2] < 3:
        return t.contiguous().clone()
    i = t[..., :3].to(torch.int32)
    y = (i[..., 0] * 299 + i[..., 1] * 587 + i[..., 2] * 114) // 1000
    return y.clamp(0, 255).to(torch.uint8)[..., None].contiguous()


rgb_to_gray_u8_hwc_simd = rgb_to_gray_u8_hwc


def resize_u8_hwc_nearest(src: torch.Tensor, out_h: int, out_w: int) -> torch.Tensor:
    """Nearest neighbour with source index (y * h) // out_h, clamped
    (legacy/src/momijo/vision/backend/cpu/resize_cpu.mojo:22-60)."""
    t = src.cpu()
    h, w = t.shape[0], t.shape[1]
    ys = (torch.arange(out_h, dtype=torch.int64) * h // max(out_h, 1)).clamp(0, h - 1)
    xs = (torch.arange(out_w, dtype=torch.int64) * w // max(out_w, 1)).clamp(0, w - 1)
    return t[ys][:, xs].contiguous()


resize_u8_hwc_nearest_simd = resize_u8_hwc_nearest


def resize_u8_hwc_nearest_tiled_into(src: torch.Tensor, dst: torch.Tensor, tile_h: int, tile_w: int) -> None:
    """Fill ``dst`` (its shape is the output size) tile by tile."""
    out_h, out_w = dst.shape[0], dst.shape[1]
    full = resize_u8_hwc_nearest(src, out_h, out_w)
    th, tw = max(1, tile_h), max(1, tile_w)
    for y0 in range(0, out_h, th):
        for x0 in range(0, out_w, tw):
            dst[y0:y0 + th, x0:x0 + tw] = full[y0:y0 + th, x0:x0 + tw]


def resize_u8_hwc_nearest_tiled(src: torch.Tensor, out_h: int, out_w: int, tile_h: int, tile_w: int) -> torch.Tensor:
    dst = torch.zeros(out_h, out_w, src.shape[2], dtype=torch.uint8)
    resize_u8_hwc_nearest_tiled_into(src, dst, tile_h, tile_w)
    return dst
