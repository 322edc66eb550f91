"""Audio helpers (legacy/src/momijo/learn/audio/signal.mojo:35-92)."""
import math

import torch


def hann_window(win_len: int) -> torch.Tensor:
    if win_len <= 1:
        return torch.ones(max(win_len, 0))
    n = torch.arange(win_len, dtype=torch.float32)
    return 0.5 - 0.5 * torch.cos(2 * math.pi * n / (win_len - 1))


def frame_signal(x: torch.Tensor, frame_len: int, hop: int):
    """List of frames (the tail that does not fill a frame is dropped)."""
    n = x.numel()
    return [x[s:s + frame_len] for s in range(0, max(n - frame_len, -1) + 1, hop)] if n >= frame_len else []


def dft_power(frame: torch.Tensor, n_fft: int) -> torch.Tensor:
    """|DFT|^2 for bins 0..n_fft/2 of the zero-padded (or truncated) frame."""
    f = torch.zeros(n_fft, dtype=torch.float32)
    k = min(frame.numel(), n_fft)
    f[:k] = frame[:k].float()
    spec = torch.fft.rfft(f)
    return spec.real ** 2 + spec.imag ** 2


def spectrogram_power(x: torch.Tensor, frame_len: int, hop: int, n_fft: int, window: bool = True):
    w = hann_window(frame_len) if window else torch.ones(frame_len)
    frames = frame_signal(x, frame_len, hop)
    if not frames:
        return torch.zeros(0, n_fft // 2 + 1)
    return torch.stack([dft_power(f.float() * w, n_fft) for f in frames])
