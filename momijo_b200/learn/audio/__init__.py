from .signal import hann_window, frame_signal, dft_power, spectrogram_power  # noqa: F401
